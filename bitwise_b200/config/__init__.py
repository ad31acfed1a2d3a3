from .base import ConfigError, read_config_json
from .favudra import FavudraConfig, FavudraLayerConfig, FavudraMixerConfig
from .kezuvik import KezuvikConfig, KezuvikLayerConfig, KezuvikMixerConfig, RotScalingConfig
from .llama import LlamaConfig, RopeScaling
from .nuderax import LatentMixerConfig, NuderaxConfig, NuderaxLayerConfig, RoutedMlpConfig
from .sebavik import BigramConfig, SebavikConfig, SebavikLayerConfig, SebavikMixerConfig, SebavikMlpConfig
from .registry import (Architecture, architecture_of, config_from_folder, known_architectures,
                       lookup_architecture, register_architecture)

__all__ = ["KezuvikConfig", "KezuvikLayerConfig", "KezuvikMixerConfig", "RotScalingConfig", "BigramConfig", "SebavikConfig", "SebavikLayerConfig", "SebavikMixerConfig", "SebavikMlpConfig", "ConfigError", "FavudraConfig", "FavudraLayerConfig", "FavudraMixerConfig", "LlamaConfig", "RopeScaling", "NuderaxConfig", "NuderaxLayerConfig", "LatentMixerConfig",
           "RoutedMlpConfig", "read_config_json", "Architecture",
           "architecture_of", "config_from_folder", "known_architectures", "lookup_architecture",
           "register_architecture"]
