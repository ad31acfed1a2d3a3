from .attention import GQAAttention
from .base import (FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, FeedForward, Mixer, Norm, PagedKVNeed,
                   PagedKVView, PagedLatentNeed, PagedLatentView, Part, PositionEncoding, SlotStateNeed, SlotStateView, StepContext, Workspace,
                   register_feed_forward, register_mixer, register_norm, register_position_encoding)
from .block import DepthMix, ParallelBlock, PreNormBlock, SandwichBlock, ScaledResidualBlock
from .token_side import TokenSide, TokenSideTable
from .embedding import OutputHead, TokenEmbedding
from .mlp import SwiGLU
from .latent_attention import LatentAttention
from .linear_recurrence import GatedLinearAttention
from .norm import LayerNorm, RMSNorm
from .rope import RotaryEncoding, inverse_frequencies
from .routed_ffn import ClampedGLU, RoutedFFN
from .scored_attention import SEQUENCE_TILE, ScoredAttention, distance_slopes
