from .decoder import DecoderModel, LayerRun, sequential_schedule
from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from . import nuderax  # noqa: F401  (registers Nuderax)
from . import favudra  # noqa: F401  (registers Favudra)
from . import sebavik  # noqa: F401  (registers Sebavik)

__all__ = ["DecoderModel", "LayerRun", "sequential_schedule"]
