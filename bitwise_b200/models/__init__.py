from .decoder import DecoderModel, LayerRun, sequential_schedule
from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from . import nuderax  # noqa: F401  (registers Nuderax)
from . import favudra  # noqa: F401  (registers Favudra)
from . import sebavik  # noqa: F401  (registers Sebavik)
from . import kezuvik  # noqa: F401  (registers Kezuvik)

__all__ = ["DecoderModel", "LayerRun", "sequential_schedule"]
