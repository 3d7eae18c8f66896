"""quench6k_b200: a single-GPU, B200-native inference engine for the Recursive Flint MoE decoder."""
__version__ = "0.1.0"

from . import config as config            # noqa: F401  (registers nothing by itself)
from .models import flint as _flint       # noqa: F401  (registers FlintForCausalLM)
from .sampling.params import SamplingParams      # noqa: F401
from .engine.engine import Engine, RequestOutput   # noqa: F401
