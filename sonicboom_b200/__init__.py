"""sonicboom_b200: a small model library with generation of its own for one B200.

Everything between a request's tokens and its next token for the Qwen2.5 dense decoder, in the
spirit of hardenedlinux/SonicBoom's generation path and built for sm_100a: typed
configuration and an architecture registry, weights by tensor name, layers put together from
parts, a paged cache with slots, one step function, a generation loop with the reference's
sampler, hand-written CUDA kernels, and a true float32 path.
"""
from .config import ConfigError, Qwen2Config, register_architecture
from .engine import Engine, StepEntry, StepError
from .models import DecoderModel, load_model, random_model
from .weights import WeightError, write_random_model

__version__ = "0.2.0"
from .buildinfo import build_info, build_info_line
__all__ = ["ConfigError", "Qwen2Config", "register_architecture", "Engine", "StepEntry",
           "StepError", "DecoderModel", "load_model", "random_model", "WeightError",
           "write_random_model", "build_info", "build_info_line"]
