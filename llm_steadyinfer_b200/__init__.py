"""A small, whole, single-GPU inference engine for the Llama 3 dense architecture on B200:
typed configuration and architecture registry, weights by tensor name, layers put together
from parts, a paged cache manager, one step function for mixed batches, a scheduler,
sampling, and hand-written sm_100a kernels with a bfloat16 and a true float32 path.
"""
from . import models as _models  # noqa: F401  (registers the architectures)

__version__ = "0.1.0"

from .engine import LLM, GenerationResult  # noqa: E402
from .sampling import SamplingParams  # noqa: E402
