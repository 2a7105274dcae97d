"""serve_b200: a small, whole inference engine for one B200, for the Llama dense decoder.

From a model folder (config.json + safetensors) or seeded random weights to
generated tokens: typed configuration and architecture registry, weights by
tensor name, layers put together from parts, a paged cache with block tables
and state slots, one step function for mixed batches, a scheduler with chunked
prefill, sampling, and hand-written sm_100a kernels underneath.
"""
from . import models, parts  # noqa: F401  (register architectures and parts)
from .config import EngineConfig, load_config, load_preset  # noqa: F401
from .engine import Engine, StepEntry  # noqa: F401

from .run import Request, generate, load_model  # noqa: F401,E402

__version__ = "0.1.0"
