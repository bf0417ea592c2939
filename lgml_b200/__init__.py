"""lgml_b200: a small, whole inference engine for one B200, after mischief/lgml.

Token ids in, next tokens out, for the Llama dense decoder: typed configuration and
an architecture registry, safetensors weights by name, layers assembled from parts, a
paged cache with block tables, one step function over mixed batches, a scheduler,
mischief/lgml's sampler, and hand-written sm_100a kernels with a true 32-bit twin.
"""
from . import models  # noqa: F401  (registers the architectures)
from .config import ConfigError, LlamaConfig, load_config
from .engine.engine import Engine
from .engine.runner import ModelRunner
from .sampling import Sampler, SamplingParams
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "LlamaConfig", "load_config", "Engine", "ModelRunner", "Sampler", "SamplingParams",
           "WeightError", "write_random_model"]
__version__ = "0.1.0"
