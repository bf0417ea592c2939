from .base import (ConfigError, ModelConfig, architecture_of, architectures, config_from_dict,
                   load_config, lookup_architecture, register_architecture)
from .llama import LlamaConfig, RopeScaling

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "RopeScaling", "architecture_of", "architectures",
           "config_from_dict", "load_config", "lookup_architecture", "register_architecture"]
