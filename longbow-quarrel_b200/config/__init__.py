from .base import ConfigError, read_config_json
from .llama import LlamaConfig, RopeScaling, FULL_ATTENTION, SLIDING_ATTENTION
from .registry import (Architecture, architecture_of, load_config, register_architecture,
                       registered_architectures)

__all__ = ["ConfigError", "read_config_json", "LlamaConfig", "RopeScaling", "FULL_ATTENTION",
           "SLIDING_ATTENTION", "Architecture", "architecture_of", "load_config",
           "register_architecture", "registered_architectures"]
