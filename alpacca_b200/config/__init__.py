from .base import ConfigError, ModelConfig
from .llama import LlamaConfig
from .registry import (Architecture, config_from_dict, get_architecture, load_config,
                       register_architecture, registered_architectures, unregister_architecture)

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "Architecture", "config_from_dict",
           "get_architecture", "load_config", "register_architecture", "registered_architectures",
           "unregister_architecture"]
