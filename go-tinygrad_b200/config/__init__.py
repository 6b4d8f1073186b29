from .llama import ConfigError, LlamaConfig, RopeScaling
from .registry import (Architecture, find_architecture, read_config_json, read_model_config,
                       register_architecture, registered_architectures, unregister_architecture)

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "Architecture", "find_architecture",
           "read_config_json", "read_model_config", "register_architecture",
           "registered_architectures", "unregister_architecture"]
