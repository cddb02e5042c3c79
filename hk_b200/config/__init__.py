from .base import (ConfigError, ModelConfig, architecture_name, config_from_dict, load_config,
                   register_architecture, resolve_architecture, supported_architectures)
from .qwen3 import Qwen3Config

__all__ = [
    "ConfigError", "ModelConfig", "Qwen3Config", "architecture_name", "config_from_dict", "load_config",
    "register_architecture", "resolve_architecture", "supported_architectures",
]
