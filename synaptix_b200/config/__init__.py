from .base import ConfigError, ModelConfig, read_config_json, take
from .qwen3 import Qwen3Config
from .registry import (ArchitectureEntry, load_config, register_architecture,
                       registered_architectures, resolve_architecture)

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "read_config_json", "take",
           "ArchitectureEntry", "load_config", "register_architecture",
           "registered_architectures", "resolve_architecture"]
