from .base import ConfigError, KeyReader, read_config_json
from .llama import LlamaConfig, RopeScaling
from .registry import (Architecture, architecture_name, register_architecture,
                       registered_architectures, resolve_architecture)

__all__ = [
    "ConfigError", "KeyReader", "read_config_json", "LlamaConfig", "RopeScaling", "Architecture",
    "architecture_name", "register_architecture", "registered_architectures", "resolve_architecture",
]
