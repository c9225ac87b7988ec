from .base import (
    Architecture,
    ConfigError,
    ModelConfig,
    load_config,
    parse_config,
    read_config_json,
    register_architecture,
    registered_architectures,
    resolve_architecture,
    unregister_architecture,
)
from .engine import EngineConfig
from .gpt2 import GPT2Config

__all__ = [
    "Architecture",
    "ConfigError",
    "EngineConfig",
    "GPT2Config",
    "ModelConfig",
    "load_config",
    "parse_config",
    "read_config_json",
    "register_architecture",
    "registered_architectures",
    "resolve_architecture",
    "unregister_architecture",
]
