"""Typed configurations and the architecture registry."""
from .base import (Architecture, ConfigError, ModelConfig, architecture_name, load_config, lookup_architecture,
                   read_config_json, register_architecture, registered_architectures, unregister_architecture)
from .qwen3 import Qwen3Config, qwen3_model_spec

__all__ = [
    "Architecture", "ConfigError", "ModelConfig", "Qwen3Config", "architecture_name", "load_config",
    "lookup_architecture", "qwen3_model_spec", "read_config_json", "register_architecture",
    "registered_architectures", "unregister_architecture",
]
