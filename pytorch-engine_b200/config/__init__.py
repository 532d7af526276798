"""Typed configurations and the registry from an architecture's name to its model."""
from .base import ConfigError, ModelConfig, read_config_dict
from .registry import (Architecture, architecture, architecture_names, architecture_of, load_config,
                       register_architecture, unregister_architecture)
from .qwen3 import Qwen3Config, preset, preset_names

__all__ = [
    "ConfigError", "ModelConfig", "read_config_dict", "Architecture", "architecture", "architecture_names",
    "architecture_of", "load_config", "register_architecture", "unregister_architecture", "Qwen3Config",
    "preset", "preset_names",
]
