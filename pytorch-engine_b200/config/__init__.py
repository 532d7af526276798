"""Typed configurations and the registry from an architecture's name to its model."""
from .base import ConfigError, ModelConfig, read_config_dict
from .registry import (Architecture, architecture, architecture_names, architecture_of, load_config, preset,
                       preset_names, register_architecture, register_preset_folder, unregister_architecture,
                       unregister_preset_folder)
from .qwen3 import Qwen3Config

__all__ = [
    "ConfigError", "ModelConfig", "read_config_dict", "Architecture", "architecture", "architecture_names",
    "architecture_of", "load_config", "register_architecture", "unregister_architecture", "Qwen3Config",
    "preset", "preset_names", "register_preset_folder", "unregister_preset_folder",
]
