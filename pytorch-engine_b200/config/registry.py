"""The one registry from an architecture's name to its model.

An architecture is a configuration class and a *plan* function that turns a configuration
into a ``ModelPlan`` (``parts/spec.py``).  ``config.json``'s ``architectures[0]`` picks the entry
everywhere: loader, engine, command line and trace replay.  The reference has no registry (it
branches on an ``arch`` string and on tensor-name presence, pygguf_engine/model.py:800, 982-1003,
pygguf_engine/gguf_parser.py:397); this table replaces those branches.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Type

from .base import ConfigError, ModelConfig, read_config_dict


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Type[ModelConfig]
    plan: Callable[[ModelConfig], Any]  # -> parts.spec.ModelPlan


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Type[ModelConfig], plan: Callable[[ModelConfig], Any],
                          *, replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise KeyError(f"architecture {name!r} is already registered")
    arch = Architecture(name, config_class, plan)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(sorted(_ARCHITECTURES)) or 'none'}"
        )
    return _ARCHITECTURES[name]


def architecture_names():
    return sorted(_ARCHITECTURES)


def architecture_of(config_dict: Dict[str, Any]) -> Architecture:
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json: missing key 'architectures' (a list whose first entry names the model)")
    return architecture(str(archs[0]))


def load_config(folder: str) -> ModelConfig:
    """Typed configuration of a model folder, class chosen by ``architectures[0]``."""
    d = read_config_dict(folder)
    return architecture_of(d).config_class.from_dict(d)
