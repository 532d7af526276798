"""The one registry from an architecture's name to its model.

An architecture is a configuration class and a *plan* function that turns a configuration
into a ``ModelPlan`` (``parts/spec.py``).  ``config.json``'s ``architectures[0]`` picks the entry
everywhere: loader, engine, command line and trace replay.  The reference has no registry (it
branches on an ``arch`` string and on tensor-name presence, pygguf_engine/model.py:800, 982-1003,
pygguf_engine/gguf_parser.py:397); this table replaces those branches.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Type

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


# ---- named presets ---------------------------------------------------------------------------------
# A preset is a config.json under another name: ``<folder>/<name>.json``.  Which configuration class reads
# it is decided by its own ``architectures[0]``, as for a model folder, so an architecture brings its presets
# by registering a folder; no size stands in code.
_PRESET_FOLDERS: List[str] = []


def register_preset_folder(folder: str) -> None:
    """Make every ``*.json`` of ``folder`` a preset (``--random NAME``, ``preset(NAME)``)."""
    folder = os.path.abspath(folder)
    if folder not in _PRESET_FOLDERS:
        _PRESET_FOLDERS.append(folder)


def unregister_preset_folder(folder: str) -> None:
    folder = os.path.abspath(folder)
    if folder in _PRESET_FOLDERS:
        _PRESET_FOLDERS.remove(folder)


def _preset_files() -> Dict[str, str]:
    found: Dict[str, str] = {}
    for folder in _PRESET_FOLDERS:
        if os.path.isdir(folder):
            for f in sorted(os.listdir(folder)):
                if f.endswith(".json"):
                    found.setdefault(f[:-5], os.path.join(folder, f))
    return found


def preset_names():
    return sorted(_preset_files())


def preset(name: str, **overrides: Any) -> ModelConfig:
    """The typed configuration of preset ``name``; ``overrides`` replace keys of its JSON first."""
    files = _preset_files()
    if name not in files:
        raise ConfigError(f"unknown preset {name!r}; known: {', '.join(sorted(files)) or 'none'}")
    with open(files[name]) as fh:
        d = json.load(fh)
    d.update(overrides)
    return architecture_of(d).config_class.from_dict(d)
