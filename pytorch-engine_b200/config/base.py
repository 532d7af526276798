"""What every architecture's typed configuration has in common.

A configuration class reads the architecture's own ``config.json`` keys, checks them, and can
write them back.  It holds numbers only; how those numbers become layers is the job of the
architecture's *plan* function (see ``config/registry.py`` and ``parts/spec.py``).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Tuple


class ConfigError(ValueError):
    """A ``config.json`` that cannot be used; the message names the key at fault."""


class ModelConfig:
    """Base class of typed configurations.

    Subclasses are frozen dataclasses that implement ``from_dict`` (validate and build) and
    ``to_dict`` (the same keys that ``config.json`` carries).  ``architecture`` is the name the
    registry knows the model by (``architectures[0]`` in ``config.json``).
    """

    architecture: str = ""

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":  # pragma: no cover - interface
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:  # pragma: no cover - interface
        raise NotImplementedError

    # ---- what the engine needs of any configuration -------------------------------------
    @property
    def max_positions(self) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    @property
    def stop_token_ids(self) -> Tuple[int, ...]:
        return ()

    @property
    def bos_token(self) -> int:
        return 0

    # ---- files ---------------------------------------------------------------------------
    @classmethod
    def from_json(cls, path: str) -> "ModelConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as fh:
            return cls.from_dict(json.load(fh))

    def save(self, folder: str) -> str:
        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, "config.json")
        with open(path, "w") as fh:
            json.dump(self.to_dict(), fh, indent=2)
            fh.write("\n")
        return path


def read_config_dict(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in model folder {folder!r}")
    with open(path) as fh:
        d = json.load(fh)
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: config.json must hold a JSON object")
    return d


def require_int(d: Dict[str, Any], key: str, *, minimum: int = 1, default: Any = None) -> int:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: missing key {key!r}")
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: {key!r} must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: {key!r} must be >= {minimum}, got {v}")
    return v


def require_float(d: Dict[str, Any], key: str, *, positive: bool = True, default: Any = None) -> float:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: missing key {key!r}")
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {key!r} must be a number, got {v!r}")
    v = float(v)
    if positive and not v > 0.0:
        raise ConfigError(f"config.json: {key!r} must be > 0, got {v}")
    return v
