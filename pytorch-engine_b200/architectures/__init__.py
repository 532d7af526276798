"""Architectures known to the registry.  Each module turns a typed configuration into a plan of
parts and registers itself under the name that ``config.json`` carries in ``architectures[0]``."""
from . import qwen3  # noqa: F401

__all__ = ["qwen3"]
