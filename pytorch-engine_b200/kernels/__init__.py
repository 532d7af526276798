"""The CUDA library of this package: build, load, and tensor-level wrappers (no fallback)."""
from . import build, lib, ops
from .lib import KernelError, library, library_path

__all__ = ["build", "lib", "ops", "KernelError", "library", "library_path"]
