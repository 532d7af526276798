"""Loads the CUDA library and declares the C signature of every entry point.

There is no fallback: if the library cannot be built or loaded, ``library()`` raises, and so does
every op in ``ops.py``.  Launchers return 0, a negative ``PE_ERR_*`` code for sizes or arguments
they refuse, or a positive CUDA runtime error number; ``check`` turns those into exceptions.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

from . import build as _build

PE_F32 = 0
PE_BF16 = 1

_ERRORS = {
    -1: "a size is outside what this kernel supports",
    -2: "bad argument",
    -3: "unsupported dtype (float32 and bfloat16 only)",
    -4: "the tensor-core kernel refuses this shape",
    -5: "a CUDA driver entry point is missing",
    -6: "the call needs more scratch than the library's built-in array holds (see csrc/attention_noalloc.h)",
}


class KernelError(RuntimeError):
    pass


_LIB: Optional[ctypes.CDLL] = None
_LIB_PATH: Optional[str] = None

P = c_void_p
I = c_int
L = c_longlong
F = c_float

_SIGNATURES = {
    "pe_embed_gather": [I, P, P, P, I, I, I, P, P],
    "pe_rmsnorm_residual": [I, P, P, P, P, P, I, I, F, P],
    "pe_rmsnorm": [I, P, P, P, I, I, F, P],
    "pe_silu_mul": [I, P, P, I, I, P],
    "pe_batch_expand": [P, P, I, P, P, P],
    "pe_qk_norm_rope_append": [I, P, L, I, I, I, I, P, P, F, P, P, I, I, P, P, P, P, P, I, I, P, P, I, P, P],
    "pe_attention_generic": [I, I, P, L, P, L, I, I, I, I, I, F, I, P, P, P, P, I, I, P, P, P, I, I, P, P],
    "pe_sample": [P, L, I, I, F, I, F, F, c_ulonglong, P, P, P, P, L, P],
    "pe_repetition_penalty": [P, L, I, I, P, I, P, F, P],
    "pe_attention_mma": [I, P, L, P, L, I, I, I, I, I, F, I, P, P, P, P, I, I, P, P, P, I, I, I, P, P],
    "pe_attention_mma_supported": [I, I, I],
    "pe_gemm_smallm": [P, L, P, P, L, I, I, I, I, I, I, P],
    "pe_gemm_smallm_supported": [I, I, I],
    "pe_gemm_umma": [P, L, P, P, L, I, I, I, I, I, I, P, P],
    "pe_gemm_umma_supported": [I, I, I, I],
    "pe_gemm_umma2": [P, L, P, P, L, I, I, I, I, I, I, P, P],
    "pe_gemm_umma2_supported": [I, I, I, I],
    "pe_gemm_umma2_qkv_rope_supported": [I, I, I, I, I, I],
    "pe_gemm_umma2_qkv_rope": [P, L, P, P, L, I, I, I, I, I, P, P, F, P, P, I, I, P, P, P, P, P, I, I, P, P, I, I, P, P],
    "pe_attention_mma_decode_blocks_per_sm": [I],
    "pe_attention_umma_prefill": [P, L, L, P, L, I, I, I, I, I, F, I, P, P, P, P, I, I, P, P, I, P, P, P],
    "pe_attention_umma_supported": [I, I, I],
    "pe_wait_probe": [P, I, P],
    "pe_attention_decode_noalloc": [I, P, L, P, L, I, I, I, I, F, I, P, P, P, P, I, I, P, P, I, I, P, P],
}
_RESTYPES = {"pe_wait_limit_polls": (L, []),
             "pe_attention_generic_scratch_floats": (L, [I, I, I, I]),
             "pe_sample_scratch_bytes": (L, [I, I, F, I, F, F])}


def library() -> ctypes.CDLL:
    """The loaded CUDA library; builds it at first use.  Raises if that is not possible."""
    global _LIB, _LIB_PATH
    if _LIB is None:
        path = _build.build()
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:  # pragma: no cover - depends on the machine
            raise KernelError(f"the CUDA library {path} could not be loaded: {exc}") from exc
        for name, argtypes in _SIGNATURES.items():
            if not hasattr(lib, name):
                continue
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        for name, (res, argtypes) in _RESTYPES.items():
            if hasattr(lib, name):
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = res
        _LIB, _LIB_PATH = lib, path
    return _LIB


def declare(name: str, argtypes, restype=c_int) -> None:
    """Declare one more entry point (kernel files added later register their launchers here)."""
    if restype is c_int:
        _SIGNATURES[name] = argtypes
    else:
        _RESTYPES[name] = (restype, argtypes)
    if _LIB is not None and hasattr(_LIB, name):
        fn = getattr(_LIB, name)
        fn.argtypes = argtypes
        fn.restype = restype


def library_path() -> Optional[str]:
    return _LIB_PATH


def check(code: int, what: str) -> None:
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, 'error ' + str(code))}")
    raise KernelError(f"{what}: CUDA error {code} at launch")
