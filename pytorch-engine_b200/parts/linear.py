"""Helpers for parts that own projection matrices."""
from __future__ import annotations

from typing import Sequence

import torch


def fuse_rows(runtime, tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    """Sibling projections stacked along the output features into one matrix, in the run dtype
    (q|k|v and gate|up, as the reference does: pygguf_engine/quant_kernels.py:1874-1893)."""
    parts = [t.to(device=runtime.device, dtype=runtime.dtype) for t in tensors]
    return torch.cat(parts, dim=0).contiguous()
