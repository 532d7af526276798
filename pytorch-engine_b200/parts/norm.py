"""RMSNorm.  Formula: ``x * rsqrt(mean(x^2) + eps) * w`` in float32
(pygguf_engine/quant_kernels.py:831-833, 1548; fused with the residual add 1595-1596)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .registry import register
from .spec import WeightDecl


@register("norm", "rmsnorm")
class RMSNorm:
    """params: ``dim``, ``eps``.  weights: ``weight [dim]`` (kept in float32)."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        return {"weight": WeightDecl((int(params["dim"]),), "norm")}

    def __init__(self, params, weights, runtime) -> None:
        self.dim = int(params["dim"])
        self.eps = float(params["eps"])
        self.runtime = runtime
        self.weight = runtime.adopt(weights["weight"], torch.float32)

    def add_forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops.rmsnorm_residual(residual, delta, self.weight, out, self.eps, rows)
        return out

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = torch.empty_like(x) if out is None else out
        ops.rmsnorm(x, self.weight, out, self.eps)
        return out
