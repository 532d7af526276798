"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))`` with gate|up as one product
(pygguf_engine/model.py:839-846, pygguf_engine/quant_kernels.py:1467-1472)."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from .linear import fuse_rows
from .registry import register
from .spec import WeightDecl


@register("feed_forward", "swiglu")
class SwiGLU:
    """params: ``hidden``, ``intermediate``.  weights: ``gate_proj, up_proj [I, H]``, ``down_proj [H, I]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, i = int(params["hidden"]), int(params["intermediate"])
        return {"gate_proj": WeightDecl((i, h)), "up_proj": WeightDecl((i, h)), "down_proj": WeightDecl((h, i))}

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])
        self.gate_up = fuse_rows(runtime, [weights["gate_proj"], weights["up_proj"]])
        self.down = runtime.adopt(weights["down_proj"])

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        rt = self.runtime
        n = x.shape[0]
        act = ctx.buffer("ffn.act", (n, self.intermediate), rt.dtype)
        if rt.takes_small_gemm(x, self.gate_up):
            # few rows: gate|up product with silu(gate) * up in its epilogue
            ops.gemm_smallm(x, self.gate_up, act, pair_offset=self.intermediate)
        elif rt.takes_large_gemm(x, self.gate_up, self.intermediate):
            # tcgen05 product over [gate rows | matching up rows] tiles, gate applied on the way out of TMEM
            # many rows: a pair of SMs per tile where the kernel takes the shape (K a multiple of 64)
            pair = rt.pair_gemm and x.shape[0] >= rt.large_gemm_rows and ops.gemm_umma2_supported(x, self.gate_up, self.intermediate)
            (ops.gemm_umma2 if pair else ops.gemm_umma)(x, self.gate_up, act, rt.status, pair_offset=self.intermediate)
        else:
            gu = ctx.buffer("ffn.gate_up", (n, 2 * self.intermediate), rt.dtype)
            rt.linear(x, self.gate_up, out=gu)
            ops.silu_mul(gu, act)
        delta = ctx.buffer("ffn.delta", (n, self.hidden), rt.dtype)
        rt.linear(act, self.down, out=delta)
        return delta
