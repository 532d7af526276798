"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from .registry import register
from .spec import WeightDecl


@register("embedding", "token_embedding")
class TokenEmbedding:
    """params: ``vocab``, ``hidden``.  weights: ``weight [vocab, hidden]``.  Output: the float32
    residual stream (pygguf_engine/model.py:2237, pygguf_engine/quant_kernels.py:1846-1847)."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        return {"weight": WeightDecl((int(params["vocab"]), int(params["hidden"])), "embedding")}

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.vocab = int(params["vocab"])
        self.hidden = int(params["hidden"])
        self.weight = runtime.adopt(weights["weight"])

    def forward(self, token_ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        ops.embed_gather(self.weight, token_ids, out, self.runtime.status)
        return out


@register("head", "linear_head")
class LinearHead:
    """params: ``vocab``, ``hidden``.  weights: ``weight [vocab, hidden]``; a tied head names the
    embedding's tensor and shares its storage (pygguf_engine/model.py:1678-1683, 2206-2214).
    Output: float32 logits."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        return {"weight": WeightDecl((int(params["vocab"]), int(params["hidden"])), "embedding")}

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.vocab = int(params["vocab"])
        self.weight = runtime.adopt(weights["weight"])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.runtime.linear(x, self.weight, out_dtype=torch.float32)
