"""Block arrangements: how two norms, a mixer and a feed-forward are wired around the residual
stream.  The stream is float32; a part's output ("delta") is added to it inside the next norm's
kernel, so a block hands its last delta on instead of adding it itself."""
from __future__ import annotations

from typing import Optional

import torch

from .registry import register


@register("arrangement", "pre_norm")
class PreNormBlock:
    """``h = x + mixer(norm1(x))``; ``out = h + ffn(norm2(h))`` (pygguf_engine/model.py:1025-1042)."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    def __init__(self, spec, parts, runtime) -> None:
        self.runtime = runtime
        self.mixer_norm = parts["mixer_norm"]
        self.mixer = parts["mixer"]
        self.ffn_norm = parts["ffn_norm"]
        self.ffn = parts["ffn"]
        self.name = spec.name

    def forward(self, stream: torch.Tensor, pending: Optional[torch.Tensor], ctx, view, writes_cache: bool = True):
        """``stream``: float32 residual ``[N, hidden]``, updated in place; ``pending``: the previous
        block's delta that is not added yet (or None).  Returns this block's own pending delta."""
        rt = self.runtime
        normed = ctx.buffer("block.normed", tuple(stream.shape), rt.dtype)
        self.mixer_norm.add_forward(stream, pending, normed)
        if writes_cache:
            mixed = self.mixer.forward(normed, ctx, view)
        else:
            mixed = self.mixer.forward(normed, ctx, view, writes_cache=False)
        self.ffn_norm.add_forward(stream, mixed, normed)
        return self.ffn.forward(normed, ctx)
