"""Rotary position encoding (split-half layout) with precomputed float32 cos/sin tables.

Formulas: ``inv_freq_j = 1 / theta^(2j / rotary_dim)`` (pygguf_engine/model.py:147-156),
``angle = position * inv_freq`` with float32 positions, then cos and sin (183-185); rotation of the
first ``rotary_dim`` features ``[x1*cos - x2*sin, x2*cos + x1*sin]``, the rest passing through
(232-251).  ``inv_freq`` is computed on the host so that it is bit-identical everywhere; the
product and cos/sin are taken on the device in float32.
"""
from __future__ import annotations

from typing import Dict

import torch

from .registry import register
from .spec import WeightDecl


@register("position", "rope")
class RotaryPosition:
    """params: ``rotary_dim`` (even, <= head size), ``theta``, ``max_positions``, ``style`` ("neox")."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    fusable_rotary = True

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        return {}

    def __init__(self, params, weights, runtime) -> None:
        self.rotary_dim = int(params["rotary_dim"])
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        style = params.get("style", "neox")
        if style != "neox":
            raise ValueError(f"rotary layout {style!r} is not built (only the split-half 'neox' layout)")
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {self.rotary_dim}")
        idx = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        inv_freq = (1.0 / (self.theta ** (idx / self.rotary_dim))).to(runtime.device)
        pos = torch.arange(0, self.max_positions, dtype=torch.float32, device=runtime.device)
        freqs = torch.outer(pos, inv_freq)
        self.cos = torch.cos(freqs).contiguous()
        self.sin = torch.sin(freqs).contiguous()

    def tables(self):
        return self.cos, self.sin, self.rotary_dim
