"""The generic decoder: builds whatever a ``ModelPlan`` describes and runs one step of it.

It knows no architecture.  Parts are looked up by kind in ``parts/registry.py``; blocks run in the
order the plan lists; each block's mixer gets the cache entry the plan assigns to it.
(The reference's counterpart is ``GGUFTransformerModel.forward``, pygguf_engine/model.py:2221-2305:
embedding, blocks, keep the wanted rows, final norm, output head, float32 logits.)
"""
from __future__ import annotations

import inspect
from typing import Dict, Optional

import torch

from ..parts.registry import lookup
from ..parts.spec import CacheRequest, ModelPlan, PartSpec


def _build_part(role: str, spec: PartSpec, weights: Dict[str, torch.Tensor], runtime, **extra):
    cls = lookup(role, spec.kind)
    local = {}
    for name in cls.weight_decls(spec.params):
        local[name] = weights[spec.weights[name]]
    accepted = inspect.signature(cls.__init__).parameters
    extra = {k: v for k, v in extra.items() if k in accepted}
    return cls(spec.params, local, runtime, **extra)


class DecoderModel:
    def __init__(self, plan: ModelPlan, weights: Dict[str, torch.Tensor], runtime) -> None:
        self.plan = plan
        self.runtime = runtime
        self.hidden = plan.hidden_size
        self.vocab = plan.vocab_size
        self.positions = {name: _build_part("position", spec, weights, runtime) for name, spec in plan.positions.items()}
        self.embedding = _build_part("embedding", plan.embedding, weights, runtime)
        self.blocks = []
        for b in plan.blocks:
            parts = {
                "mixer_norm": _build_part("norm", b.mixer_norm, weights, runtime),
                "mixer": _build_part("mixer", b.mixer, weights, runtime, positions=self.positions),
                "ffn_norm": _build_part("norm", b.ffn_norm, weights, runtime),
                "ffn": _build_part("feed_forward", b.ffn, weights, runtime),
            }
            self.blocks.append(lookup("arrangement", b.arrangement)(b, parts, runtime))
        self.final_norm = _build_part("norm", plan.final_norm, weights, runtime)
        self.head = _build_part("head", plan.head, weights, runtime)
        runtime.forget_adopted()

    def graph_safe(self) -> bool:
        """Whether a step may be recorded into a CUDA graph: every part must say so itself
        (``graph_safe = True``); a part that reads device memory on the host during its forward cannot."""
        parts = [self.embedding, self.final_norm, self.head, *self.positions.values()]
        for b in self.blocks:
            parts.append(b)
            parts.extend(getattr(b, name) for name in ("mixer_norm", "mixer", "ffn_norm", "ffn") if hasattr(b, name))
        return all(getattr(p, "graph_safe", False) for p in parts)

    def cache_requests(self) -> Dict[int, Optional[CacheRequest]]:
        """Cache entry id -> what the mixer that writes it needs."""
        reqs: Dict[int, Optional[CacheRequest]] = {}
        for run in self.plan.order:
            if not run.writes_cache or run.cache_entry in reqs:
                continue
            spec = self.plan.blocks[run.block].mixer
            cls = lookup("mixer", spec.kind)
            reqs[run.cache_entry] = cls.cache_request(spec.params) if hasattr(cls, "cache_request") else None
        for run in self.plan.order:
            if run.cache_entry not in reqs:
                raise ValueError(f"block {run.block} reads cache entry {run.cache_entry}, which no block writes")
        return reqs

    def forward(self, ctx, cache) -> torch.Tensor:
        """Run the step described by ``ctx``; returns float32 logits ``[n_want, vocab]``."""
        rt = self.runtime
        stream = ctx.buffer("model.stream", (ctx.n_tokens, self.hidden), torch.float32)
        self.embedding.forward(ctx.tokens, stream)
        pending = None
        for run in self.plan.order:
            view = cache.view(run.cache_entry)
            block = self.blocks[run.block]
            if run.writes_cache:
                pending = block.forward(stream, pending, ctx, view)
            else:
                pending = block.forward(stream, pending, ctx, view, writes_cache=False)
        if ctx.n_want == 0:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=rt.device)
        normed = ctx.buffer("model.final_normed", (ctx.n_want, self.hidden), rt.dtype)
        self.final_norm.add_forward(stream, pending, normed, rows=ctx.want_rows)
        return self.head.forward(normed)

    def weight_bytes(self) -> int:
        seen = set()
        total = 0

        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()

        visit(self.embedding)
        visit(self.final_norm)
        visit(self.head)
        for p in self.positions.values():
            visit(p)
        for b in self.blocks:
            for part in (b.mixer_norm, b.mixer, b.ffn_norm, b.ffn) if hasattr(b, "mixer_norm") else ():
                visit(part)
        return total
