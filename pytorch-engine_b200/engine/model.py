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
        self.block_parts = []     # per block: {part name: built part}
        for b in plan.blocks:
            parts = {name: _build_part(role, spec, weights, runtime, positions=self.positions)
                     for name, (role, spec) in b.parts.items()}
            self.block_parts.append(parts)
            self.blocks.append(lookup("arrangement", b.arrangement)(b, parts, runtime))
        self.final_norm = _build_part("norm", plan.final_norm, weights, runtime)
        self.head = _build_part("head", plan.head, weights, runtime)
        runtime.forget_adopted()

    def graph_safe(self) -> bool:
        """Whether a step may be recorded into a CUDA graph: every part must say so itself
        (``graph_safe = True``); a part that reads device memory on the host during its forward cannot."""
        parts = [self.embedding, self.final_norm, self.head, *self.positions.values()]
        for block, built in zip(self.blocks, self.block_parts):
            parts.append(block)
            parts.extend(built.values())
        return all(getattr(p, "graph_safe", False) for p in parts)

    @staticmethod
    def cache_key(entry: int, block_spec, mixer_name: str):
        """The cache's key for one mixer of a run: the entry number itself for a block with one mixer,
        ``(entry, mixer name)`` for a block with several."""
        return entry if len(block_spec.mixer_names()) <= 1 else (entry, mixer_name)

    def cache_requests(self) -> Dict[object, Optional[CacheRequest]]:
        """Cache key -> what the mixer that writes it needs."""
        reqs: Dict[object, Optional[CacheRequest]] = {}
        written = set()
        for run in self.plan.order:
            if not run.writes_cache or run.cache_entry in written:
                continue
            written.add(run.cache_entry)
            b = self.plan.blocks[run.block]
            for name in b.mixer_names():
                spec = b.part(name)
                cls = lookup("mixer", spec.kind)
                reqs[self.cache_key(run.cache_entry, b, name)] = (
                    cls.cache_request(spec.params) if hasattr(cls, "cache_request") else None)
        for run in self.plan.order:
            if run.cache_entry not in written:
                raise ValueError(f"block {run.block} reads cache entry {run.cache_entry}, which no block writes")
        return reqs

    def _view(self, cache, run):
        """What a block's arrangement gets as its cache view: the view of its one mixer, a dict of
        views by mixer name for a block with several, None for a block without a mixer."""
        b = self.plan.blocks[run.block]
        names = b.mixer_names()
        if not names:
            return None
        if len(names) == 1:
            return cache.view(run.cache_entry)
        return {name: cache.view((run.cache_entry, name)) for name in names}

    def forward(self, ctx, cache) -> torch.Tensor:
        """Run the step described by ``ctx``; returns float32 logits ``[n_want, vocab]``."""
        rt = self.runtime
        stream = ctx.buffer("model.stream", (ctx.n_tokens, self.hidden), torch.float32)
        self.embedding.forward(ctx.tokens, stream)
        pending = None
        for run in self.plan.order:
            view = self._view(cache, run)
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
        for built in self.block_parts:
            for part in built.values():
                visit(part)
        return total
