"""The data that describes a model: which parts, with which constants, in which order.

An architecture turns its typed configuration into a ``ModelPlan``.  The plan is plain data:
every part is a ``PartSpec`` (a registry key, the part's sizes and constants, and the checkpoint
tensor name of each of its weights); a block is an arrangement of two norms, a mixer and a
feed-forward; and the order in which blocks run is a list of ``RunStep`` entries, which may name
a block twice or let a block use the cache entry of another one.  Nothing in ``parts/`` knows
which model it is part of: the generic decoder (``engine/model.py``) builds whatever the plan
says by looking the kinds up in ``parts/registry.py``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` is the key in its registry, ``params`` its sizes and constants,
    ``weights`` maps the part's own weight names to checkpoint tensor names."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    weights: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class BlockSpec:
    """A residual block.  ``arrangement`` names how norms, mixer and feed-forward are wired
    (registry of block arrangements); the four parts are chosen independently, so two blocks of
    one model may differ in any of them."""

    arrangement: str
    mixer_norm: PartSpec
    mixer: PartSpec
    ffn_norm: PartSpec
    ffn: PartSpec
    name: str = ""


@dataclass(frozen=True)
class RunStep:
    """One entry of the execution order: run ``block``; its mixer uses cache entry ``cache``
    (default: the block's own).  ``writes_cache`` False makes the mixer read that entry without
    appending to it (a block that attends over another block's keys and values)."""

    block: int
    cache: Optional[int] = None
    writes_cache: bool = True

    @property
    def cache_entry(self) -> int:
        return self.block if self.cache is None else self.cache


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[RunStep, ...]
    final_norm: PartSpec
    head: PartSpec
    # position encodings by name; a mixer names the one it uses in params["position"]
    positions: Mapping[str, PartSpec] = field(default_factory=dict)

    def part_specs(self):
        """Every PartSpec of the plan as (label, role, spec), for the weight loader and error texts."""
        yield "embedding", "embedding", self.embedding
        for name, spec in self.positions.items():
            yield f"position {name}", "position", spec
        for i, b in enumerate(self.blocks):
            label = b.name or f"block {i}"
            yield f"{label} mixer_norm", "norm", b.mixer_norm
            yield f"{label} mixer", "mixer", b.mixer
            yield f"{label} ffn_norm", "norm", b.ffn_norm
            yield f"{label} ffn", "feed_forward", b.ffn
        yield "final_norm", "norm", self.final_norm
        yield "head", "head", self.head


@dataclass(frozen=True)
class WeightDecl:
    """What a part expects of one of its weights: shape, and the ``role`` that decides how a
    random model fills it and what the part converts it to (``matrix``/``embedding``: normal
    with the given std, run dtype; ``norm``: one plus normal, float32; ``table_int``: int32)."""

    shape: Tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class CacheRequest:
    """What a mixer needs the cache to hold per sequence.

    ``kind`` "kv": keys and values of every position, ``kv_heads x head_dim`` each, and with
    ``window`` only the last ``window`` positions need to stay.  ``kind`` "state": tensors of fixed
    shape per sequence (``state_shapes``: name -> (shape, torch dtype name)), zero when a
    sequence starts.  Entries with equal requests share one group of storage.
    """

    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shapes: Tuple[Tuple[str, Tuple[int, ...], str], ...] = ()

    def group_key(self):
        return (self.kind, self.kv_heads, self.head_dim, self.window, self.state_shapes)
