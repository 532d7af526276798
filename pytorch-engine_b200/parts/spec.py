"""The data that describes a model: which parts, with which constants, in which order.

An architecture turns its typed configuration into a ``ModelPlan``.  The plan is plain data:
every part is a ``PartSpec`` (a registry key, the part's sizes and constants, and the checkpoint
tensor name of each of its weights); a block is an arrangement and the named parts it wires (usually
two norms, a mixer and a feed-forward); and the order in which blocks run is a list of ``RunStep`` entries, which may name
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
    """A residual block: an ``arrangement`` (registry of block arrangements: how the parts are wired
    around the residual stream) and the parts themselves, by name: ``parts[name] = (role, PartSpec)``
    with ``role`` one of "norm", "mixer", "feed_forward".  The arrangement decides which names it
    wants; a block may carry four norms, two mixers or no feed-forward.  Every part is chosen
    independently, so two blocks of one model may differ in any of them.

    ``BlockSpec.standard`` builds the usual block of two norms, a mixer and a feed-forward under
    the names ``mixer_norm, mixer, ffn_norm, ffn``."""

    arrangement: str
    parts: Mapping[str, Tuple[str, PartSpec]]
    name: str = ""

    @classmethod
    def standard(cls, arrangement: str, mixer_norm: PartSpec, mixer: PartSpec, ffn_norm: PartSpec, ffn: PartSpec,
                 name: str = "") -> "BlockSpec":
        return cls(arrangement, {"mixer_norm": ("norm", mixer_norm), "mixer": ("mixer", mixer),
                                 "ffn_norm": ("norm", ffn_norm), "ffn": ("feed_forward", ffn)}, name)

    def part(self, name: str) -> PartSpec:
        return self.parts[name][1]

    def mixer_names(self) -> Tuple[str, ...]:
        """Names of the parts that are mixers, in the order the block lists them."""
        return tuple(n for n, (role, _) in self.parts.items() if role == "mixer")


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
    # checkpoint names that a file may hold beside the plan's own: ``duplicates[name] = other`` accepts
    # ``name`` if it equals tensor ``other`` (a tied head stored twice); ``ignored`` are name patterns
    # (``fnmatch``) of stored buffers that carry no weights
    duplicates: Mapping[str, str] = field(default_factory=dict)
    ignored: Tuple[str, ...] = ()

    def part_specs(self):
        """Every PartSpec of the plan as (label, role, spec), for the weight loader and error texts."""
        yield "embedding", "embedding", self.embedding
        for name, spec in self.positions.items():
            yield f"position {name}", "position", spec
        for i, b in enumerate(self.blocks):
            label = b.name or f"block {i}"
            for name, (role, spec) in b.parts.items():
                yield f"{label} {name}", role, spec
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
