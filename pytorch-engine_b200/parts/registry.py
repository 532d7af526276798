"""Registries of part classes, one per role.

A part class is registered under a ``kind``; a ``PartSpec`` with that kind makes the generic
decoder build it.  Code outside this package can register further kinds (a test registers a
toy mixer with state of its own) without touching any file here.

Interfaces (every class also has ``weight_decls(params) -> {name: WeightDecl}`` as a
classmethod and a constructor ``(params, weights, runtime)``; ``weights`` holds the tensors as
the loader read them, on the run device):

* norm:         ``forward(x, out_dtype) -> y`` and
                ``add_forward(residual_f32, delta, rows=None) -> y``: adds ``delta`` into the
                float32 residual stream in place (``rows`` given: gathers those rows instead
                and leaves the stream alone) and returns the normalised rows in the run dtype.
* position:     ``apply(q, k, positions)`` in place on ``[N, heads, d]`` tensors (views of a wider
                buffer; ``positions`` int32 on the device), or, for a rotary encoding,
                ``fusable_rotary = True`` and ``tables() -> (cos, sin, rotary_dim)`` so that a mixer
                fuses it into its own kernel.  The attention mixer takes either.
* mixer:        ``cache_request(params) -> CacheRequest | None`` (classmethod) and
                ``forward(x, ctx, cache_view) -> delta`` with ``x`` ``[N, hidden]`` in the run dtype.
* feed_forward: ``forward(x, ctx) -> delta``.
* embedding:    ``forward(token_ids_i32) -> residual stream float32 [N, hidden]``.
* head:         ``forward(x) -> logits float32 [rows, vocab]``.
* arrangement:  a class ``(block_spec, parts, runtime)`` with
                ``forward(stream, pending, ctx, cache_view) -> pending``.
"""
from __future__ import annotations

from typing import Dict

ROLES = ("norm", "position", "mixer", "feed_forward", "embedding", "head", "arrangement")
_REGISTRIES: Dict[str, Dict[str, type]] = {role: {} for role in ROLES}


def register(role: str, kind: str, cls: type = None, *, replace: bool = False):
    """Register ``cls`` as ``kind`` of ``role``; usable as a decorator when ``cls`` is omitted."""
    if role not in _REGISTRIES:
        raise KeyError(f"unknown part role {role!r}; roles: {', '.join(ROLES)}")

    def _do(c: type) -> type:
        table = _REGISTRIES[role]
        if kind in table and table[kind] is not c and not replace:
            raise KeyError(f"{role} kind {kind!r} is already registered ({table[kind].__name__})")
        table[kind] = c
        return c

    return _do if cls is None else _do(cls)


def lookup(role: str, kind: str) -> type:
    table = _REGISTRIES[role]
    if kind not in table:
        raise KeyError(f"no {role} of kind {kind!r} is registered; registered: {', '.join(sorted(table)) or 'none'}")
    return table[kind]


def unregister(role: str, kind: str) -> None:
    _REGISTRIES[role].pop(kind, None)


def registered(role: str):
    return sorted(_REGISTRIES[role])
