"""One step's batch as the kernels see it.

A step brings, for each of ``n_seqs`` sequences, ``q_len`` new tokens that follow the ``past``
tokens already in the cache.  Tokens are packed back to back without padding.  The device arrays
(all int32) are views into one buffer that is filled by a single host-to-device copy:

    tokens[n_tokens] | seq_slot[n_seqs] | seq_past[n_seqs] | seq_qstart[n_seqs+1] | want_rows[n_want]

``token_seq`` / ``token_pos`` (the batch entry and position of every token) are expanded from them
on the device.  ``decode`` is true when every sequence brings exactly one token.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..staging import PinnedStager  # noqa: F401  (used by the runner and the sampler through this module)


class BufferPool:
    """Named device buffers that persist between steps and grow on demand (never shrink)."""

    def __init__(self, device) -> None:
        self.device = torch.device(device)
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}   # (name, dtype, shape) -> view of the current buffer

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        view = self._views.get((name, dtype, shape))
        if view is not None:
            return view
        numel = 1
        for s in shape:
            numel *= s
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < numel:
            buf = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            for k in [k for k in self._views if k[0] == name and k[1] == dtype]:
                del self._views[k]                     # views of the buffer that was replaced
        if len(self._views) > 4096:                    # steps of ever new sizes: start over
            self._views.clear()
        view = buf[:numel].view(*shape)
        self._views[(name, dtype, shape)] = view
        return view

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


@dataclass
class StepEntry:
    """One sequence's share of a step: its cache slot, its next tokens, and the indices among
    these tokens whose logits are wanted (may be empty)."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepContext:
    def __init__(self, runtime, pool: BufferPool, *, n_tokens: int, n_seqs: int, max_q: int, decode: bool,
                 max_kv_len: int, n_want: int) -> None:
        self.runtime = runtime
        self.pool = pool
        self.n_tokens = n_tokens
        self.n_seqs = n_seqs
        self.max_q = max_q
        self.decode = decode
        self.max_kv_len = max_kv_len  # upper bound of any sequence's length after this step
        self.n_want = n_want
        meta = pool.get("step.meta", (n_tokens + 3 * n_seqs + 1 + n_want,), torch.int32)
        o = 0
        self.meta = meta
        self.tokens = meta[o:o + n_tokens]; o += n_tokens
        self.seq_slot = meta[o:o + n_seqs]; o += n_seqs
        self.seq_past = meta[o:o + n_seqs]; o += n_seqs
        self.seq_qstart = meta[o:o + n_seqs + 1]; o += n_seqs + 1
        self.want_rows = meta[o:o + n_want]
        self.token_seq = pool.get("step.token_seq", (n_tokens,), torch.int32)
        self.token_pos = pool.get("step.token_pos", (n_tokens,), torch.int32)

    def buffer(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        return self.pool.get(name, shape, dtype)

    def max_splits(self, split_keys: int) -> int:
        return max(1, (self.max_kv_len + split_keys - 1) // split_keys)

    @staticmethod
    def pack_meta(entries: Sequence[StepEntry], pasts: Sequence[int]) -> Tuple[List[int], int, int]:
        """The host image of the meta buffer; returns (ints, n_tokens, n_want)."""
        tokens: List[int] = []
        qstart = [0]
        want: List[int] = []
        for e in entries:
            base = len(tokens)
            n = len(e.tokens)
            for w in e.want:
                if not 0 <= w < n:
                    raise IndexError(f"wanted position {w} is outside the {n} tokens this step brings for slot {e.slot}")
                want.append(base + w)
            tokens.extend(int(t) for t in e.tokens)
            qstart.append(len(tokens))
        ints = tokens + [e.slot for e in entries] + [int(p) for p in pasts] + qstart + want
        return ints, len(tokens), len(want)
