"""The cache: a slot per sequence, pages of 64 positions, storage per group of layers.

* A *slot* stands for one live sequence: its length and, per group, its page list (and its row in
  the fixed-size state tensors).  Slots are taken when a batch starts and given back when a
  sequence ends; a slot that was given back is handed out again first.
* Keys and values live in *pages* of 64 positions.  The cache is sized in pages
  (``max_tokens / 64``), so any mix of sequence lengths whose page-rounded sum fits can be live.
* Cache entries (one per block that keeps something) with equal needs form a *group* with storage,
  page pool and page table of its own: ``[entries, 2, pages, kv_heads, 64, head_dim]`` for keys and
  values.  A group with a window gives pages back as soon as every position in them has left the
  window.  A "state" group holds tensors of fixed shape per slot, zeroed when the slot is taken.

The reference keeps one growing buffer per layer for a single sequence
(pygguf_engine/kv_cache.py:1634-1702) and per-layer recurrent state beside it (1457-1579); the
device-side position it feeds its graphs with (1847-1852) is here the per-step length array.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..parts.spec import CacheRequest
from .pages import CacheBookkeepingError, CacheFull, NumberPool

PAGE_TOKENS = 64


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


@dataclass
class CacheView:
    """What one cache entry hands to its mixer during a step."""

    kind: str
    group: "CacheGroup"
    index: int  # position of the entry inside its group's storage
    window: Optional[int] = None

    @property
    def k_pages(self) -> torch.Tensor:
        return self.group.storage[self.index, 0]

    @property
    def v_pages(self) -> torch.Tensor:
        return self.group.storage[self.index, 1]

    @property
    def page_table(self) -> torch.Tensor:
        return self.group.page_table

    @property
    def num_pages(self) -> int:
        return self.group.num_pages

    def state(self, name: str) -> torch.Tensor:
        """The fixed-size state ``[slots, *shape]`` of this entry."""
        return self.group.state_tensors[name][self.index]


@dataclass
class CacheGroup:
    request: CacheRequest
    entries: List[int] = field(default_factory=list)
    num_pages: int = 0
    pool: Optional[NumberPool] = None
    storage: Optional[torch.Tensor] = None
    page_table: Optional[torch.Tensor] = None
    pages_of_slot: Dict[int, List[int]] = field(default_factory=dict)  # logical page -> physical (-1: released)
    state_tensors: Dict[str, torch.Tensor] = field(default_factory=dict)


class PagedCache:
    def __init__(self, requests: Mapping[object, Optional[CacheRequest]], *, max_tokens: int, max_slots: int,
                 max_seq_len: int, dtype: torch.dtype, device) -> None:
        if max_tokens <= 0 or max_slots <= 0 or max_seq_len <= 0:
            raise ValueError("max_tokens, max_slots and max_seq_len must be positive")
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_tokens = pages_for(max_tokens) * PAGE_TOKENS
        self.max_slots = max_slots
        self.max_seq_len = max_seq_len
        self.table_width = pages_for(max_seq_len)
        self.slots = NumberPool(max_slots, "slot")
        self.lengths: Dict[int, int] = {}
        self.groups: List[CacheGroup] = []
        self._entry: Dict[object, Tuple[int, int]] = {}  # entry key (int, or (int, mixer name)) -> (group number, index in group)
        by_key: Dict[tuple, int] = {}
        for entry_id in sorted(requests, key=lambda e: e if isinstance(e, tuple) else (e, "")):
            req = requests[entry_id]
            if req is None:
                continue
            key = req.group_key()
            if key not in by_key:
                by_key[key] = len(self.groups)
                self.groups.append(CacheGroup(request=req))
            g = self.groups[by_key[key]]
            self._entry[entry_id] = (by_key[key], len(g.entries))
            g.entries.append(entry_id)
        for g in self.groups:
            self._allocate(g)
        # New page numbers reach the device through pinned memory and an asynchronous copy on the current
        # stream: a copy from pageable memory would make the host wait for every step still queued, once
        # per page a sequence begins.  The ring is deep enough for two steps of a full batch.
        self._stager = None
        if self.device.type == "cuda":
            from ..staging import PinnedStager
            self._stager = PinnedStager(self.device, capacity=max(64, self.table_width), depth=256)

    # ---- storage -------------------------------------------------------------------------
    def _allocate(self, g: CacheGroup) -> None:
        r = g.request
        if r.kind == "kv":
            g.num_pages = pages_for(self.max_tokens)
            g.pool = NumberPool(g.num_pages, "page")
            # zeros, not uninitialised memory: rows that were never written must hold finite values
            g.storage = torch.zeros((len(g.entries), 2, g.num_pages, r.kv_heads, PAGE_TOKENS, r.head_dim),
                                    dtype=self.dtype, device=self.device)
            g.page_table = torch.full((self.max_slots, self.table_width), -1, dtype=torch.int32, device=self.device)
        elif r.kind == "state":
            for name, shape, dtype_name in r.state_shapes:
                g.state_tensors[name] = torch.zeros((len(g.entries), self.max_slots, *shape),
                                                    dtype=getattr(torch, dtype_name), device=self.device)
        else:
            raise ValueError(f"unknown cache kind {r.kind!r} (known: 'kv', 'state')")

    def view(self, entry_id) -> Optional[CacheView]:
        if entry_id not in self._entry:
            return None
        gi, idx = self._entry[entry_id]
        g = self.groups[gi]
        return CacheView(kind=g.request.kind, group=g, index=idx, window=g.request.window)

    def nbytes(self) -> int:
        total = 0
        for g in self.groups:
            if g.storage is not None:
                total += g.storage.numel() * g.storage.element_size()
            if g.page_table is not None:
                total += g.page_table.numel() * 4
            for t in g.state_tensors.values():
                total += t.numel() * t.element_size()
        return total

    # ---- slots ---------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        slot = self.slots.take()
        self.lengths[slot] = 0
        for g in self.groups:
            if g.request.kind == "kv":
                g.pages_of_slot[slot] = []
            else:
                for t in g.state_tensors.values():
                    t[:, slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if slot not in self.lengths:
            raise CacheBookkeepingError(f"slot {slot} was freed but is not held (freed twice?)")
        for g in self.groups:
            if g.request.kind == "kv":
                g.pool.give_back_many(p for p in g.pages_of_slot.pop(slot) if p >= 0)
        del self.lengths[slot]
        self.slots.give_back(slot)

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    @property
    def live_slots(self) -> List[int]:
        return sorted(self.lengths)

    def free_pages(self) -> int:
        kv = [g.pool.free_count for g in self.groups if g.pool is not None]
        return min(kv) if kv else (1 << 30)  # nothing is paged: no page limit

    # ---- growing a sequence ----------------------------------------------------------------
    def reserve(self, slot: int, new_length: int) -> None:
        """Make sure pages exist for positions ``< new_length``; call before the step that writes them."""
        if slot not in self.lengths:
            raise CacheBookkeepingError(f"slot {slot} is not held")
        if new_length > self.max_seq_len:
            raise CacheFull(f"sequence of {new_length} tokens exceeds the cache's maximum length {self.max_seq_len}")
        need = pages_for(new_length)
        # check every group first so that a failure leaves nothing half-allocated
        for g in self.groups:
            if g.request.kind != "kv":
                continue
            missing = need - len(g.pages_of_slot[slot])
            if missing > g.pool.free_count:
                raise CacheFull(
                    f"slot {slot} needs {missing} more page(s) of {PAGE_TOKENS} tokens for length {new_length}, "
                    f"only {g.pool.free_count} of {g.num_pages} are free"
                )
        for g in self.groups:
            if g.request.kind != "kv":
                continue
            have = g.pages_of_slot[slot]
            if need > len(have):
                start = len(have)
                new_pages = g.pool.take_many(need - start)
                have.extend(new_pages)
                if self._stager is not None:
                    self._stager.send(new_pages, g.page_table[slot, start:need])
                else:
                    g.page_table[slot, start:need] = torch.tensor(new_pages, dtype=torch.int32)

    def release_reserved(self, slot: int) -> None:
        """Give back the pages that ``reserve`` took beyond the sequence's committed length (a step
        that was prepared and then not run)."""
        keep = pages_for(self.lengths[slot])
        for g in self.groups:
            if g.request.kind != "kv":
                continue
            pages = g.pages_of_slot[slot]
            g.pool.give_back_many(p for p in pages[keep:] if p >= 0)
            del pages[keep:]

    def commit(self, slot: int, new_length: int) -> None:
        """Record the length after a step and give back pages that left every window."""
        if new_length < self.lengths[slot]:
            raise CacheBookkeepingError("a sequence cannot shrink by commit(); use truncate()")
        self.lengths[slot] = new_length
        for g in self.groups:
            w = g.request.window
            if g.request.kind != "kv" or not w:
                continue
            # the next query sits at position new_length and sees keys > new_length - w
            first_needed = max(0, new_length - w + 1) // PAGE_TOKENS
            pages = g.pages_of_slot[slot]
            for logical in range(min(first_needed, len(pages))):
                if pages[logical] >= 0:
                    g.pool.give_back(pages[logical])
                    pages[logical] = -1

    def truncate(self, slot: int, length: int) -> None:
        """Forget positions ``>= length`` (pages beyond are given back).  Not possible for a group
        that has a window or fixed-size state: what they dropped or folded in cannot be brought back."""
        if length > self.lengths[slot]:
            raise CacheBookkeepingError("truncate() cannot lengthen a sequence")
        for g in self.groups:
            if g.request.kind == "state" or g.request.window:
                if length != self.lengths[slot]:
                    raise CacheBookkeepingError("a sequence with windowed or fixed-size state cannot be truncated")
        keep = pages_for(length)
        for g in self.groups:
            if g.request.kind != "kv":
                continue
            pages = g.pages_of_slot[slot]
            g.pool.give_back_many(p for p in pages[keep:] if p >= 0)
            del pages[keep:]
        self.lengths[slot] = length

    def reset(self) -> None:
        """Give every live slot back at once: all sequences are forgotten, every page is free again (the
        reference's ``clear``, pygguf_engine/kv_cache.py:2644).  Storage is not touched: nothing reads beyond a
        sequence's length, and state is zeroed when a slot is taken."""
        for slot in self.live_slots:
            self.free_slot(slot)

    def check(self) -> None:
        """Bookkeeping invariants: no page lost, held twice, or held by a slot that is not live."""
        self.slots.check()
        for g in self.groups:
            if g.request.kind != "kv":
                continue
            g.pool.check()
            seen = set()
            for slot, pages in g.pages_of_slot.items():
                if slot not in self.lengths:
                    raise CacheBookkeepingError(f"pages are recorded for slot {slot}, which is not live")
                for p in pages:
                    if p < 0:
                        continue
                    if p in seen:
                        raise CacheBookkeepingError(f"page {p} is held twice")
                    if not g.pool.is_held(p):
                        raise CacheBookkeepingError(f"page {p} is in use but marked free")
                    seen.add(p)
            if len(seen) != g.pool.held_count:
                raise CacheBookkeepingError(f"{g.pool.held_count - len(seen)} page(s) are held by no slot (lost)")
