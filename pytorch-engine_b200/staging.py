"""Small host-to-device copies that do not make the host wait."""
from __future__ import annotations

from typing import Sequence

import torch


class PinnedStager:
    """Host-to-device copies of small int32 arrays through a ring of pinned buffers.  A buffer is
    reused only after the copy that last read it has finished (an event per buffer), so the host may
    run ahead of the device by several steps."""

    def __init__(self, device, capacity: int = 1 << 16, depth: int = 4) -> None:
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.capacity = capacity
        self.bufs = [torch.empty(capacity, dtype=torch.int32, pin_memory=self.cuda) for _ in range(depth)]
        self.views = [b.numpy() for b in self.bufs]      # the same memory, for fast filling from lists
        self.events = [torch.cuda.Event() if self.cuda else None for _ in range(depth)]
        self.used = [False] * depth
        self.next = 0

    def send(self, ints: Sequence[int], dst: torch.Tensor) -> None:
        n = len(ints)
        if n > self.capacity or not self.cuda:
            dst.copy_(torch.tensor(ints, dtype=torch.int32))
            return
        i = self.next
        self.next = (i + 1) % len(self.bufs)
        if self.used[i]:
            self.events[i].synchronize()
        self.views[i][:n] = ints
        dst.copy_(self.bufs[i][:n], non_blocking=True)
        self.events[i].record()
        self.used[i] = True
