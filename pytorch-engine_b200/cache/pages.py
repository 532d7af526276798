"""Fixed-size pools of numbered things (cache pages, sequence slots) with strict bookkeeping.

A number is either free or held, never both and never twice: taking from an empty pool, giving
back a number that is not held, or one outside the pool, raises.  The most recently freed number
is handed out first, so that a slot or page that was just given back is used again at once (a
stale entry would then show in the very next batch).
"""
from __future__ import annotations

from typing import Iterable, List


class CacheFull(RuntimeError):
    """The cache has no free page or slot left for what was asked."""


class CacheBookkeepingError(RuntimeError):
    """A page or slot was freed twice, freed while not held, or is outside the pool."""


class NumberPool:
    def __init__(self, count: int, what: str = "page") -> None:
        if count < 0:
            raise ValueError(f"{what} pool size must be >= 0, got {count}")
        self.count = count
        self.what = what
        self._free: List[int] = list(range(count - 1, -1, -1))  # pop() gives 0 first
        self._held = [False] * count

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.count - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} left (all {self.count} are held)")
        n = self._free.pop()
        if self._held[n]:  # cannot happen unless the lists were corrupted
            raise CacheBookkeepingError(f"{self.what} {n} was on the free list while held")
        self._held[n] = True
        return n

    def take_many(self, k: int) -> List[int]:
        if k > len(self._free):
            raise CacheFull(f"{k} {self.what}s wanted but only {len(self._free)} of {self.count} are free")
        return [self.take() for _ in range(k)]

    def give_back(self, n: int) -> None:
        if not 0 <= n < self.count:
            raise CacheBookkeepingError(f"{self.what} {n} is outside the pool (0..{self.count - 1})")
        if not self._held[n]:
            raise CacheBookkeepingError(f"{self.what} {n} was given back but is not held (freed twice?)")
        self._held[n] = False
        self._free.append(n)

    def give_back_many(self, ns: Iterable[int]) -> None:
        for n in ns:
            self.give_back(n)

    def is_held(self, n: int) -> bool:
        return 0 <= n < self.count and self._held[n]

    def check(self) -> None:
        """Every number is exactly once either free or held."""
        seen = [0] * self.count
        for n in self._free:
            seen[n] += 1
        for n in range(self.count):
            if seen[n] + (1 if self._held[n] else 0) != 1:
                raise CacheBookkeepingError(f"{self.what} {n}: free-list count {seen[n]}, held {self._held[n]}")
