"""Host-side bookkeeping of what the cache hands out: pages of a pool and sequence slots.

Both are free lists that refuse misuse loudly: a page or slot can be neither handed out twice
nor given back twice, and giving back what was never handed out is an error.
"""
from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    """Misuse or exhaustion of the cache."""


class FreeList:
    """Ids 0..n-1; `take` hands out the lowest free id, so that freed ids are used again first."""

    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free = list(range(self.n - 1, -1, -1))      # popped from the end: lowest first
        self._held = [False] * self.n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"out of {self.what}s: all {self.n} are held")
        i = self._free.pop()
        if self._held[i]:
            raise CacheError(f"{self.what} {i} was on the free list while held")
        self._held[i] = True
        return i

    def take_many(self, k: int) -> List[int]:
        if k > len(self._free):
            raise CacheError(f"out of {self.what}s: {k} wanted, {len(self._free)} of {self.n} free")
        return [self.take() for _ in range(k)]

    def give_back(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is given back but is not held")
        self._held[i] = False
        self._free.append(i)
        # keep "lowest first": the list is short, and reuse order is part of what tests pin down
        self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return self._held[i]

    def check(self) -> None:
        """Every id is either free once or held; raises if one is lost or doubled."""
        seen = [0] * self.n
        for i in self._free:
            seen[i] += 1
        for i in range(self.n):
            if seen[i] + (1 if self._held[i] else 0) != 1:
                raise CacheError(f"{self.what} {i}: on the free list {seen[i]} times, held={self._held[i]}")
