"""Bookkeeping of the cache on the host: sequence slots and pages of positions.

A *slot* is one live sequence: its length and, for every group of layers, the
list of pages that hold its keys and values.  Pages hold ``page_size`` positions
(64: the reference's attention also works in 64-position chunks,
skyla-engine/src/arena.rs:6).  Both allocators are plain free lists that refuse
to hand out what is taken and to take back what is free, so a slot or a page can
never be lost, held twice or freed twice without an exception.
"""
from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    """Misuse of the cache: unknown slot, double free, and the like."""


class CacheFull(CacheError):
    """The request does not fit; nothing was changed and no kernel was launched.

    The reference's counterpart is "context full" (skyla-engine/src/engine.rs:99-100).
    """


class FreeList:
    """Integers ``0..n-1``; lowest free number first, so reuse is deterministic."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))  # pop() gives the lowest
        self._held = [False] * n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} in use)")
        i = self._free.pop()
        assert not self._held[i]
        self._held[i] = True
        return i

    def give_back(self, i: int) -> None:
        if not (0 <= i < self.n):
            raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is not in use: freed twice or never taken")
        self._held[i] = False
        # keep the list sorted descending so that take() returns the lowest number
        lo, hi = 0, len(self._free)
        while lo < hi:
            mid = (lo + hi) // 2
            if self._free[mid] > i:
                lo = mid + 1
            else:
                hi = mid
        self._free.insert(lo, i)

    def check(self) -> None:
        """Every number is either free or held, exactly once."""
        free = set(self._free)
        assert len(free) == len(self._free), f"{self.what}: a number is free twice"
        for i in range(self.n):
            assert self._held[i] != (i in free), f"{self.what} {i} is both free and held, or neither"
        assert sum(self._held) + len(self._free) == self.n, f"{self.what}: a number was lost"
