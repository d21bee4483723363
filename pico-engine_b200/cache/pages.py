"""Host-side bookkeeping of the cache: the free list of pages of one group and the free list
of sequence slots.  Both refuse to lose, double-hold or double-free what they manage.
"""
from __future__ import annotations

from typing import List


class CacheFull(RuntimeError):
    """More tokens (or sequences) are alive than the cache was sized for."""


class CacheStateError(RuntimeError):
    """A page or slot was given back twice, or one that was never taken."""


class FreeList:
    """Integers 0..n-1, taken and given back.  The lowest free ones are taken first, so a
    batch that follows another uses the same ones again."""

    def __init__(self, n: int, what: str):
        self.n, self.what = n, what
        self._free: List[int] = list(range(n - 1, -1, -1))     # pop() yields the lowest
        self._held = [False] * n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def take(self, count: int = 1) -> List[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}(s) wanted, {len(self._free)} of {self.n} free")
        got = [self._free.pop() for _ in range(count)]
        for i in got:
            self._held[i] = True
        return got

    def give(self, items) -> None:
        items = list(items)
        for i in items:
            if not (0 <= i < self.n) or not self._held[i]:
                raise CacheStateError(f"{self.what} {i} is given back but is not held")
            self._held[i] = False
        self._free.extend(items)
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Every item is either free or held, exactly once."""
        if len(set(self._free)) != len(self._free):
            raise CacheStateError(f"a {self.what} is in the free list twice")
        for i in range(self.n):
            if self._held[i] == (i in set(self._free)):
                raise CacheStateError(f"{self.what} {i} is {'both held and free' if self._held[i] else 'lost'}")
