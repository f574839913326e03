"""Host-side bookkeeping of the cache: which slots and which pages are held.

Pure Python, no tensors: it can be tested without a GPU.  Every misuse (double
free, freeing what was never held, running out) raises :class:`CacheError`
instead of corrupting state.  The reference has no such pool: each sequence
owns buffers that grow by reallocation in 256-token chunks
(crates/qwen35/src/state.rs:225-311).
"""
from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free slot, or not enough free pages for the tokens asked for."""


class FreeList:
    """Ids 0..n-1, handed out lowest-first and taken back; freed ids are used again."""

    def __init__(self, n: int, what: str):
        if n <= 0:
            raise CacheError(f"a pool of {what}s needs at least one, got {n}")
        self._what = what
        self._n = n
        self._free: List[int] = list(range(n - 1, -1, -1))   # pop() gives the lowest id
        self._held = [False] * n

    @property
    def capacity(self) -> int:
        return self._n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self._n - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self._n and self._held[i]

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self._what} (all {self._n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def take_many(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"{n} {self._what}s asked for, {len(self._free)} of {self._n} are free")
        return [self.take() for _ in range(n)]

    def give_back(self, i: int) -> None:
        if not 0 <= i < self._n:
            raise CacheError(f"{self._what} {i} does not exist (there are {self._n})")
        if not self._held[i]:
            raise CacheError(f"{self._what} {i} is given back but is not held")
        self._held[i] = False
        self._free.append(i)
        # keep lowest-first order cheap: only re-sort when the tail is out of order
        if len(self._free) > 1 and self._free[-1] > self._free[-2]:
            self._free.sort(reverse=True)

    def check(self) -> None:
        """Invariant: every id is either free exactly once or held, never both."""
        seen = set(self._free)
        if len(seen) != len(self._free):
            raise CacheError(f"a {self._what} is in the free list twice")
        for i in range(self._n):
            if self._held[i] == (i in seen):
                raise CacheError(f"{self._what} {i} is {'both held and free' if self._held[i] else 'lost'}")
