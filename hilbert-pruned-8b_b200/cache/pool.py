"""Index pools: pages of the key/value cache and slots of per-sequence state.

An index is either free or held by exactly one owner.  Giving back an index that is not
held, or one outside the pool, raises: a slot lost, held twice or freed twice is a fault of
the caller that must not pass silently.
"""
from __future__ import annotations

from typing import Iterable, List


class CacheFull(RuntimeError):
    """No page (or slot) is free for what was asked."""


class IndexPool:
    def __init__(self, size: int, what: str = "page"):
        if size < 0:
            raise ValueError(f"{what} pool: negative size")
        self.size = size
        self.what = what
        self._held = bytearray(size)
        # lowest index first, so that a finished batch's indices are the next ones used
        self._free: List[int] = list(range(size - 1, -1, -1))

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.size - len(self._free)

    def alloc(self, n: int = 1) -> List[int]:
        if n < 0:
            raise ValueError(f"{self.what} pool: negative count")
        if n > len(self._free):
            raise CacheFull(f"cache: {n} {self.what}s asked for, {len(self._free)} of {self.size} free")
        out = [self._free.pop() for _ in range(n)]
        for i in out:
            self._held[i] = 1
        return out

    def free(self, indices: Iterable[int]) -> None:
        indices = list(indices)
        for i in indices:
            if not 0 <= i < self.size:
                raise ValueError(f"cache: {self.what} {i} is outside the pool of {self.size}")
            if not self._held[i]:
                raise ValueError(f"cache: {self.what} {i} is given back but not held")
            self._held[i] = 0
        # keep the free list sorted so that allocation order does not depend on history
        self._free.extend(indices)
        self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return bool(self._held[i])
