"""Fixed pools of ids with reference counts: cache pages and per-request state slots.

Same contract as the reference's ``BlockAllocator``
(src/locus/kv/block_allocator.hpp:25-73, block_allocator.cpp:7-54): a free list that hands
out the most recently freed id first (ids 0, 1, 2, ... from a fresh pool), a count per id,
``retain`` to share, ``release`` to drop one reference (the id is free again at zero), and
errors on misuse (double free, retain of a free id, id out of range).  Not thread-safe; the
scheduler serialises access.
"""
from __future__ import annotations

from typing import List


class AllocatorError(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, n: int) -> None:
        if n < 0:
            raise ValueError("pool size must not be negative")
        self._n = n
        self._free: List[int] = list(range(n - 1, -1, -1))  # pop() hands out 0 first
        self._refs: List[int] = [0] * n

    @property
    def total(self) -> int:
        return self._n

    @property
    def free(self) -> int:
        return len(self._free)

    def ref_count(self, i: int) -> int:
        self._check(i)
        return self._refs[i]

    def allocate(self) -> int:
        if not self._free:
            raise AllocatorError("pool exhausted")
        i = self._free.pop()
        self._refs[i] = 1
        return i

    def allocate_many(self, n: int) -> List[int]:
        """``n`` ids, all or nothing."""
        if n > len(self._free):
            raise AllocatorError(f"pool exhausted: {n} wanted, {len(self._free)} free")
        return [self.allocate() for _ in range(n)]

    def retain(self, i: int) -> None:
        self._check(i)
        if self._refs[i] == 0:
            raise AllocatorError(f"retain of free id {i}")
        self._refs[i] += 1

    def release(self, i: int) -> bool:
        """Drop one reference; True when the id went back to the free list."""
        self._check(i)
        if self._refs[i] == 0:
            raise AllocatorError(f"release of free id {i} (freed twice)")
        self._refs[i] -= 1
        if self._refs[i] == 0:
            self._free.append(i)
            return True
        return False

    def _check(self, i: int) -> None:
        if not (0 <= i < self._n):
            raise AllocatorError(f"id {i} out of range 0..{self._n - 1}")
