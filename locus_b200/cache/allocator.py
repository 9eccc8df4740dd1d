"""Fixed pools of ids with reference counts: cache pages and per-request state slots.

Same contract as the reference's ``BlockAllocator``
(src/locus/kv/block_allocator.hpp:25-73, block_allocator.cpp:7-54): a free list that hands
out the most recently freed id first (ids 0, 1, 2, ... from a fresh pool), a count per id,
``retain`` to share, ``release`` to drop one reference (the id is free again at zero), and
errors on misuse (double free, retain of a free id, id out of range).  The pool itself is
the ``Pool`` of ``csrc/host_core.cpp``, the type the cache's own pools are made of; this
class words its return codes.  Not thread-safe; the scheduler serialises access.
"""
from __future__ import annotations

from typing import List

from . import native


class AllocatorError(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, n: int) -> None:
        if n < 0:
            raise ValueError("pool size must not be negative")
        self._lib = native.lib()
        self._pool = self._lib.locus_pool_new(n)
        self._n = n

    def __del__(self) -> None:
        pool, self._pool = getattr(self, "_pool", None), None
        if pool:
            self._lib.locus_pool_delete(pool)

    @property
    def total(self) -> int:
        return self._n

    @property
    def free(self) -> int:
        return self._lib.locus_pool_free(self._pool)

    def ref_count(self, i: int) -> int:
        r = self._lib.locus_pool_refs(self._pool, int(i))
        if r < 0:
            self._out_of_range(i)
        return r

    def allocate(self) -> int:
        i = self._lib.locus_pool_allocate(self._pool)
        if i < 0:
            raise AllocatorError("pool exhausted")
        return i

    def allocate_many(self, n: int) -> List[int]:
        """``n`` ids, all or nothing."""
        if n > self.free:
            raise AllocatorError(f"pool exhausted: {n} wanted, {self.free} free")
        return [self.allocate() for _ in range(n)]

    def retain(self, i: int) -> None:
        r = self._lib.locus_pool_retain(self._pool, int(i))
        if r == -1:
            self._out_of_range(i)
        if r == -2:
            raise AllocatorError(f"retain of free id {i}")

    def release(self, i: int) -> bool:
        """Drop one reference; True when the id went back to the free list."""
        r = self._lib.locus_pool_release(self._pool, int(i))
        if r == -1:
            self._out_of_range(i)
        if r == -2:
            raise AllocatorError(f"release of free id {i} (freed twice)")
        return r == 1

    def _out_of_range(self, i: int) -> None:
        raise AllocatorError(f"id {i} out of range 0..{self._n - 1}")
