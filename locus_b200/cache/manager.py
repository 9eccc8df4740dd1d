"""The cache manager: pages of keys and values with a block table per request, one pool per
group of layers with the same needs, and slots for per-request state of fixed size.

The reference keeps one geometry for all layers and one table per sequence
(``PagedKvCache``, src/locus/kv/paged_cache.hpp:24-202; ``ensure_capacity`` all-or-nothing,
paged_cache.cpp:62-77; ``release`` paged_cache.cpp:79-85).  Here layers are sorted into
groups by what they keep -- all keys, or a window of them, of some (kv heads, head size) --
and every group has pages and a free list of its own; a request holds one table per group.
Pages go back to their pool when the request is released and, in a window group, as soon
as every position they hold has fallen out of the window.  A request also takes one state
slot when it is opened; layers with per-request state keep a tensor
[n_state_slots, *shape] that the slot indexes.

The bookkeeping (pools, tables, what a window has passed) is host code in C++
(``csrc/host_core.cpp``); this module owns the device tensors, words the errors, and hands
the step function the native object that assembles a step's descriptors from the tables.

Device layout of a group: ``pool[call, page, 0=K|1=V, kv_head, slot_in_page, head_dim]``;
a layer call sees ``pool[call]``.  A page id means the same page in every call of the group.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..engine.batch import LayerCache
from ..parts.base import PagedKvSpec, StateSpec
from . import native
from .allocator import AllocatorError  # noqa: F401  (part of this package's interface)


class CacheError(RuntimeError):
    pass


class SeqCache:
    """What one request holds: tokens cached, one page table per group, a state slot.  A view of
    the native record; after ``release`` it reads as closed and empty."""

    __slots__ = ("seq_id", "_cache", "_handle")

    def __init__(self, cache: "CacheManager", seq_id, handle: int) -> None:
        self.seq_id = seq_id
        self._cache = cache
        self._handle = handle

    @property
    def open(self) -> bool:
        return bool(self._cache._lib.locus_cache_is_open(self._cache._core, self._handle))

    @property
    def n_tokens(self) -> int:
        return max(0, self._cache._lib.locus_cache_n_tokens(self._cache._core, self._handle))

    @property
    def state_slot(self) -> int:
        return self._cache._lib.locus_cache_state_slot(self._cache._core, self._handle)

    @property
    def tables(self) -> Dict[int, List[int]]:
        """A copy of the page table of every group; -1 = page given back (window)."""
        return {g.gid: self._cache.table_row(self, g.gid) for g in self._cache.groups}

    def pages_held(self, gid: int) -> int:
        return sum(1 for p in self._cache.table_row(self, gid) if p >= 0)


class _Group:
    def __init__(self, gid: int, spec: PagedKvSpec) -> None:
        self.gid = gid
        self.spec = spec
        self.calls: List[int] = []
        self.n_pages = 0
        self.pool: Optional[torch.Tensor] = None    # [calls, pages, planes, kv heads, page_tokens, head_dim]
        self.extra: Optional[torch.Tensor] = None   # [calls, pages, page_tokens, extra_width]


class _StateSlots:
    """Counts of the per-request state slots."""

    def __init__(self, cache: "CacheManager") -> None:
        self._cache = cache

    @property
    def free(self) -> int:
        return self._cache._lib.locus_cache_slots_free(self._cache._core)

    @property
    def total(self) -> int:
        return self._cache._lib.locus_cache_slots_total(self._cache._core)


class CacheManager:
    def __init__(self, needs: Sequence[Tuple[Optional[PagedKvSpec], Optional[StateSpec], Optional[int]]], *,
                 page_tokens: int, n_pages: int, n_state_slots: int, max_seq_tokens: int,
                 dtype: torch.dtype = torch.float32, device="cpu", allocate_device: bool = True,
                 poison: bool = False, max_step_tokens: int = 0) -> None:
        """``needs``: per entry of the model's run order, what its mixer keeps and whose cache
        it reads.  ``n_pages``: pages of a group that keeps all tokens.  ``max_step_tokens`` > 0: the most
        tokens that one step feeds to one request; a group with a window then gets only the pages that
        ``n_state_slots`` requests can hold at once (window + step, rounded up to pages, plus one each)
        instead of ``n_pages``.  ``poison``: fill pages with NaN when they are created and when they are
        given back (tests: a read of a stale or unwritten slot then shows in the logits)."""
        if page_tokens <= 0 or n_pages < 0 or n_state_slots <= 0:
            raise ValueError("page_tokens and n_state_slots must be positive")
        self.page_tokens = page_tokens
        self.n_pages = n_pages
        self.max_seq_tokens = max_seq_tokens
        self.table_width = max(1, -(-max_seq_tokens // page_tokens))
        self.dtype, self.device, self.poison = dtype, torch.device(device), poison
        self.groups: List[_Group] = []
        self._call_group: List[Optional[int]] = []
        self._call_index: List[int] = []
        self._call_writes: List[bool] = []
        by_spec: Dict[PagedKvSpec, int] = {}
        for i, (paged, state, cache_of) in enumerate(needs):
            if cache_of is not None:
                self._call_group.append(self._call_group[cache_of])
                self._call_index.append(self._call_index[cache_of])
                self._call_writes.append(False)
                continue
            self._call_writes.append(True)
            if paged is None:
                self._call_group.append(None)
                self._call_index.append(-1)
                continue
            gid = by_spec.get(paged)
            if gid is None:
                gid = len(self.groups)
                by_spec[paged] = gid
                self.groups.append(_Group(gid, paged))
            g = self.groups[gid]
            self._call_group.append(gid)
            self._call_index.append(len(g.calls))
            g.calls.append(i)
        self._lib = native.lib()
        self.max_step_tokens = max(0, int(max_step_tokens))
        for g in self.groups:
            g.n_pages = n_pages
            if g.spec.window > 0 and self.max_step_tokens > 0:
                per_request = -(-(g.spec.window + self.max_step_tokens) // page_tokens) + 1
                g.n_pages = min(n_pages, n_state_slots * per_request)
        windows = (ctypes.c_int * max(1, len(self.groups)))(*[g.spec.window for g in self.groups])
        group_pages = (ctypes.c_int * max(1, len(self.groups)))(*[g.n_pages for g in self.groups])
        self._core = self._lib.locus_cache_new(len(self.groups), windows, page_tokens, group_pages, n_state_slots,
                                               max_seq_tokens)
        if not self._core:
            raise ValueError("the native cache could not be created from these sizes")
        assert self._lib.locus_cache_table_width(self._core) == self.table_width
        self.state_slots = _StateSlots(self)
        # (group, page) pairs that a commit or a release made free
        self._freed = (ctypes.c_int * (2 * max(1, len(self.groups)) * max(1, self.table_width)))()
        self._row = (ctypes.c_int * max(1, self.table_width))()
        self._state: List[Optional[torch.Tensor]] = []
        for i, (paged, state, cache_of) in enumerate(needs):
            if cache_of is not None:
                self._state.append(self._state[cache_of])
            elif state is not None and allocate_device:
                self._state.append(torch.zeros((n_state_slots,) + tuple(state.shape), dtype=state.dtype,
                                               device=self.device))
            else:
                self._state.append(None)
        if allocate_device:
            for g in self.groups:
                shape = (len(g.calls), g.n_pages, g.spec.planes, g.spec.n_kv_heads, page_tokens, g.spec.head_dim)
                g.pool = torch.empty(shape, dtype=dtype, device=self.device)
                if g.spec.extra_width > 0:
                    g.extra = torch.empty((len(g.calls), g.n_pages, page_tokens, g.spec.extra_width), dtype=dtype,
                                          device=self.device)
                if poison:
                    g.pool.fill_(float("nan"))
                    if g.extra is not None:
                        g.extra.fill_(float("nan"))
        self._live: Dict[object, SeqCache] = {}

    # -- geometry -----------------------------------------------------------
    def bytes_per_token(self) -> int:
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.calls) * g.spec.elements_per_token() * el for g in self.groups)

    def pages_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.page_tokens)

    def free_pages(self, gid: Optional[int] = None) -> int:
        """Free pages of one group, or the smallest count over all groups."""
        if gid is not None:
            return self._lib.locus_cache_free_pages(self._core, gid)
        return min((self._lib.locus_cache_free_pages(self._core, g.gid) for g in self.groups), default=self.n_pages)

    def total_pages(self, gid: Optional[int] = None) -> int:
        """Pages of one group's pool, or the smallest pool over all groups (so that an idle cache has
        ``free_pages() == total_pages()``)."""
        if gid is not None:
            return self.groups[gid].n_pages
        return min((g.n_pages for g in self.groups), default=self.n_pages)

    def pages_needed(self, gid: int, n_tokens: int, step_tokens: int = 0) -> int:
        """Pages that a request of ``n_tokens`` tokens holds in group ``gid`` at most when no step feeds it
        more than ``step_tokens`` tokens (0: unknown): all of them, or what covers the window and a step."""
        return self._lib.locus_cache_pages_needed(self._core, gid, n_tokens, step_tokens)

    def fits_when_empty(self, n_tokens: int, step_tokens: int = 0) -> bool:
        """Whether a request of ``n_tokens`` tokens fits the pools when nothing else is held."""
        return all(self.pages_needed(g.gid, n_tokens, step_tokens) <= g.n_pages for g in self.groups)

    def layer_caches(self) -> List[LayerCache]:
        out = []
        for i, gid in enumerate(self._call_group):
            pool = None
            if gid is not None and self.groups[gid].pool is not None:
                pool = self.groups[gid].pool[self._call_index[i]]
            extra = None
            if gid is not None and self.groups[gid].extra is not None:
                extra = self.groups[gid].extra[self._call_index[i]]
            out.append(LayerCache(group=gid, pool=pool, page_tokens=self.page_tokens,
                                  state=self._state[i], writes=self._call_writes[i], extra=extra))
        return out

    # -- requests -----------------------------------------------------------
    def open(self, seq_id) -> SeqCache:
        """Start a request: takes a state slot (zeroed); raises CacheError when none is free."""
        if seq_id in self._live:
            raise CacheError(f"request {seq_id!r} is already open")
        handle = self._lib.locus_cache_open(self._core)
        if handle < 0:
            raise CacheError("no free state slot")
        seq = SeqCache(self, seq_id, handle)
        slot = seq.state_slot
        for st in self._state:
            if st is not None:
                st[slot].zero_()
        self._live[seq_id] = seq
        return seq

    def adopt_native(self, seq_id, handle: int) -> SeqCache:
        """The view of a request that native code (the scheduler) opened in this cache: zeroes its state slot
        and makes it known here, as ``open`` does."""
        if seq_id in self._live:
            raise CacheError(f"request {seq_id!r} is already open")
        seq = SeqCache(self, seq_id, handle)
        if not seq.open:
            raise CacheError(f"request {seq_id!r}: the handle is not open in this cache")
        slot = seq.state_slot
        for st in self._state:
            if st is not None:
                st[slot].zero_()
        self._live[seq_id] = seq
        return seq

    def forget_native(self, seq: SeqCache, freed_pairs: Sequence[int] = ()) -> None:
        """Native code released the request: drop its view; ``freed_pairs``: the (group, page) it freed."""
        if self._live.get(seq.seq_id) is seq:
            del self._live[seq.seq_id]
        self.poison_pairs(freed_pairs)

    def poison_pairs(self, pairs: Sequence[int]) -> None:
        if self.poison:
            for i in range(0, len(pairs) - 1, 2):
                g = self.groups[pairs[i]]
                if g.pool is not None:
                    g.pool[:, pairs[i + 1]].fill_(float("nan"))
                    if g.extra is not None:
                        g.extra[:, pairs[i + 1]].fill_(float("nan"))

    def get(self, seq_id) -> Optional[SeqCache]:
        return self._live.get(seq_id)

    def live(self) -> List[SeqCache]:
        return list(self._live.values())

    def capacity(self, seq: SeqCache) -> int:
        """Tokens the request's tables can hold without taking another page."""
        return max(0, self._lib.locus_cache_capacity(self._core, seq._handle))

    def pages_missing(self, seq: SeqCache, n_more: int) -> Dict[int, int]:
        want = self.pages_for(seq.n_tokens + n_more)
        return {g.gid: max(0, want - len(self.table_row(seq, g.gid))) for g in self.groups}

    def ensure_capacity(self, seq: SeqCache, n_more: int) -> bool:
        """Make room for ``n_more`` tokens after the cached ones, in every group, all or
        nothing: False (and nothing taken) when any group is short of pages."""
        self._check_open(seq)
        r = self._lib.locus_cache_ensure(self._core, seq._handle, int(n_more))
        if r == -2:
            raise CacheError(f"request {seq.seq_id!r}: {seq.n_tokens + n_more} tokens exceed the "
                             f"limit of {self.max_seq_tokens}")
        if r < 0:
            self._not_open(seq)
        return r == 1

    def commit(self, seq: SeqCache, n: int) -> None:
        """``n`` tokens were written after the cached ones.  Gives back window pages that no
        later query can see: a query at position p sees keys t > p - window, the next query
        is at position n_tokens, so pages wholly below n_tokens - window + 1 are dead."""
        self._check_open(seq)
        r = self._lib.locus_cache_commit(self._core, seq._handle, int(n), self._freed, len(self._freed))
        if r == -3:
            raise CacheError(f"request {seq.seq_id!r}: commit of {n} tokens beyond its capacity")
        if r < 0:
            self._not_open(seq)
        self._poison_freed(r)

    def adopt(self, seq: SeqCache, n: int) -> bool:
        """Declare ``n`` more tokens as cached without writing them: takes the pages and
        advances the count.  For measurements on synthetic cache contents only; the keys
        and values are whatever the pages hold."""
        if not self.ensure_capacity(seq, n):
            return False
        self.commit(seq, n)
        return True

    def release(self, seq: SeqCache) -> None:
        """The request ends (or is preempted): everything it holds goes back."""
        self._check_open(seq)
        r = self._lib.locus_cache_release(self._core, seq._handle, self._freed, len(self._freed))
        if r < 0:
            self._not_open(seq)
        del self._live[seq.seq_id]
        self._poison_freed(r)

    def _poison_freed(self, n_pairs: int) -> None:
        if not self.poison:
            return
        assert 2 * n_pairs <= len(self._freed)
        for i in range(n_pairs):
            g = self.groups[self._freed[2 * i]]
            if g.pool is not None:
                g.pool[:, self._freed[2 * i + 1]].fill_(float("nan"))
                if g.extra is not None:
                    g.extra[:, self._freed[2 * i + 1]].fill_(float("nan"))

    def _not_open(self, seq: SeqCache) -> None:
        raise CacheError(f"request {seq.seq_id!r} is not open in this cache")

    def _check_open(self, seq: SeqCache) -> None:
        if seq._cache is not self or self._live.get(seq.seq_id) is not seq or not seq.open:
            self._not_open(seq)

    # -- step descriptors -----------------------------------------------------
    def table_row(self, seq: SeqCache, gid: int) -> List[int]:
        """A copy of the request's page table of one group (empty once the request is closed)."""
        if seq._cache is not self:
            self._not_open(seq)
        n = self._lib.locus_cache_table(self._core, seq._handle, gid, self._row, len(self._row))
        return list(self._row[: max(0, n)])

    def slot_of(self, seq: SeqCache, gid: int, pos: int) -> int:
        page = self.table_row(seq, gid)[pos // self.page_tokens]
        if page < 0:
            raise CacheError(f"request {seq.seq_id!r}: position {pos} lies in a page already given back")
        return page * self.page_tokens + pos % self.page_tokens

    # -- invariants -----------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, held twice or free while held; state slots likewise.  Raises."""
        d = (ctypes.c_int * 3)()
        code = self._lib.locus_cache_check(self._core, d)
        if code == 1:
            raise CacheError(f"group {d[0]}: page {d[1]} is held {d[2]} times")
        if code == 2:
            raise CacheError(f"group {d[0]}: page {d[1]} is held but its count is {d[2]}")
        if code == 3:
            raise CacheError(f"group {d[0]}: {d[1]} pages lost")
        if code == 4:
            raise CacheError("a state slot is held twice")
        if code == 5:
            raise CacheError("state slots lost")
        if len(self._live) + self.state_slots.free != self.state_slots.total:
            raise CacheError("the requests known here and the native records differ")

    def __del__(self) -> None:
        core, self._core = getattr(self, "_core", None), None
        if core:
            self._lib.locus_cache_delete(core)
