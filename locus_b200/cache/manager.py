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

Device layout of a group: ``pool[call, page, 0=K|1=V, kv_head, slot_in_page, head_dim]``;
a layer call sees ``pool[call]``.  A page id means the same page in every call of the group.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..engine.batch import LayerCache
from ..parts.base import PagedKvSpec, StateSpec
from .allocator import AllocatorError, PageAllocator


class CacheError(RuntimeError):
    pass


@dataclass
class SeqCache:
    """What one request holds: tokens cached, one page table per group, a state slot."""

    seq_id: object
    n_tokens: int = 0
    tables: Dict[int, List[int]] = field(default_factory=dict)  # -1 = page given back (window)
    state_slot: int = -1
    open: bool = True

    def pages_held(self, gid: int) -> int:
        return sum(1 for p in self.tables.get(gid, ()) if p >= 0)


class _Group:
    def __init__(self, gid: int, spec: PagedKvSpec, n_pages: int) -> None:
        self.gid = gid
        self.spec = spec
        self.calls: List[int] = []
        self.allocator = PageAllocator(n_pages)
        self.pool: Optional[torch.Tensor] = None


class CacheManager:
    def __init__(self, needs: Sequence[Tuple[Optional[PagedKvSpec], Optional[StateSpec], Optional[int]]], *,
                 page_tokens: int, n_pages: int, n_state_slots: int, max_seq_tokens: int,
                 dtype: torch.dtype = torch.float32, device="cpu", allocate_device: bool = True,
                 poison: bool = False) -> None:
        """``needs``: per entry of the model's run order, what its mixer keeps and whose cache
        it reads.  ``n_pages``: pages of every group.  ``poison``: fill pages with NaN when
        they are created and when they are given back (tests: a read of a stale or unwritten
        slot then shows in the logits)."""
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
                self.groups.append(_Group(gid, paged, n_pages))
            g = self.groups[gid]
            self._call_group.append(gid)
            self._call_index.append(len(g.calls))
            g.calls.append(i)
        self.state_slots = PageAllocator(n_state_slots)
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
                shape = (len(g.calls), n_pages, 2, g.spec.n_kv_heads, page_tokens, g.spec.head_dim)
                g.pool = torch.empty(shape, dtype=dtype, device=self.device)
                if poison:
                    g.pool.fill_(float("nan"))
        self._live: Dict[object, SeqCache] = {}

    # -- geometry -----------------------------------------------------------
    def bytes_per_token(self) -> int:
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.calls) * 2 * g.spec.n_kv_heads * g.spec.head_dim * el for g in self.groups)

    def pages_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.page_tokens)

    def free_pages(self, gid: Optional[int] = None) -> int:
        """Free pages of one group, or the smallest count over all groups."""
        if gid is not None:
            return self.groups[gid].allocator.free
        return min((g.allocator.free for g in self.groups), default=self.n_pages)

    def total_pages(self) -> int:
        return self.n_pages

    def layer_caches(self) -> List[LayerCache]:
        out = []
        for i, gid in enumerate(self._call_group):
            pool = None
            if gid is not None and self.groups[gid].pool is not None:
                pool = self.groups[gid].pool[self._call_index[i]]
            out.append(LayerCache(group=gid, pool=pool, page_tokens=self.page_tokens,
                                  state=self._state[i], writes=self._call_writes[i]))
        return out

    # -- requests -----------------------------------------------------------
    def open(self, seq_id) -> SeqCache:
        """Start a request: takes a state slot (zeroed); raises CacheError when none is free."""
        if seq_id in self._live:
            raise CacheError(f"request {seq_id!r} is already open")
        try:
            slot = self.state_slots.allocate()
        except AllocatorError:
            raise CacheError("no free state slot") from None
        for st in self._state:
            if st is not None:
                st[slot].zero_()
        seq = SeqCache(seq_id=seq_id, state_slot=slot, tables={g.gid: [] for g in self.groups})
        self._live[seq_id] = seq
        return seq

    def get(self, seq_id) -> Optional[SeqCache]:
        return self._live.get(seq_id)

    def live(self) -> List[SeqCache]:
        return list(self._live.values())

    def capacity(self, seq: SeqCache) -> int:
        """Tokens the request's tables can hold without taking another page."""
        if not self.groups:
            return self.max_seq_tokens
        return min(len(seq.tables[g.gid]) for g in self.groups) * self.page_tokens

    def pages_missing(self, seq: SeqCache, n_more: int) -> Dict[int, int]:
        want = self.pages_for(seq.n_tokens + n_more)
        return {g.gid: max(0, want - len(seq.tables[g.gid])) for g in self.groups}

    def ensure_capacity(self, seq: SeqCache, n_more: int) -> bool:
        """Make room for ``n_more`` tokens after the cached ones, in every group, all or
        nothing: False (and nothing taken) when any group is short of pages."""
        self._check_open(seq)
        if seq.n_tokens + n_more > self.max_seq_tokens:
            raise CacheError(f"request {seq.seq_id!r}: {seq.n_tokens + n_more} tokens exceed the "
                             f"limit of {self.max_seq_tokens}")
        missing = self.pages_missing(seq, n_more)
        for g in self.groups:
            if missing[g.gid] > g.allocator.free:
                return False
        for g in self.groups:
            seq.tables[g.gid].extend(g.allocator.allocate_many(missing[g.gid]))
        return True

    def commit(self, seq: SeqCache, n: int) -> None:
        """``n`` tokens were written after the cached ones.  Gives back window pages that no
        later query can see: a query at position p sees keys t > p - window, the next query
        is at position n_tokens, so pages wholly below n_tokens - window + 1 are dead."""
        self._check_open(seq)
        if seq.n_tokens + n > self.capacity(seq):
            raise CacheError(f"request {seq.seq_id!r}: commit of {n} tokens beyond its capacity")
        seq.n_tokens += n
        for g in self.groups:
            w = g.spec.window
            if w <= 0:
                continue
            dead = (seq.n_tokens - w + 1) // self.page_tokens
            table = seq.tables[g.gid]
            for i in range(min(max(dead, 0), len(table))):
                if table[i] >= 0:
                    self._give_back(g, table[i])
                    table[i] = -1

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
        for g in self.groups:
            for p in seq.tables[g.gid]:
                if p >= 0:
                    self._give_back(g, p)
            seq.tables[g.gid] = []
        self.state_slots.release(seq.state_slot)
        seq.state_slot = -1
        seq.n_tokens = 0
        seq.open = False
        del self._live[seq.seq_id]

    def _give_back(self, g: _Group, page: int) -> None:
        freed = g.allocator.release(page)
        if freed and self.poison and g.pool is not None:
            g.pool[:, page].fill_(float("nan"))

    def _check_open(self, seq: SeqCache) -> None:
        if not seq.open or self._live.get(seq.seq_id) is not seq:
            raise CacheError(f"request {seq.seq_id!r} is not open in this cache")

    # -- step descriptors -----------------------------------------------------
    def table_row(self, seq: SeqCache, gid: int) -> List[int]:
        return seq.tables[gid]

    def slot_of(self, seq: SeqCache, gid: int, pos: int) -> int:
        page = seq.tables[gid][pos // self.page_tokens]
        if page < 0:
            raise CacheError(f"request {seq.seq_id!r}: position {pos} lies in a page already given back")
        return page * self.page_tokens + pos % self.page_tokens

    # -- invariants -----------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, held twice or free while held; state slots likewise.  Raises."""
        for g in self.groups:
            held: Dict[int, int] = {}
            for seq in self._live.values():
                for p in seq.tables[g.gid]:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            for p, c in held.items():
                if c != 1:
                    raise CacheError(f"group {g.gid}: page {p} is held {c} times")
                if g.allocator.ref_count(p) != 1:
                    raise CacheError(f"group {g.gid}: page {p} is held but its count is {g.allocator.ref_count(p)}")
            if len(held) + g.allocator.free != g.allocator.total:
                raise CacheError(f"group {g.gid}: {g.allocator.total - g.allocator.free - len(held)} pages lost")
        slots = [s.state_slot for s in self._live.values()]
        if len(set(slots)) != len(slots):
            raise CacheError("a state slot is held twice")
        if len(slots) + self.state_slots.free != self.state_slots.total:
            raise CacheError("state slots lost")
