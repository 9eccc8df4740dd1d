"""Page allocator and cache manager bookkeeping (no GPU): no page lost, held twice or freed
twice, under random orders of requests; window groups give pages back as the window passes;
state slots follow their requests.  Modelled on the reference's tests/test_block_allocator.cpp
and tests/test_paged_cache.cpp."""
import random

import pytest
import torch

from locus_b200.cache import AllocatorError, CacheError, CacheManager, PageAllocator
from locus_b200.parts.base import PagedKvSpec, StateSpec


def test_allocator_hands_out_ids_from_zero_and_reuses_the_last_freed():
    a = PageAllocator(4)
    assert [a.allocate() for _ in range(3)] == [0, 1, 2] and a.free == 1
    assert a.release(1) and a.allocate() == 1  # most recently freed first
    assert a.allocate() == 3
    with pytest.raises(AllocatorError, match="exhausted"):
        a.allocate()
    with pytest.raises(AllocatorError, match="exhausted"):
        a.allocate_many(1)


def test_allocator_reference_counts_and_misuse():
    a = PageAllocator(2)
    p = a.allocate()
    a.retain(p)
    assert a.ref_count(p) == 2 and not a.release(p) and a.free == 1
    assert a.release(p) and a.free == 2
    with pytest.raises(AllocatorError, match="freed twice"):
        a.release(p)
    with pytest.raises(AllocatorError, match="retain of free"):
        a.retain(p)
    with pytest.raises(AllocatorError, match="out of range"):
        a.ref_count(2)
    assert a.allocate_many(2) == [0, 1] or a.free == 0


def _needs(window=0, layers=3, state=False):
    spec = PagedKvSpec(2, 16, 0)
    out = [(spec, StateSpec((4,)) if state else None, None) for _ in range(layers)]
    if window:
        out += [(PagedKvSpec(2, 16, window), None, None) for _ in range(2)]
    return out


def mk(n_pages=8, window=0, state=False, **kw):
    return CacheManager(_needs(window, state=state), page_tokens=16, n_pages=n_pages, n_state_slots=3,
                        max_seq_tokens=kw.pop("max_seq_tokens", 256), device="cpu", **kw)


def test_capacity_in_whole_pages_all_or_nothing():
    c = mk(n_pages=4)
    s = c.open("a")
    assert c.capacity(s) == 0
    assert c.ensure_capacity(s, 1) and c.capacity(s) == 16 and c.free_pages() == 3
    assert c.ensure_capacity(s, 16) and c.free_pages() == 3  # nothing committed yet: same page suffices
    c.commit(s, 16)
    assert c.ensure_capacity(s, 17) and c.free_pages() == 1
    t = c.open("b")
    assert not c.ensure_capacity(t, 33) and c.free_pages() == 1 and t.tables[0] == []  # all or nothing
    assert c.ensure_capacity(t, 16)
    with pytest.raises(CacheError, match="beyond its capacity"):
        c.commit(t, 17)
    c.release(s)
    c.release(t)
    assert c.free_pages() == 4
    c.check_invariants()
    with pytest.raises(CacheError, match="not open"):
        c.ensure_capacity(s, 1)
    with pytest.raises(CacheError, match="not open"):
        c.release(s)


def test_groups_have_pages_of_their_own_and_windows_give_pages_back():
    c = mk(n_pages=8, window=20)
    assert len(c.groups) == 2 and c.groups[1].spec.window == 20
    lay = c.layer_caches()
    assert [l.group for l in lay] == [0, 0, 0, 1, 1]
    assert lay[0].pool.shape == (8, 2, 2, 16, 16) and lay[3].pool.data_ptr() != lay[0].pool.data_ptr()
    s = c.open("a")
    assert c.ensure_capacity(s, 70)
    assert c.free_pages(0) == 3 and c.free_pages(1) == 3
    c.commit(s, 70)
    # next query at position 70 sees keys > 50: pages 0..2 (keys 0..47) are dead in the window group
    assert s.tables[1][:3] == [-1, -1, -1] and s.tables[1][3] >= 0
    assert c.free_pages(0) == 3 and c.free_pages(1) == 6
    with pytest.raises(CacheError, match="given back"):
        c.slot_of(s, 1, 10)
    assert c.slot_of(s, 0, 10) == s.tables[0][0] * 16 + 10
    for _ in range(30):
        assert c.ensure_capacity(s, 1)
        c.commit(s, 1)
    assert s.n_tokens == 100
    assert s.pages_held(1) <= 3  # a window of 20 never holds more than ceil(20/16)+1 pages
    c.check_invariants()
    c.release(s)
    assert c.free_pages(0) == 8 and c.free_pages(1) == 8


def test_state_slots_follow_requests_and_start_at_zero():
    c = mk(state=True)
    a, b = c.open("a"), c.open("b")
    assert {a.state_slot, b.state_slot} == {0, 1}
    st = c.layer_caches()[0].state
    assert st.shape == (3, 4)
    st[a.state_slot] = 7.0
    c.release(a)
    d = c.open("d")
    assert d.state_slot == 0  # the slot that was just given back is used again
    assert float(c.layer_caches()[0].state[d.state_slot].abs().sum()) == 0.0  # zeroed on open
    c.open("e")
    with pytest.raises(CacheError, match="no free state slot"):
        c.open("f")
    with pytest.raises(CacheError, match="already open"):
        c.open("e")


def test_layer_that_reads_another_layers_cache_shares_its_pages():
    spec = PagedKvSpec(1, 16, 0)
    c = CacheManager([(spec, None, None), (spec, None, 0), (spec, None, None)], page_tokens=16, n_pages=2,
                     n_state_slots=1, max_seq_tokens=32, device="cpu")
    lay = c.layer_caches()
    assert lay[1].pool.data_ptr() == lay[0].pool.data_ptr() and not lay[1].writes and lay[2].writes
    assert c.groups[0].pool.shape[0] == 2  # two calls keep a cache, not three


def test_limit_per_request():
    c = mk(max_seq_tokens=40)
    s = c.open("a")
    with pytest.raises(CacheError, match="exceed the limit"):
        c.ensure_capacity(s, 41)


@pytest.mark.parametrize("seed", range(6))
def test_random_workload_loses_nothing(seed):
    """Random opens, growth, commits, releases and failed allocations; after every operation
    no page is lost or held twice; at the end everything is free again."""
    rng = random.Random(seed)
    c = mk(n_pages=12, window=rng.choice([0, 20, 40]), poison=True, dtype=torch.float32)
    live = {}
    ensured = {}
    for i in range(400):
        op = rng.random()
        if op < 0.2 and len(live) < 3:
            live[i] = c.open(i)
            ensured[i] = 0
        elif op < 0.7 and live:
            k = rng.choice(list(live))
            s = live[k]
            n = rng.randint(1, 40)
            if s.n_tokens + n > c.max_seq_tokens:
                continue
            before = {g.gid: c.free_pages(g.gid) for g in c.groups}
            tables = {g: list(t) for g, t in s.tables.items()}
            if c.ensure_capacity(s, n):
                c.commit(s, rng.randint(1, n))
            else:
                assert {g.gid: c.free_pages(g.gid) for g in c.groups} == before and s.tables == tables
        elif live:
            k = rng.choice(list(live))
            c.release(live.pop(k))
        c.check_invariants()
    for s in live.values():
        c.release(s)
    c.check_invariants()
    assert all(c.free_pages(g.gid) == 12 for g in c.groups) and c.state_slots.free == 3


def test_a_closed_request_stays_closed_when_its_record_is_used_again():
    """The native record of a released request is reused by the next one; the old view must not see it."""
    c = mk(n_pages=4)
    a = c.open("a")
    assert c.ensure_capacity(a, 20) and a.pages_held(0) == 2
    c.commit(a, 20)
    c.release(a)
    b = c.open("b")   # takes a's record and state slot
    assert c.ensure_capacity(b, 5)
    assert not a.open and a.n_tokens == 0 and a.state_slot == -1 and a.tables == {0: []}
    assert b.open and b.tables[0] != [] and c.capacity(a) == 0
    for call in (lambda: c.ensure_capacity(a, 1), lambda: c.commit(a, 1), lambda: c.release(a)):
        with pytest.raises(CacheError, match="not open"):
            call()
    other = mk(n_pages=4)
    with pytest.raises(CacheError, match="not open"):
        other.ensure_capacity(b, 1)   # a request of another cache
    c.release(b)
    c.check_invariants()
    assert c.free_pages() == 4 and c.state_slots.free == 3


def test_a_window_group_gets_a_pool_of_its_own_size():
    """With the step size known, a group with a window holds what the live requests can hold at once (window + step,
    in pages, plus one each), not as many pages as a group that keeps everything; requests are admitted against
    each group's own need."""
    c = CacheManager(_needs(window=20), page_tokens=16, n_pages=40, n_state_slots=3, max_seq_tokens=256,
                     dtype=torch.float32, device="cpu", max_step_tokens=32)
    full, win = c.groups
    assert (full.n_pages, win.n_pages) == (40, 3 * (-(-(20 + 32) // 16) + 1)) and win.pool.shape[1] == 15
    assert c.total_pages(0) == 40 and c.total_pages(1) == 15 and c.total_pages() == 15 == c.free_pages()
    assert c.pages_needed(0, 200, 32) == 13 and c.pages_needed(1, 200, 32) == 5 and c.pages_needed(1, 30, 32) == 2
    assert c.fits_when_empty(256, 32) and not c.fits_when_empty(41 * 16, 32)
    # three requests of 200 tokens, fed 32 at a time: the window group never runs out
    seqs = [c.open(i) for i in range(3)]
    for a in range(0, 200, 32):
        for s in seqs:
            n = min(32, 200 - a)
            assert c.ensure_capacity(s, n)
            c.commit(s, n)
            assert s.pages_held(1) <= 5
        c.check_invariants()
    assert c.free_pages(0) == 40 - 3 * 13
    for s in seqs:
        c.release(s)
    assert c.free_pages(0) == 40 and c.free_pages(1) == 15
    c.check_invariants()
    # without a step size the window group is as large as the others
    d = CacheManager(_needs(window=20), page_tokens=16, n_pages=40, n_state_slots=3, max_seq_tokens=256,
                     dtype=torch.float32, device="cpu")
    assert [g.n_pages for g in d.groups] == [40, 40]


def test_rows_without_values_and_fields_beside_the_rows():
    spec = PagedKvSpec(2, 16, 0, has_v=False, extra_width=3)
    assert spec.planes == 1 and spec.elements_per_token() == 2 * 16 + 3
    c = CacheManager([(spec, None, None), (PagedKvSpec(2, 16), None, None)], page_tokens=16, n_pages=4,
                     n_state_slots=2, max_seq_tokens=64, dtype=torch.bfloat16, device="cpu", poison=True)
    assert len(c.groups) == 2
    assert c.groups[0].pool.shape == (1, 4, 1, 2, 16, 16) and c.groups[0].extra.shape == (1, 4, 16, 3)
    assert c.groups[1].pool.shape == (1, 4, 2, 2, 16, 16) and c.groups[1].extra is None
    assert c.bytes_per_token() == 2 * ((2 * 16 + 3) + 2 * 2 * 16)
    lay = c.layer_caches()
    assert lay[0].extra.shape == (4, 16, 3) and lay[1].extra is None and lay[0].pool.shape == (4, 1, 2, 16, 16)
    s = c.open("r")
    assert c.ensure_capacity(s, 20)
    page = s.tables[0][0]
    lay[0].extra[page] = 1.0
    c.commit(s, 20)
    c.release(s)
    assert torch.isnan(lay[0].extra[page].float()).all()   # fields are poisoned with their page
