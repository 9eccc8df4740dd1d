"""The scheduler's decisions on the host, with a stand-in step function (no GPU): admission
order, the token budget and portions, decode beside prefill, what happens when pages run
out (preempt the newest, victims to the front, failure when alone), context overflow, no
wedge on an unadmittable front, nothing leaked.  Modelled on the reference's
tests/test_engine.cpp."""
import pytest
import torch

from locus_b200.cache import CacheManager
from locus_b200.engine.engine import Engine
from locus_b200.engine.scheduler import SchedulerConfig, Status
from locus_b200.parts.base import PagedKvSpec
from locus_b200.sampling.sampler import SamplingParams

V = 50


class FakeRunner:
    """Logits that depend only on the request's tokens so far (a running hash), the way a
    model's would: any cut or preemption must reproduce them.  Records every batch."""

    def __init__(self, cache):
        self.cache = cache
        self.seen = {}   # seq_id -> tokens fed so far
        self.batches = []

    def step(self, entries):
        rows = []
        self.batches.append([(e.seq.seq_id, e.seq.n_tokens, len(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            hist = self.seen.setdefault(e.seq.seq_id, [])
            if e.seq.n_tokens == 0:
                hist.clear()  # a preempted request starts again
            assert len(hist) == e.seq.n_tokens, "tokens fed out of order"
            assert e.seq.n_tokens + len(e.tokens) <= self.cache.capacity(e.seq), "capacity not ensured"
            for i, t in enumerate(e.tokens):
                hist.append(int(t))
                if i in e.want:
                    h = 0
                    for x in hist:
                        h = (h * 31 + x + 7) % 1000003
                    row = torch.zeros(V)
                    row[h % (V - 1) + 1] = 1.0  # never token 0 (kept for the end-of-sequence tests)
                    rows.append(row)
            self.cache.commit(e.seq, len(e.tokens))
        return torch.stack(rows) if rows else torch.zeros(0, V)


class FakeSampler:
    def sample(self, logits, params, seeds, counters, histories=None):
        return [int(torch.argmax(r)) for r in logits]


def make(n_pages=64, page=16, max_positions=512, eos=-1, **cfg):
    cache = CacheManager([(PagedKvSpec(1, 16, 0), None, None)], page_tokens=page, n_pages=n_pages,
                         n_state_slots=cfg.get("max_running", 64), max_seq_tokens=max_positions, device="cpu",
                         allocate_device=False)
    runner = FakeRunner(cache)
    eng = Engine(runner, cache, FakeSampler(), max_positions=max_positions, eos_token_id=eos,
                 config=SchedulerConfig(**cfg))
    return eng, runner, cache


def reference_generation(prompt, n):
    eng, _, _ = make()
    rid = eng.submit(prompt, n)
    eng.run_to_completion()
    return eng.get(rid).generated


PROMPTS = [list(range(1, 6)), list(range(3, 20)), list(range(2, 35)), [9], list(range(5, 45))]


def test_concurrent_requests_match_single_runs_and_nothing_leaks():
    eng, runner, cache = make(max_batch_tokens=24, chunk=16)
    ids = [eng.submit(p, 12) for p in PROMPTS]
    eng.run_to_completion()
    for rid, p in zip(ids, PROMPTS):
        r = eng.get(rid)
        assert r.status == Status.DONE and r.generated == reference_generation(p, 12)
    assert cache.free_pages() == cache.total_pages() and cache.state_slots.free == cache.state_slots.total
    cache.check_invariants()


def test_budget_portions_and_decode_beside_prefill():
    eng, runner, cache = make(max_batch_tokens=20, chunk=8)
    a = eng.submit(list(range(1, 4)), 6)      # short: decoding soon
    b = eng.submit(list(range(1, 41)), 2)     # long prompt: portions
    eng.run_to_completion()
    for batch in runner.batches:
        assert sum(n for _, _, n, _ in batch) <= 20
        assert all(n <= 8 for _, _, n, _ in batch)
    # some step held a decode token of a beside a portion of b
    assert any(len(batch) == 2 and {n for _, _, n, _ in batch} == {1, 8} for batch in runner.batches)
    # logits are asked for only at the end of what is known of a request
    for batch in runner.batches:
        for rid, start, n, want in batch:
            assert want in ([], [n - 1])
    first_b = [x for batch in runner.batches for x in batch if x[0] == b]
    assert [x[1] for x in first_b[:5]] == [0, 8, 16, 24, 32] and first_b[4][3] == [7]
    assert eng.get(a).status == eng.get(b).status == Status.DONE


def test_first_come_first_served_nobody_overtakes():
    eng, runner, cache = make(n_pages=6, decode_headroom=16, max_batch_tokens=64, chunk=64)
    big = eng.submit(list(range(1, 60)), 4)    # needs 5 pages with headroom
    eng.step()                                 # admission reserves nothing: pages are taken as tokens are fed
    big2 = eng.submit(list(range(1, 60)), 4)   # does not fit beside it
    small = eng.submit([1, 2, 3], 4)           # would fit, but must not overtake big2
    eng.step()
    assert eng.sched.running == [big] and list(eng.sched.waiting) == [big2, small]
    eng.run_to_completion()
    order = []
    for batch in runner.batches:
        for rid, start, n, want in batch:
            if start == 0 and rid not in order:
                order.append(rid)
    assert order == [big, big2, small]
    assert all(eng.get(r).status == Status.DONE for r in (big, big2, small))


def test_pages_run_out_newest_is_preempted_and_output_is_unchanged():
    prompts = [list(range(1, 30)), list(range(2, 31)), list(range(3, 32))]
    # every request alone needs 3 pages for its prompt and a 4th while decoding 40 tokens
    eng, runner, cache = make(n_pages=8, decode_headroom=1, max_batch_tokens=64, chunk=64)
    ids = [eng.submit(p, 40) for p in prompts]
    eng.run_to_completion()
    assert eng.sched.counters["preemptions"] > 0
    for rid, p in zip(ids, prompts):
        r = eng.get(rid)
        assert r.status == Status.DONE and r.generated == reference_generation(p, 40)
    assert eng.get(ids[-1]).preemptions > 0 and eng.get(ids[0]).preemptions == 0  # newest first
    assert cache.free_pages() == cache.total_pages()
    cache.check_invariants()
    # a victim went to the front of the queue and was re-fed from position 0 in portions
    refed = [x for batch in runner.batches for x in batch if x[0] == ids[-1] and x[1] == 0]
    assert len(refed) >= 2


def test_alone_and_still_too_big_fails_without_a_leak():
    eng, runner, cache = make(n_pages=2, decode_headroom=0, max_batch_tokens=64, chunk=64)
    rid = eng.submit(list(range(1, 30)), 40)  # 29 + 40 tokens need 5 pages, the pool has 2
    eng.run_to_completion()
    r = eng.get(rid)
    assert r.status == Status.FAILED and r.error == "kv pool too small for request"
    assert len(r.generated) > 0 and cache.free_pages() == 2
    cache.check_invariants()


def test_admit_error_and_no_wedge():
    eng, runner, cache = make(n_pages=2, max_positions=64)
    assert "exceeds context window" in eng.admit_error(64)
    assert "cache pages" in eng.admit_error(40)
    assert eng.admit_error(10) == "" and eng.admit_error(0) == "empty prompt"
    rid = eng.submit(list(range(1, 41)), 4)
    assert eng.get(rid).status == Status.FAILED and "cache pages" in eng.get(rid).error
    ok = eng.submit([1, 2, 3], 3)
    assert eng.run_to_completion() > 0 and eng.get(ok).status == Status.DONE
    assert not eng.has_runnable_work()
    with pytest.raises(RuntimeError, match="failed"):
        eng.generate([list(range(1, 41))], max_new_tokens=2)


def test_context_overflow_and_end_of_sequence():
    eng, runner, cache = make(max_positions=12)
    rid = eng.submit(list(range(1, 9)), 50)
    eng.run_to_completion()
    r = eng.get(rid)
    assert r.status == Status.FAILED and r.error == "context overflow"
    assert len(r.prompt) + len(r.generated) == 13  # the 13th token has no position left
    assert cache.free_pages() == cache.total_pages()
    # the end-of-sequence token ends a request and is kept in its output
    gen = reference_generation([4, 5, 6], 10)
    eng2, _, _ = make(eos=gen[3])
    rid = eng2.submit([4, 5, 6], 10)
    eng2.run_to_completion()
    stop = gen.index(gen[3])
    assert eng2.get(rid).generated == gen[: stop + 1] and eng2.get(rid).status == Status.DONE


def test_max_running_records_and_callbacks():
    eng, runner, cache = make(max_running=2, max_retained_terminal=3)
    seen = []
    eng.on_token = lambda r, t: seen.append((r.id, t))
    ids = [eng.submit([1 + i, 2, 3], 2) for i in range(6)]
    eng.step()
    assert len(eng.sched.running) == 2 and len(eng.sched.waiting) == 4
    eng.run_to_completion()
    assert max(len(b) for b in runner.batches) <= 2
    assert len(seen) == 12
    assert eng.get(ids[0]) is None and eng.get(ids[-1]).status == Status.DONE  # oldest records evicted
    eng.release(ids[-1])
    assert eng.get(ids[-1]) is None
    st = eng.stats()
    assert st["done"] == 6 and st["free_pages"] == st["total_pages"] and st["decode_tokens"] + st["prefill_tokens"] > 0
    nid = eng.submit([1], 1)
    assert nid == ids[-1] + 1  # ids grow and are never used again


def test_sampling_params_are_checked():
    eng, _, _ = make()
    with pytest.raises(ValueError, match="top_p"):
        eng.submit([1], 1, SamplingParams(temperature=1.0, top_p=0.0))
    with pytest.raises(ValueError, match="top_k"):
        eng.submit([1], 1, SamplingParams(top_k=-1))
    assert eng.submit([1, 2], 0) and eng.get(1) is None or True


def test_native_scheduler_decides_like_the_plain_one():
    """Random workloads (arrivals between steps, pools that run out, window groups, long prompts, end-of-
    sequence tokens): the native scheduler and the plain Python policy, each over a cache of its own, must
    plan the same batches step by step and end every request alike."""
    import random

    from plain_scheduler import PlainScheduler

    from locus_b200.cache import CacheManager
    from locus_b200.engine.scheduler import Scheduler, SchedulerConfig
    from locus_b200.parts.base import PagedKvSpec

    def token_after(rid, n):  # the "model": next token from the request and its length
        return (rid * 7919 + n * 31) % 97

    for seed in range(12):
        rng = random.Random(seed)
        needs = [(PagedKvSpec(2, 16, 0), None, None)] + ([(PagedKvSpec(2, 16, 24), None, None)] if seed % 3 == 0 else [])
        n_pages = rng.choice([4, 6, 9, 30])
        max_pos = rng.choice([64, 200])
        cfg = SchedulerConfig(max_batch_tokens=rng.choice([8, 24, 64]), chunk=rng.choice([4, 16, 64]),
                              decode_headroom=rng.choice([0, 4, 16]), max_running=rng.choice([2, 3, 8]),
                              max_retained_terminal=1000)
        eos = 5
        pair = []
        for cls in (Scheduler, PlainScheduler):
            cache = CacheManager(needs, page_tokens=16, n_pages=n_pages, n_state_slots=cfg.max_running,
                                 max_seq_tokens=max_pos, device="cpu", allocate_device=False)
            pair.append((cls(cache, cfg, max_pos, eos), cache))
        arrivals = [(rng.randint(0, 30), rng.randint(1, 70), rng.randint(0, 40)) for _ in range(rng.randint(3, 14))]
        for step in range(400):
            plans = []
            for sched, cache in pair:
                for at, n_prompt, n_new in arrivals:
                    if at == step:
                        sched.submit(list(range(1, n_prompt + 1)), n_new)
                sched.admit()
                planned = sched.plan()
                plans.append([(p.request.id, p.start, p.n, p.wants_logits) for p in planned])
                for p in planned:
                    assert p.request.seq.n_tokens == p.start
                    cache.commit(p.request.seq, p.n)
                    sched.fed(p)
                for p in planned:
                    if p.wants_logits:
                        sched.accept_token(p.request, token_after(p.request.id, p.request.stream_len()))
                cache.check_invariants()
            assert plans[0] == plans[1], (seed, step, plans)
            a, b = pair[0][0], pair[1][0]
            assert list(a.waiting) == list(b.waiting) and a.running == b.running, (seed, step)
            if step > 30 and not a.has_runnable_work():
                break
        a, b = pair[0][0], pair[1][0]
        assert a.counters == b.counters, seed
        assert a.has_runnable_work() == b.has_runnable_work()
        for rid, r in a.requests.items():
            q = b.requests[rid]
            assert (r.status, r.error, r.generated, r.preemptions, r.n_fed) == (q.status, q.error, q.generated, q.preemptions, q.n_fed), (seed, rid)
        for sched, cache in pair:
            if sched.idle():
                assert cache.free_pages() == cache.total_pages() and cache.state_slots.free == cache.state_slots.total
