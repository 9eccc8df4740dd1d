"""The engine on the GPU against the plain implementation (float64 oracle), in float32 and
in bfloat16, for three tiny configurations: every request alone and whole; most of it in
one step and the last 32 tokens one by one; in portions of changing size down to two
tokens; mixed batches of up to four live requests with so few pages that pages are used
again; long decoding across the split boundary of the decode kernel; the first tokens of
a sequence; greedy and temperature generation through the entry point; trace replay as a
program.  Pages are poisoned with NaN when created and when given back, so a read of a
stale or unwritten slot shows in the logits.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen2moe as plain
from tiny_configs import make_model_dir, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# max |error| and mean |error| of the logits, relative to the largest |logit| of the request.
# float32: rounding of float32 sums over a few hundred terms and a few layers.
# bfloat16: activations, keys and values are rounded to 8 bits of mantissa between kernels.
TOL = {torch.float32: (5e-5, 1e-5), torch.bfloat16: (2e-2, 4e-3)}
# The router of the engine sees rounded activations; where two experts' probabilities are
# this close (relative) in the oracle, either choice is right and the oracle follows the engine.
NEAR_TIE = {torch.float32: 1e-5, torch.bfloat16: 1e-2}

REQUESTS = {  # name -> (length, seed); lengths straddle page edges (16 and 64) and the 256-key split
    "A": [(5, 1), (17, 2), (33, 3), (64, 4), (200, 5)],
    "B": [(1, 1), (7, 2), (64, 3), (100, 4), (129, 5), (300, 6)],
    "C": [(2, 1), (25, 2), (49, 3), (130, 4), (290, 5)],
    "D": [(700, 1), (333, 2), (40, 3)],
}


class Case:
    def __init__(self, name, tmp, raw=None, requests=None):
        self.name = name
        self.dir = make_model_dir(tmp, name, torch.bfloat16, raw=raw)
        self.cfg, self.weights = plain.load_folder(self.dir)
        self.tokens = {f"r{i}": random_tokens(n, self.cfg["vocab_size"], 100 * s + n)
                       for i, (n, s) in enumerate(requests or REQUESTS[name])}
        self._ref = {}

    def ref(self, rid):
        """(logits, aux) of the oracle with its own routing."""
        if rid not in self._ref:
            aux = {}
            lg = plain.forward(self.cfg, self.weights, self.tokens[rid], torch.float64, aux=aux)
            self._ref[rid] = (lg, aux)
        return self._ref[rid][0]

    def near_ties(self, rid, near_tie):
        """Positions where, in some layer, the k-th and (k+1)-th expert are within ``near_tie``."""
        self.ref(rid)
        k = self.cfg["num_experts_per_tok"]
        out = set()
        for prefix, rows in self._ref[rid][1].items():
            for pos, (ids, probs) in enumerate(rows):
                top = torch.sort(probs, descending=True).values
                if k < top.shape[0] and float(top[k]) >= float(top[k - 1]) * (1 - near_tie):
                    out.add(pos)
        return out

    def ref_following(self, rid, routed, near_tie):
        """Oracle logits when the engine's routing is followed.  The engine's router sees
        rounded activations, so at a near-tie it may pick the other expert; that is allowed
        only where the oracle's own probabilities of the swapped experts are within
        ``near_tie`` (relative) of each other.  Returns (logits, number of tokens that differ)."""
        base = self.ref(rid)
        aux = self._ref[rid][1]
        forced, n_diff = {}, 0
        for prefix, per_pos in (routed or {}).items():
            own = aux[prefix]
            rows = []
            for pos in range(len(self.tokens[rid])):
                ids, probs = own[pos]
                eng = per_pos.get(pos, ids)
                if sorted(eng) != sorted(ids):
                    n_diff += 1
                    kth = min(float(probs[e]) for e in ids)
                    for e in eng:
                        assert float(probs[e]) >= kth * (1 - near_tie), (
                            f"{self.name}/{rid} {prefix} position {pos}: the engine picked expert {e} "
                            f"(p={float(probs[e]):.6f}) although the k-th best has p={kth:.6f}")
                rows.append(eng)
            forced[prefix] = rows
        if n_diff == 0:
            return base, 0
        return plain.forward(self.cfg, self.weights, self.tokens[rid], torch.float64, forced_routing=forced), n_diff


@pytest.fixture(scope="module", params=["A", "B", "C"])
def case(request, tmp_path_factory):
    return Case(request.param, tmp_path_factory.mktemp("models"))


def make_runner(case, dtype, *, page_tokens=16, n_pages=64, max_tokens=320, use_graphs=False, max_seq=None):
    from locus_b200.cache import CacheManager
    from locus_b200.engine.step import ModelRunner
    from locus_b200.models import load_model

    model = load_model(case.dir, dtype, "cuda:0")
    cache = CacheManager(model.cache_needs(), page_tokens=page_tokens, n_pages=n_pages, n_state_slots=4,
                         max_seq_tokens=max_seq or case.cfg["max_position_embeddings"], dtype=dtype, device="cuda:0",
                         poison=True)
    return ModelRunner(model, cache, max_tokens=max_tokens, max_segments=4, use_graphs=use_graphs), cache


def run_trace(runner, cache, case, steps, observe=True):
    """steps: list of lists of (request id, n tokens).  Every fed position's logits are wanted.
    A request is released after its last token.  Returns {rid: [T, V] logits}."""
    from locus_b200.engine.step import StepEntry

    fed = {}
    got = {}
    routed = {}   # rid -> {moe prefix: {position: [experts]}}
    seen = []     # this step's (prefix, ids) in layer order

    for part in runner.model.all_parts():
        if hasattr(part, "observer"):
            part.observer = (lambda prefix, ids, wts: seen.append((prefix, ids.cpu().tolist()))) if observe else None
    if observe:
        case.routed = routed
    for step in steps:
        seen.clear()
        entries, spans = [], []
        for rid, n in step:
            a = fed.get(rid, 0)
            seq = cache.get(rid) or cache.open(rid)
            assert cache.ensure_capacity(seq, n), f"out of pages for {rid}"
            entries.append(StepEntry(seq, case.tokens[rid][a : a + n], list(range(n))))
            spans.append((rid, a, n))
            fed[rid] = a + n
        logits = runner.step(entries).float().cpu()
        row = 0
        for rid, a, n in spans:
            got.setdefault(rid, []).append((a, logits[row : row + n].clone()))
            for prefix, ids in seen:
                d = routed.setdefault(rid, {}).setdefault(prefix, {})
                for i in range(n):
                    d[a + i] = ids[row + i]
            row += n
        for rid, a, n in spans:
            if fed[rid] == len(case.tokens[rid]):
                cache.release(cache.get(rid))
        cache.check_invariants()
    out = {}
    for rid, parts in got.items():
        parts.sort(key=lambda p: p[0])
        out[rid] = torch.cat([p[1] for p in parts])
        assert out[rid].shape[0] == len(case.tokens[rid])
    return out


def check(case, got, dtype, what):
    tol_max, tol_mean = TOL[dtype]
    for rid, lg in got.items():
        ref, _ = case.ref_following(rid, getattr(case, "routed", {}).get(rid), NEAR_TIE[dtype])
        scale = float(ref.abs().max())
        err = (lg.double() - ref).abs()
        assert torch.isfinite(lg).all(), f"{what} {case.name}/{rid}: logits are not finite"
        worst = int(err.max(dim=1).values.argmax())
        assert float(err.max()) <= tol_max * scale, (
            f"{what} {case.name}/{rid}: max error {float(err.max()):.3e} > {tol_max * scale:.3e}; "
            f"first position above the bound: {int((err.max(dim=1).values > tol_max * scale).nonzero()[0])}, worst {worst}")
        assert float(err.mean()) <= tol_mean * scale, f"{what} {case.name}/{rid}: mean error {float(err.mean()):.3e}"


DTYPES = [torch.float32, torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_requests_alone(case, dtype):
    runner, cache = make_runner(case, dtype)
    got = run_trace(runner, cache, case, [[(rid, len(t))] for rid, t in case.tokens.items()])
    check(case, got, dtype, "whole")
    assert cache.free_pages() == cache.total_pages()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_portions_with_head_size_128(dtype, tmp_path_factory):
    """Head size 128, pages of 64 tokens, steps of 256 and more new tokens: in bfloat16 these portions run
    on the tcgen05 attention kernel (blocks of 128 queries, two of the step's 64-query tiles each), shorter
    steps and single tokens on the other kernels, all against the same cache."""
    import locus_b200.kernels as K

    case = Case("D", tmp_path_factory.mktemp("models_d"))
    used = []
    orig = K.attn_chunk_tc
    K.attn_chunk_tc = lambda *a, **k: (used.append(1), orig(*a, **k))[1]
    try:
        for steps in ([[("r0", 700)], [("r1", 333)], [("r2", 40)]],
                      [[("r0", 300), ("r2", 40)], [("r0", 256), ("r1", 77)], [("r0", 143), ("r1", 255)], [("r0", 1), ("r1", 1)]]):
            runner, cache = make_runner(case, dtype, page_tokens=64, n_pages=24, max_tokens=768, max_seq=1024)
            got = run_trace(runner, cache, case, steps)
            check(case, got, dtype, "long portions, head size 128")
            assert cache.free_pages() == cache.total_pages()
    finally:
        K.attn_chunk_tc = orig
    assert (len(used) > 0) == (dtype == torch.bfloat16)
    assert K.attn_tc_error() == 0 if dtype == torch.bfloat16 else True


def test_short_portions_behind_a_long_context_with_head_size_128(tmp_path_factory):
    """A prompt of 4,400 tokens: most of it in one step, then portions of 100, 17, 64 and 2 tokens and single
    tokens behind more than 4,000 cached ones, a second request beside them.  In bfloat16 the short portions run on
    the tcgen05 attention kernel with the keys of every block cut into ranges that a second launch merges."""
    import locus_b200.kernels as K
    from tiny_configs import config

    raw = config("D")
    raw["max_position_embeddings"] = 8192
    case = Case("D", tmp_path_factory.mktemp("models_d_long"), raw=raw, requests=[(4400, 7), (40, 3)])
    ranges = []
    orig = K.attn_chunk_tc
    K.attn_chunk_tc = lambda *a, **k: (ranges.append((a[0].shape[0], k.get("n_splits", 1))), orig(*a, **k))[1]
    try:
        runner, cache = make_runner(case, torch.bfloat16, page_tokens=64, n_pages=80, max_tokens=4224, max_seq=8192)
        steps = [[("r0", 4200)], [("r0", 100), ("r1", 38)], [("r0", 17), ("r1", 1)], [("r0", 64), ("r1", 1)], [("r0", 2)]]
        steps += [[("r0", 1)]] * (4400 - 4383)
        got = run_trace(runner, cache, case, steps)
        check(case, got, torch.bfloat16, "short portions behind a long context")
        assert cache.free_pages() == cache.total_pages()
    finally:
        K.attn_chunk_tc = orig
    assert K.attn_tc_error() == 0
    # the long first step in one range; every short portion behind it in several
    assert ranges[0] == (4200, 1) and all(n > 1 for t, n in ranges if t < 200) and sum(t < 200 for t, n in ranges) >= 8


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_portion_with_the_shared_expert_beside_the_router(dtype, tmp_path_factory):
    """A step of more than 1,024 tokens on a model with enough experts that each gets fewer than 192 rows: the
    shared expert then starts on the side stream before the router and runs beside the selection, the layout, the
    gather and the routed products.  Run once with the picked experts read back after every router (which waits for
    the device there) and once without a wait anywhere in the step; shorter steps of the same requests take the
    other orders."""
    import locus_b200.parts.feed_forward as FF
    from tiny_configs import config

    raw = config("D")
    raw["num_experts"], raw["max_position_embeddings"] = 16, 2048
    case = Case("D", tmp_path_factory.mktemp("models_d_wide"), raw=raw, requests=[(1190, 4), (60, 5)])
    beside = []
    orig = FF.DenseMlp.forward_up

    def forward_up(self, h, rt):
        beside.append((h.shape[0], rt.side_stream is not None and torch.cuda.current_stream() == rt.side_stream))
        return orig(self, h, rt)

    FF.DenseMlp.forward_up = forward_up
    try:
        for observe in (True, False):
            runner, cache = make_runner(case, dtype, page_tokens=64, n_pages=24, max_tokens=1280, max_seq=2048)
            steps = [[("r0", 1100), ("r1", 30)], [("r0", 88), ("r1", 29)], [("r0", 1), ("r1", 1)], [("r0", 1)]]
            got = run_trace(runner, cache, case, steps, observe=observe)
            check(case, got, dtype, f"shared expert beside the router (routing read back: {observe})")
            assert cache.free_pages() == cache.total_pages()
    finally:
        FF.DenseMlp.forward_up = orig
    n_layers = raw["num_hidden_layers"]
    assert beside.count((1130, True)) == 2 * n_layers and (1130, False) not in beside
    assert beside.count((117, False)) == 2 * n_layers and (117, True) not in beside   # 65 to 1,023 tokens: no overlap
    assert beside.count((2, True)) == 2 * n_layers                                    # up to 32 tokens: early as well


@pytest.mark.parametrize("dtype", DTYPES)
def test_last_32_tokens_one_by_one(case, dtype):
    runner, cache = make_runner(case, dtype)
    steps = []
    for rid, t in case.tokens.items():
        head = max(0, len(t) - 32)
        if head:
            steps.append([(rid, head)])
        steps += [[(rid, 1)] for _ in range(len(t) - head)]
    got = run_trace(runner, cache, case, steps)
    check(case, got, dtype, "prefill then decode")


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_changing_size(case, dtype):
    runner, cache = make_runner(case, dtype)
    sizes = [2, 16, 3, 17, 2, 31, 64, 5, 2, 15, 33, 1, 2, 48]
    steps = []
    for rid, t in case.tokens.items():
        a, i = 0, 0
        while a < len(t):
            n = min(sizes[i % len(sizes)], len(t) - a)
            steps.append([(rid, n)])
            a += n
            i += 1
    got = run_trace(runner, cache, case, steps)
    check(case, got, dtype, "portions")


def mixed_steps(case, max_live=4):
    """Up to four live requests: portions of some beside single tokens of others.  Each
    request is fed in portions up to 32 tokens before its last 8 tokens go one by one."""
    todo = list(case.tokens.items())
    live, fed, steps = [], {}, []
    sizes = [7, 32, 2, 19, 16, 5]
    k = 0
    while todo or live:
        while todo and len(live) < max_live:
            live.append(todo.pop(0)[0])
        step = []
        for rid in list(live):
            n_total = len(case.tokens[rid])
            a = fed.get(rid, 0)
            left = n_total - a
            n = 1 if left <= 8 else min(sizes[k % len(sizes)], left - 8)
            k += 1
            step.append((rid, n))
            fed[rid] = a + n
            if fed[rid] == n_total:
                live.remove(rid)
        steps.append(step)
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_batches_with_pages_used_again(case, dtype):
    longest = max(len(t) for t in case.tokens.values())
    steps = mixed_steps(case)
    # just enough pages for the four largest live requests: pages of finished requests are reused
    lens = sorted((len(t) for t in case.tokens.values()), reverse=True)
    n_pages = sum(-(-n // 16) for n in lens[:4])
    runner, cache = make_runner(case, dtype, page_tokens=16, n_pages=n_pages)
    got = run_trace(runner, cache, case, steps)
    check(case, got, dtype, "mixed")
    assert cache.free_pages() == cache.total_pages()
    # once more in the same pool, other order: every page has been used before
    order = list(reversed(list(case.tokens)))
    got = run_trace(runner, cache, case, [[(rid, len(case.tokens[rid]))] for rid in order])
    check(case, got, dtype, "whole after reuse")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(case, dtype):
    """A request decoded token by token from its very first token (positions 0, 1, 2, ...),
    with 64-token pages and the CUDA graph of single-token steps, beside a second request."""
    runner, cache = make_runner(case, dtype, page_tokens=64, n_pages=12)
    rids = list(case.tokens)
    long_rid, other = rids[-1], rids[-2]
    steps = []
    n_long, n_other = len(case.tokens[long_rid]), len(case.tokens[other])
    for i in range(max(n_long, n_other)):
        step = []
        if i < n_long:
            step.append((long_rid, 1))
        if i < n_other:
            step.append((other, 1))
        steps.append(step)
    got = run_trace(runner, cache, case, steps)
    check(case, got, dtype, "token by token")
    # the same steps replayed from CUDA graphs give the same bits
    grunner, gcache = make_runner(case, dtype, page_tokens=64, n_pages=12, use_graphs=True)
    ggot = run_trace(grunner, gcache, case, steps, observe=False)
    assert grunner.stats["graph_replays"] > 0
    for rid in got:
        assert torch.equal(got[rid], ggot[rid]), f"graph replay differs for {rid}"


def test_weights_stored_in_32_bit_stay_so(case, tmp_path):
    """A folder stored in float32, run as a bfloat16 model: matrices stay float32."""
    d = make_model_dir(tmp_path, case.name, torch.float32)
    from locus_b200.models import load_model

    model = load_model(d, torch.bfloat16, "cuda:0")
    assert all(p.dtype == torch.float32 for part in model.all_parts() for p in part.params.values())
    c32 = Case.__new__(Case)
    c32.name, c32.dir = case.name, d
    c32.cfg, c32.weights = plain.load_folder(d)
    c32.tokens = {"r": random_tokens(70, c32.cfg["vocab_size"], 9)}
    c32._ref, c32.routed = {}, {}
    runner, cache = make_runner(c32, torch.bfloat16)
    got = run_trace(runner, cache, c32, [[("r", 37)], [("r", 2)]] + [[("r", 1)]] * 31)
    check(c32, got, torch.bfloat16, "float32 weights in a bfloat16 model")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generate_greedy_and_sampled(case, dtype):
    from locus_b200.engine.engine import Engine

    eng = Engine.from_model_dir(case.dir, dtype=dtype, ctx=1024, page_tokens=16, max_batch_tokens=48, chunk=16,
                                max_running=4)
    prompts = [case.tokens[r][:n] for r, n in zip(list(case.tokens)[-3:], (5, 17, 33))]
    out = eng.generate(prompts, max_new_tokens=16)
    assert eng.cache.free_pages() == eng.cache.total_pages()
    for p, o in zip(prompts, out):
        assert len(o) == 16
        # every generated token must be the arg-max of the oracle's logits, unless the two
        # best logits are closer than the rounding of this element type
        full = p + o
        ref = plain.forward(case.cfg, case.weights, full, torch.float64)
        for i, tok in enumerate(o):
            row = ref[len(p) + i - 1]
            top2 = torch.topk(row, 2).values
            margin = float(top2[0] - row[tok])
            assert margin <= TOL[torch.float32 if dtype == "float32" else torch.bfloat16][0] * float(ref.abs().max()) * 2, \
                f"token {i}: picked {tok}, margin to the best {margin:.3e}"
    # the same prompts in one batch, one by one, and in another order give the same tokens
    again = [eng.generate([p], max_new_tokens=16)[0] for p in reversed(prompts)]
    if dtype == "float32":
        assert again == list(reversed(out))
    # temperature sampling: reproducible for a seed, independent of the batch
    s1 = eng.generate(prompts, max_new_tokens=12, temperature=0.8, seed=1)
    s2 = eng.generate(prompts, max_new_tokens=12, temperature=0.8, seed=1)
    assert s1 == s2
    s3 = eng.generate(prompts, max_new_tokens=12, temperature=0.8, seed=2)
    assert s3 != s1
    assert eng.cache.free_pages() == eng.cache.total_pages()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_survives_running_out_of_pages(case, dtype):
    """A pool too small for all requests at once: the newest request is preempted and recomputed later,
    and every request still gets the tokens it gets from a large pool."""
    from locus_b200.engine.engine import Engine

    names = list(case.tokens)[-3:]
    prompts = [case.tokens[r][:n] for r, n in zip(names, (30, 41, 25))]
    big = Engine.from_model_dir(case.dir, dtype=dtype, ctx=1024, page_tokens=16, max_batch_tokens=32, chunk=16,
                                max_running=4, decode_headroom=0)
    want = big.generate(prompts, max_new_tokens=24)
    # 7 pages of 16 tokens: any single request fits (at most 65 tokens), two of them do not
    small = Engine.from_model_dir(case.dir, dtype=dtype, ctx=7 * 16, page_tokens=16, max_batch_tokens=32, chunk=16,
                                  max_running=4, decode_headroom=0)
    got = small.generate(prompts, max_new_tokens=24)
    assert small.sched.counters["preemptions"] > 0 and small.sched.counters["failed"] == 0
    assert small.cache.free_pages() == small.cache.total_pages()
    small.cache.check_invariants()
    if dtype == "float32":
        assert got == want
    else:
        # bfloat16: a recomputed request runs in other batches; a token may differ only where the oracle's
        # two best logits are within the rounding of the element type
        for p, o in zip(prompts, got):
            ref = plain.forward(case.cfg, case.weights, p + o, torch.float64)
            for i, tok in enumerate(o):
                row = ref[len(p) + i - 1]
                assert float(row.max() - row[tok]) <= TOL[torch.bfloat16][0] * float(ref.abs().max()) * 2


def test_pool_sized_by_a_share_of_free_memory(tmp_path_factory):
    """``kv_fraction`` sizes the pool from the device memory that is free after the weights are loaded."""
    from locus_b200.engine.engine import Engine

    c = Case("A", tmp_path_factory.mktemp("models_kvf"))
    free, _ = torch.cuda.mem_get_info()
    share = (64 << 20) / free   # about 64 MiB of cache
    eng = Engine.from_model_dir(c.dir, dtype="bfloat16", page_tokens=64, max_running=4, kv_fraction=share)
    held = eng.cache.total_pages() * 64 * eng.cache.bytes_per_token()
    assert 0.5 * (64 << 20) <= held <= (64 << 20) + 64 * eng.cache.bytes_per_token()
    assert eng.cache.max_seq_tokens == min(c.cfg["max_position_embeddings"], eng.cache.total_pages() * 64)
    out = eng.generate([c.tokens["r1"][:9]], max_new_tokens=4)
    assert len(out[0]) == 4 and eng.cache.free_pages() == eng.cache.total_pages()
    with pytest.raises(ValueError, match="kv_fraction"):
        Engine.from_model_dir(c.dir, dtype="bfloat16", kv_fraction=1.5)


def replay_program(case, dtype, steps, out_dir, *, max_tokens, page_tokens=64, max_live=4, extra=()):
    """Run ``steps`` (lists of (request, n new tokens), every fed position wanted) through bin/trace_run as a
    program.  Returns ({rid: [T, V] logits}, returncode, stderr) and leaves the engine's expert choices in
    ``case.routed`` as ``run_trace`` does."""
    import numpy as np

    lines, layout, fed = [], [], {}
    for no, step in enumerate(steps):
        entries, end, spans = [], [], []
        for rid, n in step:
            a = fed.get(rid, 0)
            base = rid.split("/")[-1]
            entries.append({"id": rid, "tokens": case.tokens[base][a : a + n], "want": list(range(n))})
            spans.append((rid, a, n))
            fed[rid] = a + n
            if fed[rid] == len(case.tokens[base]):
                end.append(rid)
        lines.append(json.dumps({"step": no, "entries": entries, "end": end}))
        layout.append(spans)
    dt_name = "float32" if dtype == torch.float32 else "bfloat16"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", case.dir, "--dtype", dt_name, "--out",
           str(out_dir), "--max-tokens", str(max_tokens), "--page-tokens", str(page_tokens), "--max-live", str(max_live),
           "--dump-routing", *extra]
    proc = subprocess.run(cmd, input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
    if proc.returncode != 0:
        return None, proc.returncode, proc.stderr
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    V = case.cfg["vocab_size"]
    got, routed = {}, {}
    for no, spans in enumerate(layout):
        arr = torch.from_numpy(np.fromfile(os.path.join(str(out_dir), f"{no}.f32"), dtype="<f4").reshape(-1, V).copy())
        with open(os.path.join(str(out_dir), f"{no}.route.json")) as f:
            route = json.load(f)
        assert arr.shape[0] == sum(n for _, _, n in spans)
        row = 0
        for rid, a, n in spans:
            got.setdefault(rid, []).append(arr[row : row + n])
            for prefix, ids in route.items():
                d = routed.setdefault(rid, {}).setdefault(prefix, {})
                for i in range(n):
                    d[a + i] = ids[row + i]
            row += n
    case.routed = routed
    return {rid: torch.cat(parts) for rid, parts in got.items()}, 0, proc.stderr


def check_program(case, got, dtype, what):
    """``check`` for request ids of the form <mode>/<request>: same tokens, same oracle."""
    tol_max, tol_mean = TOL[dtype]
    for rid, lg in got.items():
        base = rid.split("/")[-1]
        assert lg.shape[0] == len(case.tokens[base]), f"{what} {rid}: {lg.shape[0]} rows"
        ref, _ = case.ref_following(base, case.routed.get(rid), NEAR_TIE[dtype])
        scale = float(ref.abs().max())
        err = (lg.double() - ref).abs()
        assert torch.isfinite(lg).all(), f"{what} {case.name}/{rid}: logits are not finite"
        assert float(err.max()) <= tol_max * scale, (
            f"{what} {case.name}/{rid}: max error {float(err.max()):.3e} > {tol_max * scale:.3e}; first position "
            f"above the bound: {int((err.max(dim=1).values > tol_max * scale).nonzero()[0])}")
        assert float(err.mean()) <= tol_mean * scale, f"{what} {case.name}/{rid}: mean error {float(err.mean()):.3e}"


def four_modes(case):
    """The four ways of replaying the same requests, one after the other in one trace: whole; most of it in one step
    and the last 32 tokens one by one; portions of changing size down to two tokens; mixed, up to four live."""
    rids = list(case.tokens)
    steps = [[("whole/" + r, len(case.tokens[r]))] for r in rids]
    for r in rids:
        n = len(case.tokens[r])
        head = max(0, n - 32)
        if head:
            steps.append([("tail/" + r, head)])
        steps += [[("tail/" + r, 1)]] * (n - head)
    sizes = [2, 16, 3, 17, 2, 31, 64, 5, 2, 15, 33, 1, 2, 48]
    for r in rids:
        a, i = 0, 0
        while a < len(case.tokens[r]):
            n = min(sizes[i % len(sizes)], len(case.tokens[r]) - a)
            steps.append([("cut/" + r, n)])
            a, i = a + n, i + 1
    steps += [[("mixed/" + r, n) for r, n in step] for step in mixed_steps(case)]
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program_in_four_modes(case, dtype, tmp_path):
    """bin/trace_run as a program (its own process, the engine's model, step function, cache and kernels): the
    four ways of cutting in one trace, in a pool that holds just the four largest requests, so that every page
    is used again and again; pages of 64 tokens, and of 16 for the configuration with the window."""
    if case.name == "C" and dtype == torch.float32:
        pytest.skip("the windowed configuration replays in bfloat16; A and B in both element types")
    P = 16 if case.name == "C" else 64
    lens = sorted((len(t) for t in case.tokens.values()), reverse=True)
    max_tokens = sum(-(-n // P) * P for n in lens[:4])
    got, code, err = replay_program(case, dtype, four_modes(case), tmp_path / "out", max_tokens=max_tokens, page_tokens=P)
    assert code == 0, err[-2000:]
    assert len(got) == 4 * len(case.tokens)
    check_program(case, got, dtype, "trace_run")


def test_trace_run_program_options_and_refusals(tmp_path_factory):
    """Pages of 16 tokens with two live requests; a pool that runs out ends the program with a message and 2,
    as does a third live request when --max-live is 2."""
    case = Case("A", tmp_path_factory.mktemp("models_tr"))
    r = list(case.tokens)
    n3, n4 = len(case.tokens[r[3]]), len(case.tokens[r[4]])
    steps = [[(r[3], 30), (r[4], 2)], [(r[3], n3 - 30), (r[4], 100)], [(r[4], n4 - 102), (r[2], len(case.tokens[r[2]]))]]
    need = -(-n3 // 16) * 16 + -(-n4 // 16) * 16
    out = tmp_path_factory.mktemp("trace_out")
    got, code, err = replay_program(case, torch.float32, steps, out / "ok", max_tokens=need, page_tokens=16, max_live=2)
    assert code == 0, err[-2000:]
    check_program(case, got, torch.float32, "trace_run, pages of 16")
    # ten pages: the second step wants 4 + 7
    got, code, err = replay_program(case, torch.float32, steps, out / "short", max_tokens=160, page_tokens=16,
                                    max_live=2)
    assert code == 2 and "out of cache pages" in err
    three = [[(r[0], 2), (r[1], 2), (r[2], 2)]]
    got, code, err = replay_program(case, torch.float32, three, out / "live", max_tokens=256, page_tokens=16, max_live=2)
    assert code == 2 and "--max-live 2" in err


def _sampled(eng, prompts_and_seeds, n_new, sp, watch):
    """Submit the requests in order and run; returns the watched request's tokens and its record."""
    ids = [eng.submit(p, n_new, sp, seed) for p, seed in prompts_and_seeds]
    eng.run_to_completion()
    recs = [eng.get(i) for i in ids]
    assert all(r.status.value == "done" for r in recs), [r.error for r in recs]
    out = (list(recs[watch].generated), recs[watch].preemptions)
    for i in ids:
        eng.release(i)
    assert eng.cache.free_pages() == eng.cache.total_pages()
    return out


def test_sampled_tokens_do_not_depend_on_batching_chunking_or_preemption(tmp_path_factory):
    """tiny-B's workload: 24 samples at temperature 0.8 with seed 1.  The same request gives the same tokens alone,
    beside three others, with its prompt cut into portions of 16, and after it was preempted and recomputed: the
    draw is keyed by (seed, index of the generated token) and the logits by nothing but the request's own tokens."""
    from locus_b200.engine.engine import Engine
    from locus_b200.sampling.sampler import SamplingParams

    case = Case("B", tmp_path_factory.mktemp("models_smp"))
    sp = SamplingParams(temperature=0.8)
    r = list(case.tokens)
    mine = case.tokens[r[3]][:41]
    others = [case.tokens[r[5]][:60], case.tokens[r[4]][:30], case.tokens[r[2]][:25]]

    def engine(**kw):
        args = dict(dtype="float32", ctx=1024, page_tokens=16, max_batch_tokens=256, chunk=256, max_running=4,
                    decode_headroom=0)
        args.update(kw)
        return Engine.from_model_dir(case.dir, **args)

    alone, _ = _sampled(engine(), [(mine, 1)], 24, sp, 0)
    assert len(alone) == 24 and len(set(alone)) > 4   # sampled, not a constant
    greedy, _ = _sampled(engine(), [(mine, 1)], 24, SamplingParams(), 0)
    assert greedy != alone
    beside, _ = _sampled(engine(), [(others[0], 7), (mine, 1), (others[1], 8), (others[2], 9)], 24, sp, 1)
    assert beside == alone
    chunked, _ = _sampled(engine(max_batch_tokens=32, chunk=16), [(others[1], 5), (mine, 1)], 24, sp, 1)
    assert chunked == alone
    # a pool of 8 pages: the two requests cannot both finish in it; the newest (ours) is preempted and recomputed
    small = engine(ctx=8 * 16, max_batch_tokens=32, chunk=16)
    again, n_pre = _sampled(small, [(others[0], 7), (mine, 1)], 24, sp, 1)
    assert n_pre > 0 and small.sched.counters["failed"] == 0
    assert again == alone
    other_seed, _ = _sampled(engine(), [(mine, 2)], 24, sp, 0)
    assert other_seed != alone


@pytest.mark.parametrize("dtype", DTYPES)
def test_released_midway_and_fed_again_from_the_start(case, dtype):
    """What preemption does to a request (src/locus/engine/engine.cpp:230-239 of the reference): its pages go back
    mid-way, others take them, later it is fed again from position 0 on pages that others have used (poisoned with
    NaN in between).  Every position's logits of every feeding against the plain implementation."""
    from locus_b200.engine.step import StepEntry

    rids = list(case.tokens)
    victim, other, third = rids[-1], rids[-2], rids[-3]
    nv, no, nt = (len(case.tokens[x]) for x in (victim, other, third))
    P = 16
    runner, cache = make_runner(case, dtype, page_tokens=P, n_pages=-(-nv // P) + -(-no // P))
    cut = (2 * nv) // 3
    seen = []
    for part in runner.model.all_parts():
        if hasattr(part, "observer"):
            part.observer = lambda prefix, ids, wts: seen.append((prefix, ids.cpu().tolist()))
    feedings = {}   # name -> (request, {position: logits row}, {prefix: {position: experts}})

    def feed(name, rid, seq, a, n):
        seen.clear()
        assert cache.ensure_capacity(seq, n), f"out of pages feeding {name}"
        lg = runner.step([StepEntry(seq, case.tokens[rid][a : a + n], list(range(n)))]).float().cpu()
        _, rows, routed = feedings.setdefault(name, (rid, {}, {}))
        for i in range(n):
            rows[a + i] = lg[i].clone()
        for prefix, ids in seen:
            routed.setdefault(prefix, {}).update({a + i: ids[i] for i in range(n)})

    v = cache.open("victim")
    feed("first", victim, v, 0, cut // 2)
    o = cache.open("other")
    feed("other", other, o, 0, no // 2)
    feed("first", victim, v, cut // 2, cut - cut // 2)       # the victim is two thirds through ...
    held = v.pages_held(0)
    cache.release(v)                                          # ... and loses everything
    cache.check_invariants()
    feed("other", other, o, no // 2, no - no // 2)            # the other grows into the freed pages
    t = cache.open("third")
    feed("third", third, t, 0, nt)
    cache.release(t)
    v = cache.open("victim")                                  # readmitted: from position 0, in portions, then token by token
    a = 0
    for n in (cut // 3, 2, cut - cut // 3 - 2):
        feed("again", victim, v, a, n)
        a += n
    cache.release(o)
    while a < nv:
        n = 1 if nv - a <= 8 else min(19, nv - a - 8)
        feed("again", victim, v, a, n)
        a += n
    assert held > 0
    cache.release(v)
    assert cache.free_pages() == cache.total_pages()
    cache.check_invariants()
    tol_max, tol_mean = TOL[dtype]
    for name, (rid, rows, routed) in feedings.items():
        ref, _ = case.ref_following(rid, routed, NEAR_TIE[dtype])
        places = sorted(rows)
        assert places == list(range(len(places))) and (name == "first") == (len(places) < len(case.tokens[rid]))
        got = torch.stack([rows[p] for p in places]).double()
        assert torch.isfinite(got).all(), f"{name}: logits are not finite (a stale or poisoned page was read)"
        err = (got - ref[: len(places)]).abs()
        scale = float(ref.abs().max())
        assert float(err.max()) <= tol_max * scale, f"{name}: max error {float(err.max()):.3e} at {int(err.max(dim=1).values.argmax())}"
        assert float(err.mean()) <= tol_mean * scale, name


def test_expert_counters_through_graphs_and_the_kernel_time_table(tmp_path_factory):
    """The expert counters count once per executed step, also when decode steps are replayed from their CUDA graph
    (the counting is one more launch of the graph); the opt-in kernel time table makes steps run eagerly, names the
    entry points that ran and charges them times that fit into the wall clock of the scope."""
    import time

    import locus_b200.kernels as K
    from locus_b200.engine.moe_stats import MoeStats
    from locus_b200.engine.step import StepEntry

    case = Case("B", tmp_path_factory.mktemp("models_telemetry"))
    runner, cache = make_runner(case, torch.bfloat16, use_graphs=True)
    stats = MoeStats(runner.model)
    toks = case.tokens["r5"]
    seq = cache.open("a")

    def feed(a, n):
        assert cache.ensure_capacity(seq, n)
        return runner.step([StepEntry(seq, toks[a : a + n], [n - 1])])

    feed(0, 60)
    for i in range(60, 72):
        feed(i, 1)
    replays = runner.stats["graph_replays"]
    assert replays >= 10
    k, n_moe = case.cfg["num_experts_per_tok"], len(stats.counts)
    assert n_moe > 0 and stats.summary()["activations"] == 72 * k * n_moe
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with K.kernel_times() as kt:
        assert K.timing_active()
        for i in range(72, 76):
            feed(i, 1)
        feed(76, 24)
        table = kt.table()
    wall_ms = (time.perf_counter() - t0) * 1e3
    assert not K.timing_active() and runner.stats["graph_replays"] == replays   # nothing was replayed inside
    for what in ("embed_rows", "rmsnorm", "linear", "rope_kv_write", "attn_decode"):
        assert what in table and table[what][0] > 0, (what, sorted(table))
    total = sum(ms for _, ms in table.values())
    assert all(ms >= 0.0 for _, ms in table.values()) and 0.0 < total <= 2.0 * wall_ms + 1.0   # two streams at most
    feed(100, 1)
    assert runner.stats["graph_replays"] == replays + 1                          # and graphs again afterwards
    assert stats.summary()["activations"] == 101 * k * n_moe
    cache.release(seq)
