"""The engine's host logic on the CPU (no GPU): with the CUDA entry points replaced by their
torch twins, the real model, parts, cache manager, step function, scheduler and sampler
front end run whole prompts, portions, mixed batches with reused pages and generation, and
must agree with the plain implementation.  What this does not cover -- the kernels
themselves -- is covered by the gpu tests."""
import pytest
import torch

import emulated_kernels as EK
import plain_qwen2moe as plain
from locus_b200.cache import CacheError, CacheManager
from locus_b200.engine.engine import Engine
from locus_b200.engine.scheduler import SchedulerConfig
from locus_b200.engine.step import ModelRunner, StepEntry, StepError
from locus_b200.models import load_model
from locus_b200.sampling.sampler import Sampler
from tiny_configs import make_model_dir, random_tokens


@pytest.fixture(autouse=True)
def _emulate(monkeypatch):
    EK.install(monkeypatch)


def setup(name, tmp_path, n_pages=12, page=16, max_tokens=64):
    d = make_model_dir(tmp_path, name, torch.float32)
    cfg, W = plain.load_folder(d)
    model = load_model(d, torch.float32, "cpu")
    cache = CacheManager(model.cache_needs(), page_tokens=page, n_pages=n_pages, n_state_slots=4,
                         max_seq_tokens=cfg["max_position_embeddings"], dtype=torch.float32, device="cpu", poison=True)
    return cfg, W, model, cache, ModelRunner(model, cache, max_tokens=max_tokens, max_segments=4)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_cuts_and_mixed_batches_agree_with_plain(name, tmp_path):
    cfg, W, model, cache, runner = setup(name, tmp_path, n_pages=7)
    toks = {r: random_tokens(n, cfg["vocab_size"], n) for r, n in (("a", 45), ("b", 33), ("c", 18), ("d", 30))}
    ref = {r: plain.forward(cfg, W, t, torch.float64) for r, t in toks.items()}
    # a and b start; c joins; b ends and d takes its pages (7 pages: never room for all four)
    steps = [[("a", 20), ("b", 2)], [("a", 1), ("b", 31)], [("a", 5), ("c", 16)], [("a", 1), ("c", 1), ("d", 17)],
             [("a", 18), ("c", 1), ("d", 13)]]
    fed, got = {}, {r: [] for r in toks}
    for step in steps:
        entries = []
        for r, n in step:
            a = fed.get(r, 0)
            seq = cache.get(r) or cache.open(r)
            assert cache.ensure_capacity(seq, n), (r, n)
            entries.append(StepEntry(seq, toks[r][a : a + n], list(range(n))))
            fed[r] = a + n
        lg = runner.step(entries)
        row = 0
        for r, n in step:
            got[r].append(lg[row : row + n].clone())
            row += n
        for r, n in step:
            if fed[r] == len(toks[r]):
                cache.release(cache.get(r))
        cache.check_invariants()
    for r in toks:
        out = torch.cat(got[r]).double()
        assert out.shape == ref[r].shape
        assert float((out - ref[r]).abs().max()) <= 2e-5 * float(ref[r].abs().max()), r
    assert cache.free_pages() == cache.total_pages()


def test_step_refuses_bad_batches(tmp_path):
    cfg, W, model, cache, runner = setup("A", tmp_path)
    s = cache.open("a")
    with pytest.raises(CacheError, match="not ensured"):
        runner.step([StepEntry(s, [1, 2, 3], [2])])
    assert cache.ensure_capacity(s, 3)
    with pytest.raises(StepError, match="outside the vocabulary"):
        runner.step([StepEntry(s, [1, 256, 3], [])])
    with pytest.raises(StepError, match="wanted place"):
        runner.step([StepEntry(s, [1, 2, 3], [3])])
    with pytest.raises(StepError, match="twice"):
        runner.step([StepEntry(s, [1], []), StepEntry(s, [2], [])])
    with pytest.raises(StepError, match="no tokens"):
        runner.step([StepEntry(s, [], [])])
    with pytest.raises(StepError, match="at least one entry"):
        runner.step([])
    other = CacheManager(model.cache_needs(), page_tokens=16, n_pages=2, n_state_slots=1, max_seq_tokens=32, device="cpu")
    foreign = other.open("x")
    other.ensure_capacity(foreign, 2)
    with pytest.raises(CacheError, match="not open in the runner's cache"):
        runner.step([StepEntry(foreign, [1, 2], [])])
    assert s.n_tokens == 0  # nothing ran
    big = cache.open("big")
    assert cache.ensure_capacity(big, 70)
    with pytest.raises(StepError, match="built for 64"):
        runner.step([StepEntry(big, list(range(70)), [])])
    # context overflow is refused before launch
    cfg2, W2, model2, cache2, runner2 = setup("A", tmp_path, n_pages=20, max_tokens=300)
    s2 = cache2.open("long")
    assert cache2.ensure_capacity(s2, 256)
    runner2.step([StepEntry(s2, [1] * 256, [])])
    with pytest.raises((StepError, CacheError), match="overflow|exceed"):
        cache2.ensure_capacity(s2, 1)
        runner2.step([StepEntry(s2, [1], [0])])


@pytest.mark.parametrize("name", ["A", "B"])
def test_generation_through_the_engine_matches_plain_greedy(name, tmp_path):
    cfg, W, model, cache, runner = setup(name, tmp_path, n_pages=16)
    eng = Engine(runner, cache, Sampler("cpu", 4), max_positions=cfg["max_position_embeddings"],
                 config=SchedulerConfig(max_batch_tokens=24, chunk=16, max_running=4, decode_headroom=4))
    prompts = [random_tokens(n, cfg["vocab_size"], 7 * n) for n in (5, 17, 33)]
    out = eng.generate(prompts, max_new_tokens=6)
    for p, o in zip(prompts, out):
        assert o == plain.greedy_generate(cfg, W, p, 6, torch.float64)
    assert cache.free_pages() == cache.total_pages()
    # temperature sampling goes through the same path and is reproducible
    a = eng.generate(prompts[:2], max_new_tokens=5, temperature=0.8, seed=1)
    b = eng.generate(prompts[:2], max_new_tokens=5, temperature=0.8, seed=1)
    assert a == b and all(len(x) == 5 for x in a)
    # penalties reach the sampler with the request's history
    from locus_b200.sampling.sampler import SamplingParams
    c = eng.generate(prompts[:1], max_new_tokens=5, sampling=SamplingParams(repeat_penalty=1.5, presence_penalty=0.5))
    assert len(c[0]) == 5


def test_moe_stats_count_every_pick_and_word_the_reference_line(tmp_path):
    """The expert counters against the plain implementation's routing of the same tokens: every (layer, expert)
    count, the number of activations and the reference's one-line report."""
    from locus_b200.engine.moe_stats import MoeStats

    cfg, W, model, cache, runner = setup("B", tmp_path, n_pages=16)
    stats = MoeStats(model)
    toks = random_tokens(40, cfg["vocab_size"], 3)
    s = cache.open("a")
    fed = 0
    for n in (23, 16, 1):   # two portions and a single token
        assert cache.ensure_capacity(s, n)
        runner.step([StepEntry(s, toks[fed : fed + n], [n - 1])])
        fed += n
    aux = {}
    plain.forward(cfg, W, toks, torch.float64, aux=aux)
    table = stats.table()
    assert set(table) == set(aux) and len(table) > 0
    k = cfg["num_experts_per_tok"]
    for prefix, rows in aux.items():
        want = [0] * cfg["num_experts"]
        for ids, _ in rows:
            for e in ids:
                want[int(e)] += 1
        assert table[prefix] == want, prefix
    sm = stats.summary()
    assert sm["activations"] == 40 * k * len(table) and sm["slots"] == cfg["num_experts"] * len(table)
    assert 1 <= sm["min_unique"] <= sm["max_unique"] <= cfg["num_experts"]
    line = stats.report()
    assert line.startswith(f"moe-stats: {sm['activations']} activations; experts touched per moe layer min ")
    assert f"{sm['touched']} of {sm['slots']} (" in line and line.endswith("layer-expert slots touched")
    stats.detach()
    assert all(p.observer is None for p in stats.parts)
    assert cache.ensure_capacity(s, 1)
    runner.step([StepEntry(s, [1], [0])])
    assert stats.summary()["activations"] == sm["activations"]   # detached: counts no more


def plain_descriptors(cache, entries, chunk_tile, mma_tile):
    """The descriptors of a step, written down from their definitions with lists."""
    P, W = cache.page_tokens, cache.table_width
    out = {k: [] for k in ("tokens", "positions", "seg_q0", "seg_qn", "seg_ctx", "state_slots", "want_rows",
                           "chunk_items", "decode_items", "chunk_items64")}
    groups = {g.gid: {"slots": [], "table": []} for g in cache.groups}
    for s, e in enumerate(entries):
        n, ctx = len(e.tokens), e.seq.n_tokens
        out["seg_q0"].append(len(out["tokens"]))
        out["seg_qn"].append(n)
        out["seg_ctx"].append(ctx)
        out["state_slots"].append(e.seq.state_slot)
        out["want_rows"] += [len(out["tokens"]) + w for w in e.want]
        out["tokens"] += list(e.tokens)
        out["positions"] += list(range(ctx, ctx + n))
        if n == 1:
            out["decode_items"].append(s)
        else:
            out["chunk_items"] += [[s, q] for q in range(0, n, chunk_tile)]
            out["chunk_items64"] += [[s, q] for q in range(0, n, mma_tile)]
        for gid, row in e.seq.tables.items():
            groups[gid]["slots"] += [row[p // P] * P + p % P for p in range(ctx, ctx + n)]
            groups[gid]["table"].append(row + [-1] * (W - len(row)))
    # tiles by the position of their first query, ascending; ties keep the order of the requests
    for k in ("chunk_items", "chunk_items64"):
        out[k] = sorted(out[k], key=lambda sq: out["seg_ctx"][sq[0]] + sq[1])
    return out, groups


def test_step_descriptors_match_a_plain_assembly(tmp_path):
    """The native step assembly against the same descriptors built with Python lists: random mixed steps
    over a cache with a window group (tables with holes) beside a full one, requests that end and come back."""
    import random

    import locus_b200.kernels as K
    from locus_b200.parts.attention import CHUNK_TILE, AttentionTiles

    cfg, W, model, cache, runner = setup("C", tmp_path, n_pages=40, page=16, max_tokens=96)
    assert list(runner.plans) == [AttentionTiles.key]   # every attention layer shares the one plan
    assert any(g.spec.window > 0 for g in cache.groups) and any(g.spec.window == 0 for g in cache.groups)
    rng = random.Random(4)
    names = ["a", "b", "c", "d"]
    for it in range(60):
        entries = []
        for r in rng.sample(names, rng.randint(1, 4)):
            seq = cache.get(r) or cache.open(r)
            n = rng.choice([1, 1, 2, 3, 16, 17, 23])
            if seq.n_tokens + n > 150 or not cache.ensure_capacity(seq, n):
                cache.release(seq)
                continue
            toks = [rng.randrange(cfg["vocab_size"]) for _ in range(n)]
            entries.append(StepEntry(seq, toks, sorted(rng.sample(range(n), rng.randint(0, min(n, 3))))))
        if not entries:
            continue
        want, want_groups = plain_descriptors(cache, entries, CHUNK_TILE, K.MMA_QUERY_TILE)
        batch = runner._build(entries, fixed_shapes=False)
        tiles = batch.plans[AttentionTiles.key]   # the attention part's own work lists ride in the same buffer
        for k, v in want.items():
            got = tiles[k] if k in tiles else getattr(batch, k)
            assert got.tolist() == v, (it, k)
        assert (batch.T, batch.n_seg, batch.n_want) == (len(want["tokens"]), len(entries), len(want["want_rows"]))
        assert (tiles["n_chunk_items"], tiles["n_chunk_items64"], tiles["n_decode_items"]) == (
            len(want["chunk_items"]), len(want["chunk_items64"]), len(want["decode_items"]))
        assert batch.longest == max(e.seq.n_tokens + len(e.tokens) for e in entries) and not batch.static_shapes
        assert batch.host_seg_q0 == want["seg_q0"] and batch.host_seg_ctx == want["seg_ctx"]
        assert batch.host_seg_qn == want["seg_qn"] and batch.host_state_slots == want["state_slots"]
        for gid, g in want_groups.items():
            assert batch.groups[gid].slots.tolist() == g["slots"], (it, gid)
            assert batch.groups[gid].block_table.tolist() == g["table"], (it, gid)
        for e in entries:
            cache.commit(e.seq, len(e.tokens))
        cache.check_invariants()


def test_step_refuses_numbers_that_fit_no_field(tmp_path):
    """Token ids and wanted places far outside 32 (or 64) bits, negative ones, more wanted rows or requests
    than the runner was built for, a released request: refused with an error, nothing runs, the next good
    step is unharmed."""
    cfg, W, model, cache, runner = setup("A", tmp_path)
    s = cache.open("a")
    assert cache.ensure_capacity(s, 4)
    for bad in ([1, 2 ** 40, 3], [-1, 2, 3], [2 ** 31, 1], [1, 2 ** 70]):
        with pytest.raises(StepError, match="outside the vocabulary"):
            runner.step([StepEntry(s, bad, [])])
    for bad in ([-1], [2 ** 40], [2 ** 70]):
        with pytest.raises(StepError, match="wanted place|outside"):
            runner.step([StepEntry(s, [1, 2, 3], bad)])
    with pytest.raises(StepError, match="rows wanted"):
        small = ModelRunner(model, cache, max_tokens=64, max_segments=4, max_wanted=2)
        small.step([StepEntry(s, [1, 2, 3], [0, 1, 2])])
    others = [cache.open(f"o{i}") for i in range(3)]
    extra = CacheManager(model.cache_needs(), page_tokens=16, n_pages=2, n_state_slots=8, max_seq_tokens=32, device="cpu")
    with pytest.raises(StepError, match="requests in a step"):
        many = [StepEntry(o, [1], []) for o in others] + [StepEntry(s, [1], [])] + [StepEntry(extra.open("e"), [1], [])]
        runner.step(many)
    gone = others[0]
    cache.release(gone)
    with pytest.raises(CacheError, match="not open"):
        runner.step([StepEntry(gone, [1], [])])
    assert s.n_tokens == 0
    lg = runner.step([StepEntry(s, [1, 2, 3], [2])])   # and a good step still runs
    ref = plain.forward(cfg, W, [1, 2, 3], torch.float64)
    assert float((lg[0].double() - ref[2]).abs().max()) <= 2e-5 * float(ref.abs().max())
