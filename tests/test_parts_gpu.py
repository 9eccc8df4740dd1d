"""Each part alone on the GPU against the plain implementation's function for it, at sizes
other than the tiny models', in float32 and in bfloat16: norm, rotary table, attention
(whole prompt, then portions and single tokens against the same cache), dense MLP, sparse
mixture of experts (with and without renormalisation and shared expert), embedding and head.
The parts are built directly from their constructor arguments; no model is involved."""
import math

import pytest
import torch

import plain_qwen2moe as plain
from locus_b200 import kernels as K
from locus_b200.cache import CacheManager
from locus_b200.engine.batch import GroupBatch, Runtime, StepBatch
from locus_b200.parts import PartSpec, make_part
from locus_b200.weights.loader import random_tensor

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 3e-5, torch.bfloat16: 1.5e-2}


def fill(part, dtype, seed=0):
    """Random parameters (rounded to ``dtype``) on the device; returns them as float64 by tensor name."""
    named = {}
    shapes = part.param_shapes()
    for pname, shape in shapes.items():
        part.params[pname] = torch.empty(shape, dtype=dtype, device=DEV)
    for src in part.sources():
        t = random_tensor(seed, src.name, src.shape, src.init, dtype)
        if src.init != "norm":
            t = (t.float() * 5).to(dtype)  # larger weights: differences show
        dest = part.params[src.param]
        flat = dest.view(-1, dest.shape[-1]) if dest.dim() >= 2 else dest
        flat[src.row0 : src.row0 + src.shape[0]].copy_(t.reshape(flat[src.row0 : src.row0 + src.shape[0]].shape))
        named[src.name] = t.double()
    for sub in part.sub_parts():
        named.update(fill(sub, dtype, seed))
    return named


def rt_for(dtype, max_tokens=128):
    return Runtime(torch.device(DEV), dtype, max_tokens, 4, max_tokens)


def close(got, ref, dtype, what):
    got, ref = got.double().cpu(), ref.double().cpu()
    err, scale = float((got - ref).abs().max()), float(ref.abs().max())
    assert math.isfinite(err) and err <= TOL[dtype] * scale, f"{what}: {err:.3e} > {TOL[dtype] * scale:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    part = make_part("norm", PartSpec("rmsnorm", {"width": 200, "eps": 3e-4}), "n")
    W = fill(part, dtype)
    x = torch.randn(9, 200) * 3
    out = torch.empty(9, 200, dtype=dtype, device=DEV)
    part.forward(x.to(DEV), out)
    close(out, plain.rmsnorm(x.double(), W["n.weight"], 3e-4), dtype, "rmsnorm")


def test_rotary_table_is_computed_in_float64_and_rounded_once():
    part = make_part("position", PartSpec("rotary", {"head_dim": 48, "theta": 500000.0}), "p")
    part.bind(rt_for(torch.float32))
    t = part.rotary_table()
    i = torch.arange(24, dtype=torch.float64)
    assert t.rot_dim == 48 and not t.interleaved
    assert torch.equal(t.inv_freq.cpu(), torch.pow(torch.tensor(500000.0, dtype=torch.float64), -2 * i / 48).float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter,shape", [(72, (11, 56)), (136, (40, 120))])
def test_dense_mlp_part(dtype, inter, shape):
    T, H = shape
    part = make_part("feed_forward", PartSpec("dense_mlp", {"hidden": H, "intermediate": inter}), "m")
    W = fill(part, dtype)
    rt = rt_for(dtype)
    h = (torch.randn(T, H)).to(dtype)
    x0 = torch.randn(T, H)
    x = x0.clone().to(DEV)
    part.forward(h.to(DEV), None, x, rt)
    ref = x0.double() + plain.swiglu_mlp(h.double(), W["m.gate_proj.weight"], W["m.up_proj.weight"], W["m.down_proj.weight"])
    close(x, ref, dtype, "dense mlp adds into the residual")


def _moe_step(part, W, cfg, dtype, rt, T, seed):
    """One forward of the part on T random rows against the plain block, following the part's picks where the
    oracle has a near-tie (see test_engine_gpu.py)."""
    H, k = part.hidden, cfg["num_experts_per_tok"]
    picked = []
    part.observer = lambda prefix, ids, wts: picked.append(ids.cpu().tolist())
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(T, H, generator=g).to(dtype)
    x0 = torch.randn(T, H, generator=g)
    x = x0.clone().to(DEV)
    part.forward(h.to(DEV), None, x, rt)
    aux = {}
    plain.moe_block(h.double(), W, "f", cfg, aux=aux)
    forced = []
    for t in range(T):
        ids, probs = aux["f"][t]
        if sorted(picked[0][t]) != sorted(ids):
            kth = min(float(probs[e]) for e in ids)
            assert all(float(probs[e]) >= kth * (1 - (1e-5 if dtype == torch.float32 else 1e-2)) for e in picked[0][t])
        forced.append(picked[0][t])
    ref = x0.double() + plain.moe_block(h.double(), W, "f", cfg, forced=forced)
    close(x, ref, dtype, f"sparse moe E={part.E} k={k} T={T}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,k,norm,I,Is,T", [(8, 2, False, 32, 64, 5), (12, 3, True, 48, 0, 70), (60, 4, False, 40, 96, 300),
                                            (60, 4, True, 24, 56, 1100), (60, 4, False, 40, 96, 100)])
def test_sparse_moe_part(dtype, E, k, norm, I, Is, T):
    H = 72
    part = make_part("feed_forward", PartSpec("sparse_moe", {"hidden": H, "n_experts": E, "top_k": k, "norm_topk": norm,
                                                              "expert_intermediate": I, "shared_intermediate": Is}), "f")
    W = fill(part, dtype, seed=3)
    rt = rt_for(dtype, max_tokens=max(320, T))
    part.bind(rt)
    cfg = {"num_experts_per_tok": k, "norm_topk_prob": norm, "shared_expert_intermediate_size": Is}
    _moe_step(part, W, cfg, dtype, rt, T, 0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sparse_moe_part_steps_of_every_size_on_one_layout(dtype):
    """The expert layout is shared by the steps: a step with many rows per expert (which, in bfloat16, leaves a
    second tile list of 256 rows), then steps that sort in other ways (one launch for up to 16 tokens, tiles of 8
    rows for up to 8, the general sort above), each of which must not see the lists of the step before."""
    H, E, k, I = 72, 4, 4, 48
    assert K.expert_second_tile(100 * k, E) == 256 and K.expert_second_tile(40 * k, E) == 0
    part = make_part("feed_forward", PartSpec("sparse_moe", {"hidden": H, "n_experts": E, "top_k": k, "norm_topk": True,
                                                              "expert_intermediate": I, "shared_intermediate": 32}), "f")
    W = fill(part, dtype, seed=4)
    rt = rt_for(dtype, max_tokens=320)
    part.bind(rt)
    cfg = {"num_experts_per_tok": k, "norm_topk_prob": True, "shared_expert_intermediate_size": 32}
    for i, T in enumerate([100, 16, 300, 3, 40, 12, 120, 17]):
        _moe_step(part, W, cfg, dtype, rt, T, 10 + i)


def _attention_case(dtype, nh, nkv, hd, window, H=80, P=16):
    spec = PartSpec("attention", {"hidden": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "qkv_bias": True,
                                  "window": window, "position": PartSpec("rotary", {"head_dim": hd, "theta": 10000.0})})
    part = make_part("mixer", spec, "a")
    W = fill(part, dtype, seed=5)
    rt = rt_for(dtype, max_tokens=160)
    part.bind(rt)
    part.position.bind(rt)
    cache = CacheManager([(part.cache_needs()[0], None, None)], page_tokens=P, n_pages=16, n_state_slots=2,
                         max_seq_tokens=200, dtype=dtype, device=DEV, poison=True)
    return part, W, rt, cache


def _batch(cache, seq, n, rt):
    """Descriptors of one segment of ``n`` new tokens for request ``seq``."""
    P, ctx = cache.page_tokens, seq.n_tokens
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    table = seq.tables[0] + [-1] * (cache.table_width - len(seq.tables[0]))
    slots = [seq.tables[0][p // P] * P + p % P for p in range(ctx, ctx + n)]
    import numpy as np

    from locus_b200.parts.attention import AttentionTiles

    # the part's own step plan, built as the step function builds it: lists into a host buffer, then to the device
    plan = AttentionTiles()
    host = np.zeros(plan.capacity(n, 1), dtype=np.int32)
    res = plan.build(np.array([0], dtype=np.int32), np.array([n], dtype=np.int32), np.array([ctx], dtype=np.int32), host)
    dev = torch.from_numpy(host).to(DEV)
    tiles = {}
    for name, v in res.items():
        if isinstance(v, tuple):
            t = dev[v[0] : v[0] + v[1]]
            tiles[name] = t.view(*v[2]) if v[2] else t
        else:
            tiles[name] = v
    assert tiles["n_decode_items"] == (1 if n == 1 else 0) and tiles["n_chunk_items64"] == (-(-n // K.MMA_QUERY_TILE) if n > 1 else 0)
    b = StepBatch(T=n, n_seg=1, tokens=i32([0] * n), positions=i32(list(range(ctx, ctx + n))), seg_q0=i32([0]),
                  seg_qn=i32([n]), seg_ctx=i32([ctx]), state_slots=i32([0]), want_rows=i32([]), n_want=0,
                  longest=ctx + n, plans={AttentionTiles.key: tiles})
    b.groups[0] = GroupBatch(block_table=i32(table).view(1, -1), slots=i32(slots), page_tokens=P)
    return b


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 4, 16, 0), (6, 2, 32, 0), (5, 1, 48, 24), (2, 2, 64, 0)])
def test_attention_part_whole_then_in_portions(dtype, nh, nkv, hd, window):
    H, T = 80, 150
    part, W, rt, cache = _attention_case(dtype, nh, nkv, hd, window, H)
    h = torch.randn(T, H).to(dtype)
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "hidden_size": H, "rope_theta": 10000.0}
    Wp = {k.replace("a.", "p."): v for k, v in W.items()}
    ref = plain.attention_block(h.double(), Wp, "p", cfg, window)
    lay = cache.layer_caches()[0]
    for cuts in ([T], [33, 2, 1, 1, 64, 17, 1, 31]):
        assert sum(cuts) == T
        seq = cache.open("r")
        x = torch.zeros(T, H, device=DEV)
        a = 0
        for n in cuts:
            assert cache.ensure_capacity(seq, n)
            batch = _batch(cache, seq, n, rt)
            part.forward(h[a : a + n].to(DEV), batch, lay, x[a : a + n], rt)
            cache.commit(seq, n)
            a += n
        close(x, ref, dtype, f"attention {cuts}")
        cache.release(seq)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    emb = make_part("embedding", PartSpec("embedding", {"vocab": 331, "hidden": 56}), "e")
    head = make_part("head", PartSpec("linear", {"vocab": 331, "hidden": 56}), "h")
    We, Wh = fill(emb, dtype), fill(head, dtype, seed=2)
    toks = torch.tensor([0, 330, 17, 17, 5], dtype=torch.int32, device=DEV)
    x = torch.empty(5, 56, device=DEV)
    emb.forward(toks, x)
    assert torch.equal(x.cpu().double(), We["e.weight"][toks.cpu().long()])
    hrows = torch.randn(5, 56).to(dtype)
    logits = torch.empty(5, 331, device=DEV)
    head.forward(hrows.to(DEV), logits)
    close(logits, hrows.double() @ Wh["h.weight"].T, dtype, "head")
    tied = make_part("head", PartSpec("linear", {"vocab": 331, "hidden": 56, "tied_to": "e.weight"}), "t")
    assert [s.name for s in tied.sources()] == ["e.weight"]  # the loader gives both parts one device tensor
