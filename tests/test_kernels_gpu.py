"""Each CUDA kernel alone against its plain torch reference (tests/emulated_kernels.py, in
float64), at sizes other than the tiny models': odd widths, head sizes in steps of 16,
group ratios, page sizes, windows.  float32 kernels must agree to float32 rounding;
bfloat16 kernels to the rounding of their bfloat16 outputs (inputs are shared exactly)."""
import math

import pytest
import torch

import emulated_kernels as EK
import locus_b200.kernels as K
import plain_qwen2moe as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _precise():
    EK.PRECISE = True
    yield
    EK.PRECISE = False


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(got, ref, dtype, what, scale=None):
    got, ref = got.double().cpu(), ref.double().cpu()
    s = float(ref.abs().max()) if scale is None else scale
    tol = (2e-5 if dtype == torch.float32 else 1.2e-2) * max(s, 1e-6)
    err = float((got - ref).abs().max())
    assert math.isfinite(err) and err <= tol, f"{what}: max error {err:.3e} > {tol:.3e} (scale {s:.3e})"


DTYPES = [torch.float32, torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_rows(dtype):
    table = rnd(37, 50, dtype=dtype)
    toks = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32)
    out = torch.empty(5, 50, device=DEV)
    K.embed_rows(toks.to(DEV), table.to(DEV), out)
    assert torch.equal(out.cpu(), table[toks.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [8, 200, 2048 + 24])
def test_rmsnorm(dtype, H):
    x = rnd(7, H, seed=1, scale=3.0)
    w = rnd(H, dtype=dtype, seed=2) + 1
    out = torch.empty(7, H, dtype=dtype, device=DEV)
    K.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, out)
    ref = torch.empty(7, H, dtype=torch.float64)
    EK.rmsnorm(x, w, 1e-5, ref)
    close(out, ref, dtype, "rmsnorm")
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    out2 = torch.empty(3, H, dtype=dtype, device=DEV)
    K.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, out2, rows.to(DEV))
    close(out2, ref[rows.long()], dtype, "rmsnorm rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,k", [(8, 1), (200, 3), (4096 + 1024 + 8, 4)])
def test_rmsnorm_folds_the_expert_sum(dtype, H, k):
    """The norm that first adds a row's expert outputs gives, bit for bit, moe_combine followed by
    the plain norm, and leaves the same sum in x."""
    T = 6
    x = rnd(T, H, seed=1, scale=3.0).to(DEV)
    # the experts' rows are float32 in a float32 model and bfloat16 in a bfloat16 one; the sum is float32 either way
    pair_out = rnd(T * k, H, seed=2, scale=2.0).to(dtype).to(DEV)
    pair_pos = torch.randperm(T * k, generator=torch.Generator().manual_seed(3)).to(torch.int32).to(DEV)
    w = (rnd(H, dtype=dtype, seed=4) + 1).to(DEV)
    assert K.rmsnorm_adds(x)
    xr = x.cpu().double()
    EK.moe_combine(xr, pair_out.cpu().double(), pair_pos.cpu(), k)
    x2, out2 = x.clone(), torch.empty(T, H, dtype=dtype, device=DEV)
    K.moe_combine(x2, pair_out, pair_pos, k)
    K.rmsnorm(x2, w, 1e-6, out2)
    x1, out1 = x.clone(), torch.empty(T, H, dtype=dtype, device=DEV)
    K.rmsnorm(x1, w, 1e-6, out1, add=(pair_out, pair_pos, k))
    assert torch.equal(x1, x2) and torch.equal(out1, out2)
    close(x1, xr, torch.float32, "x + the experts' sum")
    assert not K.rmsnorm_adds(torch.zeros(2, 6))
    # with a gather of rows (one of them named twice) the sum shows in the output alone
    rows = torch.tensor([4, 1, 4], dtype=torch.int32, device=DEV)
    x3, out3 = x.clone(), torch.empty(3, H, dtype=dtype, device=DEV)
    K.rmsnorm(x3, w, 1e-6, out3, rows, add=(pair_out, pair_pos, k))
    assert torch.equal(x3, x) and torch.equal(out3, out2[rows.long()])
    with pytest.raises(K.KernelError):
        K.rmsnorm(x1, w, 1e-6, out1, add=(pair_out, pair_pos[: T * k - 1], k))


@pytest.mark.parametrize("xdt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K_", [(1, 1, 8), (5, 331, 120), (70, 130, 72), (129, 64, 2048)])
def test_linear_plain_bias_scale_accumulate(xdt, wdt, M, N, K_):
    x, w = rnd(M, K_, dtype=xdt, seed=3), rnd(N, K_, dtype=wdt, seed=4, scale=0.1)
    bias, rs = rnd(N, dtype=wdt, seed=5), rnd(M, seed=6)
    for use_bias, use_rs, acc in [(False, False, False), (True, False, False), (True, True, True)]:
        odt = torch.float32 if acc else xdt
        out0 = rnd(M, N, dtype=odt, seed=7)
        out = out0.clone().to(DEV)
        K.linear(x.to(DEV), w.to(DEV), out, bias=bias.to(DEV) if use_bias else None,
                 row_scale=rs.to(DEV) if use_rs else None, accumulate=acc)
        ref = out0.clone().double()
        EK.linear(x, w, ref, bias=bias if use_bias else None, row_scale=rs if use_rs else None, accumulate=acc)
        close(out, ref, odt, f"linear bias={use_bias} scale={use_rs} acc={acc}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_swiglu(dtype):
    x, wg, wu = rnd(33, 120, dtype=dtype, seed=1), rnd(77, 120, dtype=dtype, seed=2, scale=0.2), \
        rnd(77, 120, dtype=dtype, seed=3, scale=0.2)
    out = torch.empty(33, 77, dtype=dtype, device=DEV)
    K.linear(x.to(DEV), wg.to(DEV), out, w2=wu.to(DEV))
    ref = torch.empty(33, 77, dtype=torch.float64)
    EK.linear(x, wg, ref, w2=wu)
    close(out, ref, dtype, "swiglu")


def _route(T, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).reshape(-1)
    return ids


@pytest.mark.parametrize("T,E,k", [(1, 4, 2), (50, 7, 3), (300, 60, 4), (9, 5, 5), (2100, 60, 4), (200, 1500, 3)])
def test_moe_sort_layout(T, E, k):
    """(With up to MOE_SORT_ONE_LAUNCH_EXPERTS experts every block counts all experts' pairs itself; beyond, a
    launch of its own counts.)"""
    assert 60 < K.MOE_SORT_ONE_LAUNCH_EXPERTS < 1500
    ids = _route(T, E, k, T)
    if T == 9:
        ids[:] = 2  # every pair on one expert; others empty
    lay = K.ExpertLayout(T * k, E, 64, DEV)
    K.moe_sort(ids.to(DEV), T * k, lay)
    ref = EK.ExpertLayout(T * k, E, 64, "cpu")
    EK.moe_sort(ids, T * k, ref)
    n_tiles = int(ref.n_tiles)
    assert int(lay.n_tiles.cpu()) == n_tiles
    assert n_tiles <= lay.tiles_for(T * k)
    for name in ("counts", "offsets", "sorted_pair", "pair_pos"):
        assert torch.equal(getattr(lay, name).cpu(), getattr(ref, name)), name
    for name in ("tile_expert", "tile_row0", "tile_rows"):
        assert torch.equal(getattr(lay, name).cpu()[:n_tiles], getattr(ref, name)[:n_tiles]), name
    # a second tile list over the same rows, in tiles of another size
    K.moe_sort(ids.to(DEV), T * k, lay, 16, 40)
    EK.moe_sort(ids, T * k, ref, 16, 40)
    n1, n2 = int(ref.n_tiles), int(ref.n_tiles2)
    assert (int(lay.n_tiles.cpu()), int(lay.n_tiles2.cpu())) == (n1, n2) and n2 <= lay.tiles_for(T * k, 40) and n2 <= n1
    for name in ("tile_expert", "tile_row0", "tile_rows"):
        assert torch.equal(getattr(lay, name).cpu()[:n1], getattr(ref, name)[:n1]), name
    for name in ("tile2_expert", "tile2_row0", "tile2_rows"):
        assert torch.equal(getattr(lay, name).cpu()[:n2], getattr(ref, name)[:n2]), name
    assert int(lay.tile2_rows.cpu()[:n2].sum()) == T * k


@pytest.mark.parametrize("xdt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32)])
def test_linear_grouped_experts(xdt, wdt):
    T, E, k, H, I = 150, 6, 2, 72, 40
    ids = _route(T, E, k, 11)
    ids[: 2 * 70] = 1  # one expert with more than two row tiles
    h = rnd(T, H, dtype=xdt, seed=1)
    wg, wu = rnd(E, I, H, dtype=wdt, seed=2, scale=0.2), rnd(E, I, H, dtype=wdt, seed=3, scale=0.2)
    wd = rnd(E, H, I, dtype=wdt, seed=4, scale=0.2)
    wts = torch.rand(T * k, generator=torch.Generator().manual_seed(5))
    lay, ref_lay = K.ExpertLayout(T * k, E, 64, DEV), EK.ExpertLayout(T * k, E, 64, "cpu")
    K.moe_sort(ids.to(DEV), T * k, lay)
    EK.moe_sort(ids, T * k, ref_lay)
    act = torch.empty(T * k, I, dtype=xdt, device=DEV)
    K.linear(h.to(DEV), wg.to(DEV), act, w2=wu.to(DEV), x_rows=lay.sorted_pair, x_row_div=k, layout=lay,
             n_rows=T * k)
    ref_act = torch.empty(T * k, I, dtype=torch.float64)
    EK.linear(h, wg, ref_act, w2=wu, x_rows=ref_lay.sorted_pair, x_row_div=k, layout=ref_lay, n_rows=T * k)
    close(act, ref_act, xdt, "grouped swiglu")
    pair_out = torch.empty(T * k, H, device=DEV)
    K.linear(act, wd.to(DEV), pair_out, layout=lay, n_rows=T * k, row_scale=wts.to(DEV), scale_rows=lay.sorted_pair)
    ref_out = torch.empty(T * k, H, dtype=torch.float64)
    EK.linear(act.cpu(), wd, ref_out, layout=ref_lay, n_rows=T * k, row_scale=wts, scale_rows=ref_lay.sorted_pair)
    close(pair_out, ref_out, torch.float32 if xdt == torch.float32 else torch.bfloat16, "grouped down")
    x = rnd(T, H, seed=9)
    xd = x.clone().to(DEV)
    K.moe_combine(xd, pair_out, lay.pair_pos, k)
    xr = x.clone().double()
    EK.moe_combine(xr, pair_out.cpu().double(), ref_lay.pair_pos, k)
    close(xd, xr, torch.float32, "combine")


@pytest.mark.parametrize("xdt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("T,H,E,k,renorm", [(1, 64, 8, 2, False), (19, 200, 60, 4, False), (40, 72, 12, 3, True),
                                            (3, 2048, 5, 5, True)])
def test_router_topk(xdt, wdt, T, H, E, k, renorm):
    h, wr, wg = rnd(T, H, dtype=xdt, seed=1), rnd(E, H, dtype=wdt, seed=2, scale=0.3), rnd(1, H, dtype=wdt, seed=3, scale=0.3)
    ids = torch.zeros(T * k, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T * k, device=DEV)
    gamma = torch.zeros(T, device=DEV)
    K.router_topk(h.to(DEV), wr.to(DEV), wg.to(DEV), ids, wts, gamma, top_k=k, renorm=renorm, scale=1.5)
    rids, rw, rg = torch.zeros(T * k, dtype=torch.int32), torch.zeros(T * k, dtype=torch.float64), \
        torch.zeros(T, dtype=torch.float64)
    EK.router_topk(h, wr, wg, rids, rw, rg, top_k=k, renorm=renorm, scale=1.5)
    assert torch.equal(ids.cpu(), rids), "picked experts (and their order) differ"
    close(wts, rw, torch.float32, "router weights")
    close(gamma, rg, torch.float32, "shared gate")


@pytest.mark.parametrize("T,H,E,k,renorm", [(1, 64, 8, 2, False), (19, 200, 60, 4, False), (40, 72, 12, 3, True),
                                            (300, 2048, 60, 4, False)])
def test_router_on_tensor_cores(T, H, E, k, renorm):
    """bfloat16 path: logits by the weight-streaming kernel (any number of tokens), then selection."""
    dt = torch.bfloat16
    h, wr, wg = rnd(T, H, dtype=dt, seed=1), rnd(E, H, dtype=dt, seed=2, scale=0.3), rnd(1, H, dtype=dt, seed=3, scale=0.3)
    w_all = torch.cat([wr, wg], 0).to(DEV)
    logits = torch.full((T + 3, E + 1), float("nan"), device=DEV)
    K.router_logits(h.to(DEV), w_all, logits)
    ref_logits = h.double() @ torch.cat([wr, wg], 0).double().T
    close(logits[:T], ref_logits, torch.float32, "router logits")
    ids = torch.zeros(T * k, dtype=torch.int32, device=DEV)
    wts, gamma = torch.zeros(T * k, device=DEV), torch.zeros(T, device=DEV)
    K.router_select(logits, E, True, ids, wts, gamma, n_tokens=T, top_k=k, renorm=renorm, scale=1.5)
    rids, rw, rg = torch.zeros(T * k, dtype=torch.int32), torch.zeros(T * k, dtype=torch.float64), \
        torch.zeros(T, dtype=torch.float64)
    EK.router_topk(h, wr, wg, rids, rw, rg, top_k=k, renorm=renorm, scale=1.5)
    assert torch.equal(ids.cpu(), rids), "picked experts (and their order) differ"
    close(wts, rw, torch.float32, "router weights")
    close(gamma, rg, torch.float32, "shared gate")
    # the logits of a token do not depend on the other tokens of the batch: bit for bit
    one = torch.full((1, E + 1), float("nan"), device=DEV)
    for t in (0, T // 2, T - 1):
        K.router_logits(h[t : t + 1].to(DEV), w_all, one)
        assert torch.equal(one[0], logits[t]), f"token {t} alone differs from token {t} in the batch"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W", [8, 20, 200, 2048, 6])
def test_gather_rows(dtype, W):
    """out[i] = src[idx[i] // div], in 16-byte pieces where the rows allow it and element by element else."""
    src = rnd(37, W, dtype=dtype, seed=W).to(DEV)
    idx = torch.randint(0, 37 * 3, (90,), generator=torch.Generator().manual_seed(W)).to(torch.int32).to(DEV)
    out = torch.zeros(90, W, dtype=dtype, device=DEV)
    K.gather_rows(src, idx, 3, out, 90)
    assert torch.equal(out, src[(idx.long() // 3)])


@pytest.mark.parametrize("T,E,k,tile,gate,renorm", [(1, 4, 2, 8, True, True), (8, 60, 4, 8, True, False),
                                                     (13, 7, 3, 16, False, True), (16, 33, 16, 32, True, True),
                                                     (5, 512, 6, 8, False, False)])
def test_route_small_is_select_then_sort(T, E, k, tile, gate, renorm):
    """One launch for a decode-sized batch gives, bit for bit, what the two kernels give."""
    g = torch.Generator().manual_seed(T * 1000 + E)
    logits = (torch.randn(T, E + 1, generator=g) * 2).to(DEV)
    if T > 4:
        logits[3, : min(E, 5)] = 1.25  # ties: the lowest index wins in both
    assert K.route_small_takes(T, k, E)
    out = {}
    for name in ("two", "one"):
        ids = torch.full((T * k,), -1, dtype=torch.int32, device=DEV)
        wts, gamma = torch.zeros(T * k, device=DEV), torch.zeros(T, device=DEV)
        lay = K.ExpertLayout(T * k, E, 64, DEV)
        if name == "two":
            K.router_select(logits, E, gate, ids, wts, gamma if gate else None, n_tokens=T, top_k=k, renorm=renorm,
                            scale=0.75)
            K.moe_sort(ids, T * k, lay, tile)
        else:
            K.route_small(logits, E, gate, ids, wts, gamma if gate else None, lay, n_tokens=T, top_k=k,
                          renorm=renorm, scale=0.75, tile_m=tile)
        out[name] = (ids, wts, gamma, lay)
    (ids2, wts2, gamma2, lay2), (ids1, wts1, gamma1, lay1) = out["two"], out["one"]
    assert torch.equal(ids1, ids2) and torch.equal(wts1, wts2) and torch.equal(gamma1, gamma2)
    n_tiles = int(lay2.n_tiles.cpu())
    assert int(lay1.n_tiles.cpu()) == n_tiles
    for name in ("counts", "offsets", "sorted_pair", "pair_pos"):
        assert torch.equal(getattr(lay1, name), getattr(lay2, name)), name
    for name in ("tile_expert", "tile_row0", "tile_rows"):
        assert torch.equal(getattr(lay1, name)[:n_tiles], getattr(lay2, name)[:n_tiles]), name
    assert not K.route_small_takes(17, k, E) and not K.route_small_takes(T, k, 513)


@pytest.mark.parametrize("T,H,E,k,gate,tile", [(1, 64, 4, 2, True, 8), (8, 2048, 60, 4, True, 8), (16, 200, 64, 8, False, 16),
                                               (9, 3584, 64, 8, True, 128), (5, 72, 512, 6, False, 8)])
def test_router_in_one_launch_is_logits_then_route_small(T, H, E, k, gate, tile):
    """Logits, selection and layout of a decode-sized batch in one launch give, bit for bit, what the two launches give
    (the same kernel computes the logits; the last block routes), twice in a row (the counter returns to zero)."""
    g = torch.Generator().manual_seed(T * 7 + E)
    h = (torch.randn(T, H, generator=g)).to(torch.bfloat16).to(DEV)
    n = E + (1 if gate else 0)
    w_all = (torch.randn(n, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    rule = dict(top_k=k, renorm=True, scale=1.25)
    ids2, wts2, gamma2 = torch.full((T * k,), -1, dtype=torch.int32, device=DEV), torch.zeros(T * k, device=DEV), torch.zeros(T, device=DEV)
    logits2 = torch.zeros(T, E + 1, device=DEV)
    lay2 = K.ExpertLayout(T * k, E, 64, DEV)
    K.router_logits(h, w_all, logits2)
    K.route_small(logits2, E, gate, ids2, wts2, gamma2 if gate else None, lay2, n_tokens=T, tile_m=tile, **rule)
    counter = torch.zeros(1, dtype=torch.int32, device=DEV)
    for again in range(2):
        ids1, wts1, gamma1 = torch.full((T * k,), -1, dtype=torch.int32, device=DEV), torch.zeros(T * k, device=DEV), torch.zeros(T, device=DEV)
        logits1 = torch.zeros(T, E + 1, device=DEV)
        lay1 = K.ExpertLayout(T * k, E, 64, DEV)
        K.route_fused_small(h, w_all, logits1, E, gate, ids1, wts1, gamma1 if gate else None, lay1, counter, n_tokens=T,
                            tile_m=tile, **rule)
        assert torch.equal(logits1[:, :n], logits2[:, :n])
        assert torch.equal(ids1, ids2) and torch.equal(wts1, wts2) and torch.equal(gamma1, gamma2)
        n_tiles = int(lay2.n_tiles.cpu())
        assert int(lay1.n_tiles.cpu()) == n_tiles and int(counter.cpu()) == 0
        for name in ("counts", "offsets", "sorted_pair", "pair_pos"):
            assert torch.equal(getattr(lay1, name), getattr(lay2, name)), name
        for name in ("tile_expert", "tile_row0", "tile_rows"):
            assert torch.equal(getattr(lay1, name)[:n_tiles], getattr(lay2, name)[:n_tiles]), name


def test_router_ties_go_to_lowest_index():
    h = torch.ones(2, 16)
    wr = torch.zeros(6, 16)
    wr[4] = 0.5  # expert 4 wins, the others tie
    ids = torch.zeros(6, dtype=torch.int32, device=DEV)
    wts = torch.zeros(6, device=DEV)
    K.router_topk(h.to(DEV), wr.to(DEV), None, ids, wts, None, top_k=3, renorm=False)
    assert ids.cpu().tolist() == [4, 0, 1, 4, 0, 1]


@pytest.mark.parametrize("T,E,k,score_fn,bias,groups,used,renorm",
                         [(5, 12, 3, "sigmoid", False, 1, 1, True), (9, 60, 4, "softmax", True, 1, 1, False),
                          (16, 64, 8, "sigmoid", True, 8, 3, True), (40, 24, 5, "softmax", False, 4, 2, False),
                          (3, 9, 9, "sigmoid", True, 3, 1, False)])
def test_router_rule_score_function_bias_and_groups(T, E, k, score_fn, bias, groups, used, renorm):
    """Every selection kernel with the other rules of the reference's moe_select: sigmoid scores, a bias that
    enters the selection but not the weights, group-limited routing; against the twin and the plain function."""
    g = torch.Generator().manual_seed(T * 100 + E)
    logits = torch.randn(T, E + 1, generator=g) * 2
    sel_bias = torch.randn(E, generator=g) * 0.5 if bias else None
    rule = dict(top_k=k, renorm=renorm, scale=1.5, score_fn=score_fn, n_group=groups, n_group_used=used)
    ref_ids, ref_w = torch.zeros(T * k, dtype=torch.int32), torch.zeros(T * k)
    EK.router_select(logits, E, False, ref_ids, ref_w, None, n_tokens=T, sel_bias=sel_bias, **rule)
    for t in range(T):
        ids_p, w_p = plain.moe_select(logits[t, :E].double(), k, renorm, 1.5, score_fn,
                                      sel_bias.double() if bias else None, groups, used)
        assert ids_p == ref_ids[t * k : (t + 1) * k].tolist()
        assert torch.allclose(torch.tensor([float(x) for x in w_p]), ref_w[t * k : (t + 1) * k], rtol=1e-5, atol=1e-7)
    dev_bias = sel_bias.to(DEV) if bias else None
    # selection alone
    ids, wts = torch.full((T * k,), -1, dtype=torch.int32, device=DEV), torch.zeros(T * k, device=DEV)
    K.router_select(logits.to(DEV), E, False, ids, wts, None, n_tokens=T, sel_bias=dev_bias, **rule)
    assert torch.equal(ids.cpu(), ref_ids)
    assert torch.allclose(wts.cpu(), ref_w, rtol=1e-5, atol=1e-7)
    # selection + layout in one launch
    if K.route_small_takes(T, k, E):
        ids1, wts1 = torch.full((T * k,), -1, dtype=torch.int32, device=DEV), torch.zeros(T * k, device=DEV)
        K.route_small(logits.to(DEV), E, False, ids1, wts1, None, K.ExpertLayout(T * k, E, 64, DEV), n_tokens=T,
                      tile_m=8, sel_bias=dev_bias, **rule)
        assert torch.equal(ids1, ids) and torch.equal(wts1, wts)
    # the fused float32 router: logits = h . w^T with an identity-like weight reproduces the same logits
    h = torch.zeros(T, E + 7)
    h[:, :E] = logits[:, :E]
    wr = torch.zeros(E, E + 7)
    wr[:, :E] = torch.eye(E)
    ids2, wts2 = torch.full((T * k,), -1, dtype=torch.int32, device=DEV), torch.zeros(T * k, device=DEV)
    K.router_topk(h.to(DEV), wr.to(DEV), None, ids2, wts2, None, sel_bias=dev_bias, **rule)
    assert torch.equal(ids2.cpu(), ref_ids)
    assert torch.allclose(wts2.cpu(), ref_w, rtol=1e-5, atol=1e-7)
    with pytest.raises(K.KernelError, match="groups"):
        K.router_select(logits.to(DEV), E, False, ids, wts, None, n_tokens=T, top_k=k, renorm=renorm, n_group=E + 1)
    with pytest.raises(K.KernelError, match="score function"):
        K.router_select(logits.to(DEV), E, False, ids, wts, None, n_tokens=T, top_k=k, renorm=renorm, score_fn="relu")


@pytest.mark.parametrize("score_fn", ["softmax", "sigmoid"])
def test_router_selection_is_total_for_logits_that_are_no_numbers(score_fn):
    """NaN and infinite router logits (a broken checkpoint, an overflow upstream) must still give k distinct
    expert indices below E for every token: the indices address weights and shared memory downstream."""
    T, E, k = 6, 20, 4
    logits = torch.randn(T, E + 1, generator=torch.Generator().manual_seed(3))
    logits[0, :E] = float("nan")
    logits[1, 5] = float("inf")
    logits[2, 7] = float("nan")
    logits[3, :E] = float("-inf")
    logits[4, 2], logits[4, 9] = float("inf"), float("-inf")
    for kind in ("select", "small", "fused"):
        ids, wts = torch.full((T * k,), -1, dtype=torch.int32, device=DEV), torch.zeros(T * k, device=DEV)
        lay = K.ExpertLayout(T * k, E, 64, DEV)
        if kind == "select":
            K.router_select(logits.to(DEV), E, False, ids, wts, None, n_tokens=T, top_k=k, renorm=True, score_fn=score_fn)
            K.moe_sort(ids, T * k, lay, 8)
        elif kind == "small":
            K.route_small(logits.to(DEV), E, False, ids, wts, None, lay, n_tokens=T, top_k=k, renorm=True, tile_m=8,
                          score_fn=score_fn)
        else:
            h = torch.zeros(T, E + 4)
            h[:, :E] = logits[:, :E]
            wr = torch.zeros(E, E + 4)
            wr[:, :E] = torch.eye(E)
            K.router_topk(h.to(DEV), wr.to(DEV), None, ids, wts, None, top_k=k, renorm=True, score_fn=score_fn)
            K.moe_sort(ids, T * k, lay, 8)
        torch.cuda.synchronize()
        got = ids.cpu().view(T, k)
        assert int(got.min()) >= 0 and int(got.max()) < E, (kind, got)
        for t in range(T):
            assert len(set(got[t].tolist())) == k, (kind, t, got[t])
        assert sorted(lay.sorted_pair.cpu().tolist()) == list(range(T * k)), kind
        # the rows without bad numbers are untouched by their neighbours
        ref_ids, ref_w = torch.zeros(k, dtype=torch.int32), torch.zeros(k)
        EK.router_select(logits[5:6], E, False, ref_ids, ref_w, None, n_tokens=1, top_k=k, renorm=True, score_fn=score_fn)
        assert got[5].tolist() == ref_ids.tolist()
        assert torch.allclose(wts.cpu()[5 * k :], ref_w, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rot,inter", [(4, 4, 16, 16, False), (6, 2, 32, 32, False), (5, 1, 48, 24, False),
                                                 (2, 1, 64, 64, True)])
def test_rope_kv_write(dtype, nh, nkv, hd, rot, inter):
    T, P, pages = 9, 16, 5
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=1)
    pos = torch.tensor([0, 1, 2, 40, 41, 1000, 7, 8, 9], dtype=torch.int32)
    slots = torch.tensor([3 * P + 0, 3 * P + 1, 3 * P + 15, 0, 1, 4 * P + 7, 2 * P + 3, 2 * P + 4, 2 * P + 5],
                         dtype=torch.int32)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot).float()
    pool0 = rnd(pages, 2, nkv, P, hd, dtype=dtype, seed=2)
    pool, q = pool0.clone().to(DEV), torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, rot_dim=rot, interleaved=inter, page_tokens=P)
    K.rope_kv_write(qkv.to(DEV), pos.to(DEV), inv.to(DEV), q, pool, slots.to(DEV), **kw)
    rpool, rq = pool0.clone().double(), torch.empty(T, nh * hd, dtype=torch.float64)
    EK.rope_kv_write(qkv, pos, inv, rq, rpool, slots, **kw)
    close(q, rq, dtype, "rotated q")
    close(pool, rpool, dtype, "pages")
    # a layer that reads another layer's cache leaves the pages alone; no table: no rotation
    pool2 = pool0.clone().to(DEV)
    K.rope_kv_write(qkv.to(DEV), pos.to(DEV), None, q, pool2, slots.to(DEV), write_kv=False, **{**kw, "rot_dim": 0})
    assert torch.equal(pool2.cpu(), pool0)
    assert torch.equal(q.cpu(), qkv[:, : nh * hd])


def _paged_case(dtype, nh, nkv, hd, P, segs, seed=0, n_pages=40):
    """segs: list of (ctx, qn).  Random pool, shuffled page tables."""
    g = torch.Generator().manual_seed(seed)
    pool = rnd(n_pages, 2, nkv, P, hd, dtype=dtype, seed=seed + 1)
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max((c + n + P - 1) // P for c, n in segs)
    table = torch.full((len(segs), width), -1, dtype=torch.int32)
    used = 0
    q0s, T = [], 0
    for s, (c, n) in enumerate(segs):
        need = (c + n + P - 1) // P
        table[s, :need] = torch.tensor(perm[used : used + need], dtype=torch.int32)
        used += need
        q0s.append(T)
        T += n
    assert used <= n_pages
    q = rnd(T, nh * hd, dtype=dtype, seed=seed + 2)
    meta = dict(seg_q0=torch.tensor(q0s, dtype=torch.int32), seg_qn=torch.tensor([n for _, n in segs], dtype=torch.int32),
                seg_ctx=torch.tensor([c for c, _ in segs], dtype=torch.int32), block_table=table)
    return pool, q, meta, T


def _dev(meta):
    return {k: v.to(DEV) for k, v in meta.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,P,window", [(4, 4, 16, 16, 0), (6, 2, 32, 16, 0), (5, 1, 48, 64, 0),
                                                (2, 2, 128, 64, 0), (3, 1, 256, 16, 0), (4, 2, 64, 16, 20),
                                                (2, 1, 32, 64, 1)])
def test_attn_chunk(dtype, nh, nkv, hd, P, window):
    segs = [(0, 5), (33, 17), (100, 2), (15, 40), (64, 16)]
    pool, q, meta, T = _paged_case(dtype, nh, nkv, hd, P, segs, seed=hd)
    items = []
    for s, (c, n) in enumerate(segs):
        items += [(s, o) for o in range(0, n, 16)]
    items_t = torch.tensor(items, dtype=torch.int32)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=window, scale=1 / math.sqrt(hd))
    out = torch.zeros(T, nh * hd, dtype=dtype, device=DEV)
    K.attn_chunk(q.to(DEV), pool.to(DEV), out, items=items_t.to(DEV), n_items=len(items), **_dev(meta), **kw)
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.attn_chunk(q, pool, ref, items=items_t, n_items=len(items), **meta, **kw)
    close(out, ref, dtype, "attn_chunk")


@pytest.mark.parametrize("nh,nkv,hd,P,window", [(4, 4, 16, 16, 0), (6, 2, 32, 16, 0), (5, 1, 48, 64, 0),
                                                (2, 2, 64, 16, 0), (3, 1, 96, 64, 0), (4, 2, 128, 64, 0),
                                                (4, 2, 64, 16, 20), (2, 1, 32, 64, 1), (2, 2, 128, 16, 100),
                                                (2, 1, 80, 16, 0), (3, 3, 112, 64, 30), (2, 2, 144, 16, 0),
                                                (2, 1, 160, 64, 0), (2, 2, 176, 16, 0), (4, 2, 192, 32, 50),
                                                (2, 2, 208, 16, 0), (2, 1, 224, 64, 0), (2, 2, 240, 16, 0),
                                                (2, 1, 256, 64, 0)])
def test_attn_chunk_tensor_cores(nh, nkv, hd, P, window):
    """Portions of 2 to 200 tokens at contexts that straddle the 64-key tiles and the pages."""
    dtype = torch.bfloat16
    segs = [(0, 5), (33, 17), (100, 2), (15, 140), (64, 64), (190, 200), (63, 1 + 64)]
    pool, q, meta, T = _paged_case(dtype, nh, nkv, hd, P, segs, seed=hd + 7, n_pages=120)
    items = []
    for s, (c, n) in enumerate(segs):
        items += [(s, o) for o in range(0, n, K.MMA_QUERY_TILE)]
    items_t = torch.tensor(items, dtype=torch.int32)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=window, scale=1 / math.sqrt(hd))
    assert K.attn_chunk_mma_takes(q.to(DEV), hd)
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    K.attn_chunk_mma(q.to(DEV), pool.to(DEV), out, items=items_t.to(DEV), n_items=len(items), **_dev(meta), **kw)
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.attn_chunk(q, pool, ref, items=items_t, n_items=len(items), **meta, **kw)
    close(out, ref, dtype, "attn_chunk_mma")
    # the keys of every tile cut into ranges (more ranges than some items have tiles) and merged: the same result
    for n_splits in (2, 3, 7):
        units = len(items) * nh * n_splits * K.MMA_QUERY_TILE
        part_o = torch.full((units * hd,), float("nan"), device=DEV)
        part_ml = torch.full((units * 2,), float("nan"), device=DEV)
        out_s = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
        before = K.launches
        K.attn_chunk_mma(q.to(DEV), pool.to(DEV), out_s, items=items_t.to(DEV), n_items=len(items), n_splits=n_splits,
                         part_o=part_o, part_ml=part_ml, **_dev(meta), **kw)
        assert K.launches - before == 2
        close(out_s, ref, dtype, f"attn_chunk_mma in {n_splits} key ranges")
    with pytest.raises(K.KernelError):
        K.attn_chunk_mma(q.to(DEV), pool.to(DEV), out, items=items_t.to(DEV), n_items=len(items), n_splits=2,
                         part_o=part_o[:8], part_ml=part_ml, **_dev(meta), **kw)
    assert K.attn_chunk_mma_splits(200, 16, 100000) == 1 and K.attn_chunk_mma_splits(1, 16, 130) == 1
    assert 1 < K.attn_chunk_mma_splits(1, 16, 30000) <= K.MMA_ATTN_MAX_SPLITS


@pytest.mark.parametrize("nh,nkv,P,window", [(2, 2, 64, 0), (4, 1, 128, 0), (3, 3, 64, 100), (2, 1, 64, 1), (4, 2, 192, 333)])
def test_attn_chunk_tcgen05(nh, nkv, P, window):
    """Portions of 2 to 450 tokens at contexts that straddle the 128-key tiles and the pages; whatever lies
    in a request's pages behind its last token is NaN and must not reach the result."""
    dtype, hd = torch.bfloat16, 128
    segs = [(0, 5), (33, 17), (100, 2), (15, 140), (64, 64), (190, 200), (63, 1 + 128), (0, 450), (1000, 150)]
    pool, q, meta, T = _paged_case(dtype, nh, nkv, hd, P, segs, seed=window + 7, n_pages=80)
    for s, (c, n) in enumerate(segs):
        end = c + n
        if end % P:
            pool[int(meta["block_table"][s, end // P]), :, :, end % P :, :] = float("nan")
    items = []
    for s, (c, n) in enumerate(segs):
        items += [(s, o) for o in range(0, n, K.MMA_QUERY_TILE)]
    items_t = torch.tensor(items, dtype=torch.int32)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=window, scale=1 / math.sqrt(hd))
    assert K.attn_chunk_tc_takes(q.to(DEV), hd, P, T)
    assert not K.attn_chunk_tc_takes(q.to(DEV), hd, 48, T) and not K.attn_chunk_tc_takes(q.to(DEV), 64, P, T)
    assert not K.attn_chunk_tc_takes(q.to(DEV), hd, P, 100, 1500) and K.attn_chunk_tc_takes(q.to(DEV), hd, P, 16, 5000)
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    K.attn_chunk_tc(q.to(DEV), pool.to(DEV), out, items=items_t.to(DEV), n_items=len(items), **_dev(meta), **kw)
    assert K.attn_tc_error() == 0
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.attn_chunk(q, torch.nan_to_num(pool, nan=1e4), ref, items=items_t, n_items=len(items), **meta, **kw)
    close(out, ref, dtype, "attn_chunk_tc")
    # the key tiles of every block cut into ranges (more ranges than most blocks have tiles) and merged by a second
    # launch; the items in another order (the kernel walks the list from its end, whatever the order)
    order = torch.randperm(len(items), generator=torch.Generator().manual_seed(3))
    shuffled = items_t[order].contiguous()
    for n_splits, its in ((2, items_t), (3, shuffled), (16, items_t)):
        part_o = torch.full((T * nh * n_splits * hd,), float("nan"), device=DEV)
        part_ml = torch.full((T * nh * n_splits * 2,), float("nan"), device=DEV)
        out_s = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
        before = K.launches
        K.attn_chunk_tc(q.to(DEV), pool.to(DEV), out_s, items=its.to(DEV), n_items=len(items), n_splits=n_splits,
                        part_o=part_o, part_ml=part_ml, **_dev(meta), **kw)
        assert K.launches - before == 2 and K.attn_tc_error() == 0
        close(out_s, ref, dtype, f"attn_chunk_tc in {n_splits} key ranges")
    with pytest.raises(K.KernelError):
        K.attn_chunk_tc(q.to(DEV), pool.to(DEV), out, items=items_t.to(DEV), n_items=len(items), n_splits=2,
                        part_o=part_o[:8], part_ml=part_ml, **_dev(meta), **kw)
    with pytest.raises(K.KernelError):
        K.attn_chunk_tc(q.to(DEV), pool.to(DEV), out, items=items_t.to(DEV), n_items=len(items), n_splits=17,
                        part_o=part_o, part_ml=part_ml, **_dev(meta), **kw)
    n_sm = torch.cuda.get_device_properties(0).multi_processor_count
    assert K.attn_chunk_tc_splits(64, 16, 100000) == 1 and K.attn_chunk_tc_splits(4, 16, 600) == 1
    assert 1 < K.attn_chunk_tc_splits(4, 16, 30000) <= min(K.TC_ATTN_MAX_SPLITS, n_sm // 32)
    # the scratch of attn_chunk_tc_scratch holds every cut that attn_chunk_tc_splits chooses
    for n_items, heads in ((2, 1), (4, 16), (5, 7), (16, 4), (3, 40)):
        sp = K.attn_chunk_tc_splits(n_items, heads, 1 << 20)
        assert 64 * n_items * heads * sp * hd <= K.attn_chunk_tc_scratch()[0], (n_items, heads, sp)


def test_attn_chunk_tcgen05_one_far_key_among_thousands_in_ranges():
    """A portion of 128 tokens behind 3,900 cached ones, the keys cut into ranges: one key far back (in an early
    range) is made to carry nearly all the weight of some queries, so that a range whose maximum or denominator
    were lost in the merge would show."""
    dtype, hd, nh, nkv, P = torch.bfloat16, 128, 2, 1, 64
    segs = [(3900, 128)]
    pool, q, meta, T = _paged_case(dtype, nh, nkv, hd, P, segs, seed=5, n_pages=66)
    far = 777
    page, off = int(meta["block_table"][0, far // P]), far % P
    pool[page, 0, 0, off] = pool[page, 0, 0, off] * 0 + 4.0      # a large key ...
    q[::3] = q[::3] * 0 + 0.5                                     # ... that every third query points at
    items_t = torch.tensor([(0, o) for o in range(0, 128, K.MMA_QUERY_TILE)], dtype=torch.int32)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=0, scale=1 / math.sqrt(hd))
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.attn_chunk(q, pool, ref, items=items_t, n_items=len(items_t), **meta, **kw)
    v_far = pool[page, 1, 0, off].double()
    assert float((ref[0, :hd] - v_far).abs().max()) < 1e-2 * float(v_far.abs().max())   # the far key does dominate
    for n_splits in (1, 5, 12):
        part_o = torch.full((T * nh * n_splits * hd,), float("nan"), device=DEV)
        part_ml = torch.full((T * nh * n_splits * 2,), float("nan"), device=DEV)
        out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
        K.attn_chunk_tc(q.to(DEV), pool.to(DEV), out, items=items_t.to(DEV), n_items=len(items_t), n_splits=n_splits,
                        part_o=part_o, part_ml=part_ml, **_dev(meta), **kw)
        assert K.attn_tc_error() == 0
        close(out, ref, dtype, f"far key, {n_splits} key ranges")


@pytest.mark.parametrize("slope", [0.1, 0.01, -0.02])
def test_attn_chunk_tcgen05_scores_that_rise_or_fall_along_the_keys(slope):
    """The kernel keeps a row's weighted sum in tensor memory and rescales it only when the row's maximum has run
    ahead of the reference its probabilities are formed against by more than 2^8.  Scores that rise by 0.1 a key
    (18 powers of two a tile: a rescale at every tile), by 0.01 (a rescale every few tiles, probabilities above 1
    in between) and scores that fall (the first tile's maximum stands to the end), whole and in key ranges."""
    dtype, hd, nh, nkv, P = torch.bfloat16, 128, 2, 2, 64
    segs = [(1500, 128), (0, 200)]
    pool, q, meta, T = _paged_case(dtype, nh, nkv, hd, P, segs, seed=11, n_pages=32)
    pool = (pool.float() * 0.2).to(dtype)
    q = (q.float() * 0.2).to(dtype)
    q.view(T, nh, hd)[:, :, 0] = math.sqrt(hd)                      # score = slope * position + small noise
    for s, (c, n) in enumerate(segs):
        for t in range(c + n):
            page, off = int(meta["block_table"][s, t // P]), t % P
            pool[page, 0, :, off, 0] = slope * t
    items_t = torch.tensor([(s, o) for s, (c, n) in enumerate(segs) for o in range(0, n, K.MMA_QUERY_TILE)], dtype=torch.int32)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=0, scale=1 / math.sqrt(hd))
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.attn_chunk(q, pool, ref, items=items_t, n_items=len(items_t), **meta, **kw)
    for n_splits in (1, 5):
        part_o = torch.full((T * nh * n_splits * hd,), float("nan"), device=DEV)
        part_ml = torch.full((T * nh * n_splits * 2,), float("nan"), device=DEV)
        out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
        K.attn_chunk_tc(q.to(DEV), pool.to(DEV), out, items=items_t.to(DEV), n_items=len(items_t), n_splits=n_splits,
                        part_o=part_o, part_ml=part_ml, **_dev(meta), **kw)
        assert K.attn_tc_error() == 0
        close(out, ref, dtype, f"scores with slope {slope}, {n_splits} key ranges")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,P,window", [(4, 4, 16, 16, 0), (6, 2, 32, 64, 0), (5, 1, 48, 16, 0),
                                                (16, 16, 128, 64, 0), (2, 1, 256, 64, 0), (4, 2, 64, 16, 300),
                                                (4, 2, 128, 64, 300), (8, 8, 64, 32, 50), (6, 3, 32, 32, 0),
                                                (4, 4, 80, 16, 7), (8, 8, 96, 64, 0), (4, 2, 48, 64, 20),
                                                (3, 3, 112, 32, 0), (2, 2, 192, 16, 0)])
def test_attn_decode(dtype, nh, nkv, hd, P, window):
    segs = [(0, 1), (255, 1), (256, 1), (700, 1), (31, 1)]
    pool, q, meta, T = _paged_case(dtype, nh, nkv, hd, P, segs, seed=hd + 1, n_pages=100)
    items = torch.arange(len(segs), dtype=torch.int32)
    max_splits = 700 // K.DECODE_SPLIT + 1 + 2  # more splits than needed must not matter
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=window, scale=1 / math.sqrt(hd))
    out = torch.zeros(T, nh * hd, dtype=dtype, device=DEV)
    part_o = torch.full((len(segs) * nh * max_splits * hd,), float("nan"), device=DEV)
    part_ml = torch.full((2 * len(segs) * nh * max_splits,), float("nan"), device=DEV)
    counters = torch.zeros(len(segs) * nh, dtype=torch.int32, device=DEV)
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.attn_decode(q, pool, ref, items=items, n_items=len(segs), part_o=None, part_ml=None, counters=None,
                   max_splits=max_splits, **meta, **kw)
    # the second call finds the counters as the first left them: zero.  Where the streaming kernel runs, its two
    # variants (one or two chunks in flight per warp; the library picks by the batch) are both forced in turn
    try:
        for deep in (None, False, True):
            K.attn_decode_variant(deep)
            out.zero_()
            K.attn_decode(q.to(DEV), pool.to(DEV), out, items=items.to(DEV), n_items=len(segs), part_o=part_o,
                          part_ml=part_ml, counters=counters, max_splits=max_splits, **_dev(meta), **kw)
            close(out, ref, dtype, f"attn_decode (two chunks in flight: {deep})")
            assert int(counters.abs().sum()) == 0
    finally:
        K.attn_decode_variant(None)


@pytest.mark.parametrize("nh,nkv,hd,P,window", [(28, 4, 128, 64, 0), (6, 2, 64, 16, 0), (12, 1, 128, 16, 0), (32, 2, 64, 32, 0),
                                                (14, 2, 128, 64, 333), (8, 4, 64, 48, 40), (16, 1, 128, 64, 0)])
def test_attn_decode_grouped_queries(nh, nkv, hd, P, window, monkeypatch):
    """Several query heads per key/value head: the kernel that serves a whole group from one pass over the keys
    (tensor cores, csrc/attention_gqa.cu), against the plain attention and against the per-head kernel; groups of
    2 to 16 heads, both head sizes, windows, contexts from one key to thousands, lengths that end anywhere in a
    chunk of 16 keys."""
    segs = [(0, 1), (15, 1), (16, 1), (255, 1), (1000, 1), (2047, 1), (33, 1), (4200, 1)]
    dtype = torch.bfloat16
    pool, q, meta, T = _paged_case(dtype, nh, nkv, hd, P, segs, seed=nh + hd, n_pages=sum(-(-(c + 1) // P) for c, _ in segs) + 2)
    monkeypatch.setattr(K, "GQA_MIN_UNITS", 1)   # also the batches that the engine would give to the per-head kernels
    assert K.attn_decode_gqa_takes(dtype, nh, nkv, hd, P, len(segs))
    items = torch.tensor([3, 0, 7, 1, 2, 4, 6, 5], dtype=torch.int32)   # items in another order than the segments
    max_splits = 4200 // K.DECODE_SPLIT + 1
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=window, scale=1 / math.sqrt(hd))
    units = K.decode_units(len(segs), nh, hd, dtype, max_splits, DEV, P, nkv)
    part_o = torch.full((units * hd,), float("nan"), device=DEV)
    part_ml = torch.full((2 * units,), float("nan"), device=DEV)
    counters = torch.zeros(len(segs) * nh, dtype=torch.int32, device=DEV)
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.attn_decode(q, pool, ref, items=items, n_items=len(segs), part_o=None, part_ml=None, counters=None,
                   max_splits=max_splits, **meta, **kw)
    outs = {}
    for gqa, few in ((True, True), (True, False), (False, None)):   # both shapes of the group kernel, then per head
        K.USE_GQA_DECODE = gqa
        K.attn_decode_gqa_variant(few)
        try:
            for again in range(2):
                out = torch.zeros(T, nh * hd, dtype=dtype, device=DEV)
                pu = part_o if gqa else torch.full((len(segs) * nh * max_splits * hd,), float("nan"), device=DEV)
                pm = part_ml if gqa else torch.full((2 * len(segs) * nh * max_splits,), float("nan"), device=DEV)
                K.attn_decode(q.to(DEV), pool.to(DEV), out, items=items.to(DEV), n_items=len(segs), part_o=pu,
                              part_ml=pm, counters=counters, max_splits=max_splits, **_dev(meta), **kw)
                close(out, ref, dtype, f"attn_decode, grouped queries ({'group' if gqa else 'per head'} kernel, few pairs: {few})")
                assert int(counters.abs().sum()) == 0
            outs[gqa] = out
        finally:
            K.USE_GQA_DECODE = True
            K.attn_decode_gqa_variant(None)
    # a scratch that holds just one partial result per (request, head): one range each, still right
    tight_o = torch.full((len(segs) * nh * hd,), float("nan"), device=DEV)
    tight_ml = torch.full((2 * len(segs) * nh,), float("nan"), device=DEV)
    out = torch.zeros(T, nh * hd, dtype=dtype, device=DEV)
    K.attn_decode(q.to(DEV), pool.to(DEV), out, items=items.to(DEV), n_items=len(segs), part_o=tight_o, part_ml=tight_ml,
                  counters=counters, max_splits=max_splits, **_dev(meta), **kw)
    close(out, ref, dtype, "attn_decode, grouped queries, one range per request")
    monkeypatch.undo()
    assert K.attn_decode_gqa_takes(dtype, 28, 4, 128, 64, 4) and not K.attn_decode_gqa_takes(dtype, 28, 4, 128, 64, 3)
    assert not K.attn_decode_gqa_takes(torch.float32, nh, nkv, hd, P, 64) and not K.attn_decode_gqa_takes(dtype, 4, 4, hd, P, 64)
    assert not K.attn_decode_gqa_takes(dtype, 34, 2, hd, P, 64) and not K.attn_decode_gqa_takes(dtype, nh, nkv, 96, P, 64)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 3000])
def test_attn_decode_long_contexts(dtype, window):
    """Thousands of keys per request and very different lengths in one batch: the streaming kernel cuts
    them into many ranges (and, with few requests, into short ones)."""
    nh, nkv, hd, P = 4, 2, 128, 64
    segs = [(9000, 1), (5, 1), (4100, 1)]
    pool, q, meta, T = _paged_case(dtype, nh, nkv, hd, P, segs, seed=11, n_pages=260)
    items = torch.arange(len(segs), dtype=torch.int32)
    max_splits = 9000 // K.DECODE_SPLIT + 1
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=window, scale=1 / math.sqrt(hd))
    units = K.decode_units(len(segs), nh, hd, dtype, max_splits, DEV)
    out = torch.zeros(T, nh * hd, dtype=dtype, device=DEV)
    part_o = torch.full((units * hd,), float("nan"), device=DEV)
    part_ml = torch.full((2 * units,), float("nan"), device=DEV)
    counters = torch.zeros(len(segs) * nh, dtype=torch.int32, device=DEV)
    K.attn_decode(q.to(DEV), pool.to(DEV), out, items=items.to(DEV), n_items=len(segs), part_o=part_o,
                  part_ml=part_ml, counters=counters, max_splits=max_splits, **_dev(meta), **kw)
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.attn_decode(q, pool, ref, items=items, n_items=len(segs), part_o=None, part_ml=None, counters=None,
                   max_splits=max_splits, **meta, **kw)
    close(out, ref, dtype, "attn_decode, long")
    assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_and_respects_the_window_edge(dtype):
    """One key among hundreds carries a large score: the output must be (nearly) its value.
    With a window that ends one key short of it, the output must not contain it."""
    nh = nkv = 2
    hd, P, ctx = 64, 16, 600
    far = 3  # position of the marked key
    pool, q, meta, T = _paged_case(dtype, nh, nkv, hd, P, [(ctx, 1), (ctx - 7, 8)], seed=5, n_pages=90)
    pool *= 0.05
    q *= 0.05
    for s in range(2):
        page, off = int(meta["block_table"][s, far // P]), far % P
        pool[page, 0, :, off] = 0
        pool[page, 0, :, off, 0] = 30.0
        pool[page, 1, :, off] = 0
        pool[page, 1, :, off, 1] = 7.0
    q.view(T, nh, hd)[:, :, 0] = 8.0  # score 8 * 30 / sqrt(64) = 30 on the marked key
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, scale=1 / math.sqrt(hd))
    ms = ctx // K.DECODE_SPLIT + 1
    for window, seen in [(0, True), (ctx - far + 1, True), (ctx - far, False)]:
        out = torch.zeros(T, nh * hd, dtype=dtype, device=DEV)
        K.attn_decode(q.to(DEV), pool.to(DEV), out, items=torch.tensor([0], dtype=torch.int32, device=DEV), n_items=1,
                      part_o=torch.zeros(nh * ms * hd, device=DEV), part_ml=torch.zeros(2 * nh * ms, device=DEV),
                      counters=torch.zeros(nh, dtype=torch.int32, device=DEV), max_splits=ms, window=window, **_dev(meta), **kw)
        items = torch.tensor([[1, 0]], dtype=torch.int32)
        w2 = window - 7 if window else 0  # segment 1's last query sits at the same position as segment 0's
        K.attn_chunk(q.to(DEV), pool.to(DEV), out, items=items.to(DEV), n_items=1, window=window, **_dev(meta), **kw)
        if dtype == torch.bfloat16:  # the tensor-core kernel must see (or not see) the marked key as well
            out_tc = torch.zeros(T, nh * hd, dtype=dtype, device=DEV)
            K.attn_chunk_mma(q.to(DEV), pool.to(DEV), out_tc, items=items.to(DEV), n_items=1, window=window,
                             **_dev(meta), **kw)
            v = float(out_tc.float().cpu().view(T, nh, hd)[T - 1, 0, 1])
            assert (abs(v - 7.0) < 0.1) if seen else (abs(v) < 0.5), (window, v)
        o = out.float().cpu().view(T, nh, hd)
        for row in (0, T - 1):
            v = float(o[row, 0, 1])
            if seen:
                assert abs(v - 7.0) < 0.1, (window, row, v)
            else:
                assert abs(v) < 0.5, (window, row, v)


def test_kernels_refuse_what_they_cannot_do():
    x = torch.zeros(4, 16, device=DEV)
    with pytest.raises(K.KernelError):
        K.linear(x, torch.zeros(8, 16, device=DEV), torch.zeros(4, 8, dtype=torch.bfloat16, device=DEV), accumulate=True)
    with pytest.raises(K.KernelError):
        K.linear(x.half(), torch.zeros(8, 16, device=DEV), torch.zeros(4, 8, device=DEV))
    meta = dict(seg_q0=torch.zeros(1, dtype=torch.int32, device=DEV), seg_qn=torch.ones(1, dtype=torch.int32, device=DEV),
                seg_ctx=torch.zeros(1, dtype=torch.int32, device=DEV),
                block_table=torch.zeros(1, 1, dtype=torch.int32, device=DEV))
    with pytest.raises(K.KernelError):  # head size 24 is not a multiple of 16
        K.attn_chunk(torch.zeros(1, 24, device=DEV), torch.zeros(1, 2, 1, 16, 24, device=DEV),
                     torch.zeros(1, 24, device=DEV), items=torch.zeros(1, 2, dtype=torch.int32, device=DEV), n_items=1,
                     n_heads=1, n_kv_heads=1, head_dim=24, page_tokens=16, window=0, scale=1.0, **meta)


@pytest.mark.parametrize("V", [331, 4096, 151936])
def test_sample_greedy_and_filters(V):
    R = 6
    logits = rnd(R, V, seed=V, scale=2.0)
    logits[1, 17] = logits[1, 99] = logits[1].max() + 1  # a tie: the first maximum wins
    dl = logits.to(DEV)
    f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
    out = torch.zeros(R, dtype=torch.int32, device=DEV)
    kept = torch.zeros(R, dtype=torch.int32, device=DEV)
    temp = f32([0.0, 0.0, 0.8, 1.0, 1.3, 0.7])
    top_k = torch.tensor([0, 0, 1, 50, 0, 40], dtype=torch.int32, device=DEV)
    top_p = f32([1.0, 1.0, 1.0, 1.0, 0.6, 0.9])
    min_p = f32([0.0, 0.0, 0.0, 0.0, 0.0, 0.05])
    seeds = torch.arange(R, dtype=torch.int64, device=DEV) + 5
    import plain_qwen2moe as plain
    dists = [None, None] + [plain.kept_distribution(logits[r], float(temp[r]), int(top_k[r]), float(top_p[r]), float(min_p[r]))
                            for r in range(2, R)]
    counts = [dict() for _ in range(R)]
    n_draws = 300
    for c in range(n_draws):
        K.sample(dl, temperature=temp, top_k=top_k, top_p=top_p, min_p=min_p, seeds=seeds,
                 counters=torch.full((R,), c, dtype=torch.int64, device=DEV), out=out, kept_count=kept)
        o = out.cpu().tolist()
        for r in range(R):
            counts[r][o[r]] = counts[r].get(o[r], 0) + 1
        if c == 0:
            first, kept0 = o, kept.cpu().tolist()
    assert first[0] == int(torch.argmax(logits[0])) and first[1] == 17
    assert set(counts[0]) == {first[0]} and set(counts[2]) == {int(torch.argmax(logits[2]))}  # top_k = 1
    for r in range(3, R):
        assert kept0[r] == len(dists[r]), (r, kept0[r], len(dists[r]))
        assert set(counts[r]) <= set(dists[r]), "a token outside the kept set was drawn"
        # the most probable kept token is drawn about as often as it should be
        tok = max(dists[r], key=dists[r].get)
        p = dists[r][tok]
        sd = math.sqrt(p * (1 - p) / n_draws)
        assert abs(counts[r].get(tok, 0) / n_draws - p) < 5 * sd + 0.01, (r, p, counts[r].get(tok, 0) / n_draws)
    # same seed and counter: same token
    K.sample(dl, temperature=temp, top_k=top_k, top_p=top_p, min_p=min_p, seeds=seeds,
             counters=torch.zeros(R, dtype=torch.int64, device=DEV), out=out)
    assert out.cpu().tolist() == first


@pytest.mark.parametrize("V", [8192, 20001, 151936, 163840])
def test_sample_cluster_kernel_gives_the_one_block_kernels_tokens(V):
    """Rows of 8,192 to 163,840 tokens are sampled by a cluster of eight blocks per row that holds the row in
    registers; the one-block kernel takes every other size.  Same filters, same fixed-point sums, same draw: the
    same token and the same number of kept tokens, row by row, draw by draw."""
    R = 9
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(R, V, generator=g) * 2.5
    logits[1, 17] = logits[1, V - 1] = logits[1].max() + 1          # a tie of maxima: the first wins
    logits[7] = 0.25                                                 # every token alike
    logits[8, : V // 2] = -200.0                                     # half the row weighs nothing at all
    dl = logits.to(DEV)
    f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
    temp = f32([0.0, 0.0, 0.8, 1.0, 1.3, 0.7, 0.05, 1.0, 0.9])
    top_k = torch.tensor([0, 0, 1, 50, 0, 40, 0, 0, 7000], dtype=torch.int32, device=DEV)
    top_p = f32([1.0, 1.0, 1.0, 1.0, 0.6, 0.9, 0.95, 0.5, 0.999])
    min_p = f32([0.0, 0.0, 0.0, 0.0, 0.0, 0.05, 0.0, 0.0, 0.0])
    seeds = torch.arange(R, dtype=torch.int64, device=DEV) * 77 + 5
    res = {}
    try:
        for cluster in (True, False):
            K.sample_use_cluster(cluster)
            toks, kept_all = [], []
            for c in range(40):
                out = torch.full((R,), -1, dtype=torch.int32, device=DEV)
                kept = torch.full((R,), -1, dtype=torch.int32, device=DEV)
                K.sample(dl, temperature=temp, top_k=top_k, top_p=top_p, min_p=min_p, seeds=seeds,
                         counters=torch.full((R,), c, dtype=torch.int64, device=DEV), out=out, kept_count=kept)
                toks.append(out.cpu().tolist())
                kept_all.append(kept.cpu().tolist())
            res[cluster] = (toks, kept_all)
    finally:
        K.sample_use_cluster(True)
    assert res[True] == res[False]
    toks = res[True][0]
    assert all(0 <= t < V for row in toks for t in row)
    assert toks[0][1] == 17 and toks[0][0] == int(torch.argmax(logits[0]))
    assert len({row[7] for row in toks}) > 5            # the flat row is drawn from all over
    assert all(row[8] >= V // 2 for row in toks)        # nothing without weight is drawn


def test_sampler_front_end_at_the_full_vocabulary():
    """Sampler.sample (packed parameter upload, penalties, then the sampling kernel) on 5 rows of 151,936 logits:
    the same tokens whether the rows go to the cluster kernel or to the one-block kernel, and the same again for the
    same seeds and counters."""
    from locus_b200.sampling.sampler import GREEDY, Sampler, SamplingParams

    V, R = 151936, 5
    logits = (torch.randn(R, V, generator=torch.Generator().manual_seed(7)) * 2.0).to(DEV)
    params = [GREEDY, SamplingParams(temperature=0.8), SamplingParams(temperature=1.0, top_k=40, top_p=0.9),
              SamplingParams(temperature=0.7, top_p=0.8, min_p=0.02),
              SamplingParams(temperature=0.9, top_p=0.95, repeat_penalty=1.2, presence_penalty=0.3, repeat_last_n=16)]
    hist = [[1, 2, 3], [], [5], [7, 7], list(range(100, 140))]
    seeds = [11, 12, 13, 14, 15]
    runs = {}
    try:
        for cluster in (True, False, True):
            K.sample_use_cluster(cluster)
            s = Sampler(DEV, 8)
            runs.setdefault(cluster, []).append([s.sample(logits.clone(), params, seeds, [c] * R, hist) for c in range(12)])
    finally:
        K.sample_use_cluster(True)
    assert runs[True][0] == runs[False][0] == runs[True][1]
    toks = runs[True][0]
    assert all(row[0] == int(torch.argmax(logits[0])) for row in toks)
    assert len({row[1] for row in toks}) > 3 and all(0 <= t < V for row in toks for t in row)


def test_penalties():
    import plain_qwen2moe as plain
    V, R = 50, 3
    logits = rnd(R, V, seed=3, scale=2.0)
    hist = torch.tensor([[1, 2, 2, 2, -1, -1], [5, 5, 7, 49, 0, 0], [-1] * 6], dtype=torch.int32)
    rep, fr, pr = torch.tensor([1.3, 1.0, 1.2]), torch.tensor([0.0, 0.5, 0.1]), torch.tensor([0.2, 0.0, 0.1])
    d = logits.clone().to(DEV)
    K.apply_penalties(d, hist.to(DEV), rep.to(DEV), fr.to(DEV), pr.to(DEV))
    for r in range(R):
        h = [t for t in hist[r].tolist() if t >= 0]
        ref = plain.apply_penalties(logits[r], h, float(rep[r]), float(fr[r]), float(pr[r]), 64)
        close(d[r], ref, torch.float32, f"penalties row {r}")


# ---------------------------------------------------------------------------
# tensor-core products (csrc/gemm_tc.cu): every bfloat16 x bfloat16 call of K.linear above
# already runs on them; these add the large tiles, every grouped tile size, and the
# CUDA-core product on the same bfloat16 inputs.

@pytest.fixture
def cuda_cores_only():
    K.USE_TENSOR_CORES = False
    yield
    K.USE_TENSOR_CORES = True


def test_tensor_cores_are_what_runs_for_bfloat16():
    x, w = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV), torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV)
    assert K.tensor_cores_take(x, w)
    assert not K.tensor_cores_take(x.float(), w.float()) and not K.tensor_cores_take(x, w.float())
    assert not K.tensor_cores_take(x[:, :60], w[:, :60])  # width 60: no 16-byte rows for TMA
    assert K.tc_error() == 0


@pytest.mark.parametrize("M,N,K_", [(300, 260, 1408), (2048, 384, 2048), (17, 2048, 5632), (64, 128, 64)])
def test_linear_tensor_cores_large_tiles(M, N, K_):
    dt = torch.bfloat16
    x, w = rnd(M, K_, dtype=dt, seed=3), rnd(N, K_, dtype=dt, seed=4, scale=0.05)
    bias, rs = rnd(N, dtype=dt, seed=5), rnd(M, seed=6)
    ref = torch.empty(M, N, dtype=torch.float64)
    EK.linear(x, w, ref, bias=bias)
    out = torch.empty(M, N, dtype=dt, device=DEV)
    K.linear(x.to(DEV), w.to(DEV), out, bias=bias.to(DEV))
    close(out, ref, dt, "tensor-core linear + bias")
    res0 = rnd(M, N, seed=7)
    res = res0.clone().to(DEV)
    K.linear(x.to(DEV), w.to(DEV), res, row_scale=rs.to(DEV), accumulate=True)
    ref2 = res0.clone().double()
    EK.linear(x, w, ref2, row_scale=rs, accumulate=True)
    close(res, ref2, dt, "tensor-core linear accumulate")
    w2 = rnd(N, K_, dtype=dt, seed=8, scale=0.05)
    act = torch.empty(M, N, dtype=dt, device=DEV)
    K.linear(x.to(DEV), w.to(DEV), act, w2=w2.to(DEV))
    ref3 = torch.empty(M, N, dtype=torch.float64)
    EK.linear(x, w, ref3, w2=w2)
    close(act, ref3, dt, "tensor-core swiglu")
    assert K.tc_error() == 0


@pytest.mark.parametrize("M,N,K_,tile,splits", [(64, 2048, 2048, 64, 8), (70, 132, 5632, 32, 16), (257, 64, 200, 128, 3),
                                                (512, 2048, 1408, 256, 4), (40, 260, 72, 64, 2)])
def test_linear_tensor_cores_split_along_k(M, N, K_, tile, splits, monkeypatch):
    """A product with few tiles is cut along K: the partial sums of the parts are added up in order by a
    second kernel that also does the epilogue.  Forced plans (the last k-block ragged, more parts asked
    for than there are k-blocks) and the plan the wrapper itself makes."""
    dt = torch.bfloat16
    x, w = rnd(M, K_, dtype=dt, seed=3), rnd(N, K_, dtype=dt, seed=4, scale=0.05)
    bias, rs = rnd(N, dtype=dt, seed=5), rnd(2 * M, seed=6)
    rows = torch.randperm(2 * M, generator=torch.Generator().manual_seed(7))[:M].to(torch.int32)
    own = K.tc_plan(M, N, K_, False)
    for plan in ((tile, splits), own):
        monkeypatch.setattr(K, "tc_plan", lambda m, n, k, dual, plan=plan: plan if not dual else (min(plan[0], 128), 1))
        before = K.launches
        out = torch.empty(M, N, dtype=dt, device=DEV)
        K.linear(x.to(DEV), w.to(DEV), out, bias=bias.to(DEV))
        if plan[1] > 1:
            assert K.launches - before == 2
        ref = torch.empty(M, N, dtype=torch.float64)
        EK.linear(x, w, ref, bias=bias)
        close(out, ref, dt, f"split linear + bias {plan}")
        res0 = rnd(M, N, seed=8)
        res = res0.clone().to(DEV)
        K.linear(x.to(DEV), w.to(DEV), res, row_scale=rs.to(DEV), scale_rows=rows.to(DEV), accumulate=True)
        ref2 = res0.clone().double()
        EK.linear(x, w, ref2, row_scale=rs, scale_rows=rows, accumulate=True)
        close(res, ref2, dt, f"split linear, scaled rows added into float32 {plan}")
        # the same rows give the same bits wherever they stand in a larger product of the same plan
        if M >= 48:
            part = torch.empty(M, N, dtype=torch.float32, device=DEV)
            K.linear(x.to(DEV), w.to(DEV), part)
            again = torch.empty(M, N, dtype=torch.float32, device=DEV)
            K.linear(x.to(DEV), w.to(DEV), again)
            assert torch.equal(part, again)
    assert K.tc_error() == 0


@pytest.mark.parametrize("tile", [8, 16, 32, 64, 128])  # 8: the row-streaming kernel
def test_linear_grouped_tensor_cores_every_tile(tile):
    T, E, k, H, I = 210, 7, 3, 136, 72
    dt = torch.bfloat16
    ids = _route(T, E, k, 3)
    ids[: 3 * 60] = 4   # one crowded expert (several tiles), expert 0 possibly small
    ids[ids == 2] = 5   # expert 2 gets nothing
    h = rnd(T, H, dtype=dt, seed=1)
    wg, wu = rnd(E, I, H, dtype=dt, seed=2, scale=0.2), rnd(E, I, H, dtype=dt, seed=3, scale=0.2)
    wd = rnd(E, H, I, dtype=dt, seed=4, scale=0.2)
    wts = torch.rand(T * k, generator=torch.Generator().manual_seed(5))
    lay, ref_lay = K.ExpertLayout(T * k, E, 64, DEV), EK.ExpertLayout(T * k, E, 64, "cpu")
    K.moe_sort(ids.to(DEV), T * k, lay, tile)
    EK.moe_sort(ids, T * k, ref_lay, tile)
    assert int(lay.n_tiles.cpu()) == int(ref_lay.n_tiles) <= lay.tiles_for(T * k)
    xs = torch.empty(T * k, H, dtype=dt, device=DEV)
    K.gather_rows(h.to(DEV), lay.sorted_pair, k, xs, T * k)
    assert torch.equal(xs.cpu(), h[(ref_lay.sorted_pair.long() // k)])
    act = torch.full((T * k, I), float("nan"), dtype=dt, device=DEV)
    K.linear(xs, wg.to(DEV), act, w2=wu.to(DEV), layout=lay, n_rows=T * k)
    ref_act = torch.empty(T * k, I, dtype=torch.float64)
    EK.linear(xs.cpu(), wg, ref_act, w2=wu, layout=ref_lay, n_rows=T * k)
    close(act, ref_act, dt, f"grouped swiglu, tile {tile}")
    pair_out = torch.full((T * k, H), float("nan"), device=DEV)
    K.linear(act, wd.to(DEV), pair_out, layout=lay, n_rows=T * k, row_scale=wts.to(DEV), scale_rows=lay.sorted_pair)
    ref_out = torch.empty(T * k, H, dtype=torch.float64)
    EK.linear(act.cpu(), wd, ref_out, layout=ref_lay, n_rows=T * k, row_scale=wts, scale_rows=ref_lay.sorted_pair)
    close(pair_out, ref_out, dt, f"grouped down, tile {tile}")
    if tile == 128:
        # the second product over the same layout in tiles of 256 rows (the crowded expert has 180): the same rows out
        K.moe_sort(ids.to(DEV), T * k, lay, tile, 256)
        assert int(lay.n_tiles2.cpu()) < int(lay.n_tiles.cpu())
        out2 = torch.full((T * k, H), float("nan"), device=DEV)
        K.linear(act, wd.to(DEV), out2, layout=lay, n_rows=T * k, row_scale=wts.to(DEV), scale_rows=lay.sorted_pair,
                 second_tiles=True)
        close(out2, ref_out, dt, "grouped down, second tile list of 256 rows")
        bf = torch.full((T * k, H), float("nan"), dtype=dt, device=DEV)   # and into rows of the model's element type
        K.linear(act, wd.to(DEV), bf, layout=lay, n_rows=T * k, row_scale=wts.to(DEV), scale_rows=lay.sorted_pair,
                 second_tiles=True)
        close(bf, ref_out, dt, "grouped down, bfloat16 rows")
    assert K.tc_error() == 0


@pytest.mark.parametrize("M,N,K_", [(2, 61, 2048), (8, 2048, 1408), (9, 100, 72), (17, 331, 120), (32, 6144, 2048)])
def test_linear_skinny_rows(M, N, K_, monkeypatch):
    """2..32 rows of bfloat16: the weight-streaming tensor-core kernel, every epilogue (the wrapper sends
    it at most ``SKINNY_ROWS`` rows; the kernel takes 32)."""
    monkeypatch.setattr(K, "SKINNY_ROWS", 32)
    dt = torch.bfloat16
    x, w = rnd(M, K_, dtype=dt, seed=3), rnd(N, K_, dtype=dt, seed=4, scale=0.05)
    assert K.skinny_takes(x.to(DEV), w.to(DEV), M)
    bias, rs = rnd(N, dtype=dt, seed=5), rnd(M, seed=6)
    ref = torch.empty(M, N, dtype=torch.float64)
    EK.linear(x, w, ref, bias=bias)
    out = torch.empty(M, N, dtype=dt, device=DEV)
    K.linear(x.to(DEV), w.to(DEV), out, bias=bias.to(DEV))
    close(out, ref, dt, "skinny linear + bias")
    logits = torch.empty(M, N, device=DEV)  # float32 out, as the head and the router want it
    K.linear(x.to(DEV), w.to(DEV), logits)
    ref_l = torch.empty(M, N, dtype=torch.float64)
    EK.linear(x, w, ref_l)
    close(logits, ref_l, torch.float32, "skinny linear float32 out")
    res0 = rnd(M, N, seed=7)
    res = res0.clone().to(DEV)
    K.linear(x.to(DEV), w.to(DEV), res, row_scale=rs.to(DEV), accumulate=True)
    ref2 = res0.clone().double()
    EK.linear(x, w, ref2, row_scale=rs, accumulate=True)
    close(res, ref2, dt, "skinny accumulate")
    w2 = rnd(N, K_, dtype=dt, seed=8, scale=0.05)
    act = torch.empty(M, N, dtype=dt, device=DEV)
    K.linear(x.to(DEV), w.to(DEV), act, w2=w2.to(DEV))
    ref3 = torch.empty(M, N, dtype=torch.float64)
    EK.linear(x, w, ref3, w2=w2)
    close(act, ref3, dt, "skinny swiglu")


def test_cuda_core_product_on_bfloat16(cuda_cores_only):
    dt = torch.bfloat16
    x, w = rnd(70, 120, dtype=dt, seed=3), rnd(130, 120, dtype=dt, seed=4, scale=0.1)
    out = torch.empty(70, 130, dtype=dt, device=DEV)
    before = K.launches
    K.linear(x.to(DEV), w.to(DEV), out)
    ref = torch.empty(70, 130, dtype=torch.float64)
    EK.linear(x, w, ref)
    close(out, ref, dt, "cuda-core bf16")
    assert K.launches == before + 1
