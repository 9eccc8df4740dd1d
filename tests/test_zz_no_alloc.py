"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the kernel library cannot hand it scratch buffers: they run where device
allocation is forbidden (inside a stream callback or a section that holds an allocator
lock, or in a host that got a fixed memory budget and no allocator), or they are plain C
programs without a tensor library.  ``locus_attn_decode_static`` keeps the scratch in a
fixed 4 MiB device array inside the library instead.  This test calls it twice in a row
(the second call finds the first call's leftovers in the shared array) and compares each
result with the regular entry point's and with the plain float64 attention of
``tests/emulated_kernels.py``, checks that device memory does not move, that a call too large
for the array is refused, and that a call whose ``max_splits`` does not cover its longest
context reports it and leaves the shared counters usable.  The file sorts last so that a run that stops at
the first failure has already run every other test.
"""
import ctypes
import math

import pytest
import torch

import emulated_kernels as EK

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_FLOATS = 1 << 20
ERR_SCRATCH_TOO_SMALL = 10002


def _case(dtype, seed, n_items, nh, nkv, hd, P, ctx_list):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-(c + 1) // P) for c in ctx_list) + 3
    pool = (torch.randn(n_pages, 2, nkv, P, hd, generator=g)).to(dtype).to(DEV)
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-(c + 1) // P) for c in ctx_list)
    table = torch.full((n_items, width), -1, dtype=torch.int32)
    used = 0
    for s, c in enumerate(ctx_list):
        need = -(-(c + 1) // P)
        table[s, :need] = torch.tensor(perm[used : used + need], dtype=torch.int32)
        used += need
    q = torch.randn(n_items, nh * hd, generator=g).to(dtype).to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return dict(q=q, pool=pool, table=table.to(DEV), seg_q0=i32(list(range(n_items))), seg_qn=i32([1] * n_items),
                seg_ctx=i32(ctx_list), items=i32(list(range(n_items))))


def _call(lib, static, c, out, nh, nkv, hd, P, window, max_splits, scratch=None):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    I, F = ctypes.c_int, ctypes.c_float
    dt = 1 if c["q"].dtype == torch.bfloat16 else 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    head = [p(c["q"]), I(dt), p(c["pool"]), p(out), p(c["seg_q0"]), p(c["seg_qn"]), p(c["seg_ctx"]), p(c["table"]),
            I(c["table"].shape[1]), p(c["items"]), I(c["q"].shape[0]), I(nh), I(nkv), I(hd), I(P), I(window),
            F(1.0 / math.sqrt(hd))]
    if static:
        return lib.locus_attn_decode_static(*head, I(max_splits), stream)
    part_o, part_ml, counters = scratch
    units = min(part_o.numel() // hd, part_ml.numel() // 2)
    return lib.locus_attn_decode(*head, p(part_o), p(part_ml), p(counters), I(max_splits), ctypes.c_longlong(units),
                                 stream)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_point_matches_the_regular_one_twice(dtype):
    from locus_b200.csrc import build

    lib = build.load("attention")
    assert hasattr(lib, "locus_attn_decode_static")
    nh, nkv, hd, P = 8, 2, 64, 16
    ctxs = [[0, 255, 256, 700], [513, 31, 1023, 300]]
    from locus_b200.kernels import DECODE_SPLIT

    max_splits = 1023 // DECODE_SPLIT + 1  # the longest context below is 1023
    n = 4
    scratch = (torch.empty(n * nh * max_splits * hd, device=DEV), torch.empty(2 * n * nh * max_splits, device=DEV),
               torch.zeros(n * nh, dtype=torch.int32, device=DEV))
    # first call on this device resolves the array's address; it is made outside any capture
    cases = [_case(dtype, 11 + i, n, nh, nkv, hd, P, ctxs[i]) for i in range(2)]
    outs = [torch.zeros(n, nh * hd, dtype=dtype, device=DEV) for _ in range(2)]
    refs = [torch.zeros(n, nh * hd, dtype=dtype, device=DEV) for _ in range(2)]
    torch.cuda.synchronize()
    assert _call(lib, True, cases[0], outs[0], nh, nkv, hd, P, 0, max_splits) == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    assert _call(lib, True, cases[1], outs[1], nh, nkv, hd, P, 0, max_splits) == 0  # finds the leftovers of call 1
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the entry point moved device memory"
    for i in range(2):
        assert _call(lib, False, cases[i], refs[i], nh, nkv, hd, P, 0, max_splits, scratch) == 0
    torch.cuda.synchronize()
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    for i in range(2):
        ref = refs[i].double()
        err = float((outs[i].double() - ref).abs().max())
        assert math.isfinite(err) and err <= tol * float(ref.abs().max()), (i, err)
        assert float(outs[i].abs().max()) > 0
        plain = _plain(cases[i], nh, nkv, hd, P, 0)
        err = float((outs[i].double().cpu() - plain).abs().max())
        assert err <= tol * float(plain.abs().max()), (i, err)
    assert lib.locus_attn_error() == 0


def _plain(c, nh, nkv, hd, P, window):
    """The float64 attention of tests/emulated_kernels.py on host copies of the case."""
    EK.PRECISE = True
    try:
        ref = torch.zeros(c["q"].shape[0], nh * hd, dtype=torch.float64)
        EK.attn_decode(c["q"].cpu(), c["pool"].cpu(), ref, seg_q0=c["seg_q0"].cpu(), seg_qn=c["seg_qn"].cpu(),
                       seg_ctx=c["seg_ctx"].cpu(), block_table=c["table"].cpu(), items=c["items"].cpu(),
                       n_items=c["q"].shape[0], n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=window,
                       scale=1.0 / math.sqrt(hd), part_o=None, part_ml=None, counters=None, max_splits=1 << 20)
    finally:
        EK.PRECISE = False
    return ref


def test_too_few_splits_are_reported_and_do_not_poison_later_calls():
    """``max_splits`` below what the longest context needs: the host cannot see the context lengths, so the kernel
    notices, sets the module's error word, merges the splits that exist and returns its counters to zero.  The
    next, correct call through the shared counters is right."""
    from locus_b200.csrc import build

    lib = build.load("attention")
    nh, nkv, hd, P = 4, 2, 64, 16          # bfloat16 rows of 128 bytes with pages of 16: the split kernel
    c = _case(torch.bfloat16, 21, 3, nh, nkv, hd, P, [700, 40, 300])
    out = torch.zeros(3, nh * hd, dtype=torch.bfloat16, device=DEV)
    assert lib.locus_attn_error() == 0
    assert _call(lib, True, c, out, nh, nkv, hd, P, 0, 3) == 0     # 700 // 128 + 1 = 6 splits are needed
    torch.cuda.synchronize()
    assert lib.locus_attn_error() == 1 and lib.locus_attn_error() == 0   # reported once, then cleared
    plain = _plain(c, nh, nkv, hd, P, 0)
    err = (out.double().cpu() - plain).abs().max(dim=1).values
    assert float(err[1]) <= 1.2e-2 * float(plain.abs().max())   # the request that fits its splits is right
    assert torch.isfinite(out.float()).all()
    out.zero_()
    assert _call(lib, True, c, out, nh, nkv, hd, P, 0, 6) == 0
    torch.cuda.synchronize()
    assert lib.locus_attn_error() == 0
    assert float((out.double().cpu() - plain).abs().max()) <= 1.2e-2 * float(plain.abs().max())


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from locus_b200.csrc import build

    lib = build.load("attention")
    nh, nkv, hd, P = 16, 16, 128, 64
    n, max_splits = 40, 16
    assert n * nh * max_splits * (hd + 2) > SCRATCH_FLOATS
    c = _case(torch.bfloat16, 3, n, nh, nkv, hd, P, [5] * n)
    out = torch.full((n, nh * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    assert _call(lib, True, c, out, nh, nkv, hd, P, 0, max_splits) == ERR_SCRATCH_TOO_SMALL
    torch.cuda.synchronize()
    assert float(out.float().min()) == 7.0  # nothing ran
    # the same call with fewer splits fits
    assert 40 * nh * 1 * (hd + 2) <= SCRATCH_FLOATS
    assert _call(lib, True, c, out, nh, nkv, hd, P, 0, 1) == 0
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all() and float(out.float().min()) != 7.0
