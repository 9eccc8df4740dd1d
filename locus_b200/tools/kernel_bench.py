"""Runs one kernel of the engine on synthetic inputs, for timing and for profiler captures.

    python -m locus_b200.tools.kernel_bench linear --m 2048 --n 6144 --k 2048 [--dual] [--accumulate] [--iters 20]
    python -m locus_b200.tools.kernel_bench attn_decode --batch 8 --ctx 4000 [--heads 16 --kv-heads 16 --head-dim 128]
    python -m locus_b200.tools.kernel_bench attn_chunk --tokens 2048 --ctx 0
    python -m locus_b200.tools.kernel_bench experts --tokens 2048 [--experts 60 --top-k 4 --k 2048 --n 1408] [--part up|down]

Times with CUDA events after warm-up.  Weights rotate through enough copies that the L2
cannot hold them (``linear``); attention reads a cache larger than the L2 at the default
sizes.  Prints one line with microseconds per call, TFLOP/s and GB/s.  Under ``ncu`` use a
small ``--iters`` and ``-k regex:<kernel>``.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from .. import kernels as K


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _time(fn, iters: int, graph: bool) -> float:
    """Microseconds per call.  ``graph``: replay the calls from a CUDA graph so that the
    host's launch cost does not hide a short kernel's time."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g), K.stream_scope():
            for _ in range(iters):
                fn()
        g.replay()
        torch.cuda.synchronize()
        a, b = _events()
        a.record()
        g.replay()
        b.record()
    else:
        a, b = _events()
        a.record()
        for _ in range(iters):
            fn()
        b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def bench_linear(args) -> None:
    dev = "cuda:0"
    dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    M, N, Kd = args.m, args.n, args.k
    wbytes = N * Kd * (2 if dt == torch.bfloat16 else 4) * (2 if args.dual else 1)
    copies = max(1, min(40, int(400e6 // wbytes)))
    ws = [(torch.randn(N, Kd, device=dev) * 0.02).to(dt) for _ in range(copies)]
    w2s = [(torch.randn(N, Kd, device=dev) * 0.02).to(dt) for _ in range(copies)] if args.dual else None
    x = torch.randn(M, Kd, device=dev).to(dt)
    out = torch.zeros(M, N, device=dev, dtype=torch.float32 if args.accumulate else dt)
    state = {"i": 0}

    def fn():
        i = state["i"] % copies
        state["i"] += 1
        K.linear(x, ws[i], out, w2=w2s[i] if args.dual else None, accumulate=args.accumulate)

    us = _time(fn, args.iters, args.graph)
    flops = 2.0 * M * N * Kd * (2 if args.dual else 1)
    print(f"linear M={M} N={N} K={Kd} dual={int(args.dual)} accumulate={int(args.accumulate)} {args.dtype}: "
          f"{us:.1f} us/call  {flops / us / 1e6:.1f} TFLOP/s  weights {wbytes / us / 1e3:.1f} GB/s  "
          f"(tensor-core error word {K.tc_error() if dt == torch.bfloat16 else 0})")


def bench_experts(args) -> None:
    """The two grouped products of the routed experts as the sparse-MoE block runs them: SwiGLU of
    gate and up ([E, n, k] each) over the tokens laid out by expert, then down ([E, k, n]) with the
    routing weight of each row, into float32 rows.  Every token picks ``top_k`` distinct experts at
    random; the layers' weights rotate through copies so that the L2 cannot hold them."""
    dev = "cuda:0"
    dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    T, E, k, H, I = args.tokens, args.experts, args.top_k, args.k, args.n
    n_pairs = T * k
    g = torch.Generator(device="cpu").manual_seed(1)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).reshape(-1).to(dev)
    wts = torch.rand(n_pairs, device=dev)
    el = 2 if dt == torch.bfloat16 else 4
    layer_bytes = 3 * E * I * H * el
    copies = max(1, min(8, int(3e9 // layer_bytes)))
    gate = [(torch.randn(E, I, H, device=dev) * 0.02).to(dt) for _ in range(copies)]
    up = [(torch.randn(E, I, H, device=dev) * 0.02).to(dt) for _ in range(copies)]
    down = [(torch.randn(E, H, I, device=dev) * 0.02).to(dt) for _ in range(copies)]
    h = torch.randn(T, H, device=dev).to(dt)
    tile = args.tile or (K.FEW_ROWS if T <= K.FEW_ROWS else K.expert_tile(n_pairs, E))
    streamed = tile <= (K.SKINNY_TILE_ROWS if dt == torch.bfloat16 else K.FEW_ROWS)
    if not streamed and dt != torch.bfloat16:
        tile = 64
    lay = K.ExpertLayout(n_pairs, E, 64, dev)
    K.moe_sort(ids, n_pairs, lay, tile)
    xs = torch.empty(n_pairs, H, device=dev, dtype=dt)
    K.gather_rows(h, lay.sorted_pair, k, xs, n_pairs)
    act = torch.empty(n_pairs, I, device=dev, dtype=dt)
    pair_out = torch.empty(n_pairs, H, device=dev, dtype=torch.float32)
    state = {"i": 0}

    def fn():
        i = state["i"] % copies
        state["i"] += 1
        if args.part in ("both", "up"):
            if streamed:
                K.linear(h, gate[i], act, w2=up[i], x_rows=lay.sorted_pair, x_row_div=k, layout=lay, n_rows=n_pairs)
            else:
                K.linear(xs, gate[i], act, w2=up[i], layout=lay, n_rows=n_pairs)
        if args.part in ("both", "down"):
            K.linear(act, down[i], pair_out, layout=lay, n_rows=n_pairs, row_scale=wts, scale_rows=lay.sorted_pair)

    us = _time(fn, args.iters, args.graph)
    share = {"both": 3, "up": 2, "down": 1}[args.part]
    used = int((torch.bincount(ids.long(), minlength=E) > 0).sum())
    flops = 2.0 * n_pairs * H * I * share
    wbytes = used * I * H * el * share
    print(f"experts T={T} E={E} top_k={k} hidden={H} inner={I} part={args.part} tile={tile} {args.dtype}: "
          f"{us:.1f} us/call  {flops / us / 1e6:.1f} TFLOP/s  weights of the {used} experts used {wbytes / us / 1e3:.1f} GB/s  "
          f"(tensor-core error word {K.tc_error() if dt == torch.bfloat16 else 0})")


def _paged(args, B: int, ctx: int, new: int):
    dev = "cuda:0"
    dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    P, nh, nkv, hd = args.page_tokens, args.heads, args.kv_heads, args.head_dim
    per = -(-(ctx + new) // P)
    pool = torch.randn(B * per, 2, nkv, P, hd, device=dev).to(dt)
    table = torch.arange(B * per, dtype=torch.int32, device=dev).view(B, per).contiguous()
    q = torch.randn(B * new, nh * hd, device=dev).to(dt)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    meta = dict(seg_q0=i32([i * new for i in range(B)]), seg_qn=i32([new] * B), seg_ctx=i32([ctx] * B), block_table=table)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=args.window, scale=1 / math.sqrt(hd))
    return pool, q, torch.empty_like(q), meta, kw, i32


def bench_attn_decode(args) -> None:
    B, ctx = args.batch, args.ctx
    pool, q, out, meta, kw, i32 = _paged(args, B, ctx, 1)
    ms = ctx // K.DECODE_SPLIT + 1
    po = torch.empty(B * args.heads * ms * args.head_dim, device="cuda:0")
    pm = torch.empty(2 * B * args.heads * ms, device="cuda:0")
    items = i32(list(range(B)))
    cnt = torch.zeros(B * args.heads, dtype=torch.int32, device="cuda:0")

    def fn():
        K.attn_decode(q, pool, out, items=items, n_items=B, part_o=po, part_ml=pm, counters=cnt, max_splits=ms,
                      **meta, **kw)

    us = _time(fn, args.iters, args.graph)
    byts = B * (ctx + 1) * 2 * args.kv_heads * args.head_dim * pool.element_size()
    print(f"attn_decode batch={B} ctx={ctx} heads={args.heads}/{args.kv_heads} head_dim={args.head_dim} {args.dtype}: "
          f"{us:.1f} us/call  cache read {byts / us / 1e3:.1f} GB/s")


def bench_attn_chunk(args) -> None:
    T, ctx = args.tokens, args.ctx
    pool, q, out, meta, kw, i32 = _paged(args, 1, ctx, T)
    mma = K.attn_chunk_mma_takes(q, args.head_dim) and not args.cuda_cores
    tile = K.MMA_QUERY_TILE if mma else 16
    items = torch.tensor([(0, o) for o in range(0, T, tile)], dtype=torch.int32, device="cuda:0")

    tc = mma and not args.mma_sync and K.attn_chunk_tc_takes(q, args.head_dim, args.page_tokens, T, ctx + T)

    extra = {}
    n_splits = 1
    if tc:
        n_splits = K.attn_chunk_tc_splits(items.shape[0], args.heads, ctx + T) if args.key_ranges < 0 else args.key_ranges
        if n_splits > 1:
            n_o, n_ml = T * args.heads * n_splits * args.head_dim, T * args.heads * n_splits * 2
            extra = dict(n_splits=n_splits, part_o=torch.empty(n_o, device="cuda:0"), part_ml=torch.empty(n_ml, device="cuda:0"))
    elif mma:
        n_splits = K.attn_chunk_mma_splits(items.shape[0], args.heads, ctx + T) if args.key_ranges < 0 else args.key_ranges
        if n_splits > 1:
            n_o, n_ml = K.attn_chunk_mma_scratch(args.head_dim)
            extra = dict(n_splits=n_splits, part_o=torch.empty(n_o, device="cuda:0"), part_ml=torch.empty(n_ml, device="cuda:0"))

    def fn():
        call = K.attn_chunk_tc if tc else (K.attn_chunk_mma if mma else K.attn_chunk)
        call(q, pool, out, items=items, n_items=items.shape[0], **meta, **kw, **extra)

    us = _time(fn, args.iters, args.graph)
    flops = 4.0 * args.heads * args.head_dim * (T * ctx + T * (T + 1) / 2)
    print(f"attn_chunk tokens={T} ctx={ctx} heads={args.heads}/{args.kv_heads} head_dim={args.head_dim} "
          f"{f'tcgen05, {n_splits} key ranges' if tc else (f'mma.sync, {n_splits} key ranges' if mma else 'cuda cores')}: {us:.1f} us/call  {flops / us / 1e6:.1f} TFLOP/s (causal flops)")


def bench_sample(args) -> None:
    """The sampling kernel on --rows rows of --vocab random float32 logits: greedy, temperature 0.8 alone, with
    top-k 50, with top-p 0.9, with top-k 50 + top-p 0.9 + min-p 0.05.  --one-block keeps every row on the one-block
    kernel (up to 16 rows of 8,192 to 163,840 tokens otherwise go to the cluster kernel)."""
    dev = "cuda:0"
    R, V = args.rows, args.vocab
    K.sample_use_cluster(not args.one_block)
    logits = torch.randn(R, V, device=dev, generator=torch.Generator(dev).manual_seed(1)) * 3
    full = lambda v, dt: torch.full((R,), v, dtype=dt, device=dev)
    out = torch.zeros(R, dtype=torch.int32, device=dev)
    seeds, ctr = torch.arange(R, dtype=torch.int64, device=dev), torch.zeros(R, dtype=torch.int64, device=dev)
    for name, t, k, p, m in (("greedy", 0.0, 0, 1.0, 0.0), ("temperature", 0.8, 0, 1.0, 0.0), ("top-k 50", 0.8, 50, 1.0, 0.0),
                             ("top-p 0.9", 0.8, 0, 0.9, 0.0), ("top-k + top-p + min-p", 0.8, 50, 0.9, 0.05)):
        kw = dict(temperature=full(t, torch.float32), top_k=full(k, torch.int32), top_p=full(p, torch.float32),
                  min_p=full(m, torch.float32), seeds=seeds, counters=ctr, out=out)
        us = _time(lambda: K.sample(logits, **kw), args.iters, args.graph)
        print(f"sample rows={R} vocab={V} {'one block a row' if args.one_block else 'default'} {name}: {us:.1f} us/call")
    K.sample_use_cluster(True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kernel_bench")
    ap.add_argument("kernel", choices=["linear", "attn_decode", "attn_chunk", "experts", "sample"])
    ap.add_argument("--rows", type=int, default=8, help="sample: rows of logits")
    ap.add_argument("--vocab", type=int, default=151936, help="sample: logits of a row")
    ap.add_argument("--one-block", action="store_true", help="sample: never the cluster kernel")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--graph", action="store_true", help="time a CUDA graph of the calls")
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--dual", action="store_true", help="SwiGLU of two weight matrices")
    ap.add_argument("--accumulate", action="store_true", help="add into a float32 output")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4000)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-tokens", type=int, default=64)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--experts", type=int, default=60)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--tile", type=int, default=0, help="experts: rows of a tile instead of the engine's choice")
    ap.add_argument("--part", default="both", choices=["both", "up", "down"], help="experts: which product")
    ap.add_argument("--skinny-rows", type=int, default=-1,
                    help="linear: most rows that go to the weight-streaming kernel instead of the engine's limit")
    ap.add_argument("--token-tile", type=int, default=0,
                    help="linear: token tile of the tcgen05 kernel instead of the engine's choice")
    ap.add_argument("--splits", type=int, default=0,
                    help="linear: with --token-tile, parts along K (0 = not split)")
    ap.add_argument("--cuda-cores", action="store_true", help="attn_chunk: the CUDA-core kernel")
    ap.add_argument("--key-ranges", type=int, default=-1,
                    help="attn_chunk, tensor-core kernels: ranges the keys are cut into (default: the engine's choice)")
    ap.add_argument("--mma-sync", action="store_true", help="attn_chunk: the mma.sync kernel where tcgen05 would run")
    args = ap.parse_args(argv)
    if args.skinny_rows >= 0:
        K.SKINNY_ROWS = args.skinny_rows
        K.FEW_ROWS = min(K.FEW_ROWS, args.skinny_rows)
    if args.token_tile:
        K.tc_plan = lambda m, n, k, dual: (args.token_tile, max(1, args.splits))
    if not torch.cuda.is_available():
        print("kernel_bench: no CUDA device", file=sys.stderr)
        return 1
    {"linear": bench_linear, "attn_decode": bench_attn_decode, "attn_chunk": bench_attn_chunk,
     "experts": bench_experts, "sample": bench_sample}[args.kernel](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
