"""What each kernel of a decode step adds to the step's time: the step is replayed from its CUDA graph with one
kernel (or family of kernels) left out at a time.

The durations of a launch list (one kernel after the other, cold cache) do not say this: inside the graph the
kernels overlap (programmatic dependent launch, the shared expert on a side stream), and a kernel's share is what
the step gains when it is gone.  The results of an ablated step are wrong by construction; only its time is read.
Leaving the router out leaves the expert layout as the last full step wrote it.

    python -m locus_b200.tools.step_ablation [--config a27b] [--batch 8,1] [--context 4096] [--steps 24]

Sizes come from bench.py's configurations (random weights); prints one line per case and a JSON object at the end.
"""
import argparse
import json
import os
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="step_ablation")
    ap.add_argument("--config", default="a27b")
    ap.add_argument("--batch", default="8,1", help="batch sizes, comma separated")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=24)
    ap.add_argument("--warmup", type=int, default=6)
    ap.add_argument("--only", default="", help="comma separated case names (default: all)")
    args = ap.parse_args(argv)

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    import bench  # the repository's bench.py: the configurations' sizes

    import locus_b200.kernels as K
    import locus_b200.models  # noqa: F401
    from locus_b200.cache import CacheManager
    from locus_b200.config import find_arch
    from locus_b200.engine.step import ModelRunner, StepEntry
    from locus_b200.models.model import Model
    from locus_b200.weights.loader import RandomSource, load_weights

    dev, dtype = "cuda:0", torch.bfloat16
    conf = bench.CONFIGS[args.config]
    raw = dict(conf["raw"])
    raw["max_position_embeddings"] = max(raw["max_position_embeddings"], args.context + 64)
    entry = find_arch(raw["architectures"][0])
    cfg = entry.parse_config(raw)
    model = Model(entry.build_plan(cfg), dtype, dev)
    load_weights(model, RandomSource(model, conf["seed"], dtype, dev))
    batches = [int(b) for b in args.batch.split(",")]
    P, ctx, max_b = 64, args.context, max(batches)
    cache = CacheManager(model.cache_needs(), page_tokens=P, n_pages=max_b * (ctx // P + 2), n_state_slots=max_b,
                         max_seq_tokens=ctx + 64, dtype=dtype, device=dev)
    for g in cache.groups:
        g.pool.view(-1).uniform_(-1, 1)
    gen = torch.Generator().manual_seed(1)
    V, H = cfg.vocab_size, cfg.hidden_size

    def measure(n_batch: int, patch) -> float:
        runner = ModelRunner(model, cache, max_tokens=64, max_segments=max_b, max_wanted=max_b, use_graphs=False)
        seqs = [cache.open(f"s{i}") for i in range(n_batch)]
        for s in seqs:
            assert cache.adopt(s, ctx - args.steps - args.warmup - 2)
        toks = torch.randint(0, V, (args.steps + args.warmup + 1, n_batch), generator=gen).tolist()

        def one(i):
            for s in seqs:
                assert cache.ensure_capacity(s, 1)
            runner.step([StepEntry(s, [toks[i][j]], [0]) for j, s in enumerate(seqs)])

        one(args.steps + args.warmup)   # a whole step outside any graph: the expert layout that "no router" keeps
        for n, f in patch.items():
            setattr(K, n, f)
        runner.use_graphs = True        # the graph is captured with the patch in place
        for i in range(args.warmup):
            one(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.warmup, args.warmup + args.steps):
            one(i)
        b.record()
        torch.cuda.synchronize()
        for s in seqs:
            cache.release(s)
        return a.elapsed_time(b) / args.steps

    names = ("rmsnorm", "rope_kv_write", "route_fused_small", "attn_decode", "linear")
    orig = {n: getattr(K, n) for n in names}

    def noop(*a, **k):
        return None

    def linear_without(pred):
        def f(x, w, out, **kw):
            if pred(w, kw):
                return None
            return orig["linear"](x, w, out, **kw)
        return f

    shared = getattr(cfg, "shared_expert_intermediate_size", 0)
    cases = {
        "base": {},
        "no norms": {"rmsnorm": noop},
        "no rotary encoding and cache write": {"rope_kv_write": noop},
        "no router (stale expert layout)": {"route_fused_small": noop},
        "no attention": {"attn_decode": noop},
        "no q/k/v product": {"linear": linear_without(lambda w, kw: w.dim() == 2 and w.shape[1] == H and w.shape[0] not in (H, V)
                                                      and kw.get("w2") is None and shared not in tuple(w.shape))},
        "no output projection": {"linear": linear_without(lambda w, kw: w.dim() == 2 and tuple(w.shape) == (H, H))},
        "no shared expert": {"linear": linear_without(lambda w, kw: w.dim() == 2 and shared in tuple(w.shape))},
        "no experts gate/up": {"linear": linear_without(lambda w, kw: w.dim() == 3 and kw.get("w2") is not None)},
        "no experts down": {"linear": linear_without(lambda w, kw: w.dim() == 3 and kw.get("w2") is None)},
        "no experts": {"linear": linear_without(lambda w, kw: w.dim() == 3)},
        "no head": {"linear": linear_without(lambda w, kw: w.dim() == 2 and w.shape[0] == V)},
    }
    if args.only:
        cases = {k: v for k, v in cases.items() if k in args.only.split(",")}
    res = {}
    try:
        for n_batch in batches:
            for name, patch in cases.items():
                for n, f in orig.items():
                    setattr(K, n, f)
                ms = measure(n_batch, patch)
                res[f"batch {n_batch}, {name}"] = round(ms, 4)
                print(f"batch {n_batch}, {name}: {ms:.3f} ms/step", flush=True)
    finally:
        for n, f in orig.items():
            setattr(K, n, f)
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
