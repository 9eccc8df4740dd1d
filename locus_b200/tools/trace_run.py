"""Trace replay: feed given token ids through a model step by step and write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Reads one JSON object per line from standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

runs each step's entries as ONE batch through the framework's own model, step function,
cache manager and kernels (the ones generation uses; nothing here computes anything), and
for a step in which logits are wanted writes ``<out>/<step>.f32``: float32 little-endian,
[wanted, vocab], in the order of the entries and of their ``want``.  After every step it
prints ``done <step>`` and flushes.  ``end`` names requests that are finished after the
step; their pages and state slot go back to the pool.  It samples nothing.

``--max-tokens N``: the most tokens live requests hold at any time, each request's count
rounded up to a whole page; the cache pool is made for exactly this many, so pages are used
again as requests end.  ``--page-tokens`` (64) and ``--max-live`` (4) are the engine's page size
and the most requests that are live at a time.  ``--dump-routing`` also writes
``<out>/<step>.route.json`` for every step: {feed-forward prefix: [picked experts of row 0, of
row 1, ...]} over all rows of the step in batch order, so that a comparison can tell which side of
a near-tie between two experts the engine took.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PAGE_TOKENS = 64   # defaults of --page-tokens and --max-live
MAX_LIVE = 4


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, dest="max_tokens")
    ap.add_argument("--max-step-tokens", type=int, default=0,
                    help="most tokens in one step (default: --max-tokens)")
    ap.add_argument("--page-tokens", type=int, default=PAGE_TOKENS, dest="page_tokens",
                    help=f"tokens per cache page (default {PAGE_TOKENS})")
    ap.add_argument("--max-live", type=int, default=MAX_LIVE, dest="max_live",
                    help=f"most requests live at a time (default {MAX_LIVE})")
    ap.add_argument("--dump-routing", action="store_true", dest="dump_routing",
                    help="write <step>.route.json: the experts picked for every row of the step")
    args = ap.parse_args(argv)
    if args.page_tokens < 1 or args.max_live < 1 or args.max_tokens < 1:
        ap.error("--page-tokens, --max-live and --max-tokens must be positive")

    import torch

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 1
    from ..cache.manager import CacheError, CacheManager
    from ..engine.engine import parse_dtype
    from ..engine.step import ModelRunner, StepEntry
    from ..models.model import load_model

    os.makedirs(args.out, exist_ok=True)
    print(f"[trace_run] loading {args.model} as {args.dtype}", file=sys.stderr, flush=True)
    model = load_model(args.model, parse_dtype(args.dtype), "cuda:0")
    P = args.page_tokens
    n_pages = max(1, -(-args.max_tokens // P))
    max_seq = min(model.plan.max_positions, n_pages * P)
    cache = CacheManager(model.cache_needs(), page_tokens=P, n_pages=n_pages,
                         n_state_slots=args.max_live, max_seq_tokens=max_seq, dtype=model.dtype, device=model.device)
    step_tokens = args.max_step_tokens or max(args.max_tokens, 1)
    runner = ModelRunner(model, cache, max_tokens=step_tokens, max_segments=args.max_live, max_wanted=step_tokens)
    routing = {}
    if args.dump_routing:
        for part in model.all_parts():
            if hasattr(part, "observer"):
                part.observer = lambda prefix, ids, wts: routing.__setitem__(prefix, ids.cpu().tolist())
    print("[trace_run] ready", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            seq = cache.get(e["id"])
            if seq is None:
                try:
                    seq = cache.open(e["id"])
                except CacheError as err:
                    print(f"trace_run: step {step}: cannot open request {e['id']!r}: {err} (--max-live {args.max_live})",
                          file=sys.stderr)
                    return 2
            if not cache.ensure_capacity(seq, len(e["tokens"])):
                print(f"trace_run: step {step}: out of cache pages for request {e['id']!r} "
                      f"(--max-tokens {args.max_tokens})", file=sys.stderr)
                return 2
            entries.append(StepEntry(seq, e["tokens"], e.get("want", [])))
        if entries:
            routing.clear()
            logits = runner.step(entries)
            if args.dump_routing:
                with open(os.path.join(args.out, f"{step}.route.json"), "w", encoding="utf-8") as f:
                    json.dump(routing, f)
            if logits.shape[0]:
                arr = logits.detach().to("cpu", torch.float32).contiguous().numpy()
                arr.astype("<f4", copy=False).tofile(os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.synchronize()
            runner.check_device_errors()  # a bounded wait of a tensor-core pipeline that ran out: fail here
        for rid in rec.get("end", []):
            seq = cache.get(rid)
            if seq is not None:
                cache.release(seq)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
