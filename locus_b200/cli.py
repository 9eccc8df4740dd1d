"""``locus-run``: generate from a model folder on the command line.

    locus-run [options] <model_dir> <prompt> [n_tokens=64]

In the manner of the reference's ``locus-run`` (tools/run_main.cpp:16-137; flags
tools/backend_cli.hpp:164-282): the same positional arguments, ``--ctx``, ``--concurrent``,
``--batch-decode``, ``--no-batch-prefill``, ``--archs``, ``--backends``, ``--quants``,
``--tokenizers``, ``--capabilities`` and ``-h``, a banner with the model's sizes on stderr
and, with ``--concurrent N``, a ``bench:`` line with the aggregate tokens per second.  This
engine takes token ids, not text: ``<prompt>`` is a list of ids ("5,17,3" or "5 17 3"),
``@file`` with such a list, or ``random:LEN``; generated ids are printed as they come.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List


def _parse_prompt(text: str, vocab: int, seed: int) -> List[int]:
    if text.startswith("random:"):
        import torch

        g = torch.Generator().manual_seed(seed)
        return torch.randint(0, vocab, (int(text[7:]),), generator=g).tolist()
    if text.startswith("@"):
        with open(text[1:], "r", encoding="utf-8") as f:
            text = f.read()
    ids = [int(t) for t in text.replace(",", " ").split()]
    if not ids:
        raise ValueError("empty prompt")
    return ids


def _print_archs() -> None:
    from . import models  # noqa: F401
    from .config import archs

    print("architectures:")
    for a in archs():
        print(f"  {a.name:24s} {a.description}")


def _print_backends() -> None:
    print("backends:\n  cuda-sm100a              hand-written CUDA kernels for NVIDIA B200 (the only backend)")


def _print_quants() -> None:
    print("weight element types:\n  BF16  F16 (read as BF16)  F32   (no quantised formats)")


def _print_tokenizers() -> None:
    print("tokenizers:\n  (none: prompts and outputs are token ids)")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="locus-run", description="Generate token ids from a model folder on one B200.",
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model", nargs="?", help="folder with config.json and model.safetensors")
    ap.add_argument("prompt", nargs="?", help='token ids "5,17,3", @file, or random:LEN')
    ap.add_argument("n_tokens", nargs="?", type=int, default=64, help="tokens to generate (default 64)")
    ap.add_argument("--backend", default="", help="select the math backend (see --backends)")
    ap.add_argument("--backends", action="store_true", help="list available backends and exit")
    ap.add_argument("--archs", action="store_true", help="list supported architectures and exit")
    ap.add_argument("--quants", action="store_true", help="list loadable weight element types and exit")
    ap.add_argument("--tokenizers", action="store_true", help="list tokenizer families and exit")
    ap.add_argument("--capabilities", action="store_true", help="list archs+backends+quants+tokenizers, exit")
    ap.add_argument("--ctx", type=int, default=0, help="cap the KV pool at N tokens (default min(model context, 4096))")
    ap.add_argument("--kv-fraction", type=float, default=0.0,
                    help="instead of --ctx: size the KV pool to this share of the free device memory")
    ap.add_argument("--concurrent", type=int, default=1, help="submit the prompt N times and report aggregate tok/s")
    ap.add_argument("--batch-decode", action="store_true", help="decode all running requests in one batch (always on here)")
    ap.add_argument("--no-batch-prefill", action="store_true", help="force per-token prompt ingestion")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--repeat-last-n", type=int, default=64)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--page-tokens", type=int, default=64)
    ap.add_argument("--chunk", type=int, default=2048, help="longest portion of a prompt in one step")
    ap.add_argument("--max-batch-tokens", type=int, default=2048, help="tokens of one step")
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="write a random-weights model folder from --config into <model_dir> first")
    ap.add_argument("--config", default="", help="config.json for --random-weights")
    ap.add_argument("--stats", action="store_true", help="print engine counters at exit")
    ap.add_argument("--moe-stats", action="store_true",
                    help="count the picked experts per layer and print the reference's moe-stats line at exit "
                         "(also switched on by the environment variable LOCUS_MOE_STATS)")
    ap.add_argument("--kernel-times", action="store_true",
                    help="run every step eagerly and print, at exit, the time per kernel entry point")
    return ap


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.backends:
        _print_backends()
        return 0
    if args.archs:
        _print_archs()
        return 0
    if args.quants:
        _print_quants()
        return 0
    if args.tokenizers:
        _print_tokenizers()
        return 0
    if args.capabilities:
        _print_archs(); print(); _print_backends(); print(); _print_quants(); print(); _print_tokenizers()
        return 0
    if not args.model or not args.prompt:
        print("usage: locus-run [options] <model_dir> <prompt> [n_tokens]\nsee locus-run --help", file=sys.stderr)
        return 2
    if args.backend not in ("", "cuda-sm100a"):
        print(f"error: unknown backend {args.backend!r} (see --backends)", file=sys.stderr)
        return 1
    try:
        import torch

        from . import models  # noqa: F401
        from .engine.engine import Engine
        from .sampling.sampler import SamplingParams

        if args.random_weights is not None:
            if not args.config:
                raise ValueError("--random-weights needs --config FILE")
            from .engine.engine import parse_dtype
            from .weights.loader import write_random_model

            with open(args.config, "r", encoding="utf-8") as f:
                raw = json.load(f)
            write_random_model(raw, args.random_weights, args.model, parse_dtype(args.dtype),
                               device="cuda:0" if torch.cuda.is_available() else "cpu")
        chunk = 1 if args.no_batch_prefill else args.chunk
        conc = max(1, args.concurrent)
        eng = Engine.from_model_dir(args.model, dtype=args.dtype, ctx=args.ctx, page_tokens=args.page_tokens,
                                    max_batch_tokens=max(args.max_batch_tokens, conc), chunk=chunk,
                                    max_running=max(conc, 1), kv_fraction=args.kv_fraction)
        plan = eng.model.plan
        cfg = plan.config
        print(f"{torch.cuda.get_device_name(0)} | backend=cuda-sm100a | dtype={args.dtype} | layers={len(plan.layers)} "
              f"embd={plan.hidden_size} heads={getattr(cfg, 'num_attention_heads', '?')}/"
              f"{getattr(cfg, 'num_key_value_heads', '?')} vocab={plan.vocab_size}", file=sys.stderr)
        ids = _parse_prompt(args.prompt, plan.vocab_size, args.seed)
        moe_stats = kernel_times = None
        if args.moe_stats or os.environ.get("LOCUS_MOE_STATS") is not None:   # moe_stats.cpp:23-27
            from .engine.moe_stats import MoeStats

            moe_stats = MoeStats(eng.model)
        if args.kernel_times:
            from . import kernels as K

            kernel_times = K.kernel_times()
            kernel_times.__enter__()
        sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                            repeat_penalty=args.repeat_penalty, frequency_penalty=args.frequency_penalty,
                            presence_penalty=args.presence_penalty, repeat_last_n=args.repeat_last_n)
        if conc == 1:
            print(" ".join(str(t) for t in ids), end="", flush=True)
            eng.on_token = lambda r, t: print(f" {t}", end="", flush=True)
            rid = eng.submit(ids, args.n_tokens, sp, args.seed)
            eng.run_to_completion()
            print()
            r = eng.get(rid)
            if r.error:
                print(f"error: {r.error}", file=sys.stderr)
                return 1
        else:
            rids = [eng.submit(ids, args.n_tokens, sp, args.seed + i) for i in range(conc)]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            eng.run_to_completion()
            torch.cuda.synchronize()
            sec = time.perf_counter() - t0
            total = sum(len(eng.get(r).generated) for r in rids)
            print(f"bench: {conc} seqs, {total} tokens, {sec:.2f}s, {total / sec if sec > 0 else 0.0:.1f} tok/s "
                  f"(batch_decode=1 batch_prefill={0 if args.no_batch_prefill else 1})", file=sys.stderr)
        if args.stats:
            print(json.dumps(eng.stats()), file=sys.stderr)
        if kernel_times is not None:
            kernel_times.__exit__(None, None, None)
            table = kernel_times.table()
            total = sum(ms for _, ms in table.values()) or 1.0
            print("kernel-times: entry point, launches, ms, share (eager steps)", file=sys.stderr)
            for what, (n, ms) in sorted(table.items(), key=lambda kv: -kv[1][1]):
                print(f"kernel-times: {what:<20} {n:>8} {ms:>10.3f} {100.0 * ms / total:>5.1f}%", file=sys.stderr)
        if moe_stats is not None:
            print(moe_stats.report(), file=sys.stderr)
    except Exception as e:  # the reference prints "error: <what>" and returns 1 (run_main.cpp:133-136)
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
