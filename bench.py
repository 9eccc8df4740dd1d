#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second of Qwen1.5-MoE-A2.7B layer
sizes (random weights, bfloat16) at batch 8 and context 4096, with the prefill of one
2,048-token prompt and decode at batch 1 and 64 beside it.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  ``value``: decoded tokens per second of K decode steps timed on the
device with CUDA events (token ids are synthetic; every step reads far more than the L2
holds: all weights it uses plus the cache of the live requests).  ``e2e``: the same through
the Python entry point (``Engine.step``): host token ids in through pinned memory, sampled
ids back to the host, every step.  ``prefill``: one 2,048-token prompt in one step.
``roofline``: bytes a decode step has to read / its time, against the measured copy
bandwidth.  The engine is a single-GPU engine: ``--gpus N`` with N > 1 prints a line saying
so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

A27B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 16, "num_key_value_heads": 16,
    "head_dim": 128, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 8192, "decoder_sparse_step": 1, "num_experts": 60, "num_experts_per_tok": 4,
    "norm_topk_prob": False, "moe_intermediate_size": 1408, "shared_expert_intermediate_size": 5632,
    "intermediate_size": 5632, "qkv_bias": True, "tie_word_embeddings": False, "use_sliding_window": False,
    "mlp_only_layers": [], "hidden_act": "silu", "eos_token_id": -1,
}
MODEL_LAYERS = 24
PREFILL_TOKENS = 2048


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 8:
                        continue
                    try:
                        sm.append(float(c[0])); mx.append(float(c[1]))
                    except ValueError:
                        continue
                    for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[4:8]):
                        if v.lower().startswith("active"):
                            reasons.add(name)
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        return out


def linear_params_per_token(cfg, n_layers):
    """Weights one token multiplies with, per layer kinds, and the head."""
    H, hd = cfg["hidden_size"], cfg["head_dim"]
    q, kv = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    attn = (q + 2 * kv) * H + H * q
    router = cfg["num_experts"] * H + H
    expert = 3 * cfg["moe_intermediate_size"] * H
    shared = 3 * cfg["shared_expert_intermediate_size"] * H
    per_layer = attn + router + cfg["num_experts_per_tok"] * expert + shared
    return n_layers * per_layer, attn, router, expert, shared


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL_LAYERS, help="fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip cannot install the reference (a C++/CMake project: neither setup.py nor pyproject.toml); "
                          "its CUDA backend is an sm_50 per-call matvec offload that needs a GGUF file with a tokenizer"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    K_steps, W = args.steps, max(3, args.warmup)

    import torch

    import locus_b200.kernels as K
    import locus_b200.models  # noqa: F401
    from locus_b200.cache import CacheManager
    from locus_b200.config import find_arch
    from locus_b200.engine.engine import Engine
    from locus_b200.engine.scheduler import SchedulerConfig
    from locus_b200.engine.step import ModelRunner, StepEntry
    from locus_b200.models.model import Model
    from locus_b200.sampling.sampler import GREEDY, Sampler
    from locus_b200.weights.loader import RandomSource, load_weights

    dev = "cuda:0"
    torch.cuda.set_device(0)
    raw = dict(A27B, num_hidden_layers=args.layers)
    if args.context > raw["max_position_embeddings"]:
        raw["max_position_embeddings"] = args.context  # a longer synthetic context than the model was trained for
    entry = find_arch("Qwen2MoeForCausalLM")
    cfg = entry.parse_config(raw)
    t0 = time.time()
    model = Model(entry.build_plan(cfg), torch.bfloat16, dev)
    load_weights(model, RandomSource(model, 2, torch.bfloat16, dev))
    torch.cuda.synchronize()
    print(f"[bench] {args.layers}-layer model, {model.param_bytes() / 1e9:.1f} GB of weights, built in {time.time() - t0:.0f}s",
          file=sys.stderr, flush=True)

    P = 64
    ctx = args.context
    max_b = args.batch if args.no_points else max(64, args.batch)
    n_pages = max(max_b * (-(-ctx // P)), -(-PREFILL_TOKENS // P))
    cache = CacheManager(model.cache_needs(), page_tokens=P, n_pages=n_pages, n_state_slots=max_b,
                         max_seq_tokens=max(ctx, PREFILL_TOKENS),
                         dtype=torch.bfloat16, device=dev)
    for g in cache.groups:  # synthetic cache contents for the steps that start from an adopted context
        flat = g.pool.view(-1)
        step = 1 << 28
        for i in range(0, flat.numel(), step):
            flat[i : i + step].uniform_(-1.0, 1.0)
    runner = ModelRunner(model, cache, max_tokens=PREFILL_TOKENS, max_segments=max_b, max_wanted=max_b, use_graphs=True)
    sampler = Sampler(dev, max_b)
    gen = torch.Generator().manual_seed(2)
    V = cfg.vocab_size
    pk = peaks()

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---- prefill: one 2,048-token prompt in one step
    prompt = torch.randint(0, V, (PREFILL_TOKENS,), generator=gen).tolist()
    times = []
    for i in range(2 + 3):
        seq = cache.open("prefill")
        assert cache.ensure_capacity(seq, PREFILL_TOKENS)
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        runner.step([StepEntry(seq, prompt, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(a.elapsed_time(b))
        cache.release(seq)
    pre_ms = min(times)
    lin, attn_p, router_p, expert_p, shared_p = linear_params_per_token(raw, args.layers)
    T = PREFILL_TOKENS
    flops = 2.0 * lin * T + 2.0 * V * cfg.hidden_size \
        + args.layers * 2.0 * cfg.num_attention_heads * cfg.head_dim * T * T  # causal QK^T and PV
    prefill = {"value": T / (pre_ms / 1e3), "tokens": T, "ms": pre_ms,
               "frac": flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), "tflops": flops / (pre_ms / 1e3) / 1e12}
    print(f"[bench] prefill {T} tokens: {pre_ms:.2f} ms", file=sys.stderr, flush=True)

    # ---- decode steps on the device
    def decode_run(B, steps, warm, sample_clocks=False):
        seqs = [cache.open(f"d{B}_{i}") for i in range(B)]
        start = ctx - (steps + warm) - 1
        for s in seqs:
            assert cache.adopt(s, start)
        toks = torch.randint(0, V, (steps + warm, B), generator=gen).tolist()
        params, zeros = [GREEDY] * B, [0] * B

        def one(i):
            for s in seqs:
                assert cache.ensure_capacity(s, 1)
            logits = runner.step([StepEntry(s, [toks[i][j]], [0]) for j, s in enumerate(seqs)])
            sampler.sample_device(logits, params, zeros, zeros)

        for i in range(warm):
            one(i)
        torch.cuda.synchronize()
        clocks = ClockSampler()
        if sample_clocks:
            clocks.start()
            time.sleep(0.3)
        l0, k0 = runner.launch_counter, K.launches
        a, b = ev(), ev()
        a.record()
        for i in range(warm, warm + steps):
            one(i)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        launches = (runner.launch_counter - l0) + steps  # + the sampling kernel of every step
        ck = clocks.stop() if sample_clocks else None
        # distinct experts of one more step, counted from the router's picks
        picked = []
        for part in model.all_parts():
            if hasattr(part, "observer"):
                part.observer = lambda prefix, ids, wts: picked.append(int(torch.unique(ids).numel()))
        runner.use_graphs = False
        for s in seqs:
            assert cache.ensure_capacity(s, 1)
        runner.step([StepEntry(s, [toks[0][j]], [0]) for j, s in enumerate(seqs)])
        runner.use_graphs = True
        for part in model.all_parts():
            if hasattr(part, "observer"):
                part.observer = None
        n_ctx = seqs[0].n_tokens
        for s in seqs:
            cache.release(s)
        el = 2
        weight_bytes = el * (args.layers * (attn_p + router_p + shared_p) + sum(picked) * expert_p + V * cfg.hidden_size)
        kv_bytes = B * n_ctx * cache.bytes_per_token()
        return ms, launches, ck, weight_bytes, kv_bytes, (sum(picked) / max(1, len(picked)))

    ms8, launches, clocks, wbytes, kvbytes, experts_hit = decode_run(args.batch, K_steps, W, sample_clocks=True)
    value = args.batch / (ms8 / 1e3)
    achieved = (wbytes + kvbytes) / (ms8 / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                "weight_gb": wbytes / 1e9, "kv_gb": kvbytes / 1e9, "experts_per_layer": experts_hit, "peaks": pk["source"]}
    print(f"[bench] decode batch {args.batch}: {ms8:.3f} ms/step", file=sys.stderr, flush=True)
    points = {}
    if not args.no_points:
        for B in (1, 64):
            steps_b = max(8, K_steps // 2)
            ms, _, _, _, _, _ = decode_run(B, steps_b, W)
            points[f"decode_b{B}"] = B / (ms / 1e3)
            print(f"[bench] decode batch {B}: {ms:.3f} ms/step", file=sys.stderr, flush=True)

    # ---- end to end through Engine.step: host ids in, sampled ids out, every step
    e2e = None
    if not args.no_e2e:
        B = args.batch
        eng = Engine(runner, cache, sampler, max_positions=cfg.max_position_embeddings,
                     config=SchedulerConfig(max_batch_tokens=PREFILL_TOKENS, chunk=PREFILL_TOKENS, max_running=max_b,
                                            decode_headroom=16))
        # Requests that finish their prompt early decode while the others still prefill; nobody may
        # reach its length limit (or the context limit) inside the timed steps, or the batch would shrink.
        prefill_steps = -(-(B * ctx) // PREFILL_TOKENS) + 2
        n_new = K_steps + W + prefill_steps + 2
        n_prompt = ctx - n_new - 1
        rids = [eng.submit(torch.randint(0, V, (n_prompt,), generator=gen).tolist(), n_new, GREEDY, 0)
                for _ in range(B)]
        while any(eng.get(r).n_fed < n_prompt for r in rids):
            eng.step()
        for _ in range(W):
            eng.step()
        h0, s0, d0 = runner.stats["h2d_bytes"], sampler.h2d_bytes, sampler.d2h_bytes
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for _ in range(K_steps):
            eng.step()
        torch.cuda.synchronize()
        sec = time.perf_counter() - t1
        assert all(eng.get(r).status.value == "running" and len(eng.get(r).generated) >= K_steps + W for r in rids), \
            "a request left the batch inside the timed steps"
        e2e = {"value": B * K_steps / sec, "unit": "tokens/s",
               "h2d_bytes_per_step": (runner.stats["h2d_bytes"] - h0 + sampler.h2d_bytes - s0) / K_steps,
               "d2h_bytes_per_step": (sampler.d2h_bytes - d0) / K_steps, "ms_per_step": sec * 1e3 / K_steps}
        eng.run_to_completion()
        print(f"[bench] end to end batch {B}: {sec * 1e3 / K_steps:.3f} ms/step", file=sys.stderr, flush=True)

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen1.5-MoE-A2.7B layer sizes, bf16, context {ctx})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K_steps, "warmup": W, "ms_per_step": ms8,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": "Qwen1.5-MoE-A2.7B layer sizes, random weights seed 2", "layers": args.layers,
            "layers_of_model": MODEL_LAYERS, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "vocab": V, "experts": cfg.num_experts,
            "top_k": cfg.num_experts_per_tok, "moe_intermediate": cfg.moe_intermediate_size,
            "shared_intermediate": cfg.shared_expert_intermediate_size, "global_batch": args.batch, "seq_len": ctx,
            "parallelism": "1 GPU", "page_tokens": P,
            "l2": "no flush: every step reads its weights and cache, far more than the 126 MB L2",
            "cache_fill": "device-timed steps start from an adopted synthetic cache; e2e prompts are prefilled",
        },
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e, "gpu_launches": launches,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
