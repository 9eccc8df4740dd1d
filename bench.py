#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second of Qwen1.5-MoE-A2.7B layer
sizes (random weights, bfloat16) at batch 8 and context 4096, with the prefill of one
2,048-token prompt and decode at batch 1 and 64 beside it.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config a27b|57b-a14b] [--dtype bf16|fp32] [--trace]

With no options: the headline configuration.  ``--config 57b-a14b``: the Qwen2-57B-A14B layer sizes
(28 layers, 114.8 GB of weights), decode from 8,192-token contexts and a 32,768-token prefill in portions
of 2,048.  ``--dtype fp32``: the true 32-bit path (CUDA-core products, float32 cache).  ``--trace``: adds
a mixed continuous-batching trace through ``Engine`` (32 requests, prompts uniform in [16, 4096], decode
lengths uniform in [1, 512], one arrival every 4 steps, portions of 512 tokens).

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
Q57B = dict(A27B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
            max_position_embeddings=32768, num_experts=64, num_experts_per_tok=8, moe_intermediate_size=2560,
            shared_expert_intermediate_size=20480, intermediate_size=18944)
# name -> raw config, weight seed, context the decode steps end at (0: prompt + steps), prompt length the decode
# steps start from (0: so that they end at the context), prefill tokens, name in the metric
CONFIGS = {
    "a27b": dict(raw=A27B, seed=2, context=4096, prompt=0, prefill=2048, name="Qwen1.5-MoE-A2.7B"),
    "57b-a14b": dict(raw=Q57B, seed=4, context=0, prompt=8192, prefill=32768, name="Qwen2-57B-A14B", step_tokens=8192),
}
# Most tokens of one step: a longer prefill runs in portions of this size.  Every step streams all experts' weights,
# so a model with large experts gains from longer portions (the 57B sizes' 32,768-token prompt: 1,481 ms in portions of
# 2,048, 1,335 ms of 4,096, 1,268 ms of 8,192); a configuration may name its own, --step-tokens overrides.
STEP_TOKENS = 2048


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
    ap.add_argument("--config", default="a27b", choices=sorted(CONFIGS))
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=0, help="context at which the decode steps end")
    ap.add_argument("--trace", action="store_true", help="add the mixed continuous-batching trace through Engine")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--step-tokens", type=int, default=0, help="most tokens of a step (default: the configuration's)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a C++/CMake project that pip cannot install (no setup.py or pyproject.toml); "
                          "built with CMake, its only path for this architecture is the float32 CPU forward, measured at "
                          "580 to 8,400 decoded tokens/s on models of 0.2 to 1.6 M parameters (tests/golden/golden.json), "
                          "which cannot run 8 prompts of 4,070 tokens at 14.3 B parameters inside a benchmark run"}))
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
    conf = CONFIGS[args.config]
    STEP_TOKENS = args.step_tokens or conf.get("step_tokens", globals()["STEP_TOKENS"])
    MODEL_LAYERS = conf["raw"]["num_hidden_layers"]
    PREFILL_TOKENS = conf["prefill"]
    args.layers = args.layers or MODEL_LAYERS
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    el = 2 if args.dtype == "bf16" else 4
    # the context at which the timed decode steps end: given, or the configuration's, or its prompt length plus the steps
    ctx = args.context or conf["context"] or conf["prompt"] + K_steps + W + 1
    raw = dict(conf["raw"], num_hidden_layers=args.layers)
    if max(ctx, PREFILL_TOKENS) > raw["max_position_embeddings"]:
        raw["max_position_embeddings"] = max(ctx, PREFILL_TOKENS)  # a longer synthetic context than the model was trained for
    if args.trace:
        raw["max_position_embeddings"] = max(raw["max_position_embeddings"], 8192)
    entry = find_arch("Qwen2MoeForCausalLM")
    cfg = entry.parse_config(raw)
    t0 = time.time()
    model = Model(entry.build_plan(cfg), dtype, dev)
    load_weights(model, RandomSource(model, conf["seed"], dtype, dev))
    torch.cuda.synchronize()
    print(f"[bench] {args.layers}-layer model, {model.param_bytes() / 1e9:.1f} GB of weights, built in {time.time() - t0:.0f}s",
          file=sys.stderr, flush=True)

    P = 64
    max_b = args.batch if args.no_points else max(64, args.batch)
    pages_wanted = max(max_b * (-(-ctx // P)), -(-PREFILL_TOKENS // P))
    # the cache takes what the device has left after the weights and the step's buffers; if the largest batch's
    # contexts do not fit, the points that do not fit are left out and named
    per_page = CacheManager(model.cache_needs(), page_tokens=P, n_pages=0, n_state_slots=1, max_seq_tokens=1, dtype=dtype,
                            allocate_device=False).bytes_per_token() * P
    free, _ = torch.cuda.mem_get_info()
    n_pages = min(pages_wanted, int((free - (12 << 30)) // per_page))
    TRACE_CONTEXT = 8192   # the trace's requests hold up to 4,096 + 512 tokens
    max_seq = max(ctx, PREFILL_TOKENS, TRACE_CONTEXT if args.trace else 0)
    cache = CacheManager(model.cache_needs(), page_tokens=P, n_pages=n_pages, n_state_slots=max_b,
                         max_seq_tokens=max_seq, dtype=dtype, device=dev)
    for g in cache.groups:  # synthetic cache contents for the steps that start from an adopted context
        flat = g.pool.view(-1)
        step = 1 << 28
        for i in range(0, flat.numel(), step):
            flat[i : i + step].uniform_(-1.0, 1.0)
    runner = ModelRunner(model, cache, max_tokens=STEP_TOKENS, max_segments=max_b, max_wanted=max_b, use_graphs=True)
    sampler = Sampler(dev, max_b)
    gen = torch.Generator().manual_seed(2)
    V = cfg.vocab_size
    pk = peaks()

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def checked(what):
        """After a timed region (the read synchronises, so never inside one): a kernel that gave up a bounded wait
        ended with invalid output, and a number measured on it means nothing."""
        try:
            runner.check_device_errors()
        except RuntimeError as e:
            raise SystemExit(f"bench.py: {what}: {e}")

    # ---- prefill: one prompt of PREFILL_TOKENS tokens, in one step or in portions of STEP_TOKENS
    prompt = torch.randint(0, V, (PREFILL_TOKENS,), generator=gen).tolist()
    portions = [(a, min(STEP_TOKENS, PREFILL_TOKENS - a)) for a in range(0, PREFILL_TOKENS, STEP_TOKENS)]
    times = []
    for i in range(2 + 3 if len(portions) == 1 else 1 + 2):
        seq = cache.open("prefill")
        assert cache.ensure_capacity(seq, PREFILL_TOKENS)
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for p0, n in portions:
            runner.step([StepEntry(seq, prompt[p0 : p0 + n], [n - 1] if p0 + n == PREFILL_TOKENS else [])])
        b.record()
        torch.cuda.synchronize()
        if i >= (2 if len(portions) == 1 else 1):
            times.append(a.elapsed_time(b))
        cache.release(seq)
    checked("prefill")
    pre_ms = min(times)
    lin, attn_p, router_p, expert_p, shared_p = linear_params_per_token(raw, args.layers)
    T = PREFILL_TOKENS
    flops = 2.0 * lin * T + 2.0 * V * cfg.hidden_size \
        + args.layers * 2.0 * cfg.num_attention_heads * cfg.head_dim * T * T  # causal QK^T and PV
    # float32 runs on the CUDA cores: 128 FMA lanes per SM
    peak_flops = pk["bf16_tflops"] * 1e12 if args.dtype == "bf16" else 148 * 128 * 2 * 1.965e9
    prefill = {"value": T / (pre_ms / 1e3), "tokens": T, "ms": pre_ms, "portions": len(portions),
               "frac": flops / (pre_ms / 1e3) / peak_flops, "tflops": flops / (pre_ms / 1e3) / 1e12,
               "peak_tflops": peak_flops / 1e12}
    print(f"[bench] prefill {T} tokens: {pre_ms:.2f} ms", file=sys.stderr, flush=True)

    # ---- decode steps on the device
    def decode_run(B, steps, warm, sample_clocks=False):
        start = ctx - (steps + warm) - 1
        if B * (-(-ctx // P)) > cache.total_pages():
            return None
        seqs = [cache.open(f"d{B}_{i}") for i in range(B)]
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
        checked(f"decode at batch {B}")
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
        weight_bytes = el * (args.layers * (attn_p + router_p + shared_p) + sum(picked) * expert_p + V * cfg.hidden_size)
        kv_bytes = B * n_ctx * cache.bytes_per_token()
        return ms, launches, ck, weight_bytes, kv_bytes, (sum(picked) / max(1, len(picked)))

    main_run = decode_run(args.batch, K_steps, W, sample_clocks=True)
    if main_run is None:
        raise SystemExit(f"bench.py: the cache of {args.batch} requests of {ctx} tokens does not fit beside the weights")
    ms8, launches, clocks, wbytes, kvbytes, experts_hit = main_run
    value = args.batch / (ms8 / 1e3)
    achieved = (wbytes + kvbytes) / (ms8 / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                "weight_gb": wbytes / 1e9, "kv_gb": kvbytes / 1e9, "experts_per_layer": experts_hit, "peaks": pk["source"]}
    print(f"[bench] decode batch {args.batch}: {ms8:.3f} ms/step", file=sys.stderr, flush=True)
    points = {}
    if not args.no_points:
        for B in (1, 64):
            steps_b = max(8, K_steps // 2)
            run = decode_run(B, steps_b, W)
            if run is None:
                points[f"decode_b{B}"] = None   # this batch's cache does not fit beside the weights (named in config)
                continue
            ms, _, _, wb, kb, _ = run
            points[f"decode_b{B}"] = B / (ms / 1e3)
            points[f"decode_b{B}_hbm_frac"] = (wb + kb) / (ms / 1e3) / 1e9 / pk["hbm_gbs"]
            print(f"[bench] decode batch {B}: {ms:.3f} ms/step", file=sys.stderr, flush=True)

    # ---- end to end through Engine.step: host ids in, sampled ids out, every step
    e2e = None
    if not args.no_e2e:
        B = args.batch
        eng = Engine(runner, cache, sampler, max_positions=cfg.max_position_embeddings,
                     config=SchedulerConfig(max_batch_tokens=STEP_TOKENS, chunk=STEP_TOKENS, max_running=max_b,
                                            decode_headroom=16))
        # Requests that finish their prompt early decode while the others still prefill; nobody may
        # reach its length limit (or the context limit) inside the timed steps, or the batch would shrink.
        prefill_steps = -(-(B * ctx) // STEP_TOKENS) + 2
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
        eng.run_to_completion()   # reads the device error words at its end
        print(f"[bench] end to end batch {B}: {sec * 1e3 / K_steps:.3f} ms/step", file=sys.stderr, flush=True)

    # ---- a mixed continuous-batching trace through Engine: arrivals while others decode, portions of 512
    trace = None
    if args.trace:
        n_req, arrive_every, chunk = 32, 4, 512
        eng = Engine(runner, cache, sampler, max_positions=cfg.max_position_embeddings,
                     config=SchedulerConfig(max_batch_tokens=STEP_TOKENS, chunk=chunk, max_running=max_b, decode_headroom=16))
        tg = torch.Generator().manual_seed(conf["seed"] + 100)
        lens = torch.randint(16, 4097, (n_req,), generator=tg).tolist()
        news = torch.randint(1, 513, (n_req,), generator=tg).tolist()
        prompts = [torch.randint(0, V, (n,), generator=tg).tolist() for n in lens]
        steps0 = eng.timing["steps"]
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        rids, n_steps = [], 0
        while len(rids) < n_req or eng.has_runnable_work():
            if len(rids) < n_req and n_steps % arrive_every == 0:
                rids.append(eng.submit(prompts[len(rids)], news[len(rids)], GREEDY, 0))
            eng.step()
            n_steps += 1
        torch.cuda.synchronize()
        sec = time.perf_counter() - t1
        eng.check_device_errors()
        recs = [eng.get(r) for r in rids]
        bad = [(r.id, r.status.value, r.error, len(r.generated), n) for r, n in zip(recs, news)
               if r.status.value != "done" or len(r.generated) != n]
        if bad:
            raise SystemExit(f"bench.py: trace requests failed: {bad[:4]}")
        gen_tokens = sum(news)
        trace = {"requests": n_req, "prompt_tokens": sum(lens), "generated_tokens": gen_tokens, "steps": n_steps,
                 "seconds": sec, "tokens_per_s": (sum(lens) + gen_tokens) / sec, "generated_per_s": gen_tokens / sec,
                 "chunk": chunk, "arrival_every_steps": arrive_every, "preemptions": eng.sched.counters["preemptions"]}
        for r in rids:
            eng.release(r)
        print(f"[bench] trace: {n_steps} steps in {sec:.2f} s", file=sys.stderr, flush=True)

    dt_name = "bf16" if args.dtype == "bf16" else "fp32"
    line = {
        "metric": f"decode tok/s at batch {args.batch} ({conf['name']} layer sizes, {dt_name}, context {ctx})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K_steps, "warmup": W, "ms_per_step": ms8,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dt_name, "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": f"{conf['name']} layer sizes, random weights seed {conf['seed']}", "layers": args.layers,
            "layers_of_model": MODEL_LAYERS, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "vocab": V, "experts": cfg.num_experts,
            "top_k": cfg.num_experts_per_tok, "moe_intermediate": cfg.moe_intermediate_size,
            "shared_intermediate": cfg.shared_expert_intermediate_size, "global_batch": args.batch, "seq_len": ctx,
            "parallelism": "1 GPU", "page_tokens": P, "prefill_tokens": PREFILL_TOKENS, "cache_tokens": n_pages * P,
            "l2": "no flush: every step reads its weights and cache, far more than the 126 MB L2",
            "cache_fill": "device-timed steps start from an adopted synthetic cache; e2e prompts are prefilled",
        },
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e, "gpu_launches": launches,
        "clocks": clocks,
    }
    if trace is not None:
        line["trace"] = trace
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
