"""Continuous batching through :class:`Engine` on random weights: N requests of P prompt tokens and G
new tokens each, submitted at once; prints generated and total tokens per second.

    python -m locus_b200.tools.serve_bench --requests 64 --prompt 512 --new 128 [--layers 24] [--kv-fraction 0.3]

The model has the layer sizes of Qwen1.5-MoE-A2.7B unless ``--config FILE`` names another config.json.
Everything goes through the public entry point (``Engine.generate``): admission, portions of prompts
beside decode tokens, device sampling, finishing and freeing.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch

A27B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 16, "num_key_value_heads": 16,
    "head_dim": 128, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 8192, "decoder_sparse_step": 1, "num_experts": 60, "num_experts_per_tok": 4,
    "norm_topk_prob": False, "moe_intermediate_size": 1408, "shared_expert_intermediate_size": 5632,
    "intermediate_size": 5632, "qkv_bias": True, "tie_word_embeddings": False, "use_sliding_window": False,
    "mlp_only_layers": [], "hidden_act": "silu", "eos_token_id": -1,
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="serve_bench")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=128)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has")
    ap.add_argument("--config", default="", help="config.json of the model to build (default: A2.7B sizes)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--kv-fraction", type=float, default=0.3)
    ap.add_argument("--max-running", type=int, default=64)
    ap.add_argument("--max-batch-tokens", type=int, default=2048)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--repeats", type=int, default=2)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("serve_bench: no CUDA device", file=sys.stderr)
        return 1
    from .. import models  # noqa: F401
    from ..config import find_arch
    from ..config.base import arch_name_of
    from ..engine.engine import Engine, parse_dtype
    from ..models.model import Model
    from ..weights.loader import RandomSource, load_weights

    raw = dict(A27B)
    if args.config:
        with open(args.config, "r", encoding="utf-8") as f:
            raw = json.load(f)
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    entry = find_arch(arch_name_of(raw))
    cfg = entry.parse_config(raw)
    dt = parse_dtype(args.dtype)
    model = Model(entry.build_plan(cfg), dt, "cuda:0")
    load_weights(model, RandomSource(model, 2, dt, "cuda:0"))
    eng = Engine.from_model(model, kv_fraction=args.kv_fraction, max_running=args.max_running,
                            max_batch_tokens=args.max_batch_tokens, chunk=args.max_batch_tokens)
    print(f"pool of {eng.cache.total_pages() * eng.cache.page_tokens} tokens, {args.max_running} requests at a time",
          file=sys.stderr)
    gen = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, model.plan.vocab_size, (args.prompt,), generator=gen).tolist()
               for _ in range(args.requests)]
    N, P, G = args.requests, args.prompt, args.new
    for rep in range(args.repeats):
        steps0 = eng.timing["steps"]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = eng.generate(prompts, max_new_tokens=G, temperature=args.temperature, seed=1)
        torch.cuda.synchronize()
        dt_s = time.perf_counter() - t0
        assert all(len(o) == G for o in out)
        print(f"{N} x ({P} + {G}) tokens in {dt_s:.3f} s: {N * G / dt_s:.0f} generated tokens/s, "
              f"{N * (P + G) / dt_s:.0f} tokens/s in all, {eng.timing['steps'] - steps0} steps"
              + ("  (first run: graphs are captured)" if rep == 0 else ""))
    assert eng.cache.free_pages() == eng.cache.total_pages()
    return 0


if __name__ == "__main__":
    sys.exit(main())
