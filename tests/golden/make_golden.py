#!/usr/bin/env python3
"""Makes tests/golden/golden.json: logits of the reference's own C++ model code for tiny
random qwen2moe models.

    python tests/golden/make_golden.py /path/to/locus-source [build-dir]

Builds the reference's library on the CPU (CUDA and Vulkan switched off), compiles
ref_harness.cpp against it, writes each case's weights (drawn exactly as the random-weights
mode of the engine draws them: locus_b200.weights.random_init, a function of seed, tensor name
and element index) in the tensor names
and layouts the reference reads (GGUF names, experts stacked [E][I][H]), runs the harness
and stores config, seed, tensor list, tokens and logits.  tests/test_plain.py regenerates the
same weights and compares the plain implementation with these logits.

Model cases: what the reference can express for this architecture -- every layer a mixture of
experts, no renormalisation of the top-k weights, gated shared expert, q/k/v bias, head size
hidden / heads, tied or untied head.

Selection cases: the reference's ``moe_select`` (src/locus/model/llama.cpp:900-980) called directly on
rows of router logits with the options that its qwen2moe loader fixes (renormalised top-k weights:
llama.cpp:966-978; a weight scale; sigmoid scores; a selection bias; group-limited routing); the
picked experts and their weights are stored and compared with ``plain.moe_select``.

It also times the reference's CPU forward on the model cases (batched prefill of the case's tokens
repeated to 128, then 32 greedy decode steps; scalar and avx2 backends) and stores the tokens per
second under "timing": the only speed of the reference for this architecture that can be had here.
"""
import json
import os
import struct
import subprocess
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = [
    {"name": "tiny-A (2 layers, 8 experts top-2, MHA, untied head)", "seed": 0, "tokens_seed": 11, "n_tokens": 12,
     "config": {"num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 4,
                "head_dim": 16, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
                "max_position_embeddings": 256, "decoder_sparse_step": 1, "num_experts": 8, "num_experts_per_tok": 2,
                "norm_topk_prob": False, "moe_intermediate_size": 32, "shared_expert_intermediate_size": 64,
                "intermediate_size": 96, "tie_word_embeddings": False}},
    {"name": "B-like (3 layers all MoE, 12 experts top-3, GQA 6:2, head 32, theta 1e6, tied head)", "seed": 1,
     "tokens_seed": 12, "n_tokens": 20,
     "config": {"num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2,
                "head_dim": 32, "vocab_size": 512, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
                "max_position_embeddings": 512, "decoder_sparse_step": 1, "num_experts": 12, "num_experts_per_tok": 3,
                "norm_topk_prob": False, "moe_intermediate_size": 48, "shared_expert_intermediate_size": 128,
                "intermediate_size": 256, "tie_word_embeddings": True}},
]


SELECT_CASES = [
    # name, E, k, renorm, scoring, groups, groups used, bias, scale, rows
    ("tiny-B router: 12 experts top-3, renormalised", 12, 3, True, "softmax", 1, 1, False, 1.0, 48),
    ("8 experts top-2, renormalised, scale 2.5", 8, 2, True, "softmax", 1, 1, False, 2.5, 32),
    ("60 experts top-4, plain softmax", 60, 4, False, "softmax", 1, 1, False, 1.0, 32),
    ("16 experts top-4, sigmoid scores, selection bias, renormalised", 16, 4, True, "sigmoid", 1, 1, True, 1.0, 32),
    ("32 experts top-6 in 3 of 8 groups, sigmoid, bias", 32, 6, True, "sigmoid", 8, 3, True, 1.5, 32),
    ("24 experts top-5 in 2 of 4 groups, softmax", 24, 5, False, "softmax", 4, 2, False, 1.0, 32),
]

sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from locus_b200.weights.random_init import random_tensor  # noqa: E402


def draw(seed, name, shape, init):
    return random_tensor(seed, name, shape, init, torch.float32)


def select_inputs(case_index, E, rows, has_bias):
    """Router logits (and the bias) of a selection case: seeded draws, some rows with exact ties."""
    logits = random_tensor(100 + case_index, "router_logits", (rows, E), "linear", torch.float32) * 100.0
    logits[1, : min(E, 4)] = 0.75      # a tie among the first experts: the lowest index wins
    logits[2, :] = 0.0                  # everything ties
    bias = random_tensor(100 + case_index, "selection_bias", (E,), "linear", torch.float32) * 10.0 if has_bias else None
    return logits, bias


def tensor_list(cfg):
    """(checkpoint name, shape, init) of every tensor, in the engine's naming."""
    H, nh, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    E, I, Is, V = cfg["num_experts"], cfg["moe_intermediate_size"], cfg["shared_expert_intermediate_size"], cfg["vocab_size"]
    out = [("model.embed_tokens.weight", [V, H], "linear")]
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}"
        out += [(f"{p}.input_layernorm.weight", [H], "norm"), (f"{p}.post_attention_layernorm.weight", [H], "norm")]
        for n, rows in (("q_proj", nh * hd), ("k_proj", nkv * hd), ("v_proj", nkv * hd)):
            out += [(f"{p}.self_attn.{n}.weight", [rows, H], "linear"), (f"{p}.self_attn.{n}.bias", [rows], "bias")]
        out.append((f"{p}.self_attn.o_proj.weight", [H, nh * hd], "linear"))
        out.append((f"{p}.mlp.gate.weight", [E, H], "linear"))
        for e in range(E):
            out += [(f"{p}.mlp.experts.{e}.gate_proj.weight", [I, H], "linear"),
                    (f"{p}.mlp.experts.{e}.up_proj.weight", [I, H], "linear"),
                    (f"{p}.mlp.experts.{e}.down_proj.weight", [H, I], "linear")]
        out += [(f"{p}.mlp.shared_expert.gate_proj.weight", [Is, H], "linear"),
                (f"{p}.mlp.shared_expert.up_proj.weight", [Is, H], "linear"),
                (f"{p}.mlp.shared_expert.down_proj.weight", [H, Is], "linear"),
                (f"{p}.mlp.shared_expert_gate.weight", [1, H], "linear")]
    out.append(("model.norm.weight", [H], "norm"))
    if not cfg["tie_word_embeddings"]:
        out.append(("lm_head.weight", [V, H], "linear"))
    return out


def gguf_tensors(cfg, W):
    """The reference's names and layouts (ggml dims: fastest first)."""
    E = cfg["num_experts"]
    out = [("token_embd.weight", W["model.embed_tokens.weight"])]
    for l in range(cfg["num_hidden_layers"]):
        p, b = f"model.layers.{l}", f"blk.{l}."
        out += [(b + "attn_norm.weight", W[f"{p}.input_layernorm.weight"]),
                (b + "ffn_norm.weight", W[f"{p}.post_attention_layernorm.weight"])]
        for n, gname in (("q_proj", "attn_q"), ("k_proj", "attn_k"), ("v_proj", "attn_v")):
            out += [(b + gname + ".weight", W[f"{p}.self_attn.{n}.weight"]), (b + gname + ".bias", W[f"{p}.self_attn.{n}.bias"])]
        out.append((b + "attn_output.weight", W[f"{p}.self_attn.o_proj.weight"]))
        out.append((b + "ffn_gate_inp.weight", W[f"{p}.mlp.gate.weight"]))
        for n, gname in (("gate_proj", "ffn_gate_exps"), ("up_proj", "ffn_up_exps"), ("down_proj", "ffn_down_exps")):
            out.append((b + gname + ".weight", torch.stack([W[f"{p}.mlp.experts.{e}.{n}.weight"] for e in range(E)])))
        out += [(b + "ffn_gate_shexp.weight", W[f"{p}.mlp.shared_expert.gate_proj.weight"]),
                (b + "ffn_up_shexp.weight", W[f"{p}.mlp.shared_expert.up_proj.weight"]),
                (b + "ffn_down_shexp.weight", W[f"{p}.mlp.shared_expert.down_proj.weight"]),
                (b + "ffn_gate_inp_shexp.weight", W[f"{p}.mlp.shared_expert_gate.weight"])]
    out.append(("output_norm.weight", W["model.norm.weight"]))
    if "lm_head.weight" in W:
        out.append(("output.weight", W["lm_head.weight"]))
    return out


def wstr(f, s):
    b = s.encode()
    f.write(struct.pack("<I", len(b)) + b)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of the reference> [build folder]")
    ref = sys.argv[1]
    build = sys.argv[2] if len(sys.argv) > 2 else tempfile.mkdtemp(prefix="locus_ref_build_")
    subprocess.check_call(["cmake", "-S", ref, "-B", build, "-DCMAKE_BUILD_TYPE=Release",
                           "-DCMAKE_DISABLE_FIND_PACKAGE_CUDAToolkit=ON", "-DCMAKE_DISABLE_FIND_PACKAGE_Vulkan=ON"],
                          stdout=subprocess.DEVNULL)
    subprocess.check_call(["cmake", "--build", build, "--target", "locus", "-j", "8"], stdout=subprocess.DEVNULL)
    lib = None
    for root, _, files in os.walk(build):
        for fn in files:
            if fn in ("liblocus.a", "liblocus.so"):
                lib = os.path.join(root, fn)
    exe = os.path.join(build, "ref_harness")
    subprocess.check_call(["g++", "-std=c++20", "-O2", "-I", os.path.join(ref, "src"), "-I", os.path.join(ref, "tests"),
                           os.path.join(HERE, "ref_harness.cpp"), lib, "-lpthread", "-o", exe])
    golden = {"reference": "garana/locus 0.1.0, LlamaModel::forward on the scalar backend", "cases": []}
    for case in CASES:
        cfg = case["config"]
        tl = tensor_list(cfg)
        W = {n: draw(case["seed"], n, s, i) for n, s, i in tl}
        g = torch.Generator().manual_seed(case["tokens_seed"])
        tokens = torch.randint(0, cfg["vocab_size"], (case["n_tokens"],), generator=g).tolist()
        path = os.path.join(build, "case.bin")
        ku = [("qwen2moe.embedding_length", cfg["hidden_size"]), ("qwen2moe.block_count", cfg["num_hidden_layers"]),
              ("qwen2moe.attention.head_count", cfg["num_attention_heads"]),
              ("qwen2moe.attention.head_count_kv", cfg["num_key_value_heads"]),
              ("qwen2moe.feed_forward_length", cfg["intermediate_size"]),
              ("qwen2moe.context_length", cfg["max_position_embeddings"]),
              ("qwen2moe.expert_count", cfg["num_experts"]), ("qwen2moe.expert_used_count", cfg["num_experts_per_tok"])]
        kf = [("qwen2moe.attention.layer_norm_rms_epsilon", cfg["rms_norm_eps"]), ("qwen2moe.rope.freq_base", cfg["rope_theta"])]
        gt = gguf_tensors(cfg, W)
        with open(path, "wb") as f:
            f.write(struct.pack("<I", len(ku)))
            for k, v in ku:
                wstr(f, k); f.write(struct.pack("<I", v))
            f.write(struct.pack("<I", len(kf)))
            for k, v in kf:
                wstr(f, k); f.write(struct.pack("<f", v))
            f.write(struct.pack("<I", len(gt)))
            for name, t in gt:
                wstr(f, name)
                dims = list(reversed(t.shape))
                f.write(struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims))
                f.write(t.contiguous().numpy().astype("<f4").tobytes())
            f.write(struct.pack("<I", len(tokens)) + struct.pack(f"<{len(tokens)}i", *tokens))
        out = subprocess.check_output([exe, "logits", path]).decode().split("\n")
        n, V = (int(x) for x in out[0].split())
        logits = [[float(x) for x in out[1 + i].split()] for i in range(n)]
        assert all(len(r) == V for r in logits)
        golden["cases"].append({"name": case["name"], "seed": case["seed"], "config": cfg, "tokens": tokens,
                                "tensors": [[n, s, i] for n, s, i in tl], "logits": logits})
        print(f"{case['name']}: {n} positions x {V} logits")
        # the reference's speed on this model: 128 prompt tokens in one batched prefill, 32 decode steps
        long_tokens = (tokens * (128 // len(tokens) + 1))[:128]
        tpath = os.path.join(build, "case_time.bin")
        with open(path, "rb") as f:
            blob = f.read()
        with open(tpath, "wb") as f:
            f.write(blob[: len(blob) - 4 - 4 * len(tokens)])
            f.write(struct.pack("<I", len(long_tokens)) + struct.pack(f"<{len(long_tokens)}i", *long_tokens))
        for backend in ("scalar", "avx2"):
            best = None
            for _ in range(3):
                res = subprocess.check_output([exe, "time", tpath, backend, "32"]).decode().split()
                if res[0] == "unavailable":
                    break
                n_pre, t_pre, n_dec, t_dec = int(res[0]), float(res[1]), int(res[2]), float(res[3])
                cur = {"prefill_tokens": n_pre, "prefill_tok_s": n_pre / t_pre, "decode_tokens": n_dec,
                       "decode_tok_s": n_dec / t_dec}
                if best is None or cur["decode_tok_s"] > best["decode_tok_s"]:
                    best = cur
            if best is not None:
                golden.setdefault("timing", []).append(dict(best, case=case["name"], backend=backend,
                                                            threads=os.cpu_count()))
                print(f"  {backend}: prefill {best['prefill_tok_s']:.0f} tok/s, decode {best['decode_tok_s']:.0f} tok/s")
    golden["select"] = []
    for ci, (name, E, k, renorm, scoring, groups, used, has_bias, scale, rows) in enumerate(SELECT_CASES):
        logits, bias = select_inputs(ci, E, rows, has_bias)
        path = os.path.join(build, "select.bin")
        with open(path, "wb") as f:
            f.write(struct.pack("<7I", E, k, int(renorm), 1 if scoring == "softmax" else 2, groups, used, int(has_bias)))
            f.write(struct.pack("<f", scale))
            if has_bias:
                f.write(bias.numpy().astype("<f4").tobytes())
            f.write(struct.pack("<I", rows))
            f.write(logits.contiguous().numpy().astype("<f4").tobytes())
        lines = [l.split() for l in subprocess.check_output([exe, "select", path]).decode().strip().split("\n")]
        assert len(lines) == rows and all(len(l) == 2 * k for l in lines)
        golden["select"].append({"name": name, "index": ci, "n_experts": E, "top_k": k, "renorm": renorm,
                                 "score_fn": scoring, "n_group": groups, "n_group_used": used, "bias": has_bias,
                                 "scale": scale, "rows": rows, "ids": [[int(x) for x in l[:k]] for l in lines],
                                 "weights": [[float(x) for x in l[k:]] for l in lines]})
        print(f"select: {name}: {rows} rows")
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(golden, f)
    print("wrote", os.path.join(HERE, "golden.json"))


if __name__ == "__main__":
    main()
