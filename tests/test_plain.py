"""The plain implementation itself (no GPU): closed forms of its parts, the architecture's
properties the reference tests (tests/test_moe.cpp:238-845: identical experts are a dense
model, a forced router is that expert, the gate touches only the shared expert), its
sampling helpers, and the golden logits that the reference's own C++ code produced."""
import json
import math
import os
import sys

import pytest
import torch

import plain_qwen2moe as plain
from tiny_configs import make_model_dir, random_tokens

HERE = os.path.dirname(os.path.abspath(__file__))


def test_rmsnorm_softmax_silu_closed_forms():
    x = torch.tensor([[3.0, 4.0]])
    out = plain.rmsnorm(x, torch.tensor([1.0, 2.0]), 0.0)
    assert torch.allclose(out, torch.tensor([[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]]))
    p = plain.softmax(torch.tensor([1.0, 1.0, 1.0, 1.0]))
    assert torch.allclose(p, torch.full((4,), 0.25))
    assert torch.allclose(plain.silu_mul(torch.tensor([0.0, 20.0]), torch.tensor([5.0, 2.0])),
                          torch.tensor([0.0, 40.0]), atol=1e-6)


def test_rope_identity_at_zero_norm_kept_and_relative():
    x = torch.randn(3, 2, 16, dtype=torch.float64)
    assert torch.equal(plain.rope_half_split(x[:1], torch.tensor([0]), 10000.0), x[:1])
    y = plain.rope_half_split(x, torch.tensor([5, 17, 400]), 10000.0)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # the score of a rotated pair depends only on the distance of the positions
    q, k = torch.randn(1, 1, 16, dtype=torch.float64), torch.randn(1, 1, 16, dtype=torch.float64)
    s = lambda a, b: float((plain.rope_half_split(q, torch.tensor([a]), 1e6) * plain.rope_half_split(k, torch.tensor([b]), 1e6)).sum())
    assert abs(s(10, 3) - s(107, 100)) < 1e-9
    # pairs are (i, i + half), not (2i, 2i + 1)
    e = torch.zeros(1, 1, 4, dtype=torch.float64)
    e[0, 0, 0] = 1.0
    r = plain.rope_half_split(e, torch.tensor([1]), 10000.0)[0, 0]
    assert abs(float(r[0]) - math.cos(1.0)) < 1e-12 and abs(float(r[2]) - math.sin(1.0)) < 1e-12 and float(r[1]) == 0


def test_attention_is_causal_grouped_and_windowed():
    T, nh, nkv, hd = 6, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, dtype=torch.float64) for n in (nh, nkv, nkv))
    o = plain.attention(q, k, v)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 3], v[0, 1])  # one key: its value; head 3 -> kv 1
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, 9.0
    assert torch.allclose(plain.attention(q, k2, v2)[:4], o[:4])  # the future does not matter
    w1 = plain.attention(q, k, v, window=1)
    assert torch.allclose(w1, v.repeat_interleave(2, dim=1))  # window 1: each token sees itself
    w3 = plain.attention(q, k, v, window=3)
    assert torch.allclose(w3[:3], o[:3]) and not torch.allclose(w3[5], o[5])


def test_moe_select_order_ties_and_renorm():
    r = torch.tensor([0.1, 2.0, 0.1, 1.0, 0.1])
    ids, w = plain.moe_select(r, 3, False)
    assert ids == [1, 3, 0]  # the tie among 0, 2, 4 goes to the lowest index
    p = plain.softmax(r)
    assert all(abs(float(a) - float(p[i])) < 1e-7 for a, i in zip(w, ids))
    ids2, w2 = plain.moe_select(r, 3, True)
    assert ids2 == ids and abs(sum(float(x) for x in w2) - 1.0) < 1e-6


def _weights(name, tmp_path):
    d = make_model_dir(tmp_path, name, torch.float32)
    return plain.load_folder(d)


def test_identical_experts_are_a_dense_model(tmp_path):
    cfg, W = _weights("B", tmp_path)
    cfg["norm_topk_prob"] = True
    p = "model.layers.1.mlp"
    for e in range(1, cfg["num_experts"]):
        for n in ("gate_proj", "up_proj", "down_proj"):
            W[f"{p}.experts.{e}.{n}.weight"] = W[f"{p}.experts.0.{n}.weight"]
    h = torch.randn(5, cfg["hidden_size"], dtype=torch.float64)
    Wd = {k: v.double() for k, v in W.items()}
    cfg2 = dict(cfg, shared_expert_intermediate_size=0)
    out = plain.moe_block(h, Wd, p, cfg2)
    dense = plain.swiglu_mlp(h, Wd[f"{p}.experts.0.gate_proj.weight"], Wd[f"{p}.experts.0.up_proj.weight"],
                             Wd[f"{p}.experts.0.down_proj.weight"])
    assert torch.allclose(out, dense, atol=1e-12)


def test_forced_router_is_that_expert_and_gate_touches_only_the_shared_expert(tmp_path):
    cfg, W = _weights("A", tmp_path)
    Wd = {k: v.double() for k, v in W.items()}
    p = "model.layers.0.mlp"
    h = torch.randn(4, cfg["hidden_size"], dtype=torch.float64)
    nos = dict(cfg, shared_expert_intermediate_size=0, num_experts_per_tok=1)
    Wd[f"{p}.gate.weight"] = torch.zeros_like(Wd[f"{p}.gate.weight"])  # all logits tie: the lowest index, expert 0
    out = plain.moe_block(h, Wd, p, nos)
    e0 = plain.swiglu_mlp(h, *(Wd[f"{p}.experts.0.{n}.weight"] for n in ("gate_proj", "up_proj", "down_proj")))
    assert torch.allclose(out, e0 / cfg["num_experts"], atol=1e-12)  # p = 1/E without renormalisation
    base = plain.moe_block(h, Wd, p, cfg)
    Wg = dict(Wd)
    Wg[f"{p}.shared_expert_gate.weight"] = Wd[f"{p}.shared_expert_gate.weight"] + 3.0
    assert not torch.allclose(plain.moe_block(h, Wg, p, cfg), base)
    Wz = dict(Wg)
    Wz[f"{p}.shared_expert.down_proj.weight"] = torch.zeros_like(Wd[f"{p}.shared_expert.down_proj.weight"])
    Wz0 = dict(Wd)
    Wz0[f"{p}.shared_expert.down_proj.weight"] = Wz[f"{p}.shared_expert.down_proj.weight"]
    assert torch.equal(plain.moe_block(h, Wz, p, cfg), plain.moe_block(h, Wz0, p, cfg))


def test_forward_float32_close_to_float64_and_window_matters(tmp_path):
    for name in "ABC":
        cfg, W = _weights(name, tmp_path)
        toks = random_tokens(40, cfg["vocab_size"], 1)
        a, b = plain.forward(cfg, W, toks, torch.float32), plain.forward(cfg, W, toks, torch.float64)
        assert float((a.double() - b).abs().max()) < 1e-4 * float(b.abs().max())
        assert torch.allclose(plain.forward(cfg, W, toks[:17], torch.float64), b[:17], atol=1e-12)  # causal
    cfg, W = _weights("C", tmp_path)
    toks = random_tokens(40, cfg["vocab_size"], 1)
    full = plain.forward(dict(cfg, use_sliding_window=False), W, toks, torch.float64)
    win = plain.forward(cfg, W, toks, torch.float64)
    assert torch.allclose(full[:24], win[:24], atol=1e-12) and not torch.allclose(full[30:], win[30:], atol=1e-6)


def test_sampling_helpers():
    logits = torch.tensor([1.0, 3.0, 3.0, -2.0, 0.5])
    assert plain.argmax(logits) == 1
    d = plain.kept_distribution(logits, 1.0)
    assert abs(sum(d.values()) - 1.0) < 1e-12 and len(d) == 5
    assert set(plain.kept_distribution(logits, 1.0, top_k=2)) == {1, 2}
    assert set(plain.kept_distribution(logits, 1.0, top_p=0.5)) == {1, 2}
    assert set(plain.kept_distribution(logits, 1.0, top_p=0.3)) == {1}
    assert set(plain.kept_distribution(logits, 1.0, min_p=0.1)) == {0, 1, 2}
    pen = plain.apply_penalties(logits, [1, 1, 3], 2.0, 0.5, 0.25, 64)
    assert float(pen[1]) == 3.0 / 2 - (0.5 * 2 + 0.25) and float(pen[3]) == -2.0 * 2 - 0.75 and float(pen[0]) == 1.0
    assert torch.equal(plain.apply_penalties(logits, [1], 2.0, 0, 0, 0), logits)  # empty window


def test_golden_logits_of_the_reference():
    """tests/golden/ holds logits computed by the reference's own C++ model code (compiled
    on the CPU by tests/golden/make_golden.py) for seeded tiny models; see its README."""
    path = os.path.join(HERE, "golden", "golden.json")
    if not os.path.isfile(path):
        pytest.skip("no golden file committed")
    with open(path) as f:
        golden = json.load(f)
    from locus_b200.weights.random_init import random_tensor

    for case in golden["cases"]:
        cfg = case["config"]
        W = {name: random_tensor(case["seed"], name, shape, init, torch.float32) for name, shape, init in case["tensors"]}
        ref = torch.tensor(case["logits"], dtype=torch.float64)
        got = plain.forward(cfg, W, case["tokens"], torch.float32)
        scale = float(ref.abs().max())
        assert float((got.double() - ref).abs().max()) <= 2e-5 * scale, case["name"]


def test_golden_selections_of_the_reference():
    """The reference's own moe_select (src/locus/model/llama.cpp:900-980), called directly by
    tests/golden/ref_harness.cpp with the options its qwen2moe loader fixes: renormalised weights
    (tiny-B's norm_topk_prob), a weight scale, sigmoid scores, a selection bias, groups."""
    path = os.path.join(HERE, "golden", "golden.json")
    if not os.path.isfile(path):
        pytest.skip("no golden file committed")
    with open(path) as f:
        golden = json.load(f)
    sys.path.insert(0, os.path.join(HERE, "golden"))
    from make_golden import select_inputs

    assert len(golden["select"]) >= 6
    for case in golden["select"]:
        E, k = case["n_experts"], case["top_k"]
        logits, bias = select_inputs(case["index"], E, case["rows"], case["bias"])
        for r in range(case["rows"]):
            ids, w = plain.moe_select(logits[r], k, case["renorm"], case["scale"], case["score_fn"], bias,
                                      case["n_group"], case["n_group_used"])
            assert ids == case["ids"][r], (case["name"], r)
            ref = torch.tensor(case["weights"][r], dtype=torch.float64)
            got = torch.tensor([float(x) for x in w], dtype=torch.float64)
            assert float((got - ref).abs().max()) <= 2e-6 * max(1.0, float(ref.abs().max())), (case["name"], r)
            if case["renorm"]:
                assert abs(float(got.sum()) - case["scale"]) < 1e-5
