"""Generality of the cache, of the step's work lists and of the router, with pieces that exist only in this
file: a mixer that keeps ONE row per token (keys only, no values) and a per-token field beside it, and that
plans its own tiles of queries for every step (a ``StepPlan`` whose lists ride in the step's buffer);
and the framework's sparse mixture of experts with sigmoid scores, a selection bias and group-limited routing.
Nothing under ``locus_b200`` knows of them.  The toy is registered, written as a model folder, loaded, stepped
in portions and mixed batches from few pages, and compared with a plain whole-sequence computation, on the GPU
and, with the kernels replaced by their torch twins, on the CPU.
"""
import math
import os

import numpy as np
import pytest
import torch

import plain_qwen2moe as plain
from locus_b200.cache import CacheManager
from locus_b200.config.base import ArchEntry, register_arch
from locus_b200.engine.step import ModelRunner, StepEntry
from locus_b200.models import load_model
from locus_b200.parts import LayerCall, LayerSpec, Mixer, ModelPlan, PagedKvSpec, PartSpec, TensorSource, register_mixer
from locus_b200.parts.base import StepPlan
from locus_b200.weights.loader import write_random_model
from tiny_configs import random_tokens

TILE = 4


class ToyTiles(StepPlan):
    """Tiles of TILE queries over every segment, as (segment, first query, queries) triples, and their number."""

    key = ("toy.key_only.tiles", TILE)

    def capacity(self, max_tokens, max_segments):
        return 3 * (max_tokens // TILE + max_segments)

    def build(self, seg_q0, seg_qn, seg_ctx, out):
        n = 0
        for s, qn in enumerate(seg_qn.tolist()):
            for q in range(0, qn, TILE):
                out[3 * n : 3 * n + 3] = (s, q, min(TILE, qn - q))
                n += 1
        return {"tiles": (0, 3 * n, (-1, 3)), "n_tiles": n}


class KeyOnlyMixer(Mixer):
    """Per token the cache holds a key row k_t = Wk . h_t (one head) and, beside it, the scalar
    g_t = sigmoid(wg . h_t).  out_t = Wo . sum_{s <= t} softmax_s(q_t . k_s / sqrt(d)) g_s k_s : the keys serve as
    values, scaled by the stored field.  Works tile by tile through its own step plan."""

    def __init__(self, prefix, *, hidden, dim):
        super().__init__(prefix)
        self.hidden, self.dim = hidden, dim

    def param_shapes(self):
        return {"wq": (self.dim, self.hidden), "wk": (self.dim, self.hidden), "wg": (1, self.hidden),
                "wo": (self.hidden, self.dim)}

    def sources(self):
        return [TensorSource(f"{self.prefix}.{n}.weight", shape, n) for n, shape in self.param_shapes().items()]

    def cache_needs(self):
        return PagedKvSpec(1, self.dim, window=0, has_v=False, extra_width=1), None

    def step_plans(self):
        return [ToyTiles()]

    def forward(self, h, batch, cache, residual, rt):
        assert cache.pool.shape[1:] == (1, 1, cache.page_tokens, self.dim) and cache.extra.shape[1:] == (cache.page_tokens, 1)
        gb = batch.groups[cache.group]
        P = gb.page_tokens
        hf = h.float()
        q = hf @ self.params["wq"].float().T
        k = hf @ self.params["wk"].float().T
        g = torch.sigmoid(hf @ self.params["wg"].float().T)
        slots = gb.slots[: batch.T].long()
        cache.pool[slots // P, 0, 0, slots % P] = k.to(cache.pool.dtype)
        cache.extra[slots // P, slots % P] = g.to(cache.extra.dtype)
        plan = batch.plans[ToyTiles.key]
        table = gb.block_table.cpu()
        for s, q0, n in plan["tiles"].cpu().tolist()[: plan["n_tiles"]]:
            row0, ctx = batch.host_seg_q0[s] + q0, batch.host_seg_ctx[s] + q0
            pos = torch.arange(ctx + n, device=h.device)
            pages = table[s, : (ctx + n + P - 1) // P].to(h.device).long()
            keys = cache.pool[pages, 0, 0].reshape(-1, self.dim)[: ctx + n].float()
            gate = cache.extra[pages].reshape(-1)[: ctx + n].float()
            sc = (q[row0 : row0 + n] @ keys.T) / math.sqrt(self.dim)
            sc = sc.masked_fill(pos[None, :] > (ctx + torch.arange(n, device=h.device))[:, None], float("-inf"))
            mixed = torch.softmax(sc, dim=-1) @ (keys * gate[:, None])
            residual[row0 : row0 + n] += mixed @ self.params["wo"].float().T


register_mixer("toy_key_only", KeyOnlyMixer)

TOY3 = {"architectures": ["Toy3ForCausalLM"], "hidden": 40, "vocab": 83, "dim": 24, "experts": 12, "top_k": 3,
        "inter": 16, "groups": 4, "groups_used": 2, "eps": 1e-5, "max_positions": 160}


def toy3_plan(cfg):
    H = cfg["hidden"]
    norm = PartSpec("rmsnorm", {"width": H, "eps": cfg["eps"]})
    moe = PartSpec("sparse_moe", {"hidden": H, "n_experts": cfg["experts"], "top_k": cfg["top_k"], "norm_topk": True,
                                  "expert_intermediate": cfg["inter"], "shared_intermediate": 0, "weight_scale": 1.5,
                                  "score_fn": "sigmoid", "selection_bias": True, "n_group": cfg["groups"],
                                  "n_group_used": cfg["groups_used"]})
    mixer = PartSpec("toy_key_only", {"hidden": H, "dim": cfg["dim"]})
    layers = [LayerSpec(f"toy3.layers.{l}", PartSpec("pre_norm", {"hidden": H, "mixer_prefix": "mix"}), norm, mixer, moe)
              for l in range(2)]
    return ModelPlan(architecture="Toy3ForCausalLM", hidden_size=H, vocab_size=cfg["vocab"],
                     max_positions=cfg["max_positions"], eos_token_id=-1,
                     embedding=PartSpec("embedding", {"vocab": cfg["vocab"], "hidden": H, "prefix": "toy3.embed"}),
                     layers=layers, order=[LayerCall(0), LayerCall(1)],
                     final_norm=PartSpec("rmsnorm", {"width": H, "eps": cfg["eps"], "prefix": "toy3.norm"}),
                     head=PartSpec("linear", {"vocab": cfg["vocab"], "hidden": H, "prefix": "toy3.head"}), config=cfg)


register_arch(ArchEntry("Toy3ForCausalLM", "test-only toy: key-only cache with a per-token field, own step plan, "
                        "sigmoid-scored grouped router", lambda raw: dict(raw), toy3_plan))


def toy3_plain(cfg, W, tokens):
    W = {k: v.double() for k, v in W.items()}
    T, d = len(tokens), cfg["dim"]
    x = W["toy3.embed.weight"][torch.tensor(tokens)]
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for l in range(2):
        p = f"toy3.layers.{l}"
        h = plain.rmsnorm(x, W[f"{p}.input_layernorm.weight"], cfg["eps"])
        q, k = h @ W[f"{p}.mix.wq.weight"].T, h @ W[f"{p}.mix.wk.weight"].T
        g = torch.sigmoid(h @ W[f"{p}.mix.wg.weight"].T)
        sc = (q @ k.T / math.sqrt(d)).masked_fill(~causal, float("-inf"))
        x = x + (torch.softmax(sc, -1) @ (k * g)) @ W[f"{p}.mix.wo.weight"].T
        h = plain.rmsnorm(x, W[f"{p}.post_attention_layernorm.weight"], cfg["eps"])
        r = h @ W[f"{p}.mlp.gate.weight"].T
        out = torch.zeros_like(h)
        for t in range(T):
            ids, wts = plain.moe_select(r[t], cfg["top_k"], True, 1.5, "sigmoid", W[f"{p}.mlp.gate.selection_bias"],
                                        cfg["groups"], cfg["groups_used"])
            for e, w in zip(ids, wts):
                out[t] += w * plain.swiglu_mlp(h[t : t + 1], W[f"{p}.mlp.experts.{e}.gate_proj.weight"],
                                               W[f"{p}.mlp.experts.{e}.up_proj.weight"],
                                               W[f"{p}.mlp.experts.{e}.down_proj.weight"])[0]
        x = x + out
    return plain.rmsnorm(x, W["toy3.norm.weight"], cfg["eps"]) @ W["toy3.head.weight"].T


def run_toy3(device, tmp_path):
    d = write_random_model(TOY3, 11, os.path.join(str(tmp_path), "toy3"), torch.float32)
    cfg, W = plain.load_folder(d)
    # the stored selection bias is drawn like a bias, N(0, 0.02): far too small to matter beside sigmoid scores of
    # about one half.  Scale it up in the file's copy and in the model alike, so that the bias decides picks.
    model = load_model(d, torch.float32, device)
    for l in range(2):
        name = f"toy3.layers.{l}.mlp.gate.selection_bias"
        W[name] = W[name] * 10.0
        model.blocks[l].ff.params["sel_bias"].mul_(10.0)
    needs = model.cache_needs()
    assert needs[0][0] == PagedKvSpec(1, cfg["dim"], 0, False, 1)
    cache = CacheManager(needs, page_tokens=16, n_pages=9, n_state_slots=3, max_seq_tokens=128, dtype=torch.float32,
                         device=device, poison=True)
    assert len(cache.groups) == 1 and cache.groups[0].pool.shape == (2, 9, 1, 1, 16, cfg["dim"])
    assert cache.groups[0].extra.shape == (2, 9, 16, 1)
    assert cache.bytes_per_token() == 2 * (cfg["dim"] + 1) * 4     # one row and one field per token and layer
    runner = ModelRunner(model, cache, max_tokens=64, max_segments=3)
    assert list(runner.plans) == [ToyTiles.key]
    for part in model.all_parts():
        part.bind(runner.rt)   # the bias was changed after binding
    toks = {"a": random_tokens(70, cfg["vocab"], 1), "b": random_tokens(41, cfg["vocab"], 2), "c": random_tokens(7, cfg["vocab"], 3)}
    refs = {k: toy3_plain(cfg, W, v) for k, v in toks.items()}
    steps = [[("a", 23)], [("a", 5), ("b", 30)], [("a", 1), ("b", 1), ("c", 7)], [("a", 41), ("b", 10)]]
    fed, got = {}, {k: [] for k in toks}
    for step in steps:
        entries = []
        for rid, n in step:
            a = fed.get(rid, 0)
            seq = cache.get(rid) or cache.open(rid)
            assert cache.ensure_capacity(seq, n)
            entries.append(StepEntry(seq, toks[rid][a : a + n], list(range(n))))
            fed[rid] = a + n
        lg = runner.step(entries).double().cpu()
        row = 0
        for rid, n in step:
            got[rid].append(lg[row : row + n].clone())
            row += n
        for rid, n in step:
            if fed[rid] == len(toks[rid]):
                cache.release(cache.get(rid))
        cache.check_invariants()
    for rid in toks:
        out = torch.cat(got[rid])
        assert torch.isfinite(out).all()
        err = float((out - refs[rid]).abs().max())
        assert err <= 5e-5 * float(refs[rid].abs().max()), (rid, err)
    assert cache.free_pages() == cache.total_pages()


@pytest.mark.gpu
def test_key_only_cache_own_step_plan_and_sigmoid_router_on_the_gpu(tmp_path):
    run_toy3("cuda:0", tmp_path)


def test_key_only_cache_own_step_plan_and_sigmoid_router_host_logic(tmp_path, monkeypatch):
    import emulated_kernels as EK

    EK.install(monkeypatch)
    run_toy3("cpu", tmp_path)


def test_the_toy_plan_writes_its_lists_behind_the_descriptors():
    plan = ToyTiles()
    out = np.zeros(plan.capacity(32, 3), dtype=np.int32)
    res = plan.build(np.array([0, 9, 10], dtype=np.int32), np.array([9, 1, 6], dtype=np.int32),
                     np.array([0, 40, 3], dtype=np.int32), out)
    assert res["n_tiles"] == 6 and res["tiles"][:2] == (0, 18)
    assert out[:18].reshape(-1, 3).tolist() == [[0, 0, 4], [0, 4, 4], [0, 8, 1], [1, 0, 1], [2, 0, 4], [2, 4, 2]]
