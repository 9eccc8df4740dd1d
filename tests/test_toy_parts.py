"""Generality of the parts: a toy architecture, defined here and nowhere in the framework,
with a mixer that keeps per-request state of its own (a running mean), a run order that
names layers twice and lets one call read another call's cache.  It is registered, written
as a model folder, loaded, stepped in portions and mixed batches, and compared with a plain
whole-sequence computation.  Runs on the GPU (marked gpu) and, with the kernels replaced
by their torch twins, on the CPU.
"""
import os

import pytest
import torch

import plain_qwen2moe as plain
from locus_b200.cache import CacheManager
from locus_b200.config.base import ArchEntry, register_arch
from locus_b200.engine.step import ModelRunner, StepEntry
from locus_b200.models import load_model
from locus_b200.parts import (LayerCall, LayerSpec, Mixer, ModelPlan, PartSpec, StateSpec, TensorSource,
                              register_mixer)
from locus_b200.weights.loader import write_random_model
from tiny_configs import random_tokens


class RunningMeanMixer(Mixer):
    """out_t = W . mean(h_0 .. h_t) over the request's tokens so far.  State per request:
    the running sum [H] and the count [1], float32; no pages."""

    def __init__(self, prefix, *, hidden):
        super().__init__(prefix)
        self.hidden = hidden

    def param_shapes(self):
        return {"w": (self.hidden, self.hidden)}

    def sources(self):
        return [TensorSource(self.prefix + ".w.weight", (self.hidden, self.hidden), "w")]

    def cache_needs(self):
        return None, StateSpec((self.hidden + 1,), torch.float32)

    def forward(self, h, batch, cache, residual, rt):
        w = self.params["w"].float()
        for q0, qn, ctx, slot in zip(batch.host_seg_q0, batch.host_seg_qn, batch.host_seg_ctx, batch.host_state_slots):
            st = cache.state[slot]
            assert int(st[-1]) == ctx, "state and position disagree"
            csum = torch.cumsum(h[q0 : q0 + qn].float(), 0) + st[:-1]
            cnt = st[-1] + torch.arange(1, qn + 1, device=h.device, dtype=torch.float32)
            residual[q0 : q0 + qn] += (csum / cnt[:, None]) @ w.T
            st[:-1] = csum[-1]
            st[-1] = cnt[-1]


register_mixer("toy_running_mean", RunningMeanMixer)

TOY = {"architectures": ["ToyForCausalLM"], "hidden": 48, "vocab": 97, "heads": 3, "head_dim": 16, "inter": 40,
       "eps": 1e-5, "theta": 10000.0, "max_positions": 128}


def toy_plan(cfg):
    H = cfg["hidden"]
    norm = PartSpec("rmsnorm", {"width": H, "eps": cfg["eps"]})
    ff = PartSpec("dense_mlp", {"hidden": H, "intermediate": cfg["inter"]})
    att = PartSpec("attention", {"hidden": H, "n_heads": cfg["heads"], "n_kv_heads": 1, "head_dim": cfg["head_dim"],
                                 "qkv_bias": False, "position": PartSpec("rotary", {"head_dim": cfg["head_dim"],
                                                                                    "theta": cfg["theta"]})})
    layers = [
        LayerSpec("toy.layers.0", PartSpec("pre_norm", {"hidden": H}), norm, att, ff),
        LayerSpec("toy.layers.1", PartSpec("pre_norm", {"hidden": H, "mixer_prefix": "mean"}), norm,
                  PartSpec("toy_running_mean", {"hidden": H}), ff),
    ]
    # layer 0, layer 1, layer 1 again (state of its own), layer 0 again reading the first call's cache
    order = [LayerCall(0), LayerCall(1), LayerCall(1), LayerCall(0, cache_of=0)]
    return ModelPlan(architecture="ToyForCausalLM", hidden_size=H, vocab_size=cfg["vocab"],
                     max_positions=cfg["max_positions"], eos_token_id=-1,
                     embedding=PartSpec("embedding", {"vocab": cfg["vocab"], "hidden": H, "prefix": "toy.embed"}),
                     layers=layers, order=order,
                     final_norm=PartSpec("rmsnorm", {"width": H, "eps": cfg["eps"], "prefix": "toy.norm"}),
                     head=PartSpec("linear", {"vocab": cfg["vocab"], "hidden": H, "tied_to": "toy.embed.weight", "prefix": "toy.head"}),
                     config=cfg)


register_arch(ArchEntry("ToyForCausalLM", "test-only toy with a stateful mixer", lambda raw: dict(raw), toy_plan))


def toy_plain(cfg, W, tokens):
    """Whole-sequence float64 computation of the toy model."""
    W = {k: v.double() for k, v in W.items()}
    T, H, nh, hd = len(tokens), cfg["hidden"], cfg["heads"], cfg["head_dim"]
    x = W["toy.embed.weight"][torch.tensor(tokens)]
    pos = torch.arange(T)
    kv0 = None
    for call, (layer, reads_first) in enumerate([(0, False), (1, False), (1, False), (0, True)]):
        p = f"toy.layers.{layer}"
        h = plain.rmsnorm(x, W[f"{p}.input_layernorm.weight"], cfg["eps"])
        if layer == 0:
            a = f"{p}.self_attn"
            q = plain.rope_half_split((h @ W[f"{a}.q_proj.weight"].T).view(T, nh, hd), pos, cfg["theta"])
            if reads_first:
                k, v = kv0
            else:
                k = plain.rope_half_split((h @ W[f"{a}.k_proj.weight"].T).view(T, 1, hd), pos, cfg["theta"])
                v = (h @ W[f"{a}.v_proj.weight"].T).view(T, 1, hd)
                kv0 = (k, v)
            x = x + plain.attention(q, k, v).reshape(T, nh * hd) @ W[f"{a}.o_proj.weight"].T
        else:
            mean = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=h.dtype)[:, None]
            x = x + mean @ W[f"{p}.mean.w.weight"].T
        h = plain.rmsnorm(x, W[f"{p}.post_attention_layernorm.weight"], cfg["eps"])
        x = x + plain.swiglu_mlp(h, W[f"{p}.mlp.gate_proj.weight"], W[f"{p}.mlp.up_proj.weight"],
                                 W[f"{p}.mlp.down_proj.weight"])
    return plain.rmsnorm(x, W["toy.norm.weight"], cfg["eps"]) @ W["toy.embed.weight"].T


def run_toy(device, tmp_path):
    d = write_random_model(TOY, 3, os.path.join(str(tmp_path), "toy"), torch.float32)
    cfg, W = plain.load_folder(d)
    model = load_model(d, torch.float32, device)
    needs = model.cache_needs()
    assert [n[0] is not None for n in needs] == [True, False, False, True] and needs[3][2] == 0
    assert needs[1][1].shape == (49,)
    cache = CacheManager(needs, page_tokens=16, n_pages=10, n_state_slots=3, max_seq_tokens=128, dtype=torch.float32,
                         device=device, poison=True)
    assert len(cache.groups) == 1 and cache.groups[0].pool.shape[0] == 1  # one call keeps pages
    lay = cache.layer_caches()
    assert lay[1].state.data_ptr() != lay[2].state.data_ptr()  # a layer named twice has state per call
    runner = ModelRunner(model, cache, max_tokens=64, max_segments=3)
    toks = {"a": random_tokens(50, 97, 1), "b": random_tokens(37, 97, 2), "c": random_tokens(9, 97, 3)}
    refs = {k: toy_plain(cfg, W, v) for k, v in toks.items()}
    steps = [[("a", 20)], [("a", 3), ("b", 30)], [("a", 1), ("b", 1), ("c", 9)], [("a", 26), ("b", 6)]]
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
    for rid in toks:
        out = torch.cat(got[rid])
        err = float((out - refs[rid]).abs().max())
        assert err <= 5e-5 * float(refs[rid].abs().max()), (rid, err)
    # a state slot that is used again starts from zero
    seq = cache.open("again")
    assert cache.ensure_capacity(seq, 9)
    lg = runner.step([StepEntry(seq, toks["c"], [8])]).double().cpu()
    assert float((lg[0] - refs["c"][8]).abs().max()) <= 5e-5 * float(refs["c"].abs().max())
    cache.release(seq)
    cache.check_invariants()
    assert cache.free_pages() == cache.total_pages()


@pytest.mark.gpu
def test_toy_architecture_on_the_gpu(tmp_path):
    run_toy("cuda:0", tmp_path)


def test_toy_architecture_host_logic(tmp_path, monkeypatch):
    import emulated_kernels as EK

    EK.install(monkeypatch)
    run_toy("cpu", tmp_path)
