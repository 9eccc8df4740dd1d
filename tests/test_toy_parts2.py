"""More generality of the parts, again with pieces that exist only in this file: a feed-forward
with routing of its own (one expert per token, picked by the largest router logit), a position
encoding that is not a rotation (it marks positions additively in q and k through ``apply``),
and a post-norm arrangement.  They are registered, put into a plan beside the framework's own
attention and sparse-MoE parts, written as a model folder, loaded, stepped in portions and mixed
batches, and compared with a plain whole-sequence computation.

The plan also checks the rule of pending additions: the framework's sparse-MoE block may leave
its experts' sum to the next block's first norm only if that block's arrangement takes it; the
post-norm arrangement of this file knows nothing of that, so the sum must have been added
before it runs.
"""
import math
import os

import pytest
import torch

import plain_qwen2moe as plain
from locus_b200.cache import CacheManager
from locus_b200.config.base import ArchEntry, register_arch
from locus_b200.engine.step import ModelRunner, StepEntry
from locus_b200.models import load_model
from locus_b200.parts import (Arrangement, FeedForward, LayerCall, LayerSpec, ModelPlan, PartSpec, PositionEncoding,
                              TensorSource, make_part, register_arrangement, register_feed_forward,
                              register_position)
from locus_b200.weights.loader import write_random_model
from tiny_configs import random_tokens


class SwitchFeedForward(FeedForward):
    """One expert per token: e = argmax(R . h) (lowest index on ties), out = D_e . relu(U_e . h)."""

    def __init__(self, prefix, *, hidden, n_experts, inner):
        super().__init__(prefix)
        self.hidden, self.E, self.inner = hidden, n_experts, inner

    def param_shapes(self):
        return {"router": (self.E, self.hidden), "up": (self.E * self.inner, self.hidden),
                "down": (self.E * self.hidden, self.inner)}

    def sources(self):
        out = [TensorSource(f"{self.prefix}.router.weight", (self.E, self.hidden), "router")]
        for e in range(self.E):
            out.append(TensorSource(f"{self.prefix}.expert{e}.up.weight", (self.inner, self.hidden), "up", e * self.inner))
            out.append(TensorSource(f"{self.prefix}.expert{e}.down.weight", (self.hidden, self.inner), "down",
                                    e * self.hidden))
        return out

    def forward(self, h, batch, residual, rt):
        hf = h.float()
        pick = torch.argmax(hf @ self.params["router"].float().T, dim=-1)
        up = self.params["up"].float().view(self.E, self.inner, self.hidden)
        down = self.params["down"].float().view(self.E, self.hidden, self.inner)
        for e in range(self.E):
            rows = torch.nonzero(pick == e).flatten()
            if rows.numel():
                residual[rows] += torch.relu(hf[rows] @ up[e].T) @ down[e].T


class MarkedPositions(PositionEncoding):
    """Not a rotation: element 0 of every head of q gets + sin(pos * w), element 1 of every head of k
    gets + cos(pos * w).  No rotary table, so the attention part calls ``apply``."""

    def __init__(self, prefix, *, head_dim, omega):
        super().__init__(prefix)
        self.head_dim, self.omega = head_dim, omega

    def apply(self, q, k, positions):
        ang = positions.to(torch.float32) * self.omega
        q[:, 0 :: self.head_dim] += torch.sin(ang)[:, None].to(q.dtype)
        k[:, 1 :: self.head_dim] += torch.cos(ang)[:, None].to(k.dtype)


class PostNorm(Arrangement):
    """x = norm1(x + mixer(x)); x = norm2(x + ff(x)).  Takes no pending additions."""

    def __init__(self, prefix, *, hidden, norm, mixer, feed_forward):
        super().__init__(prefix)
        self.hidden = hidden
        self.mixer = make_part("mixer", mixer, prefix + ".mix")
        self.ff = make_part("feed_forward", feed_forward, prefix + ".ff")
        self.norm1 = make_part("norm", norm, prefix + ".norm1")
        self.norm2 = make_part("norm", norm, prefix + ".norm2")

    def sub_parts(self):
        return [self.mixer, self.ff, self.norm1, self.norm2]

    def forward(self, x, batch, cache, rt):
        T = batch.T
        h = rt.rows("toy2.h", self.hidden, rt.dtype, T)
        y = rt.rows("toy2.y", self.hidden, torch.float32, T)
        for part, norm, is_mixer in ((self.mixer, self.norm1, True), (self.ff, self.norm2, False)):
            h.copy_(x)
            if is_mixer:
                part.forward(h, batch, cache, x, rt)
            else:
                part.forward(h, batch, x, rt)
            norm.forward(x, y)
            x.copy_(y)


register_feed_forward("toy_switch", SwitchFeedForward)
register_position("toy_marked", MarkedPositions)
register_arrangement("toy_post_norm", PostNorm)

TOY2 = {"architectures": ["Toy2ForCausalLM"], "hidden": 40, "vocab": 83, "heads": 2, "kv_heads": 2, "head_dim": 16,
        "experts": 5, "top_k": 2, "expert_inner": 24, "shared_inner": 16, "switch_experts": 3, "switch_inner": 20,
        "eps": 1e-6, "omega": 0.37, "max_positions": 96}


def toy2_plan(cfg):
    H = cfg["hidden"]
    norm = PartSpec("rmsnorm", {"width": H, "eps": cfg["eps"]})
    att = PartSpec("attention", {"hidden": H, "n_heads": cfg["heads"], "n_kv_heads": cfg["kv_heads"],
                                 "head_dim": cfg["head_dim"], "qkv_bias": True,
                                 "position": PartSpec("toy_marked", {"head_dim": cfg["head_dim"], "omega": cfg["omega"]})})
    moe = PartSpec("sparse_moe", {"hidden": H, "n_experts": cfg["experts"], "top_k": cfg["top_k"], "norm_topk": True,
                                  "expert_intermediate": cfg["expert_inner"], "shared_intermediate": cfg["shared_inner"]})
    switch = PartSpec("toy_switch", {"hidden": H, "n_experts": cfg["switch_experts"], "inner": cfg["switch_inner"]})
    layers = [
        LayerSpec("toy2.layers.0", PartSpec("pre_norm", {"hidden": H}), norm, att, moe),   # leaves nothing pending: see below
        LayerSpec("toy2.layers.1", PartSpec("toy_post_norm", {"hidden": H}), norm, att, switch),
        LayerSpec("toy2.layers.2", PartSpec("pre_norm", {"hidden": H}), norm, att, moe),   # may leave its sum to layer 3's norm
        LayerSpec("toy2.layers.3", PartSpec("pre_norm", {"hidden": H}), norm, att, switch),
    ]
    return ModelPlan(architecture="Toy2ForCausalLM", hidden_size=H, vocab_size=cfg["vocab"],
                     max_positions=cfg["max_positions"], eos_token_id=-1,
                     embedding=PartSpec("embedding", {"vocab": cfg["vocab"], "hidden": H, "prefix": "toy2.embed"}),
                     layers=layers, order=[LayerCall(i) for i in range(4)],
                     final_norm=PartSpec("rmsnorm", {"width": H, "eps": cfg["eps"], "prefix": "toy2.norm"}),
                     head=PartSpec("linear", {"vocab": cfg["vocab"], "hidden": H, "prefix": "toy2.head"}),
                     config=cfg)


register_arch(ArchEntry("Toy2ForCausalLM", "test-only toy: routed feed-forward, marked positions, post-norm",
                        lambda raw: dict(raw), toy2_plan))


def toy2_plain(cfg, W, tokens):
    """Whole-sequence float64 computation of the second toy model."""
    W = {k: v.double() for k, v in W.items()}
    T, H, nh, nkv, hd = len(tokens), cfg["hidden"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    x = W["toy2.embed.weight"][torch.tensor(tokens)]
    ang = torch.arange(T, dtype=torch.float64) * cfg["omega"]

    def attn(h, a):
        q = (h @ W[f"{a}.q_proj.weight"].T + W[f"{a}.q_proj.bias"]).view(T, nh, hd).clone()
        k = (h @ W[f"{a}.k_proj.weight"].T + W[f"{a}.k_proj.bias"]).view(T, nkv, hd).clone()
        v = (h @ W[f"{a}.v_proj.weight"].T + W[f"{a}.v_proj.bias"]).view(T, nkv, hd)
        q[:, :, 0] += torch.sin(ang)[:, None]
        k[:, :, 1] += torch.cos(ang)[:, None]
        return plain.attention(q, k, v).reshape(T, nh * hd) @ W[f"{a}.o_proj.weight"].T

    def switch(h, p):
        pick = torch.argmax(h @ W[f"{p}.router.weight"].T, dim=-1)
        out = torch.zeros_like(h)
        for t in range(T):
            e = int(pick[t])
            out[t] = torch.relu(h[t] @ W[f"{p}.expert{e}.up.weight"].T) @ W[f"{p}.expert{e}.down.weight"].T
        return out

    moe_cfg = {"num_experts_per_tok": cfg["top_k"], "norm_topk_prob": True,
               "shared_expert_intermediate_size": cfg["shared_inner"]}
    for l in range(4):
        p = f"toy2.layers.{l}"
        if l == 1:  # post-norm
            x = plain.rmsnorm(x + attn(x, f"{p}.mix"), W[f"{p}.norm1.weight"], cfg["eps"])
            x = plain.rmsnorm(x + switch(x, f"{p}.ff"), W[f"{p}.norm2.weight"], cfg["eps"])
            continue
        x = x + attn(plain.rmsnorm(x, W[f"{p}.input_layernorm.weight"], cfg["eps"]), f"{p}.self_attn")
        h = plain.rmsnorm(x, W[f"{p}.post_attention_layernorm.weight"], cfg["eps"])
        x = x + (plain.moe_block(h, W, f"{p}.mlp", moe_cfg) if l in (0, 2) else switch(h, f"{p}.mlp"))
    return plain.rmsnorm(x, W["toy2.norm.weight"], cfg["eps"]) @ W["toy2.head.weight"].T


def run_toy2(device, tmp_path):
    d = write_random_model(TOY2, 5, os.path.join(str(tmp_path), "toy2"), torch.float32)
    cfg, W = plain.load_folder(d)
    model = load_model(d, torch.float32, device)
    assert [b.takes_pending_add for b in model.blocks] == [True, False, True, True]
    cache = CacheManager(model.cache_needs(), page_tokens=16, n_pages=12, n_state_slots=3, max_seq_tokens=96,
                         dtype=torch.float32, device=device, poison=True)
    runner = ModelRunner(model, cache, max_tokens=64, max_segments=3)
    # what each sparse-MoE block did with its experts' sum
    from locus_b200.engine import batch as batch_mod

    left = []
    orig = batch_mod.Runtime.leave_pending
    batch_mod.Runtime.leave_pending = lambda self, add: (left.append(add), orig(self, add))[1]
    try:
        toks = {"a": random_tokens(41, 83, 1), "b": random_tokens(30, 83, 2), "c": random_tokens(5, 83, 3)}
        refs = {k: toy2_plain(cfg, W, v) for k, v in toks.items()}
        steps = [[("a", 17)], [("a", 2), ("b", 23)], [("a", 1), ("b", 1), ("c", 5)], [("a", 21), ("b", 6)]]
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
    finally:
        batch_mod.Runtime.leave_pending = orig
    # layer 2's block left its sum to layer 3's norm in every step; layer 0's, before the post-norm block, never did
    assert len(left) == len(steps)
    for rid in toks:
        out = torch.cat(got[rid])
        err = float((out - refs[rid]).abs().max())
        assert math.isfinite(err) and err <= 5e-5 * float(refs[rid].abs().max()), (rid, err)
    cache.check_invariants()
    assert cache.free_pages() == cache.total_pages()


@pytest.mark.gpu
def test_second_toy_architecture_on_the_gpu(tmp_path):
    run_toy2("cuda:0", tmp_path)


def test_second_toy_architecture_host_logic(tmp_path, monkeypatch):
    import emulated_kernels as EK

    EK.install(monkeypatch)
    run_toy2("cpu", tmp_path)
