"""A plain, slow implementation of Qwen1.5-MoE for whole sequences, written from the
formulas of the reference (garana/locus).  No cache, no batching tricks, one function per
part; it shares no code with ``locus_b200``.  Weights come as a dict of tensors keyed by
checkpoint name; everything is computed in ``dtype`` (float32 like the reference, or
float64 as an oracle with negligible rounding).

Anchoring: ``tests/golden/`` holds logits that the reference's own C++ model code
(compiled here on the CPU) produced for a tiny random model; ``tests/test_plain.py``
compares this file with them.  Options the reference cannot express (dense layers by
``decoder_sparse_step``, ``norm_topk_prob`` for this architecture, a window) rest on the
formulas alone.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """src/locus/backend/cpu_ops.cpp:1687-1699: x * (1 / sqrt(mean(x^2) + eps)) * w."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    scale = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return x * scale * w


def softmax(x: torch.Tensor) -> torch.Tensor:
    """src/locus/backend/cpu_ops.cpp:1721-1734: exp(x - max) / sum."""
    e = torch.exp(x - x.max(dim=-1, keepdim=True).values)
    return e / e.sum(dim=-1, keepdim=True)


def silu_mul(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """src/locus/backend/cpu_ops.cpp:1736-1743: g / (1 + exp(-g)) * u."""
    return g / (1.0 + torch.exp(-g)) * u


def rope_half_split(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """src/locus/backend/cpu_ops.cpp:1849-1872 with the angle of cpu_ops.cpp:1807-1814:
    per head, pairs (i, i + hd/2) rotated by pos * theta^(-2i/hd).  x: [T, heads, hd]."""
    hd = x.shape[-1]
    half = hd // 2
    i = torch.arange(half, dtype=x.dtype)
    inv = torch.pow(torch.tensor(theta, dtype=x.dtype), -2.0 * i / hd)
    ang = positions.to(x.dtype)[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """src/locus/model/arch.cpp:668-695: for head h with kv head h // (heads / kv_heads),
    scores = q.k / sqrt(hd) over keys 0..pos, softmax, weighted sum of v.  q: [T, nh, hd];
    k, v: [T, nkv, hd].  ``window`` > 0: query p sees keys t with p - window < t <= p."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    for h in range(nh):
        kvh = h // group
        for p in range(T):
            lo = max(0, p - window + 1) if window > 0 else 0
            s = (k[lo : p + 1, kvh] @ q[p, h]) * scale
            a = softmax(s)
            out[p, h] = a @ v[lo : p + 1, kvh]
    return out


def moe_select(router_logits: torch.Tensor, top_k: int, norm_topk: bool, scale: float = 1.0,
               score_fn: str = "softmax", sel_bias: Optional[torch.Tensor] = None, n_group: int = 1,
               n_group_used: int = 1):
    """src/locus/model/llama.cpp:900-980: scores = softmax over all experts (llama.cpp:903-904) or a
    sigmoid of each logit (:905-909); selection scores = scores + bias (:913-918); with groups, a group's
    score is the sum of its two best selection scores and all but the best ``n_group_used`` groups are
    masked to -1e30 (:919-951); k rounds of arg-max with strict '>' (ties to the lowest index, :952-965);
    weight = score / wsum * scale, wsum = sum of the picked scores when renormalising, else 1 (:966-978).
    One token: router_logits [E] -> (ids [k], weights [k]) in pick order."""
    E = router_logits.shape[0]
    p = softmax(router_logits) if score_fn == "softmax" else 1.0 / (1.0 + torch.exp(-router_logits))
    sel = p.clone()
    if sel_bias is not None:
        sel = sel + sel_bias.to(sel.dtype)
    if n_group > 1:
        per = E // n_group
        gscore = []
        for g in range(n_group):
            top1 = top2 = -1e30
            for e in range(g * per, (g + 1) * per):
                v = float(sel[e])
                if v > top1:
                    top1, top2 = v, top1
                elif v > top2:
                    top2 = v
            gscore.append(top1 + (top2 if per > 1 else 0.0))
        keep: List[int] = []
        for _ in range(n_group_used):
            best = -1
            for g in range(n_group):
                if g not in keep and (best < 0 or gscore[g] > gscore[best]):
                    best = g
            keep.append(best)
        for e in range(E):
            if e // per not in keep:
                sel[e] = -1e30
    picked: List[int] = []
    for _ in range(top_k):
        best = -1
        for e in range(E):
            if e in picked:
                continue
            if best < 0 or sel[e] > sel[best]:
                best = e
        picked.append(best)
    wsum = sum(p[e] for e in picked) if norm_topk else 1.0
    return picked, [p[e] / wsum * scale for e in picked]


def swiglu_mlp(h: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """src/locus/model/llama.cpp:493-503 / 1026-1043: Wdown . (silu(Wgate.h) * (Wup.h))."""
    return silu_mul(h @ wg.T, h @ wu.T) @ wd.T


def moe_block(h: torch.Tensor, W: Dict[str, torch.Tensor], prefix: str, cfg: dict, forced=None,
              aux: Optional[dict] = None) -> torch.Tensor:
    """src/locus/model/llama.cpp:992-1077: routed experts summed in pick order, then the
    shared expert scaled by sigmoid(w_gate . h) (llama.cpp:1062-1076).  h: [T, H].

    ``forced``: per token, the experts to use instead of the selection (their weights still
    come from this function's own probabilities) -- tests use it to follow an engine whose
    router, fed rounded activations, chose the other side of a near-tie.  ``aux`` collects the
    selection and the probabilities per token."""
    r = h @ W[f"{prefix}.gate.weight"].T
    k, norm = cfg["num_experts_per_tok"], cfg.get("norm_topk_prob", False)
    picks = []
    for t in range(h.shape[0]):
        ids, wts = moe_select(r[t], k, norm)
        if aux is not None:
            aux.setdefault(prefix, []).append((list(ids), softmax(r[t])))
        if forced is not None and sorted(forced[t]) != sorted(ids):
            p = softmax(r[t])
            ids = list(forced[t])
            wsum = sum(p[e] for e in ids) if norm else 1.0
            wts = [p[e] / wsum for e in ids]
        picks.append((ids, wts))
    # every expert once, over the tokens that picked it (its weights are read once, not per token)
    picked_out = [[None] * k for _ in picks]
    for e in sorted({e for ids, _ in picks for e in ids}):
        who = [(t, s) for t, (ids, _) in enumerate(picks) for s, x in enumerate(ids) if x == e]
        y = swiglu_mlp(h[torch.tensor([t for t, _ in who])], W[f"{prefix}.experts.{e}.gate_proj.weight"],
                       W[f"{prefix}.experts.{e}.up_proj.weight"], W[f"{prefix}.experts.{e}.down_proj.weight"])
        for i, (t, s) in enumerate(who):
            picked_out[t][s] = y[i]
    out = torch.zeros_like(h)
    for t, (ids, wts) in enumerate(picks):
        for s in range(len(ids)):
            out[t] = out[t] + wts[s] * picked_out[t][s]
    if cfg.get("shared_expert_intermediate_size", 0) > 0:
        z = h @ W[f"{prefix}.shared_expert_gate.weight"][0]
        gamma = 1.0 / (1.0 + torch.exp(-z))
        out = out + gamma[:, None] * swiglu_mlp(h, W[f"{prefix}.shared_expert.gate_proj.weight"],
                                                W[f"{prefix}.shared_expert.up_proj.weight"],
                                                W[f"{prefix}.shared_expert.down_proj.weight"])
    return out


def is_moe_layer(cfg: dict, l: int) -> bool:
    return (cfg.get("num_experts", 0) > 0 and l not in cfg.get("mlp_only_layers", [])
            and (l + 1) % cfg.get("decoder_sparse_step", 1) == 0)


def layer_window(cfg: dict, l: int) -> int:
    if cfg.get("use_sliding_window", False) and l >= cfg.get("max_window_layers", cfg["num_hidden_layers"]):
        return cfg["sliding_window"]
    return 0


def attention_block(h: torch.Tensor, W: Dict[str, torch.Tensor], prefix: str, cfg: dict, window: int) -> torch.Tensor:
    """src/locus/model/arch.cpp:596-696 and src/locus/model/llama.cpp:487: q, k, v with bias,
    rotation of q and k, causal attention, output projection without bias."""
    T = h.shape[0]
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    pos = torch.arange(T)

    def proj(name):
        y = h @ W[f"{prefix}.{name}.weight"].T
        b = W.get(f"{prefix}.{name}.bias")
        return y + b if b is not None else y

    q = rope_half_split(proj("q_proj").view(T, nh, hd), pos, cfg["rope_theta"])
    k = rope_half_split(proj("k_proj").view(T, nkv, hd), pos, cfg["rope_theta"])
    v = proj("v_proj").view(T, nkv, hd)
    o = attention(q, k, v, window).reshape(T, nh * hd)
    return o @ W[f"{prefix}.o_proj.weight"].T


class _CastOnRead:
    """The checkpoint's tensors, converted to the working type when read (a large model converted
    as a whole would not fit in memory).  ``weights`` may be any mapping, also one that makes a
    tensor only when it is asked for."""

    def __init__(self, weights, dtype):
        self.weights = weights
        self.dtype = dtype

    def __getitem__(self, name):
        return self.weights[name].to(self.dtype)

    def __contains__(self, name):
        return name in self.weights

    def get(self, name, default=None):
        return self[name] if name in self.weights else default

    def rows(self, name, idx):
        """Rows ``idx`` of a matrix, without converting the rest of it."""
        return self.weights[name][idx].to(self.dtype)


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int],
            dtype: torch.dtype = torch.float32, forced_routing: Optional[dict] = None,
            aux: Optional[dict] = None, positions: Optional[Sequence[int]] = None) -> torch.Tensor:
    """src/locus/model/llama.cpp:426-515: embed; per layer x += attn(norm(x)), x += ffn(norm(x));
    final norm; head (the embedding when tied).  Returns logits [T, vocab] for every position, or for
    ``positions`` only.
    ``forced_routing``: {"model.layers.N.mlp": [experts of token 0, of token 1, ...]}."""
    W = _CastOnRead(weights, dtype)
    eps = cfg["rms_norm_eps"]
    x = W.rows("model.embed_tokens.weight", torch.tensor(list(tokens), dtype=torch.long))
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}"
        h = rmsnorm(x, W[f"{p}.input_layernorm.weight"], eps)
        x = x + attention_block(h, W, f"{p}.self_attn", cfg, layer_window(cfg, l))
        h = rmsnorm(x, W[f"{p}.post_attention_layernorm.weight"], eps)
        if is_moe_layer(cfg, l):
            x = x + moe_block(h, W, f"{p}.mlp", cfg, (forced_routing or {}).get(f"{p}.mlp"), aux)
        else:
            x = x + swiglu_mlp(h, W[f"{p}.mlp.gate_proj.weight"], W[f"{p}.mlp.up_proj.weight"],
                               W[f"{p}.mlp.down_proj.weight"])
    h = rmsnorm(x, W["model.norm.weight"], eps)
    if positions is not None:
        h = h[torch.tensor(list(positions), dtype=torch.long)]
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else W["lm_head.weight"]
    return h @ head.T


def argmax(logits: torch.Tensor) -> int:
    """src/locus/model/llama.cpp:1237-1245: the first maximum wins."""
    best = 0
    for i in range(1, logits.shape[0]):
        if logits[i] > logits[best]:
            best = i
    return best


def greedy_generate(cfg: dict, weights, prompt: Sequence[int], n_new: int, dtype=torch.float32) -> List[int]:
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        t = int(torch.argmax(forward(cfg, weights, toks, dtype)[-1]).item())
        out.append(t)
        toks.append(t)
    return out


def apply_penalties(logits: torch.Tensor, history: Sequence[int], repeat_penalty: float, frequency_penalty: float,
                    presence_penalty: float, repeat_last_n: int) -> torch.Tensor:
    """src/locus/model/sampling.cpp:16-43."""
    out = logits.clone()
    if repeat_penalty == 1.0 and frequency_penalty == 0.0 and presence_penalty == 0.0:
        return out
    hist = list(history)[-repeat_last_n:] if repeat_last_n > 0 else []
    counts: Dict[int, int] = {}
    for t in hist:
        counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        if t >= out.shape[0]:
            continue
        l = out[t]
        if repeat_penalty != 1.0:
            l = l / repeat_penalty if l > 0 else l * repeat_penalty
        out[t] = l - (frequency_penalty * c + presence_penalty)
    return out


def kept_distribution(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0,
                      min_p: float = 0.0) -> Dict[int, float]:
    """src/locus/model/sampling.cpp:67-134: candidates sorted by logit, top-k cut, softmax
    of (logit - max) / T in double, top-p prefix, min-p cut; returns {token: probability}
    renormalised over the kept tokens (the reference draws uniformly in [0, kept_sum))."""
    order = sorted(range(logits.shape[0]), key=lambda i: (-float(logits[i]), i))
    if 0 < top_k < len(order):
        order = order[:top_k]
    mx = float(logits[order[0]])
    w = [math.exp((float(logits[i]) - mx) / temperature) for i in order]
    total = sum(w)
    keep = len(order)
    if top_p < 1.0:
        cum = 0.0
        for j, wj in enumerate(w):
            cum += wj / total
            if cum >= top_p:
                keep = j + 1
                break
    if min_p > 0.0:
        thresh = min_p * (w[0] / total)
        for j in range(1, keep):
            if w[j] / total < thresh:
                keep = j
                break
    kept_sum = sum(w[:keep])
    return {order[j]: w[j] / kept_sum for j in range(keep)}


def load_folder(model_dir: str):
    """(config dict, weights dict) of a model folder, read with the safetensors library."""
    import json
    import os

    from safetensors import safe_open

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            weights[k] = f.get_tensor(k)
    return cfg, weights
