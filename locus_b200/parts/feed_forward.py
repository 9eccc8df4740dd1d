"""Feed-forward parts: the dense SwiGLU MLP and the sparse mixture of experts.

Dense (src/locus/model/llama.cpp:493-503 of the reference):
    out = Wdown . (silu(Wgate . h) * (Wup . h)),  silu(g) = g / (1 + exp(-g))
    (``silu_mul``, src/locus/backend/cpu_ops.cpp:1736-1743).

Sparse (``moe_ffn`` llama.cpp:992-1077, ``moe_select`` llama.cpp:900-980):
    r = Wr . h; p = softmax(r) over all experts; pick top-k by k rounds of arg-max with
    strict '>' (ties to the lowest index); weight w_e = p_e / wsum * scale with
    wsum = sum of picked p_e when ``norm_topk`` else 1; out = sum over picked e, in pick
    order, of w_e * SwiGLU_e(h); then the shared expert, scaled by
    sigmoid(w_shared_gate . h) when it is gated (llama.cpp:1062-1076), is added.

The batched form lays the (token, slot) pairs out by expert, runs each expert over its
tokens, and sums each token's pairs in slot order without atomics (the reference's
``moe_ffn_batch``, llama.cpp:1079-1235, does the same to stay byte-identical).
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import FeedForward, PendingAdd, TensorSource, register_feed_forward


class DenseMlp(FeedForward):
    def __init__(self, prefix: str, *, hidden: int, intermediate: int) -> None:
        super().__init__(prefix)
        self.hidden, self.inter = int(hidden), int(intermediate)

    def param_shapes(self):
        return {"w_gate": (self.inter, self.hidden), "w_up": (self.inter, self.hidden),
                "w_down": (self.hidden, self.inter)}

    def sources(self):
        p = self.prefix
        return [
            TensorSource(f"{p}.gate_proj.weight", (self.inter, self.hidden), "w_gate"),
            TensorSource(f"{p}.up_proj.weight", (self.inter, self.hidden), "w_up"),
            TensorSource(f"{p}.down_proj.weight", (self.hidden, self.inter), "w_down"),
        ]

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def forward(self, h, batch, residual, rt, row_scale=None) -> None:
        self.forward_down(self.forward_up(h, rt), residual, rt, row_scale)

    # The two products on their own, for a caller that has something to do between them (the shared expert of a
    # routed feed-forward starts before the router has made the scale of its second product).
    def forward_up(self, h, rt) -> torch.Tensor:
        act = rt.rows(f"dense_mlp.act{self.inter}", self.inter, rt.dtype, h.shape[0])
        K.linear(h, self.params["w_gate"], act, w2=self.params["w_up"])
        return act

    def forward_down(self, act, residual, rt, row_scale=None) -> None:
        K.linear(act, self.params["w_down"], residual, accumulate=True, row_scale=row_scale)


# Up to this many tokens in a step the shared expert's first product starts beside the router instead of behind it
# (decode steps of the 2.7B sizes at 4,096 tokens of context: 1.995 -> 1.81 ms at one request, 4.14 -> 3.97 at 8,
# 6.83 -> 6.40 at 16, 9.00 -> 8.88 at 32; at 64 the router and the product get in each other's way: 13.27 -> 13.37).
SHARED_EARLY_TOKENS = 32
SHARED_OVERLAP_FROM = 1024   # steps of at least this many tokens ...
SHARED_OVERLAP_ROWS = 192    # ... and at most this many rows per routed expert run the shared expert on the side stream


class SparseMoe(FeedForward):
    """Softmax top-k routed SwiGLU experts plus an optional (gated) shared SwiGLU expert."""

    def __init__(self, prefix: str, *, hidden: int, n_experts: int, top_k: int, norm_topk: bool,
                 expert_intermediate: int, shared_intermediate: int = 0, shared_gate: bool = True,
                 weight_scale: float = 1.0, score_fn: str = "softmax", selection_bias: bool = False,
                 n_group: int = 1, n_group_used: int = 1) -> None:
        """``score_fn``: "softmax" over all experts or "sigmoid" of each router logit; ``selection_bias``:
        a float32 tensor ``<prefix>.gate.selection_bias`` [n_experts] is added to the scores for the
        selection only; ``n_group`` > 1: group-limited routing with ``n_group_used`` groups (the
        parameters of the reference's ``moe_select``, src/locus/model/llama.cpp:900-980)."""
        super().__init__(prefix)
        if not (1 <= top_k <= n_experts):
            raise ValueError(f"sparse_moe: top_k {top_k} must be within 1..{n_experts}")
        if score_fn not in K.SCORE_FUNCTIONS:
            raise ValueError(f"sparse_moe: score function {score_fn!r} (known: {', '.join(K.SCORE_FUNCTIONS)})")
        if not (1 <= n_group <= 32) or n_experts % n_group or not (1 <= n_group_used <= n_group):
            raise ValueError(f"sparse_moe: {n_group} groups ({n_group_used} used) do not fit {n_experts} experts")
        self.score_fn, self.has_sel_bias = score_fn, bool(selection_bias)
        self.n_group, self.n_group_used = int(n_group), int(n_group_used)
        self.hidden, self.E, self.k = int(hidden), int(n_experts), int(top_k)
        self.norm_topk, self.I, self.Is = bool(norm_topk), int(expert_intermediate), int(shared_intermediate)
        self.shared_gate = bool(shared_gate) and self.Is > 0
        self.weight_scale = float(weight_scale)
        self.shared = (DenseMlp(prefix + ".shared_expert", hidden=hidden, intermediate=self.Is)
                       if self.Is > 0 else None)
        self._layout = None
        self._scratch = None
        self._router_all = None
        # telemetry hook: called with (prefix, ids [T, k], weights [T, k]) after routing; the
        # reference counts expert hits per layer the same way (src/locus/model/moe_stats.cpp:23-78)
        self.observer = None

    def sub_parts(self):
        return [self.shared] if self.shared is not None else []

    def param_shapes(self):
        s = {
            "router": (self.E, self.hidden),
            "gate_exps": (self.E, self.I, self.hidden),
            "up_exps": (self.E, self.I, self.hidden),
            "down_exps": (self.E, self.hidden, self.I),
        }
        if self.shared_gate:
            s["shared_gate"] = (1, self.hidden)
        if self.has_sel_bias:
            s["sel_bias"] = (self.E,)
        return s

    def sources(self):
        p = self.prefix
        out = [TensorSource(f"{p}.gate.weight", (self.E, self.hidden), "router")]
        for e in range(self.E):
            out.append(TensorSource(f"{p}.experts.{e}.gate_proj.weight", (self.I, self.hidden), "gate_exps", e * self.I))
            out.append(TensorSource(f"{p}.experts.{e}.up_proj.weight", (self.I, self.hidden), "up_exps", e * self.I))
            out.append(TensorSource(f"{p}.experts.{e}.down_proj.weight", (self.hidden, self.I), "down_exps",
                                    e * self.hidden))
        if self.shared_gate:
            out.append(TensorSource(f"{p}.shared_expert_gate.weight", (1, self.hidden), "shared_gate"))
        if self.has_sel_bias:
            out.append(TensorSource(f"{p}.gate.selection_bias", (self.E,), "sel_bias", 0, "bias"))
        return out

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv", "moe_route", "elementwise"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def bind(self, rt) -> None:
        self._layout = rt.shared_object(
            ("expert_layout", self.E, self.k),
            lambda: K.ExpertLayout(rt.max_tokens * self.k, self.E, 64, rt.device),
        )
        self._scratch = rt.shared_object(
            ("router_scratch", self.E + 1),
            lambda: K.RouterScratch(rt.max_tokens, self.E + 1, rt.device),
        )
        self._router_all = None
        bias = self.params.get("sel_bias")
        self._rule = dict(top_k=self.k, renorm=self.norm_topk, scale=self.weight_scale, score_fn=self.score_fn,
                          sel_bias=bias.float().contiguous() if bias is not None else None, n_group=self.n_group,
                          n_group_used=self.n_group_used)
        r, g = self.params["router"], self.params.get("shared_gate")
        if (rt.dtype == torch.bfloat16 and r.dtype == torch.bfloat16 and self.hidden % 8 == 0
                and (g is None or g.dtype == torch.bfloat16)):
            # router rows and the gate row as one matrix (a copy of a few hundred KB)
            self._router_all = torch.cat([r, g.view(1, -1)], 0).contiguous() if g is not None else r

    def forward(self, h, batch, residual, rt) -> None:
        T = h.shape[0]
        n_pairs = T * self.k
        ids = rt.buf("moe.ids", (rt.max_tokens * self.k,), torch.int32)
        wts = rt.buf("moe.wts", (rt.max_tokens * self.k,), torch.float32)
        gamma = rt.buf("moe.gamma", (rt.max_tokens,), torch.float32) if self.shared_gate else None
        lay = self._layout
        # which kernels the expert products run on decides the row tile of the expert layout
        tile = K.FEW_ROWS if T <= K.FEW_ROWS else K.expert_tile(n_pairs, self.E)
        widths_ok = self.I % 8 == 0 and self.hidden % 8 == 0
        all_bf16 = (K.tensor_cores_take(h, self.params["gate_exps"]) and widths_ok
                    and self.params["down_exps"].dtype == torch.bfloat16)
        if not all_bf16 and widths_ok and n_pairs <= K.FEW_ROWS * self.E:
            # No tensor-core form (float32) and a handful of rows per expert: tiles of 8 rows on the row-streaming
            # kernel read an expert's weights once per tile, where the CUDA-core product would compute a 64-row
            # tile for every expert that has a row.
            tile = K.FEW_ROWS
        streamed = (all_bf16 and tile <= K.SKINNY_TILE_ROWS) or (widths_ok and tile <= K.FEW_ROWS)
        if not streamed and not all_bf16:
            tile = 64
        sorted_already = False
        # The shared expert needs only h for its first product: for a few tokens, where no kernel fills the GPU, it
        # starts on the side stream beside the router; its second product waits for the router's gate (below).
        # Long portions, too, while the routed experts wait for their weights rather than for the tensor cores
        # (fewer than about 190 rows per expert: flops / peak < bytes / bandwidth): the shared expert's products,
        # which are bound by the tensor cores, then run beside the router, the selection, the layout and the gather
        # and fill what the routed products leave idle.  (2,048 tokens of the 2.7B sizes in one step 12.6 -> 11.7 ms,
        # in two steps of 1,024 17.5 -> 15.2 ms; steps of 512 tokens lose, 27.6 -> 28.7 ms, and so do the 57B sizes'
        # steps of 4,096 and 8,192 tokens, whose experts are bound by the tensor cores: 1,254 -> 1,289 ms.)
        long_overlap = T >= SHARED_OVERLAP_FROM and n_pairs <= SHARED_OVERLAP_ROWS * self.E
        overlap = self.shared is not None and (T <= 64 or long_overlap)
        shared_act = None
        if overlap and (T <= SHARED_EARLY_TOKENS or long_overlap):
            with rt.side():
                shared_act = self.shared.forward_up(h, rt)
        if self._router_all is not None and K.USE_TENSOR_CORES:
            # bfloat16: router (and gate) logits on the tensor cores, one kernel for every batch shape
            logits = self._scratch.logits.view(rt.max_tokens, self.E + 1)
            if K.route_small_takes(T, self.k, self.E):
                # a decode-sized batch: logits, selection and the expert layout in one launch
                K.route_fused_small(h, self._router_all, logits, self.E, self.shared_gate, ids, wts, gamma, lay,
                                    self._scratch.fused_counter, n_tokens=T, tile_m=tile, **self._rule)
                sorted_already = True
            else:
                K.router_logits(h, self._router_all, logits)
                K.router_select(logits, self.E, self.shared_gate, ids, wts, gamma, n_tokens=T, **self._rule)
        else:
            K.router_topk(h, self.params["router"], self.params.get("shared_gate"), ids, wts, gamma,
                          scratch=self._scratch, **self._rule)
        if self.observer is not None:
            self.observer(self.prefix, ids[:n_pairs].view(T, self.k), wts[:n_pairs].view(T, self.k))
        # The rest of the shared expert runs beside the routed experts on the side stream and is joined before the
        # combine (both add into the residual, so they must not overlap there).
        if overlap:
            with rt.side():
                if shared_act is not None:
                    self.shared.forward_down(shared_act, residual, rt, row_scale=gamma)
                else:
                    self.shared.forward(h, batch, residual, rt, row_scale=gamma)
        act = rt.rows(f"moe.act{self.I}", self.I, rt.dtype, n_pairs, per_token=self.k)
        if not sorted_already:
            # the second product of the tensor-core path may walk the layout in larger tiles
            tile2 = K.expert_second_tile(n_pairs, self.E) if (all_bf16 and not streamed) else 0
            K.moe_sort(ids, n_pairs, lay, tile, tile2)
        if streamed or not all_bf16:
            # few rows per expert (or no tensor-core form): the kernels gather the token rows themselves
            K.linear(h, self.params["gate_exps"], act, w2=self.params["up_exps"], x_rows=lay.sorted_pair,
                     x_row_div=self.k, layout=lay, n_rows=n_pairs)
        else:
            # tcgen05 kernel: TMA reads whole row ranges, so lay the tokens out in expert order first
            xs = rt.rows("moe.x_sorted", self.hidden, rt.dtype, n_pairs, per_token=self.k)
            K.gather_rows(h, lay.sorted_pair, self.k, xs, n_pairs)
            K.linear(xs, self.params["gate_exps"], act, w2=self.params["up_exps"], layout=lay, n_rows=n_pairs)
        # the experts' weighted outputs, one row per (token, slot): in the model's element type (in bfloat16 a row is
        # rounded once more, like every activation between kernels; their sum, the residual stream, stays float32)
        pair_dt = torch.bfloat16 if (all_bf16 and rt.dtype == torch.bfloat16) else torch.float32
        pair_out = rt.rows("moe.pair_out", self.hidden, pair_dt, n_pairs, per_token=self.k)
        K.linear(act, self.params["down_exps"], pair_out, layout=lay, n_rows=n_pairs, row_scale=wts,
                 scale_rows=lay.sorted_pair, lists_ready=True, second_tiles=True)
        if overlap:
            rt.join()
        if self.shared is not None and not overlap:
            self.shared.forward(h, batch, residual, rt, row_scale=gamma)
        if rt.defer_add and K.rmsnorm_adds(residual):
            # the sum of the experts' outputs is folded into the next block's first norm
            rt.leave_pending(PendingAdd(pair_out, lay.pair_pos, self.k))
        else:
            K.moe_combine(residual, pair_out, lay.pair_pos, self.k)


register_feed_forward("dense_mlp", DenseMlp)
register_feed_forward("sparse_moe", SparseMoe)
