"""Attention mixer over the paged cache: grouped-query attention with optional q/k/v bias,
a position encoding, an optional window, and an output projection.

Per token, as the reference computes it (``qwen2moe_attention``,
src/locus/model/arch.cpp:596-696): q = Wq.h + bq, k = Wk.h + bk, v = Wv.h + bv
(arch.cpp:618-620, 650-655); q and k rotated (arch.cpp:621-622, 656-657), v not; k and v
written to the cache at the token's position; for head h with kv head h // (heads/kv_heads):
scores = q.k * 1/sqrt(head_dim) over the keys 0..pos (arch.cpp:668-681), softmax
(arch.cpp:682), weighted sum of v (arch.cpp:683-694); output = Wo.concat(heads), added to
the residual stream (src/locus/model/llama.cpp:487-490).

The three projections are one product against the stacked weight [(heads + 2 kv_heads) *
head_dim, hidden]; that is layout only.  Scores, softmax and the weighted sum are float32.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels as K
from .base import Mixer, PagedKvSpec, PartSpec, StepPlan, TensorSource, make_part, register_mixer

CHUNK_TILE = 16  # queries per work item of the CUDA-core chunk kernel


class AttentionTiles(StepPlan):
    """The work lists of this file's attention kernels: tiles of 16 queries (CUDA-core kernel) and of 64 queries
    (tensor-core kernels) over the segments with more than one new token, and the segments with exactly one
    (the decode kernel).  One plan serves every attention layer of a model.  The lists are made by two small
    native helpers (csrc/host_core.cpp: ``locus_plan_query_tiles``, ``locus_plan_segments_with``).  The tiles are
    listed by the position of their first query, ascending, across requests: the kernels walk a list from its end,
    so the tiles with the most keys start first (``locus_sort_tiles_by_position``)."""

    key = ("attention.tiles", CHUNK_TILE, K.MMA_QUERY_TILE)

    def __init__(self) -> None:
        from ..cache import native

        self._lib = native.lib()

    def capacity(self, max_tokens: int, max_segments: int) -> int:
        tiles = max_tokens // CHUNK_TILE + max_tokens // K.MMA_QUERY_TILE + 2 * max_segments
        return 2 * tiles + max_segments

    def build(self, seg_q0, seg_qn, seg_ctx, out):
        n_seg, qn, cap = len(seg_qn), seg_qn.ctypes.data, len(out)
        base = out.ctypes.data
        n16 = self._lib.locus_plan_query_tiles(n_seg, qn, CHUNK_TILE, 2, base, cap)
        o64 = 2 * max(n16, 0)
        n64 = self._lib.locus_plan_query_tiles(n_seg, qn, K.MMA_QUERY_TILE, 2, base + 4 * o64, cap - o64)
        o1 = o64 + 2 * max(n64, 0)
        n1 = self._lib.locus_plan_segments_with(n_seg, qn, 1, base + 4 * o1, cap - o1)
        if n16 < 0 or n64 < 0 or n1 < 0:
            raise ValueError("attention: the step has more tiles than the plan's capacity holds")
        ctx = seg_ctx.ctypes.data
        self._lib.locus_sort_tiles_by_position(n16, base, ctx)
        self._lib.locus_sort_tiles_by_position(n64, base + 4 * o64, ctx)
        return {"chunk_items": (0, 2 * n16, (-1, 2)), "n_chunk_items": n16,
                "chunk_items64": (o64, 2 * n64, (-1, 2)), "n_chunk_items64": n64,
                "decode_items": (o1, n1, None), "n_decode_items": n1}


class Attention(Mixer):
    def __init__(self, prefix: str, *, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 qkv_bias: bool, o_bias: bool = False, window: int = 0,
                 position: PartSpec = PartSpec("none"), softmax_scale: Optional[float] = None) -> None:
        super().__init__(prefix)
        if n_heads % n_kv_heads:
            raise ValueError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if head_dim % 16 or not (16 <= head_dim <= 256):
            raise ValueError(f"attention: head_dim {head_dim} is not a multiple of 16 in 16..256 "
                             "(the attention kernels take no other head size)")
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim = hidden, n_heads, n_kv_heads, head_dim
        self.qkv_bias, self.o_bias, self.window = bool(qkv_bias), bool(o_bias), int(window)
        self.scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = make_part("position", position, prefix + ".position")
        self.q_dim = n_heads * head_dim
        self.kv_dim = n_kv_heads * head_dim

    def sub_parts(self):
        return [self.position]

    # -- weights ------------------------------------------------------------
    def param_shapes(self):
        shapes = {"wqkv": (self.q_dim + 2 * self.kv_dim, self.hidden), "wo": (self.hidden, self.q_dim)}
        if self.qkv_bias:
            shapes["bqkv"] = (self.q_dim + 2 * self.kv_dim,)
        if self.o_bias:
            shapes["bo"] = (self.hidden,)
        return shapes

    def sources(self):
        p = self.prefix
        rows = [("q_proj", 0, self.q_dim), ("k_proj", self.q_dim, self.kv_dim),
                ("v_proj", self.q_dim + self.kv_dim, self.kv_dim)]
        out = [TensorSource(f"{p}.{n}.weight", (size, self.hidden), "wqkv", row0) for n, row0, size in rows]
        if self.qkv_bias:
            out += [TensorSource(f"{p}.{n}.bias", (size,), "bqkv", row0, "bias") for n, row0, size in rows]
        out.append(TensorSource(f"{p}.o_proj.weight", (self.hidden, self.q_dim), "wo"))
        if self.o_bias:
            out.append(TensorSource(f"{p}.o_proj.bias", (self.hidden,), "bo", 0, "bias"))
        return out

    def kernel_modules(self, dtype):
        return ["elementwise", "gemm_simt", "gemv", "attention"] + (["gemm_skinny", "gemm_tc", "attention_mma", "attention_tc", "attention_gqa"] if dtype == torch.bfloat16 else [])

    def cache_needs(self):
        return PagedKvSpec(self.n_kv_heads, self.head_dim, self.window), None

    def step_plans(self):
        return [AttentionTiles()]

    # -- forward ------------------------------------------------------------
    def forward(self, h, batch, cache, residual, rt) -> None:
        T = batch.T
        gb = batch.groups[cache.group]
        qkv = rt.rows("attention.qkv", self.q_dim + 2 * self.kv_dim, rt.dtype, T)
        K.linear(h, self.params["wqkv"], qkv, bias=self.params.get("bqkv"))
        table = self.position.rotary_table()
        if table is None:
            # an encoding without a rotary table transforms q and k in place itself
            self.position.apply(qkv[:, : self.q_dim], qkv[:, self.q_dim : self.q_dim + self.kv_dim],
                                batch.positions)
        q = rt.rows("attention.q", self.q_dim, rt.dtype, T)
        K.rope_kv_write(
            qkv, batch.positions, table.inv_freq if table else None, q, cache.pool, gb.slots,
            n_heads=self.n_heads, n_kv_heads=self.n_kv_heads, head_dim=self.head_dim,
            rot_dim=table.rot_dim if table else 0, interleaved=table.interleaved if table else False,
            page_tokens=gb.page_tokens, write_kv=cache.writes,
        )
        o = rt.rows("attention.o", self.q_dim, rt.dtype, T)
        common = dict(seg_q0=batch.seg_q0, seg_qn=batch.seg_qn, seg_ctx=batch.seg_ctx,
                      block_table=gb.block_table, n_heads=self.n_heads, n_kv_heads=self.n_kv_heads,
                      head_dim=self.head_dim, page_tokens=gb.page_tokens, window=self.window,
                      scale=self.scale)
        tiles = batch.plans[AttentionTiles.key]
        # splits of 128 keys that cover the longest context (all that the block table can describe when the
        # step's launches must not depend on its lengths)
        cap_splits = (gb.block_table.shape[1] * gb.page_tokens - 1) // K.DECODE_SPLIT + 1
        max_splits = cap_splits if batch.static_shapes else min(cap_splits, (max(batch.longest, 1) - 1) // K.DECODE_SPLIT + 1)
        if tiles["n_chunk_items"]:
            # few query tiles behind a long context: the keys of every tile are cut into ranges
            keys = max_splits * K.DECODE_SPLIT
            if self.window > 0:
                keys = min(keys, self.window + K.TC_ATTN_QUERY_BLOCK)
            if K.attn_chunk_tc_takes(q, self.head_dim, gb.page_tokens, T, keys):
                n_splits = K.attn_chunk_tc_splits(tiles["n_chunk_items64"], self.n_heads, keys)
                part_o = part_ml = None
                if n_splits > 1:
                    n_o, n_ml = K.attn_chunk_tc_scratch()
                    part_o = rt.buf("attention.chunk_tc_part_o", (n_o,), torch.float32)
                    part_ml = rt.buf("attention.chunk_tc_part_ml", (n_ml,), torch.float32)
                K.attn_chunk_tc(q, cache.pool, o, items=tiles["chunk_items64"], n_items=tiles["n_chunk_items64"],
                                n_splits=n_splits, part_o=part_o, part_ml=part_ml, **common)
            elif K.attn_chunk_mma_takes(q, self.head_dim):
                n_splits = K.attn_chunk_mma_splits(tiles["n_chunk_items64"], self.n_heads, keys)
                part_o = part_ml = None
                if n_splits > 1:
                    n_o, n_ml = K.attn_chunk_mma_scratch(self.head_dim)
                    part_o = rt.buf("attention.chunk_part_o", (n_o,), torch.float32)
                    part_ml = rt.buf("attention.chunk_part_ml", (n_ml,), torch.float32)
                K.attn_chunk_mma(q, cache.pool, o, items=tiles["chunk_items64"], n_items=tiles["n_chunk_items64"],
                                 n_splits=n_splits, part_o=part_o, part_ml=part_ml, **common)
            else:
                K.attn_chunk(q, cache.pool, o, items=tiles["chunk_items"], n_items=tiles["n_chunk_items"], **common)
        if tiles["n_decode_items"]:
            n = tiles["n_decode_items"]
            # scratch sized once, for the longest context that the block table can describe
            units = K.decode_units(rt.max_segments, self.n_heads, self.head_dim, q.dtype, cap_splits, rt.device,
                                   gb.page_tokens, self.n_kv_heads)
            part_o = rt.buf("attention.part_o", (units * self.head_dim,), torch.float32)
            part_ml = rt.buf("attention.part_ml", (2 * units,), torch.float32)
            counters = rt.shared_object(
                ("attention.counters", rt.max_segments * self.n_heads),
                lambda: torch.zeros(rt.max_segments * self.n_heads, dtype=torch.int32, device=rt.device),
            )
            K.attn_decode(q, cache.pool, o, items=tiles["decode_items"], n_items=n, part_o=part_o,
                          part_ml=part_ml, counters=counters, max_splits=max_splits, **common)
        K.linear(o, self.params["wo"], residual, bias=self.params.get("bo"), accumulate=True)


register_mixer("attention", Attention)
