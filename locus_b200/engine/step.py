"""The step function: one ragged batch of (request, its next tokens) through the model.

``ModelRunner.step(entries)`` runs exactly the tokens it is given -- portions of prompts
beside single decoded tokens, cut anywhere -- as one batch against the cache that earlier
steps left, writes their keys and values, and returns float32 logits at the wanted places.
The reference has three entry points for this (``forward``, ``forward_batch``,
``forward_batch_decode``, src/locus/model/llama.hpp:173-241) and never mixes prompt
portions with decode tokens in one call (src/locus/engine/engine.cpp:527-539, 608-618);
here there is one call.

Preconditions are checked on the host before anything is launched (the reference does the
same, src/locus/model/llama.cpp:432-445, 575-578): token ids in range, capacity ensured by
the caller (``CacheManager.ensure_capacity``), positions within the model's limit.  All
descriptors of a step travel to the device as one pinned int32 buffer.

Steps that consist of one new token per request can be replayed from a CUDA graph keyed
by the number of requests; every other shape is launched kernel by kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheError, CacheManager, SeqCache
from .. import kernels as K
from ..kernels import DECODE_SPLIT
from .batch import GroupBatch, Runtime, StepBatch

CHUNK_TILE = 16  # queries per work item of the chunk attention kernel


class StepError(ValueError):
    pass


@dataclass
class StepEntry:
    seq: SeqCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


class ModelRunner:
    def __init__(self, model, cache: CacheManager, *, max_tokens: int, max_segments: int,
                 max_wanted: Optional[int] = None, use_graphs: bool = False) -> None:
        self.model = model
        self.cache = cache
        self.device = model.device
        self.max_tokens = max_tokens
        self.max_segments = max_segments
        self.max_wanted = max_wanted if max_wanted is not None else max_tokens
        self.use_graphs = use_graphs
        self.rt = Runtime(self.device, model.dtype, max_tokens, max_segments, self.max_wanted)
        model.bind(self.rt)
        self.layer_caches = cache.layer_caches()
        G = len(cache.groups)
        W = cache.table_width
        items_max = max_tokens // CHUNK_TILE + max_segments + 1
        size = (max_tokens * (2 + G) + max_segments * (5 + G * W) + self.max_wanted + 4 * items_max)
        # two pinned staging buffers, used in turn: a buffer is rewritten only after the copy
        # that read it has finished (its event), so steps may be queued without a host sync
        on_gpu = self.device.type == "cuda"
        self._hosts = [torch.empty(size, dtype=torch.int32, pin_memory=on_gpu) for _ in range(2)]
        self._host_events = [torch.cuda.Event() if on_gpu else None for _ in range(2)]
        self._host_used = [False, False]
        self._host_turn = 0
        self._dev = torch.empty(size, dtype=torch.int32, device=self.device)
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self._graph_logits: Dict[int, torch.Tensor] = {}
        self._graph_launches: Dict[int, int] = {}
        self.launch_counter = 0
        self.stats = {"steps": 0, "tokens": 0, "graph_replays": 0, "h2d_bytes": 0}

    # ------------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        plan = self.model.plan
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.max_segments:
            raise StepError(f"{len(entries)} requests in a step, the runner was built for {self.max_segments}")
        seen = set()
        T = 0
        n_want = 0
        for e in entries:
            if id(e.seq) in seen:
                raise StepError(f"request {e.seq.seq_id!r} appears twice in a step")
            seen.add(id(e.seq))
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.seq.seq_id!r}: no tokens in its entry")
            for t in e.tokens:
                if not (0 <= int(t) < plan.vocab_size):
                    raise StepError(f"request {e.seq.seq_id!r}: token {t} outside the vocabulary "
                                    f"0..{plan.vocab_size - 1}")
            if e.seq.n_tokens + n > plan.max_positions:
                raise StepError(f"request {e.seq.seq_id!r}: context overflow, {e.seq.n_tokens + n} tokens "
                                f"exceed max_position_embeddings {plan.max_positions}")
            if not e.seq.open or self.cache.get(e.seq.seq_id) is not e.seq:
                raise CacheError(f"request {e.seq.seq_id!r} is not open in the runner's cache")
            if e.seq.n_tokens + n > self.cache.capacity(e.seq):
                raise CacheError(f"request {e.seq.seq_id!r}: capacity for {n} more tokens was not ensured")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {e.seq.seq_id!r}: wanted place {w} is not among its {n} tokens")
            T += n
            n_want += len(e.want)
        if T > self.max_tokens:
            raise StepError(f"{T} tokens in a step, the runner was built for {self.max_tokens}")
        if n_want > self.max_wanted:
            raise StepError(f"{n_want} logits rows wanted, the runner was built for {self.max_wanted}")

    def _build(self, entries: Sequence[StepEntry], fixed_splits: bool) -> StepBatch:
        cache = self.cache
        P = cache.page_tokens
        W = cache.table_width
        tokens: List[int] = []
        positions: List[int] = []
        seg_q0, seg_qn, seg_ctx, slots_state, want_rows = [], [], [], [], []
        chunk_items: List[int] = []
        chunk_items64: List[int] = []
        decode_items: List[int] = []
        longest = 0
        for s, e in enumerate(entries):
            n, ctx = len(e.tokens), e.seq.n_tokens
            seg_q0.append(len(tokens))
            seg_qn.append(n)
            seg_ctx.append(ctx)
            slots_state.append(e.seq.state_slot)
            for w in e.want:
                want_rows.append(len(tokens) + int(w))
            tokens.extend(int(t) for t in e.tokens)
            positions.extend(range(ctx, ctx + n))
            longest = max(longest, ctx + n)
            if n == 1:
                decode_items.append(s)
            else:
                for q in range(0, n, CHUNK_TILE):
                    chunk_items.extend((s, q))
                for q in range(0, n, K.MMA_QUERY_TILE):
                    chunk_items64.extend((s, q))
        T, n_seg = len(tokens), len(entries)
        fields = [tokens, positions, seg_q0, seg_qn, seg_ctx, slots_state, want_rows, chunk_items, decode_items,
                  chunk_items64]
        group_fields = []
        for g in cache.groups:
            slots: List[int] = []
            table: List[int] = []
            for e in entries:
                row = e.seq.tables[g.gid]
                ctx = e.seq.n_tokens
                for pos in range(ctx, ctx + len(e.tokens)):
                    page = row[pos // P]
                    if page < 0:
                        raise CacheError(f"request {e.seq.seq_id!r}: position {pos} lies in a page given back")
                    slots.append(page * P + pos % P)
                table.extend(row)
                table.extend([-1] * (W - len(row)))
            group_fields.append((slots, table))
            fields.extend((slots, table))
        off = 0
        views = []
        turn = self._host_turn
        self._host_turn ^= 1
        if self._host_used[turn] and self._host_events[turn] is not None:
            self._host_events[turn].synchronize()
        host = self._hosts[turn]
        hn = host.numpy()
        for f in fields:
            n = len(f)
            if n:
                hn[off : off + n] = f
            views.append((off, n))
            off += n
        self._dev[:off].copy_(host[:off], non_blocking=True)
        if self._host_events[turn] is not None:
            self._host_events[turn].record()
            self._host_used[turn] = True
        self.stats["h2d_bytes"] += off * 4

        def dv(i):
            o, n = views[i]
            return self._dev[o : o + n]

        max_splits = (cache.max_seq_tokens - 1) // DECODE_SPLIT + 1 if fixed_splits else (longest - 1) // DECODE_SPLIT + 1
        batch = StepBatch(
            T=T, n_seg=n_seg, tokens=dv(0), positions=dv(1), seg_q0=dv(2), seg_qn=dv(3), seg_ctx=dv(4),
            state_slots=dv(5), want_rows=dv(6), n_want=len(want_rows),
            chunk_items=dv(7).view(-1, 2), n_chunk_items=len(chunk_items) // 2,
            chunk_items64=dv(9).view(-1, 2), n_chunk_items64=len(chunk_items64) // 2,
            decode_items=dv(8), n_decode_items=len(decode_items), max_splits=max_splits,
            host_seg_q0=seg_q0, host_seg_qn=seg_qn, host_seg_ctx=seg_ctx, host_state_slots=slots_state,
        )
        for gi, g in enumerate(cache.groups):
            batch.groups[g.gid] = GroupBatch(block_table=dv(10 + 2 * gi + 1).view(n_seg, W), slots=dv(10 + 2 * gi),
                                             page_tokens=P)
        return batch

    def check_device_errors(self) -> None:
        """Raise if a kernel recorded a fault since the last check (a bounded wait of the
        tensor-core pipeline that ran out).  Synchronises the device."""
        if self.device.type == "cuda" and "gemm_tc" in K._LIBS:
            code = K.tc_error()
            if code:
                raise RuntimeError(f"tensor-core kernel fault: a pipeline wait ran out (code {code}: "
                                   "1 = loader, 2 = MMA issuer, 3 = epilogue); results since the last check are invalid")
        if self.device.type == "cuda" and "attention_tc" in K._LIBS:
            code = K.attn_tc_error()
            if code:
                raise RuntimeError(f"tensor-core attention fault: a pipeline wait ran out or shared memory was "
                                   f"misaligned (code {code}); results since the last check are invalid")

    # ------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens; returns logits [n_wanted, vocab] (float32, on the device,
        rows in the order of the entries and of their ``want``; valid until the next step).
        The requests' token counts are advanced."""
        self._validate(entries)
        decode_only = all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        graphed = self.use_graphs and decode_only and self.device.type == "cuda"
        batch = self._build(entries, fixed_splits=graphed)
        before = K.launches
        if graphed:
            key = len(entries)
            g = self._graphs.get(key)
            if g is None:
                with K.stream_scope():
                    logits = self.model.forward(batch, self.layer_caches)  # also allocates every buffer
                self._graph_launches[key] = K.launches - before
                torch.cuda.synchronize(self.device)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g), K.stream_scope(), K.pdl_scope():
                    out = self.model.forward(batch, self.layer_caches)
                self._graphs[key] = g
                self._graph_logits[key] = out
                self.launch_counter += self._graph_launches[key]
            else:
                g.replay()
                self.stats["graph_replays"] += 1
                logits = self._graph_logits[key]
                self.launch_counter += self._graph_launches[key]
        else:
            with K.stream_scope():
                logits = self.model.forward(batch, self.layer_caches)
            self.launch_counter += K.launches - before
        for e in entries:
            self.cache.commit(e.seq, len(e.tokens))
        self.stats["steps"] += 1
        self.stats["tokens"] += batch.T
        return logits
