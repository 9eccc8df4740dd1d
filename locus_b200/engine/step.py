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
from typing import Dict, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheError, CacheManager, SeqCache
from .. import kernels as K
from .batch import GroupBatch, Runtime, StepBatch


class StepError(ValueError):
    pass


@dataclass
class StepEntry:
    seq: SeqCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


class _BuildArgs:
    """The arrays that carry a step's entries to the native assembly and its layout back, made once."""

    def __init__(self, max_tokens: int, max_segments: int, max_wanted: int, n_groups: int) -> None:
        self.counts = np.zeros(max_segments, dtype=np.int32)
        self.want_counts = np.zeros(max_segments, dtype=np.int32)
        self.handles = np.zeros(max_segments, dtype=np.int64)
        self.tokens = np.zeros(max(1, max_tokens), dtype=np.int64)
        self.wants = np.zeros(max(1, max_wanted), dtype=np.int64)
        self.layout = np.zeros(2 * (ModelRunner._N_FIELDS + 2 * n_groups), dtype=np.int32)
        self.info = np.zeros(8, dtype=np.int32)
        for name in ("counts", "want_counts", "handles", "tokens", "wants", "layout", "info"):
            setattr(self, "p_" + name, getattr(self, name).ctypes.data)


class ModelRunner:
    _N_FIELDS = 7  # fields of a step before the per-group ones (csrc/host_core.cpp: locus_step_build)

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
        # the parts' own step plans (work lists of their kernels), one of each kind, behind the descriptors
        self.plans = {}
        for part in model.all_parts():
            for pl in (part.step_plans() if hasattr(part, "step_plans") else []):
                self.plans.setdefault(pl.key, pl)
        self._plan_caps = {key: int(pl.capacity(max_tokens, max_segments)) for key, pl in self.plans.items()}
        size = (max_tokens * (2 + G) + max_segments * (4 + G * W) + self.max_wanted + sum(self._plan_caps.values()))
        # two pinned staging buffers, used in turn: a buffer is rewritten only after the copy
        # that read it has finished (its event), so steps may be queued without a host sync
        on_gpu = self.device.type == "cuda"
        self._hosts = [torch.empty(size, dtype=torch.int32, pin_memory=on_gpu) for _ in range(2)]
        self._host_events = [torch.cuda.Event() if on_gpu else None for _ in range(2)]
        self._host_used = [False, False]
        self._host_turn = 0
        self._host_ptrs = [h.data_ptr() for h in self._hosts]
        self._host_np = [h.numpy() for h in self._hosts]
        self._dev = torch.empty(size, dtype=torch.int32, device=self.device)
        self._args = _BuildArgs(max_tokens, max_segments, self.max_wanted, G)
        self._views: Dict[bytes, list] = {}
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self._graph_logits: Dict[int, torch.Tensor] = {}
        self._graph_launches: Dict[int, int] = {}
        self.launch_counter = 0
        self.stats = {"steps": 0, "tokens": 0, "graph_replays": 0, "h2d_bytes": 0}

    # ------------------------------------------------------------------
    def _build(self, entries: Sequence[StepEntry], fixed_shapes: bool) -> StepBatch:
        """Check the entries and write the step's descriptors: one native call that reads the
        requests' page tables where they live and fills the pinned staging buffer, then one
        copy to the device."""
        cache, plan = self.cache, self.model.plan
        n_seg = len(entries)
        if n_seg == 0:
            raise StepError("a step needs at least one entry")
        if n_seg > self.max_segments:
            raise StepError(f"{n_seg} requests in a step, the runner was built for {self.max_segments}")
        live = cache._live
        for e in entries:
            if live.get(e.seq.seq_id) is not e.seq:
                raise CacheError(f"request {e.seq.seq_id!r} is not open in the runner's cache")
        a = self._args
        counts = [len(e.tokens) for e in entries]
        want_counts = [len(e.want) for e in entries]
        T_all, W_all = sum(counts), sum(want_counts)
        if T_all > self.max_tokens:
            raise StepError(f"{T_all} tokens in a step, the runner was built for {self.max_tokens}")
        if W_all > self.max_wanted:
            raise StepError(f"{W_all} logits rows wanted, the runner was built for {self.max_wanted}")
        a.counts[:n_seg] = counts
        a.want_counts[:n_seg] = want_counts
        a.handles[:n_seg] = [e.seq._handle for e in entries]
        try:
            a.tokens[:T_all] = [t for e in entries for t in e.tokens]
            a.wants[:W_all] = [w for e in entries for w in e.want]
        except OverflowError:
            raise StepError("a token id or wanted place does not fit 64 bits: outside the vocabulary") from None

        turn = self._host_turn
        if self._host_used[turn] and self._host_events[turn] is not None:
            self._host_events[turn].synchronize()
        host = self._hosts[turn]
        code = cache._lib.locus_step_build(
            cache._core, n_seg, a.p_handles, a.p_counts, a.p_tokens, a.p_want_counts, a.p_wants, plan.vocab_size,
            plan.max_positions, self.max_tokens, self.max_segments, self.max_wanted,
            self._host_ptrs[turn], host.numel(), a.p_layout, a.p_info)
        info = a.info
        if code:
            self._raise_build_error(code, entries, int(info[6]), int(info[7]))
        self._host_turn ^= 1
        layout = a.layout
        off = int(layout[-2]) + int(layout[-1])
        hn = self._host_np[turn]

        def hseg(i):
            return hn[layout[2 * i] : layout[2 * i] + layout[2 * i + 1]]

        # every distinct plan of the model's parts writes its work lists behind the descriptors
        planned = []
        if self.plans:
            seg_q0, seg_qn, seg_ctx = hseg(2), hseg(3), hseg(4)
            for key, pl in self.plans.items():
                cap = self._plan_caps[key]
                res = pl.build(seg_q0, seg_qn, seg_ctx, hn[off : off + cap])
                used = 0
                for name, v in res.items():
                    if isinstance(v, tuple):
                        if v[0] < 0 or v[1] < 0 or v[0] + v[1] > cap:
                            raise StepError(f"step plan {key!r}: list {name!r} lies outside the plan's capacity of {cap}")
                        used = max(used, v[0] + v[1])
                planned.append((key, off, tuple(sorted(res.items()))))
                off += used
        self._dev[:off].copy_(host[:off], non_blocking=True)
        if self._host_events[turn] is not None:
            self._host_events[turn].record()
            self._host_used[turn] = True
        self.stats["h2d_bytes"] += off * 4

        # the device views of a layout are made once: steps of the same shape (every decode step of
        # a batch size) have the same layout
        key = (layout.tobytes(), tuple(planned))
        views = self._views.get(key)
        if views is None:
            if len(self._views) > 256:
                self._views.clear()
            fields = [self._dev[int(layout[2 * i]) : int(layout[2 * i]) + int(layout[2 * i + 1])]
                      for i in range(len(layout) // 2)]
            W = cache.table_width
            for gi in range(len(cache.groups)):
                fields[self._N_FIELDS + 2 * gi + 1] = fields[self._N_FIELDS + 2 * gi + 1].view(n_seg, W)
            plans = {}
            for pkey, base, items in planned:
                d = {}
                for name, v in items:
                    if isinstance(v, tuple):
                        t = self._dev[base + v[0] : base + v[0] + v[1]]
                        d[name] = t.view(*v[2]) if len(v) > 2 and v[2] else t
                    else:
                        d[name] = v
                plans[pkey] = d
            views = (fields, plans)
            self._views[key] = views
        fields, plans = views
        batch = StepBatch(
            T=int(info[0]), n_seg=n_seg, tokens=fields[0], positions=fields[1], seg_q0=fields[2], seg_qn=fields[3],
            seg_ctx=fields[4], state_slots=fields[5], want_rows=fields[6], n_want=int(info[1]),
            longest=cache.max_seq_tokens if fixed_shapes else int(info[2]), static_shapes=fixed_shapes, plans=plans,
            host_seg_q0=hseg(2).tolist(), host_seg_qn=hseg(3).tolist(), host_seg_ctx=hseg(4).tolist(),
            host_state_slots=hseg(5).tolist(),
        )
        for gi, g in enumerate(cache.groups):
            batch.groups[g.gid] = GroupBatch(block_table=fields[self._N_FIELDS + 2 * gi + 1],
                                             slots=fields[self._N_FIELDS + 2 * gi], page_tokens=cache.page_tokens)
        return batch

    def _raise_build_error(self, code: int, entries, at: int, value: int) -> None:
        """Words the native step assembly's refusal (its codes are listed in csrc/host_core.cpp)."""
        plan = self.model.plan
        e = entries[at] if 0 <= at < len(entries) else None
        who = repr(e.seq.seq_id) if e is not None else "?"
        n = len(e.tokens) if e is not None else 0
        if code == 3:
            raise StepError(f"request {who} appears twice in a step")
        if code == 4:
            raise StepError(f"request {who}: no tokens in its entry")
        if code == 5:
            raise StepError(f"request {who}: token {int(e.tokens[value])} outside the vocabulary "
                            f"0..{plan.vocab_size - 1}")
        if code == 6:
            raise StepError(f"request {who}: context overflow, {value} tokens exceed max_position_embeddings "
                            f"{plan.max_positions}")
        if code == 7:
            raise CacheError(f"request {who} is not open in the runner's cache")
        if code == 8:
            raise CacheError(f"request {who}: capacity for {n} more tokens was not ensured")
        if code == 9:
            raise StepError(f"request {who}: wanted place {int(e.want[value])} is not among its {n} tokens")
        if code == 12:
            raise CacheError(f"request {who}: position {value} lies in a page given back")
        raise StepError(f"the step could not be assembled (code {code})")

    def check_device_errors(self) -> None:
        """Raise if a kernel recorded a fault since the last check (a bounded wait of the
        tensor-core pipeline that ran out).  Synchronises the device."""
        if self.device.type == "cuda" and "gemm_tc" in K._LIBS:
            code = K.tc_error()
            if code:
                raise RuntimeError(f"tensor-core kernel fault: a pipeline wait ran out (code {code}: "
                                   "1 = loader, 2 = MMA issuer, 3 = epilogue); results since the last check are invalid")
        if self.device.type == "cuda" and "attention" in K._LIBS:
            code = K.attn_error()
            if code:
                raise RuntimeError(f"decode attention fault (code {code}): the step's split count did not cover its "
                                   "longest context; results since the last check are invalid")
        if self.device.type == "cuda" and "attention_gqa" in K._LIBS:
            code = K.attn_gqa_error()
            if code:
                raise RuntimeError(f"grouped-query decode attention fault (code {code}): a wait for a bulk copy ran out; "
                                   "results since the last check are invalid")
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
        decode_only = all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        graphed = self.use_graphs and decode_only and self.device.type == "cuda" and not K.timing_active()
        batch = self._build(entries, fixed_shapes=graphed)
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
