"""A model built from a plan: the parts, their weights, and the forward pass of one step.

``Model`` instantiates every part the plan names, collects the checkpoint tensors they
declare, and runs the layers in the plan's order.  Nothing in here depends on a particular
architecture: the architecture is the plan.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..config.base import load_config
from ..engine.batch import LayerCache, Runtime, StepBatch
from ..parts.base import (ModelPlan, PagedKvSpec, Part, PartSpec, StateSpec, TensorSource,
                          iter_parts, make_part)


def _split_prefix(spec: PartSpec) -> Tuple[PartSpec, str]:
    args = dict(spec.args)
    prefix = args.pop("prefix")
    return PartSpec(spec.kind, args), prefix


class Model:
    def __init__(self, plan: ModelPlan, dtype: torch.dtype, device="cuda:0") -> None:
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"model element type must be float32 or bfloat16, got {dtype}")
        self.plan = plan
        self.dtype = dtype
        self.device = torch.device(device)
        spec, prefix = _split_prefix(plan.embedding)
        self.embedding = make_part("embedding", spec, prefix)
        self.blocks: List[Part] = []
        for ls in plan.layers:
            self.blocks.append(make_part(
                "arrangement", ls.arrangement, ls.prefix,
                norm=ls.norm, mixer=ls.mixer, feed_forward=ls.feed_forward,
            ))
        spec, prefix = _split_prefix(plan.final_norm)
        self.final_norm = make_part("norm", spec, prefix)
        spec, prefix = _split_prefix(plan.head)
        self.head = make_part("head", spec, prefix)
        for i, call in enumerate(plan.order):
            if not (0 <= call.layer < len(self.blocks)):
                raise ValueError(f"run order entry {i} names layer {call.layer} of {len(self.blocks)}")
            if call.cache_of is not None:
                if not (0 <= call.cache_of < i):
                    raise ValueError(f"run order entry {i}: cache_of must name an earlier entry")
                if plan.order[call.cache_of].cache_of is not None:
                    raise ValueError(f"run order entry {i}: cache_of must name an entry with a cache of its own")
        self.rt: Optional[Runtime] = None
        self.loaded = False

    # -- structure ----------------------------------------------------------
    def top_parts(self) -> List[Part]:
        return [self.embedding] + self.blocks + [self.final_norm, self.head]

    def all_parts(self):
        for p in self.top_parts():
            yield from iter_parts(p)

    def tensor_sources(self) -> List[Tuple[Part, TensorSource]]:
        out = []
        for p in self.all_parts():
            for s in p.sources():
                out.append((p, s))
        return out

    def kernel_modules(self) -> List[str]:
        mods = {"sampling"}
        for p in self.all_parts():
            mods.update(p.kernel_modules(self.dtype))
        return sorted(mods)

    def cache_needs(self) -> List[Tuple[Optional[PagedKvSpec], Optional[StateSpec], Optional[int]]]:
        """For every entry of the run order: (paged spec, state spec, cache_of)."""
        out = []
        for call in self.plan.order:
            paged, state = self.blocks[call.layer].mixer.cache_needs()
            out.append((paged, state, call.cache_of))
        return out

    def param_bytes(self) -> int:
        seen = set()
        total = 0
        for p in self.all_parts():
            for t in p.params.values():
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    # -- lifecycle ----------------------------------------------------------
    def bind(self, rt: Runtime) -> None:
        """After the weights are loaded: build the kernels, let the parts set up device tables."""
        if not self.loaded:
            raise RuntimeError("bind() before the weights are loaded")
        from ..csrc import build
        build.ensure(self.kernel_modules())
        self.rt = rt
        for p in self.all_parts():
            p.bind(rt)

    # -- forward ------------------------------------------------------------
    def forward(self, batch: StepBatch, caches: List[LayerCache]) -> torch.Tensor:
        """Run the step's tokens through every layer call; float32 logits [n_want, vocab]."""
        rt = self.rt
        T = batch.T
        x = rt.rows("model.x", self.plan.hidden_size, torch.float32, T)
        self.embedding.forward(batch.tokens, x)
        order = self.plan.order
        for i, (call, cache) in enumerate(zip(order, caches)):
            # a block may leave its last addition to the residual stream to the next block's first norm,
            # the last block to the final norm
            rt.defer_add = i + 1 == len(order) or self.blocks[order[i + 1].layer].takes_pending_add
            self.blocks[call.layer].forward(x, batch, cache, rt)
        rt.defer_add = False
        # what the last block left undone only matters in the rows whose logits are wanted
        pending = rt.take_pending()
        n = batch.n_want
        logits = rt.buf("model.logits", (rt.max_wanted, self.plan.vocab_size), torch.float32)[:n]
        if n:
            hw = rt.buf("model.h_want", (rt.max_wanted, self.plan.hidden_size), rt.dtype)[:n]
            self.final_norm.forward(x, hw, rows=batch.want_rows, add=pending)
            self.head.forward(hw, logits)
        return logits


def load_model(model_dir: str, dtype: torch.dtype, device="cuda:0") -> Model:
    """Model of a folder (config.json + safetensors), weights on the device."""
    from ..weights.loader import load_weights
    from ..weights.safetensors_io import ModelFiles

    entry, cfg = load_config(model_dir)
    model = Model(entry.build_plan(cfg), dtype, device)
    files = ModelFiles(model_dir)
    try:
        load_weights(model, files)
    finally:
        files.close()
    return model
