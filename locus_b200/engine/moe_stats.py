"""Which experts the router picks, counted per mixture-of-experts layer.

The reference keeps a counter per (layer, expert) when ``LOCUS_MOE_STATS`` is set and prints one
line at exit: activations, the fewest and most experts a layer touched, and the share of
(layer, expert) slots touched (src/locus/model/moe_stats.cpp:23-78).  Here the counters live on the
device: every routed feed-forward hands its picks to an observer, which adds them to the layer's
row with one scatter-add on the stream of the step, so nothing waits and the addition is recorded
into a decode step's CUDA graph like any other launch (a replayed step counts again).  Reading the
counters (``table``, ``summary``, ``report``) waits for the device.
"""
from __future__ import annotations

from typing import Dict, List

import torch


class MoeStats:
    def __init__(self, model) -> None:
        self.parts = [p for p in model.all_parts() if hasattr(p, "observer") and hasattr(p, "E")]
        self.counts: Dict[str, torch.Tensor] = {}
        for p in self.parts:
            device = p.params["router"].device if getattr(p, "params", None) and "router" in p.params else "cpu"
            self.counts[p.prefix] = torch.zeros(p.E, dtype=torch.int64, device=device)
            p.observer = self._record

    def _record(self, prefix: str, ids: torch.Tensor, wts: torch.Tensor) -> None:
        idx = ids.reshape(-1).to(torch.int64)
        self.counts[prefix].scatter_add_(0, idx, torch.ones_like(idx))

    def detach(self) -> None:
        """Stop counting (the parts' observers are cleared)."""
        for p in self.parts:
            if p.observer == self._record:
                p.observer = None

    def table(self) -> Dict[str, List[int]]:
        """{feed-forward prefix: picks per expert}, in the model's layer order."""
        return {k: v.cpu().tolist() for k, v in self.counts.items()}

    def summary(self) -> Dict[str, int]:
        """The reference's figures: a layer that was never routed (no step yet, or a dense layer) is
        not part of the working set (moe_stats.cpp:57-64)."""
        activations = touched = slots = 0
        uniques = []
        for row in self.table().values():
            unique = sum(1 for c in row if c > 0)
            activations += sum(row)
            if unique > 0:
                slots += len(row)
                touched += unique
                uniques.append(unique)
        return {"activations": activations, "min_unique": min(uniques) if uniques else 0,
                "max_unique": max(uniques) if uniques else 0, "touched": touched, "slots": slots}

    def report(self) -> str:
        """The reference's line (moe_stats.cpp:66-78)."""
        s = self.summary()
        pct = 100.0 * s["touched"] / s["slots"] if s["slots"] else 0.0
        return (f"moe-stats: {s['activations']} activations; experts touched per moe layer min {s['min_unique']} / "
                f"max {s['max_unique']}; {s['touched']} of {s['slots']} ({pct:.1f}%) layer-expert slots touched")
