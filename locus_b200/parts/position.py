"""Rotary position encoding as a table of inverse frequencies.

The reference rotates, per head, the pairs (i, i + head_dim/2) ("half-split") by the
angle ``pos * base^(-2i/head_dim)`` (``rope_neox_yarn``,
src/locus/backend/cpu_ops.cpp:1849-1872; angle cpu_ops.cpp:1807-1814), after the bias and
before the key is cached.  Here the per-pair inverse frequency is computed once on the
host in float64, rounded to float32, and handed to the kernel that also writes K and V;
the angle ``float(pos) * inv_freq[i]`` and its sine and cosine are float32 on the device.
``rot_dim`` < head_dim leaves the tail of each head unrotated; ``interleaved`` pairs
(2i, 2i+1) instead.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, RotaryTable, register_position


class Rotary(PositionEncoding):
    def __init__(self, prefix: str, *, head_dim: int, theta: float, rot_dim: Optional[int] = None,
                 interleaved: bool = False) -> None:
        super().__init__(prefix)
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rot_dim = int(rot_dim) if rot_dim is not None else self.head_dim
        self.interleaved = bool(interleaved)
        if self.rot_dim % 2 or not (0 < self.rot_dim <= self.head_dim):
            raise ValueError(f"rotary: rot_dim {self.rot_dim} must be even and within head_dim {self.head_dim}")
        self._table: Optional[RotaryTable] = None

    def inv_freq_host(self) -> torch.Tensor:
        i = torch.arange(self.rot_dim // 2, dtype=torch.float64)
        return torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rot_dim).to(torch.float32)

    def bind(self, rt) -> None:
        self._table = RotaryTable(self.inv_freq_host().to(rt.device), self.rot_dim, self.interleaved)

    def rotary_table(self) -> Optional[RotaryTable]:
        return self._table


class NoPosition(PositionEncoding):
    """No position encoding at all (q and k are used as projected)."""

    def __init__(self, prefix: str) -> None:
        super().__init__(prefix)

    def rotary_table(self):
        return None

    def apply(self, q, k, positions) -> None:
        return None


register_position("rotary", Rotary)
register_position("none", NoPosition)
