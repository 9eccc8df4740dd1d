"""RMSNorm(eps): out = x * rsqrt(mean(x^2) + eps) * w, statistics in float32.

Formula and multiplication order of the reference's ``rmsnorm``
(src/locus/backend/cpu_ops.cpp:1687-1699): no mean subtraction, no bias, the weight used
as stored (not 1 + w).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from .base import Norm, TensorSource, register_norm


class RMSNorm(Norm):
    def __init__(self, prefix: str, *, width: int, eps: float) -> None:
        super().__init__(prefix)
        self.width = int(width)
        self.eps = float(eps)

    def param_shapes(self):
        return {"weight": (self.width,)}

    def sources(self):
        return [TensorSource(self.prefix + ".weight", (self.width,), "weight", 0, "norm")]

    def kernel_modules(self, dtype):
        return ["elementwise"]

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None, add=None) -> None:
        if add is not None and not K.rmsnorm_adds(x):
            add.apply(x)
            add = None
        K.rmsnorm(x, self.params["weight"], self.eps, out, rows,
                  add=None if add is None else (add.pair_out, add.pair_pos, add.top_k))


register_norm("rmsnorm", RMSNorm)
