"""Seeded random weights that are the same bits on every device.

The value of element ``i`` of tensor ``name`` under ``seed`` is a pure function of
(seed, name, i): a 64-bit key from sha256("seed:name"), a 64-bit integer mix of key and index
(the finaliser of SplitMix64), the top 53 bits as a uniform number in (0, 1), and the normal
quantile of that number by a rational approximation (P. J. Acklam's; relative error about 1e-9).
Every step uses only operations that IEEE 754 defines exactly and that libraries implement so --
integer arithmetic, float64 add, multiply and divide, one step per tensor operation so that
nothing is contracted into a fused multiply-add -- and the logarithm and the square root of the
tails are computed here from those operations (exponent split off with integer arithmetic and a
fixed-length series for the mantissa; a fixed number of Newton steps from a constant) instead of
by a device's math library, whose square root was seen to differ in the last bit between the
host and the GPU.  So the CPU and the GPU draw identical float32
values in any order and in slices of any size, and a model made on the device can be checked
against an implementation that draws its weights on the host.

The reference's own tests fill synthetic models from a counter as well (a linear congruential
generator in [-0.1, 0.1], tests/test_moe.cpp:22-33); it has no seeded normal initialisation.
"""
from __future__ import annotations

import hashlib
from typing import Tuple

import torch

_MASK64 = (1 << 64) - 1
SLICE = 1 << 22  # elements drawn at a time: bounds the float64 temporaries (about 0.5 GB on the device)

# Acklam's coefficients of the normal quantile: central region |u - 0.5| <= 0.47575, tails beyond
_A = (-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02, 1.383577518672690e+02,
      -3.066479806614716e+01, 2.506628277459239e+00)
_B = (-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02, 6.680131188771972e+01,
      -1.328068155288572e+01)
_C = (-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00, -2.549732539343734e+00,
      4.374664141464968e+00, 2.938163982698783e+00)
_D = (7.784695709041462e-03, 3.224671290700398e-01, 2.445134137142996e+00, 3.754408661907416e+00)
_P_LOW = 0.02425
_LN2 = 0.6931471805599453
_SQRT_HALF_BITS = 0x6A09E667F3BCD  # mantissa bits of sqrt(2): mantissas above it belong to the next exponent


def _s64(v: int) -> int:
    """A 64-bit pattern as the signed integer that torch's int64 holds."""
    v &= _MASK64
    return v - (1 << 64) if v >> 63 else v


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of tensor ``name`` under ``seed``."""
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _lsr(z: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right of int64 bit patterns."""
    return (z >> n) & ((1 << (64 - n)) - 1)


def _mix(key: int, start: int, count: int, device) -> torch.Tensor:
    """The 64-bit mix of (key, index) for indices start .. start + count - 1, as int64 bit patterns."""
    idx = torch.arange(start + 1, start + count + 1, dtype=torch.int64, device=device)
    z = idx * _s64(0x9E3779B97F4A7C15) + _s64(key)
    z = (z ^ _lsr(z, 30)) * _s64(0xBF58476D1CE4E5B9)
    z = (z ^ _lsr(z, 27)) * _s64(0x94D049BB133111EB)
    return z ^ _lsr(z, 31)


def uniform_slice(key: int, start: int, count: int, device="cpu") -> torch.Tensor:
    """float64 uniforms in (0, 1): (top 53 bits + 0.5) / 2^53, exact."""
    z = _lsr(_mix(key, start, count, device), 11)
    return (z.to(torch.float64) + 0.5) * (1.0 / 9007199254740992.0)


def _horner(coeffs, x: torch.Tensor) -> torch.Tensor:
    acc = torch.full_like(x, coeffs[0])
    for c in coeffs[1:]:
        acc = acc * x
        acc = acc + c
    return acc


def _log(x: torch.Tensor) -> torch.Tensor:
    """Natural logarithm of positive normal float64 numbers from exactly defined operations:
    x = m * 2^e with m in [sqrt(1/2), sqrt(2)); log m = 2 atanh((m - 1) / (m + 1)) by its series
    up to the 27th power (|s| < 0.172: the rest is below 1e-22)."""
    bits = x.view(torch.int64)
    e = _lsr(bits, 52) - 1023
    mant = bits & ((1 << 52) - 1)
    high = mant > _SQRT_HALF_BITS
    e = e + high.to(torch.int64)
    m = (mant | torch.where(high, torch.full_like(mant, 1022 << 52), torch.full_like(mant, 1023 << 52))).view(torch.float64)
    s = (m - 1.0) / (m + 1.0)
    s2 = s * s
    acc = torch.full_like(s, 1.0 / 27.0)
    for n in range(25, 0, -2):
        acc = acc * s2
        acc = acc + 1.0 / n
    return (acc * s) * 2.0 + e.to(torch.float64) * _LN2


def _sqrt_7_to_80(x: torch.Tensor) -> torch.Tensor:
    """Square root of float64 numbers clamped to [7, 80]: nine Newton steps from 5 (the error of the start,
    at most 90 %, squares with every step and is below 1e-16 after seven)."""
    x = x.clamp(7.0, 80.0)
    y = torch.full_like(x, 5.0)
    for _ in range(9):
        y = (y + x / y) * 0.5
    return y


def normal_slice(key: int, start: int, count: int, device="cpu") -> torch.Tensor:
    """float64 standard normal draws of elements start .. start + count - 1."""
    u = uniform_slice(key, start, count, device)
    # central region
    q = u - 0.5
    r = q * q
    central = (_horner(_A, r) * q) / (_horner(_B + (1.0,), r))
    # tails, computed for the lower tail of min(u, 1 - u) and mirrored
    lower = u < 0.5
    pt = torch.where(lower, u, 1.0 - u)
    t = _sqrt_7_to_80(_log(pt) * -2.0)   # -2 log p of a tail lies within 7.4 .. 75
    tail = _horner(_C, t) / _horner(_D + (1.0,), t)
    tail = torch.where(lower, tail, -tail)
    return torch.where(pt < _P_LOW, tail, central)


_INIT = {"linear": (0.0, 0.02), "bias": (0.0, 0.02), "norm": (1.0, 0.01)}


def init_kinds() -> Tuple[str, ...]:
    return tuple(_INIT)


def random_tensor(seed: int, name: str, shape, init: str, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """The random-weights mode's value of tensor ``name``: mean + std * normal in float64, rounded once to
    float32 and from there to ``dtype``.  ``init``: "linear" and "bias" N(0, 0.02), "norm" 1 + N(0, 0.01)."""
    try:
        mean, std = _INIT[init]
    except KeyError:
        raise ValueError(f"unknown init kind {init!r}") from None
    key = tensor_key(seed, name)
    n = 1
    for d in shape:
        n *= int(d)
    out = torch.empty(n, dtype=dtype, device=device)
    for start in range(0, n, SLICE):
        count = min(SLICE, n - start)
        v = normal_slice(key, start, count, device) * std
        if mean:
            v = v + mean
        out[start : start + count] = v.to(torch.float32).to(dtype)
    return out.view(tuple(int(d) for d in shape))
