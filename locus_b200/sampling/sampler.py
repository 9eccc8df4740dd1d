"""Sampling parameters and the device sampler.

Names, defaults and meanings follow the reference's ``SamplingParams``
(src/locus/model/sampling.hpp:23-40); the filters are applied in its order
(sampling.hpp:65-68, src/locus/model/sampling.cpp:45-148): penalties -> top-k ->
temperature softmax -> top-p -> min-p -> draw.  ``temperature <= 0`` is greedy arg-max
(the first maximum wins, src/locus/model/llama.cpp:1237-1245) and touches no random state.

Where this differs from the reference: the draw uses a counter-based generator keyed by
(seed, index of the generated token) instead of a per-request ``std::mt19937_64``, so a
request's samples do not depend on what else is in the batch or on preemption; and tokens
whose weight ties with the cut-off of top-k / top-p are all kept.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import kernels as K


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repeat_last_n: int = 64

    def has_penalties(self) -> bool:
        return not (self.repeat_penalty == 1.0 and self.frequency_penalty == 0.0 and self.presence_penalty == 0.0)

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be within (0, 1]")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must be within [0, 1]")
        if self.repeat_penalty <= 0.0:
            raise ValueError("repeat_penalty must be positive")
        if self.repeat_last_n < 0:
            raise ValueError("repeat_last_n must not be negative")


GREEDY = SamplingParams()


class Sampler:
    """Samples one token per logits row on the device.  Per-row parameters travel in one
    pinned buffer; the result comes back as int32."""

    def __init__(self, device, max_rows: int, max_history: int = 64) -> None:
        """``max_history``: tokens of history per row that the penalty buffers hold at first; they
        grow to the largest ``repeat_last_n`` that a request brings."""
        self.device = torch.device(device)
        self.max_rows = max_rows
        self._pin = self.device.type == "cuda"
        R = max_rows
        # One packed block of per-row parameters, host (pinned) and device, so that a step uploads them with one
        # copy: int64 seed, counter; float32 temperature, top_p, min_p, repeat, frequency, presence; int32 top_k.
        self._block_bytes = (2 * 8 + 6 * 4 + 4) * R
        self._hblock = torch.zeros(self._block_bytes, dtype=torch.uint8, pin_memory=self._pin)
        self._dblock = torch.zeros(self._block_bytes, dtype=torch.uint8, device=self.device)

        def views(block):
            return (block[: 16 * R].view(torch.int64), block[16 * R : 40 * R].view(torch.float32),
                    block[40 * R :].view(torch.int32))

        self._hl, self._hf, self._hi = views(self._hblock)
        self._dl, self._df, self._di = views(self._dblock)
        # numpy views of the host block: assigning a Python list to a slice of them costs a few microseconds,
        # a torch.tensor() per field cost ten times that
        self._nl, self._nf, self._ni = self._hl.numpy().reshape(2, R), self._hf.numpy().reshape(6, R), self._hi.numpy()
        self._out = torch.zeros(R, dtype=torch.int32, device=self.device)
        self._out_host = torch.zeros(R, dtype=torch.int32, pin_memory=self._pin)
        self.max_history = 0
        self._grow_history(max(1, max_history))
        # rows 0 .. _greedy_rows - 1 of the device blocks hold plain greedy parameters (0: not known to)
        self._greedy_rows = 0
        self.d2h_bytes = 0
        self.h2d_bytes = 0

    def _grow_history(self, n: int) -> None:
        """Room for ``n`` tokens of history per row (the only allocation after construction: a request
        with a longer ``repeat_last_n`` than any before it)."""
        if n <= self.max_history:
            return
        cap = max(64, self.max_history)
        while cap < n:
            cap *= 2
        self.max_history = cap
        self._hh = torch.full((self.max_rows, cap), -1, dtype=torch.int32, pin_memory=self._pin)
        self._dh = torch.full((self.max_rows, cap), -1, dtype=torch.int32, device=self.device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               counters: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """One token for each row of ``logits`` [R, V].  ``counters[i]``: index of the token
        being generated for request i (the draw's counter).  ``histories``: recent tokens of
        each request (at least its last ``repeat_last_n``), needed only when a row has penalties."""
        tokens = self.sample_device(logits, params, seeds, counters, histories)
        R = logits.shape[0]
        self._out_host[:R].copy_(tokens[:R], non_blocking=False)
        self.d2h_bytes += 4 * R
        return self._out_host[:R].tolist()

    def sample_device(self, logits, params, seeds, counters, histories=None) -> torch.Tensor:
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"{R} rows, the sampler was built for {self.max_rows}")
        if len(params) != R:
            raise ValueError(f"{len(params)} sampling parameters for {R} rows of logits")
        all_greedy = all(p.temperature <= 0.0 and not p.has_penalties() for p in params)
        Rm = self.max_rows
        # a batch of plain greedy rows needs no upload while the device rows it uses are known to be greedy
        if not (all_greedy and R <= self._greedy_rows):
            nf = self._nf
            nf[0, :R] = [p.temperature for p in params]
            nf[1, :R] = [p.top_p for p in params]
            nf[2, :R] = [p.min_p for p in params]
            nf[3, :R] = [p.repeat_penalty for p in params]
            nf[4, :R] = [p.frequency_penalty for p in params]
            nf[5, :R] = [p.presence_penalty for p in params]
            self._ni[:R] = [p.top_k for p in params]
            self._nl[0, :R] = [int(s) & 0x7FFFFFFFFFFFFFFF for s in seeds]
            self._nl[1, :R] = [int(c) for c in counters]
            self._dblock.copy_(self._hblock, non_blocking=True)
            self.h2d_bytes += self._block_bytes
            # rows beyond R keep what an earlier batch left: greedy only if they were and this batch is
            self._greedy_rows = max(R, self._greedy_rows) if all_greedy else 0
        if any(p.has_penalties() for p in params):
            if histories is None:
                raise ValueError("penalties need the requests' token histories")
            need = max(min(p.repeat_last_n, len(h)) for p, h in zip(params, histories))
            self._grow_history(need)
            n_hist = max(1, need)
            hist = self._hh.view(-1)[: R * n_hist].view(R, n_hist)
            nh = hist.numpy()
            nh.fill(-1)
            for i, (p, h) in enumerate(zip(params, histories)):
                n = min(p.repeat_last_n, len(h)) if p.has_penalties() else 0
                if n:
                    nh[i, :n] = h[len(h) - n :]
            dh = self._dh.view(-1)[: R * n_hist].view(R, n_hist)
            dh.copy_(hist, non_blocking=True)
            self.h2d_bytes += 4 * R * n_hist
            K.apply_penalties(logits, dh, self._df[3 * Rm :], self._df[4 * Rm :], self._df[5 * Rm :])
        K.sample(logits, temperature=self._df[:Rm], top_k=self._di[:Rm], top_p=self._df[Rm : 2 * Rm],
                 min_p=self._df[2 * Rm : 3 * Rm], seeds=self._dl[:Rm], counters=self._dl[Rm:], out=self._out)
        return self._out
