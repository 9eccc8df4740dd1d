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


GREEDY = SamplingParams()


class Sampler:
    """Samples one token per logits row on the device.  Per-row parameters travel in one
    pinned buffer; the result comes back as int32."""

    def __init__(self, device, max_rows: int, max_history: int = 64) -> None:
        self.device = torch.device(device)
        self.max_rows = max_rows
        self.max_history = max_history
        pin = self.device.type == "cuda"
        R = max_rows
        # float block: temperature, top_p, min_p, repeat, freq, presence ; int block: top_k
        self._hf = torch.zeros(6 * R, dtype=torch.float32, pin_memory=pin)
        self._df = torch.zeros(6 * R, dtype=torch.float32, device=self.device)
        self._hi = torch.zeros(R * (1 + max_history), dtype=torch.int32, pin_memory=pin)
        self._di = torch.zeros(R * (1 + max_history), dtype=torch.int32, device=self.device)
        self._hl = torch.zeros(2 * R, dtype=torch.int64, pin_memory=pin)
        self._dl = torch.zeros(2 * R, dtype=torch.int64, device=self.device)
        self._out = torch.zeros(R, dtype=torch.int32, device=self.device)
        self._out_host = torch.zeros(R, dtype=torch.int32, pin_memory=pin)
        self._all_greedy_loaded = False
        self.d2h_bytes = 0
        self.h2d_bytes = 0

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               counters: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """One token for each row of ``logits`` [R, V].  ``counters[i]``: index of the token
        being generated for request i (the draw's counter).  ``histories``: recent tokens of
        each request, needed only when a row has penalties."""
        tokens = self.sample_device(logits, params, seeds, counters, histories)
        R = logits.shape[0]
        self._out_host[:R].copy_(tokens[:R], non_blocking=False)
        self.d2h_bytes += 4 * R
        return self._out_host[:R].tolist()

    def sample_device(self, logits, params, seeds, counters, histories=None) -> torch.Tensor:
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"{R} rows, the sampler was built for {self.max_rows}")
        all_greedy = all(p.temperature <= 0.0 and not p.has_penalties() for p in params)
        Rm = self.max_rows
        if not (all_greedy and self._all_greedy_loaded):
            hf = self._hf
            for i, p in enumerate(params):
                hf[i] = p.temperature
                hf[Rm + i] = p.top_p
                hf[2 * Rm + i] = p.min_p
                hf[3 * Rm + i] = p.repeat_penalty
                hf[4 * Rm + i] = p.frequency_penalty
                hf[5 * Rm + i] = p.presence_penalty
                self._hi[i] = p.top_k
                self._hl[i] = int(seeds[i]) & 0x7FFFFFFFFFFFFFFF
                self._hl[Rm + i] = int(counters[i])
            self._df.copy_(self._hf, non_blocking=True)
            self._di[:Rm].copy_(self._hi[:Rm], non_blocking=True)
            self._dl.copy_(self._hl, non_blocking=True)
            self.h2d_bytes += 6 * 4 * Rm + 4 * Rm + 16 * Rm
            self._all_greedy_loaded = all_greedy
        if any(p.has_penalties() for p in params):
            if histories is None:
                raise ValueError("penalties need the requests' token histories")
            H = self.max_history
            hist = self._hi[Rm : Rm + R * H].view(R, H)
            hist.fill_(-1)
            for i, (p, h) in enumerate(zip(params, histories)):
                n = min(p.repeat_last_n, H, len(h))
                if n:
                    hist[i, :n] = torch.tensor(list(h[len(h) - n :]), dtype=torch.int32)
            dh = self._di[Rm : Rm + R * H]
            dh.copy_(self._hi[Rm : Rm + R * H], non_blocking=True)
            self.h2d_bytes += 4 * R * H
            K.apply_penalties(logits, dh.view(R, H), self._df[3 * Rm :], self._df[4 * Rm :], self._df[5 * Rm :])
        K.sample(logits, temperature=self._df[:Rm], top_k=self._di[:Rm], top_p=self._df[Rm : 2 * Rm],
                 min_p=self._df[2 * Rm : 3 * Rm], seeds=self._dl[:Rm], counters=self._dl[Rm:], out=self._out)
        return self._out
