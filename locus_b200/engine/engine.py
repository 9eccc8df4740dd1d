"""The engine: requests in, tokens out.  ``submit`` / ``step`` / ``run_to_completion`` /
``get`` / ``release`` mirror the reference's ``Engine``
(src/locus/engine/engine.hpp:155-181); ``generate`` is the Python entry point (the reference
has no Python binding).  One iteration: admit, plan a batch, run the step function, sample
for the requests whose last known token was in the batch, finish and free.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..sampling.sampler import GREEDY, Sampler, SamplingParams
from .scheduler import Request, Scheduler, SchedulerConfig, Status
from .step import ModelRunner, StepEntry


class Engine:
    def __init__(self, runner, cache: CacheManager, sampler, *, max_positions: int, eos_token_id: int = -1,
                 config: Optional[SchedulerConfig] = None) -> None:
        """``runner.step(entries)`` -> logits rows; ``sampler.sample(logits, params, seeds,
        counters, histories)`` -> token ids.  Both can be stand-ins on the host, so that the
        scheduler is testable without a GPU."""
        self.runner = runner
        self.cache = cache
        self.sampler = sampler
        self.cfg = config or SchedulerConfig()
        self.sched = Scheduler(cache, self.cfg, max_positions, eos_token_id)
        self.on_token: Optional[Callable[[Request, int], None]] = None
        self.timing = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "step_seconds": 0.0}

    # -- construction from a model folder -------------------------------------
    @classmethod
    def from_model_dir(cls, model_dir: str, *, dtype: str = "bfloat16", ctx: int = 0, page_tokens: int = 64,
                       max_batch_tokens: int = 2048, chunk: int = 2048, max_running: int = 64,
                       decode_headroom: int = 16, device: str = "cuda:0", use_graphs: bool = True,
                       max_seq_tokens: int = 0, kv_fraction: float = 0.0) -> "Engine":
        """``ctx``: tokens the cache pool holds in all (default: min(model context, 4096), the
        reference's default, src/locus/model/llama.cpp:389-398).  ``kv_fraction`` > 0 instead sizes
        the pool to that fraction of the device memory that is free once the weights are loaded (the
        way to use a 180 GB device for many long requests); a request may then grow to the model's
        context."""
        from ..models.model import load_model

        model = load_model(model_dir, parse_dtype(dtype), device)
        return cls.from_model(model, ctx=ctx, page_tokens=page_tokens, max_batch_tokens=max_batch_tokens,
                              chunk=chunk, max_running=max_running, decode_headroom=decode_headroom,
                              use_graphs=use_graphs, max_seq_tokens=max_seq_tokens, kv_fraction=kv_fraction)

    @classmethod
    def from_model(cls, model, *, ctx: int = 0, page_tokens: int = 64, max_batch_tokens: int = 2048,
                   chunk: int = 2048, max_running: int = 64, decode_headroom: int = 16,
                   use_graphs: bool = True, max_seq_tokens: int = 0, kv_fraction: float = 0.0) -> "Engine":
        plan = model.plan
        if kv_fraction > 0:
            if not (kv_fraction <= 1.0) or model.device.type != "cuda":
                raise ValueError("kv_fraction is a share (0, 1] of the free memory of a CUDA device")
            per_token = CacheManager(model.cache_needs(), page_tokens=page_tokens, n_pages=0, n_state_slots=1,
                                     max_seq_tokens=1, dtype=model.dtype, allocate_device=False).bytes_per_token()
            free, _ = torch.cuda.mem_get_info(model.device)
            ctx = int(free * kv_fraction) // max(1, per_token * page_tokens) * page_tokens
            if ctx < page_tokens:
                raise ValueError(f"kv_fraction {kv_fraction} of {free} free bytes holds no page of {page_tokens} tokens")
            if max_seq_tokens <= 0:
                max_seq_tokens = min(plan.max_positions, ctx)
        if ctx <= 0:
            ctx = min(plan.max_positions, 4096)
        if max_seq_tokens <= 0:
            max_seq_tokens = min(plan.max_positions, ctx)
        n_pages = -(-ctx // page_tokens)
        cache = CacheManager(model.cache_needs(), page_tokens=page_tokens, n_pages=n_pages,
                             n_state_slots=max_running, max_seq_tokens=max_seq_tokens, dtype=model.dtype,
                             device=model.device, max_step_tokens=min(chunk, max_batch_tokens))
        max_tokens = max(max_batch_tokens, max_running)
        runner = ModelRunner(model, cache, max_tokens=max_tokens, max_segments=max_running,
                             max_wanted=max_running, use_graphs=use_graphs)
        sampler = Sampler(model.device, max_running)
        cfg = SchedulerConfig(max_batch_tokens=max_batch_tokens, chunk=chunk, decode_headroom=decode_headroom,
                              max_running=max_running)
        eng = cls(runner, cache, sampler, max_positions=plan.max_positions, eos_token_id=plan.eos_token_id,
                  config=cfg)
        eng.model = model
        return eng

    # -- requests -------------------------------------------------------------
    def submit(self, prompt: Sequence[int], max_new_tokens: int, sampling: SamplingParams = GREEDY,
               seed: int = 0) -> int:
        sampling.validate()
        return self.sched.submit(prompt, max_new_tokens, sampling, seed)

    def get(self, rid: int) -> Optional[Request]:
        return self.sched.get(rid)

    def release(self, rid: int) -> None:
        self.sched.release_record(rid)

    def admit_error(self, n_prompt: int) -> str:
        return self.sched.admit_error(n_prompt)

    def has_runnable_work(self) -> bool:
        return self.sched.has_runnable_work()

    # -- the loop -------------------------------------------------------------
    def step(self) -> bool:
        """One iteration; True while requests are waiting or running."""
        s = self.sched
        s.admit()
        planned = s.plan()
        if planned:
            t0 = time.perf_counter()
            entries = [StepEntry(p.request.seq, p.request.stream_slice(p.start, p.start + p.n),
                                 [p.n - 1] if p.wants_logits else []) for p in planned]
            logits = self.runner.step(entries)
            for p in planned:
                s.fed(p)
            wanting = [p for p in planned if p.wants_logits]
            if wanting:
                reqs = [p.request for p in wanting]
                tokens = self.sampler.sample(
                    logits, [r.sampling for r in reqs], [r.seed for r in reqs],
                    [len(r.generated) for r in reqs],
                    [_history_tail(r) for r in reqs] if any(r.sampling.has_penalties() for r in reqs) else None,
                )
                for r, tok in zip(reqs, tokens):
                    s.accept_token(r, tok)
                    if self.on_token is not None:
                        self.on_token(r, int(tok))
            self.timing["steps"] += 1
            if self.timing["steps"] % 256 == 1 and hasattr(self.runner, "check_device_errors"):
                self.runner.check_device_errors()  # the first step and every 256th
            self.timing["step_seconds"] += time.perf_counter() - t0
            for p in planned:
                self.timing["decode_tokens" if p.n == 1 and p.start >= len(p.request.prompt) else "prefill_tokens"] += p.n
        return bool(s.waiting or s.running)

    def run_to_completion(self, max_steps: int = 0) -> int:
        """Step until nothing is left or nothing can run (engine.cpp:408-416); returns steps."""
        n = 0
        while self.has_runnable_work():
            self.step()
            n += 1
            if max_steps and n >= max_steps:
                break
        self.check_device_errors()
        return n

    def check_device_errors(self) -> None:
        """Raise if a kernel recorded a fault since the last check (the runner's error words; reading
        them synchronises the device).  The reference fails a request with a reason rather than
        returning garbage (src/locus/engine/engine.cpp:198-211); a kernel whose bounded wait ran out
        ends with invalid output, so tokens must not be handed out before this was read."""
        check = getattr(self.runner, "check_device_errors", None)
        if check is not None:
            check()

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 64, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, seed: int = 0,
                 sampling: Optional[SamplingParams] = None) -> List[List[int]]:
        """Generated token ids of every prompt (token ids in, token ids out).  Request i is
        seeded with ``seed + i``.  A request that fails raises ``RuntimeError``."""
        sp = sampling or SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p)
        ids = [self.submit(p, max_new_tokens, sp, seed + i) for i, p in enumerate(prompts)]
        self.run_to_completion()
        out = []
        for rid in ids:
            r = self.get(rid)
            if r is None or r.status == Status.FAILED:
                raise RuntimeError(f"request {rid} failed: {r.error if r else 'record evicted'}")
            if r.status != Status.DONE:
                raise RuntimeError(f"request {rid} could not run: {self.admit_error(len(r.prompt)) or 'queue blocked'}")
            out.append(list(r.generated))
            self.release(rid)
        return out

    def stats(self) -> Dict[str, object]:
        d = dict(self.timing)
        d.update(self.sched.counters)
        d["free_pages"] = self.cache.free_pages()
        d["total_pages"] = self.cache.total_pages()
        d["waiting"] = len(self.sched.waiting)
        d["running"] = len(self.sched.running)
        return d


def _history_tail(r: Request) -> List[int]:
    """The last ``repeat_last_n`` tokens of a request (prompt, then generated): what the penalties see."""
    n = r.sampling.repeat_last_n if r.sampling.has_penalties() else 0
    if n <= 0:
        return []
    g = r.generated
    if len(g) >= n:
        return g[len(g) - n :]
    p = r.prompt
    return list(p[max(0, len(p) - (n - len(g))) :]) + list(g)


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
             "f32": torch.float32}
    try:
        return table[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r} (bfloat16 or float32)") from None
