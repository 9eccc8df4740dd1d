"""The scheduler's policy written down in plain Python over the cache manager's public interface:
the comparison for the native scheduler (csrc/host_core.cpp, locus_sched_*), which must take the same
decisions step by step.  Policy of the reference's ``Engine`` (src/locus/engine/engine.cpp:503-634):
first come first served admission against free pages (nothing reserved, no overtaking), preemption of
the newest admitted request when pages run out (victims to the front of the queue, recomputed later),
failure when the newest is alone, context overflow; decode tokens first, then portions in admission
order under one token budget.
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Dict, List, Optional, Sequence

from locus_b200.cache.manager import CacheManager
from locus_b200.engine.scheduler import Planned, Request, SchedulerConfig, Status
from locus_b200.sampling.sampler import GREEDY, SamplingParams


class PlainScheduler:
    def __init__(self, cache: CacheManager, config: SchedulerConfig, max_positions: int,
                 eos_token_id: int = -1) -> None:
        self.cache = cache
        self.cfg = config
        self.max_positions = max_positions
        self.eos = eos_token_id
        self.waiting: Deque[int] = deque()
        self.running: List[int] = []
        self.requests: Dict[int, Request] = {}
        self._terminal: Deque[int] = deque()
        self._next_id = 1
        self.counters = {"preemptions": 0, "failed": 0, "done": 0, "admitted": 0}

    # -- submission ---------------------------------------------------------
    def admit_error(self, n_prompt: int) -> str:
        """Why a prompt of this length can never run; empty when it can (engine.cpp:54-68)."""
        if n_prompt <= 0:
            return "empty prompt"
        if n_prompt >= self.max_positions:
            return f"prompt length {n_prompt} exceeds context window {self.max_positions}"
        if n_prompt + 1 > self.cache.max_seq_tokens:
            return (f"prompt length {n_prompt} exceeds the cache's limit of "
                    f"{self.cache.max_seq_tokens} tokens per request")
        want = self.cache.pages_for(n_prompt + self.cfg.decode_headroom)
        if want > self.cache.total_pages():
            return f"prompt needs {want} cache pages but the pool holds only {self.cache.total_pages()}"
        return ""

    def submit(self, prompt: Sequence[int], max_new_tokens: int, sampling: SamplingParams = GREEDY,
               seed: int = 0) -> int:
        rid = self._next_id  # ids grow and are never used again (engine.cpp:33)
        self._next_id += 1
        r = Request(id=rid, prompt=[int(t) for t in prompt], max_new_tokens=int(max_new_tokens),
                    sampling=sampling, seed=seed)
        self.requests[rid] = r
        err = self.admit_error(len(r.prompt))
        if err:
            self._fail(r, err)
        elif r.max_new_tokens <= 0:
            self._finish(r, Status.DONE)
        else:
            self.waiting.append(rid)
        return rid

    def get(self, rid: int) -> Optional[Request]:
        return self.requests.get(rid)

    def release_record(self, rid: int) -> None:
        r = self.requests.get(rid)
        if r is not None and r.status in (Status.DONE, Status.FAILED):
            del self.requests[rid]
            try:
                self._terminal.remove(rid)
            except ValueError:
                pass

    def has_runnable_work(self) -> bool:
        """False when nothing runs and the front of the queue cannot be admitted even with
        the whole pool free: park, do not spin (engine.cpp:70-89)."""
        if self.running:
            return True
        if not self.waiting:
            return False
        r = self.requests[self.waiting[0]]
        return self.cache.pages_for(r.stream_len() + self.cfg.decode_headroom) <= self.cache.total_pages()

    def idle(self) -> bool:
        return not self.running and not self.waiting

    # -- one iteration --------------------------------------------------------
    def admit(self) -> None:
        while self.waiting and len(self.running) < self.cfg.max_running:
            r = self.requests[self.waiting[0]]
            want = self.cache.pages_for(r.stream_len() + self.cfg.decode_headroom)
            if want > self.cache.free_pages() or self.cache.state_slots.free == 0:
                break  # first come first served: nobody overtakes the front
            self.waiting.popleft()
            r.seq = self.cache.open(r.id)
            r.status = Status.RUNNING
            r.n_fed = 0
            self.running.append(r.id)
            self.counters["admitted"] += 1

    def plan(self) -> List[Planned]:
        """Choose this step's tokens and take their pages.  Decode tokens (one left to feed)
        first, then portions in admission order under the budget."""
        planned: Dict[int, Planned] = {}
        budget = self.cfg.max_batch_tokens
        # context overflow: the next token to feed has no position left
        for rid in list(self.running):
            r = self.requests[rid]
            if r.n_fed + 1 > self.max_positions or r.n_fed + 1 > self.cache.max_seq_tokens:
                self._fail(r, "context overflow")
        order = [rid for rid in self.running if self.requests[rid].stream_len() - self.requests[rid].n_fed == 1]
        order += [rid for rid in self.running if self.requests[rid].stream_len() - self.requests[rid].n_fed > 1]
        for rid in order:
            r = self.requests.get(rid)
            if r is None or r.status != Status.RUNNING or budget <= 0:
                continue
            left = r.stream_len() - r.n_fed
            n = min(left, budget, self.cfg.chunk,
                    self.max_positions - r.n_fed, self.cache.max_seq_tokens - r.n_fed)
            if n <= 0:
                continue
            ok = self._make_room(r, n, planned)
            if not ok:
                continue
            planned[rid] = Planned(r, r.n_fed, n, wants_logits=(r.n_fed + n == r.stream_len()))
            budget -= n
        # keep admission order in the batch: rows of a request do not depend on it, but a
        # stable order makes steps reproducible
        return [planned[rid] for rid in self.running if rid in planned]

    def _make_room(self, r: Request, n: int, planned: Dict[int, Planned]) -> bool:
        while not self.cache.ensure_capacity(r.seq, n):
            victim = self.requests[self.running[-1]]
            if victim is r:
                if len(self.running) == 1:
                    self._fail(r, "kv pool too small for request")
                return False  # newest but not alone: sit this step out
            planned.pop(victim.id, None)
            self._preempt(victim)
        return True

    def _preempt(self, victim: Request) -> None:
        self.cache.release(victim.seq)
        victim.seq = None
        victim.n_fed = 0
        victim.status = Status.WAITING
        victim.preemptions += 1
        self.running.remove(victim.id)
        self.waiting.appendleft(victim.id)  # victims go to the front
        self.counters["preemptions"] += 1

    def fed(self, p: Planned) -> None:
        p.request.n_fed += p.n

    def accept_token(self, r: Request, token: int) -> bool:
        """Append a sampled token; True when the request is finished by it (end-of-sequence
        token, which is kept in ``generated`` as in the reference, or the length limit)."""
        r.generated.append(int(token))
        if int(token) == self.eos or len(r.generated) >= r.max_new_tokens:
            self._finish(r, Status.DONE)
            return True
        return False

    # -- endings --------------------------------------------------------------
    def _finish(self, r: Request, status: Status) -> None:
        if r.seq is not None:
            self.cache.release(r.seq)
            r.seq = None
        if r.id in self.running:
            self.running.remove(r.id)
        r.status = status
        self.counters["done" if status == Status.DONE else "failed"] += 1
        self._terminal.append(r.id)
        while len(self._terminal) > self.cfg.max_retained_terminal:
            old = self._terminal.popleft()
            self.requests.pop(old, None)

    def _fail(self, r: Request, why: str) -> None:
        r.error = why
        self._finish(r, Status.FAILED)
