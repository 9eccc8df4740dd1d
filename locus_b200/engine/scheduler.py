"""The scheduler: admits requests, cuts prompts into portions under a token budget, puts
decode tokens and portions into one batch per step, finishes requests and frees what they
hold; and decides what happens when pages run out.

Policy of the reference's ``Engine`` (src/locus/engine/engine.cpp:503-634):

* Admission is first come, first served: the front of the waiting queue is admitted while
  fewer than ``max_running`` requests run and the pool has free pages for
  prompt + generated + ``decode_headroom`` tokens; a front that does not fit blocks the
  queue, later arrivals never overtake (engine.cpp:505-524).  The check reserves nothing;
  pages are taken as tokens are fed.
* A request whose prompt can never fit is refused at once: ``admit_error``
  (engine.cpp:54-68).
* When ``ensure_capacity`` fails for a request r, the newest admitted request is preempted:
  its pages are given back, its progress is reset and it goes to the FRONT of the waiting
  queue, to be recomputed later (engine.cpp:230-239, 482-494, 582-601).  If r is itself
  the newest: alone, it fails with "kv pool too small for request"; else it sits the step out.
* A request whose next token would pass the context limit fails with "context overflow"
  (engine.cpp:198-200, 576-580).
* Finished and failed requests release everything; their records are kept up to
  ``max_retained_terminal`` (engine.cpp:241-273).

Where this differs: prompt portions and decode tokens share one batch and one budget
(``max_batch_tokens``: decode tokens first, the rest to portions in admission order, each
at most ``chunk`` tokens), and a preempted request re-feeds prompt + generated tokens as
one stream in portions.

The decisions are made by host code in C++ (``csrc/host_core.cpp``: ``locus_sched_*``), next
to the cache whose pages it takes and gives back; it keeps lengths and states and reports
what it decided as events.  This class keeps the records with their tokens, applies the
events to them and mirrors the queues.
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

import ctypes

from ..cache import native
from ..cache.manager import CacheManager, SeqCache
from ..sampling.sampler import GREEDY, SamplingParams


class Status(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    DONE = "done"
    FAILED = "failed"


@dataclass
class Request:
    id: int
    prompt: List[int]
    max_new_tokens: int
    sampling: SamplingParams = GREEDY
    seed: int = 0
    generated: List[int] = field(default_factory=list)
    status: Status = Status.WAITING
    error: str = ""
    seq: Optional[SeqCache] = None
    n_fed: int = 0          # tokens of prompt + generated that went through the model
    preemptions: int = 0

    def stream_len(self) -> int:
        return len(self.prompt) + len(self.generated)

    def stream_slice(self, a: int, b: int) -> List[int]:
        n = len(self.prompt)
        if b <= n:
            return self.prompt[a:b]
        if a >= n:
            return self.generated[a - n : b - n]
        return self.prompt[a:] + self.generated[: b - n]


@dataclass
class SchedulerConfig:
    # A step streams the weights of every expert that any of its tokens picked (all of them from a few
    # dozen tokens on), so long portions pay: at the A2.7B sizes a 4,096-token prompt runs at 70 k tokens/s
    # in portions of 512 and at 144 k in portions of 2,048.
    max_batch_tokens: int = 2048  # tokens of one step, decode tokens and portions together
    chunk: int = 2048             # longest portion of one request in one step
    decode_headroom: int = 16     # tokens of room required at admission beyond what is known
    max_running: int = 64
    max_retained_terminal: int = 1024


@dataclass
class Planned:
    request: Request
    start: int      # first stream index fed in this step
    n: int          # tokens fed
    wants_logits: bool


class Scheduler:
    _EV_ADMITTED, _EV_PREEMPTED, _EV_FAILED, _EV_DONE = 1, 2, 3, 4
    _WHY = {1: "context overflow", 2: "kv pool too small for request"}

    def __init__(self, cache: CacheManager, config: SchedulerConfig, max_positions: int,
                 eos_token_id: int = -1) -> None:
        self.cache = cache
        self.cfg = config
        self.max_positions = max_positions
        self.eos = eos_token_id
        self.waiting: Deque[int] = deque()   # mirrors of the native queues
        self.running: List[int] = []
        self.requests: Dict[int, Request] = {}
        self._terminal: Deque[int] = deque()
        self._next_id = 1
        self.counters = {"preemptions": 0, "failed": 0, "done": 0, "admitted": 0}
        self._lib = native.lib()
        self._core = self._lib.locus_sched_new(cache._core, config.max_batch_tokens, config.chunk,
                                               config.decode_headroom, config.max_running, max_positions)
        if not self._core:
            raise ValueError("scheduler: token budget, portion size and max_running must be positive")
        self._ids = (ctypes.c_int64 * 4096)()
        self._plan = (ctypes.c_int64 * (4 * max(1, config.max_running)))()
        self._pairs = (ctypes.c_int * 4096)()

    def __del__(self) -> None:
        core, self._core = getattr(self, "_core", None), None
        if core:
            self._lib.locus_sched_delete(core)

    # -- what the native side decided -----------------------------------------
    def _sync(self) -> None:
        """Apply the native side's events to the records, poison the pages it freed (tests), mirror the queues."""
        lib, core = self._lib, self._core
        changed = False
        while True:
            n = lib.locus_sched_events(core, self._ids, len(self._ids) // 3)
            changed = changed or n > 0
            for i in range(n):
                kind, rid, arg = self._ids[3 * i], self._ids[3 * i + 1], self._ids[3 * i + 2]
                r = self.requests[rid]
                if kind == self._EV_ADMITTED:
                    r.seq = self.cache.adopt_native(r.id, arg)
                    r.status = Status.RUNNING
                    r.n_fed = 0
                    self.counters["admitted"] += 1
                elif kind == self._EV_PREEMPTED:
                    self.cache.forget_native(r.seq)
                    r.seq = None
                    r.n_fed = 0
                    r.status = Status.WAITING
                    r.preemptions += 1
                    self.counters["preemptions"] += 1
                elif kind == self._EV_FAILED:
                    r.error = self._WHY.get(arg, "failed")
                    self._record_end(r, Status.FAILED)
                else:
                    self._record_end(r, Status.DONE)
            if n < len(self._ids) // 3:
                break
        while True:
            n = lib.locus_sched_freed(core, self._pairs, len(self._pairs))
            self.cache.poison_pairs(self._pairs[: 2 * n])
            if 2 * n < len(self._pairs):
                break
        if changed:   # the queues only change with an event
            self.waiting = deque(self._queue(0))
            self.running = self._queue(1)

    def _queue(self, which: int) -> List[int]:
        n = self._lib.locus_sched_count(self._core, which)
        if n > len(self._ids):
            self._ids = (ctypes.c_int64 * (2 * n))()
        n = self._lib.locus_sched_queue(self._core, which, self._ids, len(self._ids))
        return list(self._ids[:n])

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
        n = n_prompt + self.cfg.decode_headroom
        for g in self.cache.groups:
            want = self.cache.pages_needed(g.gid, n, self.cfg.chunk)
            if want > g.n_pages:
                return f"prompt needs {want} cache pages but the pool holds only {g.n_pages}"
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
            r.error = err
            self._record_end(r, Status.FAILED)   # never reaches the native queue
        elif r.max_new_tokens <= 0:
            self._record_end(r, Status.DONE)
        else:
            self._lib.locus_sched_add(self._core, rid, len(r.prompt))
            self.waiting.append(rid)
        return rid

    def get(self, rid: int) -> Optional[Request]:
        return self.requests.get(rid)

    def release_record(self, rid: int) -> None:
        r = self.requests.get(rid)
        if r is not None and r.status in (Status.DONE, Status.FAILED):
            self._drop(rid)
            try:
                self._terminal.remove(rid)
            except ValueError:
                pass

    def _drop(self, rid: int) -> None:
        self.requests.pop(rid, None)
        self._lib.locus_sched_forget(self._core, rid)

    def has_runnable_work(self) -> bool:
        """False when nothing runs and the front of the queue cannot be admitted even with
        the whole pool free: park, do not spin (engine.cpp:70-89)."""
        if self.running:
            return True
        if not self.waiting:
            return False
        r = self.requests[self.waiting[0]]
        return self.cache.fits_when_empty(r.stream_len() + self.cfg.decode_headroom, self.cfg.chunk)

    def idle(self) -> bool:
        return not self.running and not self.waiting

    # -- one iteration --------------------------------------------------------
    def admit(self) -> None:
        """First come first served while requests fit (see the module's text); native."""
        if self._lib.locus_sched_admit(self._core):
            self._sync()

    def plan(self) -> List[Planned]:
        """Choose this step's tokens and take their pages.  Decode tokens (one left to feed)
        first, then portions in admission order under the budget; native."""
        n = self._lib.locus_sched_plan(self._core, self._plan, len(self._plan) // 4)
        self._sync()
        out = []
        for i in range(n):
            rid, start, cnt, wants = (self._plan[4 * i + j] for j in range(4))
            out.append(Planned(self.requests[rid], int(start), int(cnt), bool(wants)))
        return out

    def fed(self, p: Planned) -> None:
        p.request.n_fed += p.n
        self._lib.locus_sched_fed(self._core, p.request.id, p.n)

    def accept_token(self, r: Request, token: int) -> bool:
        """Append a sampled token; True when the request is finished by it (end-of-sequence
        token, which is kept in ``generated`` as in the reference, or the length limit)."""
        r.generated.append(int(token))
        finished = int(token) == self.eos or len(r.generated) >= r.max_new_tokens
        self._lib.locus_sched_token(self._core, r.id, 1 if finished else 0)
        if finished:
            self._sync()
        return finished

    # -- endings --------------------------------------------------------------
    def _record_end(self, r: Request, status: Status) -> None:
        """The record of a request that ended (the native side has given back what it held)."""
        if r.seq is not None:
            self.cache.forget_native(r.seq)
            r.seq = None
        r.status = status
        self.counters["done" if status == Status.DONE else "failed"] += 1
        self._terminal.append(r.id)
        while len(self._terminal) > self.cfg.max_retained_terminal:
            self._drop(self._terminal.popleft())
