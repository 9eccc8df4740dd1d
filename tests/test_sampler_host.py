"""The sampler's front end and the engine's error reporting on the CPU, with the CUDA entry points
replaced by their torch twins: which per-row parameters reach the kernel after batches of changing size
and kind, how much history the penalties see, and that a kernel fault recorded on the device ends
``generate`` with an error instead of tokens."""
import pytest
import torch

import emulated_kernels as EK
import plain_qwen2moe as plain
from locus_b200.engine.engine import Engine, _history_tail
from locus_b200.engine.scheduler import Request, SchedulerConfig
from locus_b200.sampling.sampler import GREEDY, Sampler, SamplingParams


@pytest.fixture(autouse=True)
def _emulate(monkeypatch):
    EK.install(monkeypatch)


def rows(n, v=97, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, v, generator=g) * 3.0


def test_greedy_rows_after_a_sampled_and_a_shorter_greedy_batch_are_greedy():
    """Five sampled rows, then two greedy rows, then five greedy rows: rows 2..4 of the device blocks must not
    still hold temperature 0.8 (the upload of a greedy batch may be skipped only for rows known to be greedy)."""
    s = Sampler("cpu", 8)
    hot = SamplingParams(temperature=0.8, top_p=0.9)
    lg = rows(5)
    s.sample(lg.clone(), [hot] * 5, [11] * 5, [0] * 5)
    s.sample(lg[:2].clone(), [GREEDY] * 2, [0] * 2, [0] * 2)
    for trial in range(4):  # a sampled row would differ from arg-max in some trial
        lg = rows(5, seed=trial + 1)
        assert s.sample(lg.clone(), [GREEDY] * 5, [0] * 5, [trial] * 5) == lg.argmax(1).tolist()
    assert float(s._df[:5].abs().max()) == 0.0
    # and the skipped upload stays skipped only as far as it is safe
    before = s.h2d_bytes
    s.sample(rows(3).clone(), [GREEDY] * 3, [0] * 3, [0] * 3)
    assert s.h2d_bytes == before
    s.sample(rows(7).clone(), [GREEDY] * 7, [0] * 7, [0] * 7)
    assert s.h2d_bytes > before


def test_mixed_rows_keep_their_own_parameters():
    s = Sampler("cpu", 4)
    lg = rows(3, seed=5)
    out = s.sample(lg.clone(), [GREEDY, SamplingParams(temperature=1.0, top_k=1), GREEDY], [3, 4, 5], [0, 0, 0])
    assert out == lg.argmax(1).tolist()  # top_k = 1 keeps the best token only
    with pytest.raises(ValueError, match="sampling parameters"):
        s.sample(lg.clone(), [GREEDY], [0], [0])


def test_penalties_see_repeat_last_n_tokens_however_many():
    V = 300
    s = Sampler("cpu", 2)
    history = list(range(200))                      # 200 distinct tokens
    p = SamplingParams(presence_penalty=100.0, repeat_last_n=150)
    lg = torch.zeros(1, V)
    lg[0, 60] = 1.0                                 # among the last 150 (50..199): penalised
    lg[0, 10] = 0.5                                 # older than that: not
    want = plain.apply_penalties(lg[0].double(), history, 1.0, 0.0, 100.0, 150)
    assert s.sample(lg.clone(), [p], [0], [0], [history]) == [int(want.argmax())] == [10]
    assert s.max_history >= 150
    # a window of 64 (the default) would have left token 60 alone
    assert s.sample(lg.clone(), [SamplingParams(presence_penalty=100.0)], [0], [0], [history]) == [60]
    with pytest.raises(ValueError, match="repeat_last_n"):
        SamplingParams(repeat_last_n=-1).validate()


def test_history_tail_is_the_end_of_prompt_plus_generated():
    def req(prompt, generated, n):
        r = Request.__new__(Request)
        r.prompt, r.generated = prompt, generated
        r.sampling = SamplingParams(repeat_penalty=1.1, repeat_last_n=n)
        return r

    assert _history_tail(req([1, 2, 3], [4, 5], 4)) == [2, 3, 4, 5]
    assert _history_tail(req([1, 2, 3], [4, 5], 2)) == [4, 5]
    assert _history_tail(req([1, 2, 3], [4, 5], 64)) == [1, 2, 3, 4, 5]
    assert _history_tail(req([1, 2, 3], [], 2)) == [2, 3]
    assert _history_tail(req([1, 2, 3], [4], 0)) == []


class _FaultyRunner:
    """A step function whose device records a fault in its third step: logits still come back, the
    error word is set from then on."""

    def __init__(self, cache, vocab):
        self.cache, self.vocab, self.checked, self.steps = cache, vocab, 0, 0

    def step(self, entries):
        self.steps += 1
        for e in entries:
            self.cache.commit(e.seq, len(e.tokens))
        return torch.zeros(sum(len(e.want) for e in entries), self.vocab)

    def check_device_errors(self):
        self.checked += 1
        if self.steps >= 3:
            raise RuntimeError("tensor-core kernel fault: a pipeline wait ran out (code 2)")


def test_generate_raises_when_the_device_recorded_a_fault(tmp_path):
    from locus_b200.cache import CacheManager
    from locus_b200.parts.base import PagedKvSpec

    cache = CacheManager([(PagedKvSpec(1, 16), None, None)], page_tokens=16, n_pages=8, n_state_slots=2,
                         max_seq_tokens=128, dtype=torch.float32, device="cpu")
    runner = _FaultyRunner(cache, 32)
    eng = Engine(runner, cache, Sampler("cpu", 2), max_positions=128,
                 config=SchedulerConfig(max_batch_tokens=16, chunk=16, max_running=2, decode_headroom=2))
    with pytest.raises(RuntimeError, match="pipeline wait ran out"):
        eng.generate([[1, 2, 3]], max_new_tokens=5)
    assert runner.steps == 5 and runner.checked == 2  # after the first step (nothing yet) and at the end
