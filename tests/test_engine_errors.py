"""Errors reach the caller: a raised device status ends the step's requests with an error, and an
exception in the engine's thread leaves nobody waiting.  A stand-in step function and sampler are
used, so no device is needed (the reference prints such errors and goes on, src/engine.cc:330-333)."""
import time
from types import SimpleNamespace

import pytest
import torch

from firefly_b200.cache import PagedKVSpec
from firefly_b200.engine.engine import Engine, EngineOptions, ResultQueue
from firefly_b200.engine.request import GenerationRequest
from firefly_b200.sampling.params import SamplingParams


class _Read:
    def __init__(self, code):
        self._code = code

    def code(self):
        return self._code


class StandInRunner:
    """Advances the caches like the real step function and reports a status the test sets."""

    def __init__(self, cache):
        self.cache = cache
        self.status_now = 0
        self.fail_at_step = None
        self.raise_at_step = None
        self.steps = 0
        self.cleared = 0

    def step(self, entries):
        self.steps += 1
        if self.raise_at_step == self.steps:
            raise RuntimeError("stand-in step function broke")
        if self.fail_at_step == self.steps:
            self.status_now = 4
        for e in entries:
            self.cache.advance(e.cache, len(e.tokens))
        return torch.zeros(sum(len(e.want) for e in entries), 8)

    def queue_status_read(self):
        return _Read(self.status_now)

    def clear_status(self):
        self.status_now = 0
        self.cleared += 1

    def check_status(self):
        pass


class StandInSampler:
    def sample(self, logits, params, counters):
        return [3] * logits.shape[0]


def _engine(queue=None, **opts):
    model = SimpleNamespace(rt=SimpleNamespace(device=torch.device("cpu"), dtype=torch.float32),
                            spec=SimpleNamespace(max_positions=256, vocab_size=8),
                            cache_slot_specs=lambda: {0: PagedKVSpec(1, 4, None)})
    options = EngineOptions(num_kv_blocks=64, kv_block_size=4, use_cuda_graphs=False, max_prefill_chunk_size=8, **opts)
    eng = Engine(model, options=options, result_queue=queue, runner=None if False else object(), sampler=StandInSampler())
    eng.runner = StandInRunner(eng.cache)
    return eng


def test_raised_status_ends_the_steps_requests_and_the_engine_goes_on():
    eng = _engine()
    a = GenerationRequest("a", [1, 2, 3], SamplingParams(max_tokens=5))
    b = GenerationRequest("b", [4, 5], SamplingParams(max_tokens=5))
    eng.add_request(a)
    eng.add_request(b)
    eng.runner.fail_at_step = 2
    outs = eng.step()                                       # step 1: both prompts, fine
    assert sorted(o.request_id for o in outs) == ["a", "b"] and not any(o.is_finished for o in outs)
    outs = eng.step()                                       # step 2 raises the status word
    assert sorted(o.request_id for o in outs) == ["a", "b"] and all(o.is_finished for o in outs)
    assert all(o.finish_reason.startswith("error: device status 4") and "block table" in o.finish_reason
               for o in outs)
    assert eng.runner.cleared == 1 and eng.stats["device_errors"] == 1
    assert not eng.has_unfinished_requests()
    eng.cache.check()
    assert eng.cache.num_free_blocks == 64                   # their pages are back
    # the next request is served as if nothing had happened
    c = GenerationRequest("c", [1], SamplingParams(max_tokens=2))
    eng.add_request(c)
    while eng.has_unfinished_requests():
        eng.step()
    assert c.finish_reason == "length" and c.generated_tokens == [3, 3]


def test_status_of_steps_without_sampled_tokens_is_looked_at_now_and_then():
    eng = _engine()
    eng.STATUS_EVERY = 3
    a = GenerationRequest("a", list(range(1, 8)) * 8, SamplingParams(max_tokens=2))       # 56 tokens, 7 portions of 8
    eng.add_request(a)
    eng.runner.fail_at_step = 1
    outs = []
    for _ in range(3):
        outs += eng.step()
    assert len(outs) == 1 and outs[0].finish_reason.startswith("error: device status 4")


def test_exception_in_the_loop_thread_finishes_everyone_and_is_raised_by_stop():
    q = ResultQueue()
    eng = _engine(q)
    eng.runner.raise_at_step = 2
    eng.start()
    eng.async_generate("a", [1, 2, 3], max_tokens=50)
    eng.async_generate("b", [1] * 40, max_tokens=50)         # still in its prompt when the loop breaks
    got = {}
    deadline = time.time() + 20
    while len(got) < 2 and time.time() < deadline:
        out = q.pop(timeout=0.5)
        if out is not None and out.is_finished:
            got[out.request_id] = out.finish_reason
    assert set(got) == {"a", "b"}
    assert all(r.startswith("error: engine loop failed: RuntimeError: stand-in step function broke") for r in got.values())
    with pytest.raises(RuntimeError, match="engine loop ended with an error"):
        eng.stop()
    eng.stop()                                               # a second stop has nothing left to raise
