"""The scheduler's decisions (no GPU): budgets, order, portions, finishing, and
what happens when pages run out."""
import random

import pytest

from firefly_b200.cache import CacheManager, PagedKVSpec
from firefly_b200.engine.request import GenerationRequest, RequestStatus
from firefly_b200.engine.scheduler import Scheduler
from firefly_b200.sampling import SamplingParams

V = 1000


def next_token(tokens):
    """A stand-in for the model: the next token is a function of all tokens so far,
    so any error in what is fed (order, loss, repeat) changes the output."""
    h = 1469598103934665603
    for t in tokens:
        h = ((h ^ (t + 1)) * 1099511628211) & ((1 << 64) - 1)
    return h % V


def make(num_blocks=64, block=16, chunk=256, budget=8192, limit=64, max_len=4096, eos=()):
    cache = CacheManager({0: PagedKVSpec(2, 16), 1: PagedKVSpec(2, 16)}, block_size=block,
                         num_blocks=num_blocks, max_requests=limit)
    return Scheduler(cache, max_batch_size_limit=limit, max_prefill_chunk_size=chunk,
                     max_num_batched_tokens=budget, max_model_len=max_len, eos_token_ids=eos), cache


def run(sched, cache, log=None, max_steps=100000):
    """The engine loop with the stand-in model.  Returns per-step item lists."""
    steps = []
    while sched.has_unfinished_requests():
        batch = sched.step()
        assert batch.items or batch.failed or batch.preempted, "no progress"
        fed = []
        for it in batch.items:
            req = it.request
            assert it.start == req.context_len
            toks = req.tokens_between(it.start, it.start + it.num_tokens)
            assert len(toks) == it.num_tokens
            fed.append((req.id, it.start, it.num_tokens, it.samples))
            cache.advance(req.cache, it.num_tokens)
        for it in batch.items:
            if it.samples:
                req = it.request
                all_toks = req.prompt_tokens + req.generated_tokens
                assert req.context_len == len(all_toks)
                sched.append_token(req, next_token(all_toks))
        cache.check()
        steps.append(fed)
        assert len(steps) < max_steps
    return steps


def alone(prompt, n):
    toks = list(prompt)
    out = []
    for _ in range(n):
        out.append(next_token(toks))
        toks.append(out[-1])
    return out


def req(i, n_prompt, max_tokens=8, seed=0, **kw):
    rng = random.Random(seed * 1000 + i)
    return GenerationRequest(f"r{i}", [rng.randrange(V) for _ in range(n_prompt)],
                             SamplingParams(max_tokens=max_tokens, **kw))


def test_prompt_is_cut_into_portions_then_decoded():
    sched, cache = make(chunk=17, num_blocks=8)
    r = req(0, 40)
    sched.add_request(r)
    steps = run(sched, cache)
    assert [s[0][2] for s in steps[:3]] == [17, 17, 6]            # as the reference cuts it
    assert [s[0][3] for s in steps[:3]] == [False, False, True]
    assert all(s == [("r0", 40 + i, 1, True)] for i, s in enumerate(steps[3:]))
    assert r.generated_tokens == alone(r.prompt_tokens, 8) and r.finish_reason == "length"
    assert r.status is RequestStatus.FINISHED and cache.num_free_blocks == 8 and not cache.live


def test_prompts_are_not_cut_while_nobody_decodes():
    """With ``whole_prompts_when_idle`` a portion may fill the step's token budget as long as no
    request is decoding; as soon as one is, later prompts come in portions of the configured size.
    The tokens produced do not depend on it."""
    for idle_whole in (False, True):
        sched, cache = make(chunk=64, budget=1000, num_blocks=256)
        sched.whole_prompts_when_idle = idle_whole
        a, b = req(0, 700, max_tokens=20), req(1, 500, max_tokens=3)
        sched.add_request(a)
        first = sched.step()
        assert [(it.request.id, it.num_tokens) for it in first.items] == [("r0", 700 if idle_whole else 64)]
        for it in first.items:
            cache.advance(it.request.cache, it.num_tokens)
            if it.samples:
                sched.append_token(a, next_token(a.prompt_tokens))
        sched.add_request(b)                        # arrives while (or before) r0 decodes
        steps = run(sched, cache)
        portions_b = [n for step in steps for (rid, _, n, _) in step if rid == "r1"]
        if idle_whole:
            # r0 was decoding when r1 came in: r1 is cut into portions of 64
            assert portions_b[:7] == [64] * 7 and max(portions_b) == 64
        assert a.generated_tokens == alone(a.prompt_tokens, 20) and b.generated_tokens == alone(b.prompt_tokens, 3)
    # the budget still bounds a whole prompt
    sched, cache = make(chunk=64, budget=300, num_blocks=256)
    sched.whole_prompts_when_idle = True
    sched.add_request(req(2, 700, max_tokens=1))
    assert [it.num_tokens for it in sched.step().items] == [300]


def test_token_budget_and_limits_hold():
    sched, cache = make(chunk=64, budget=100, limit=3, num_blocks=200)
    rs = [req(i, 150 + 10 * i, max_tokens=5) for i in range(6)]
    for r in rs:
        sched.add_request(r)
    steps = run(sched, cache)
    for fed in steps:
        assert sum(n for _, _, n, _ in fed) <= 100
        assert all(n <= 64 for _, _, n, _ in fed)
        assert len(fed) <= 3
    # decodes and prompt portions share steps
    assert any(any(n == 1 for *_, n, _ in fed) and any(n > 1 for *_, n, _ in fed) for fed in steps)
    for r in rs:
        assert r.generated_tokens == alone(r.prompt_tokens, 5)
    # first come, first served
    first_seen = []
    for fed in steps:
        for rid, *_ in fed:
            if rid not in first_seen:
                first_seen.append(rid)
    assert first_seen == [r.id for r in rs]


def test_active_requests_go_first():
    sched, cache = make(chunk=32, budget=40, num_blocks=100)
    a, b = req(0, 10, max_tokens=20), req(1, 100, max_tokens=3)
    sched.add_request(a)
    run_one = sched.step()
    for it in run_one.items:
        cache.advance(it.request.cache, it.num_tokens)
        sched.append_token(it.request, 1)
    sched.add_request(b)
    batch = sched.step()
    assert [(it.request.id, it.num_tokens) for it in batch.items] == [("r0", 1), ("r1", 32)]


def test_pages_run_out_preempts_newest_and_everyone_finishes():
    # the reference's livelock case: 4 pages of 16, two prompts of 30 tokens
    sched, cache = make(num_blocks=4, chunk=256)
    a, b = req(0, 30, max_tokens=12), req(1, 30, max_tokens=12)
    sched.add_request(a)
    sched.add_request(b)
    run(sched, cache)
    assert a.generated_tokens == alone(a.prompt_tokens, 12)
    assert b.generated_tokens == alone(b.prompt_tokens, 12)     # recomputed after preemption: same tokens
    assert b.num_preemptions >= 1 and a.num_preemptions == 0     # the oldest is never the victim
    assert cache.num_free_blocks == 4 and not cache.live


def test_request_that_cannot_fit_alone_fails_with_error():
    sched, cache = make(num_blocks=4)
    big, ok = req(0, 100), req(1, 20, max_tokens=4)
    sched.add_request(big)
    sched.add_request(ok)
    run(sched, cache)
    assert big.finish_reason.startswith("error") and "pages" in big.finish_reason
    assert ok.generated_tokens == alone(ok.prompt_tokens, 4)
    # grows past the pool while decoding, alone
    sched, cache = make(num_blocks=2)
    r = req(2, 30, max_tokens=50)
    sched.add_request(r)
    run(sched, cache)
    assert r.finish_reason.startswith("error") and len(r.generated_tokens) == 3   # 30 + 3 = 33 > 32
    assert cache.num_free_blocks == 2


def test_eos_and_length():
    sched, cache = make()
    r = req(0, 5, max_tokens=50)
    want = alone(r.prompt_tokens, 50)
    sched, cache = make(eos=[want[6]])
    sched.add_request(r)
    run(sched, cache)
    k = want.index(want[6])
    assert r.generated_tokens == want[:k + 1] and r.finish_reason == "eos"
    r2 = GenerationRequest("x", list(r.prompt_tokens), SamplingParams(max_tokens=9, ignore_eos=True))
    sched.add_request(r2)
    run(sched, cache)
    assert r2.generated_tokens == want[:9] and r2.finish_reason == "length"
    # the model length ends a request too
    sched, cache = make(max_len=12)
    r3 = req(3, 8, max_tokens=50)
    sched.add_request(r3)
    run(sched, cache)
    assert r3.get_total_len() == 12 and r3.finish_reason == "length"
    with pytest.raises(ValueError, match="empty"):
        sched.add_request(GenerationRequest("e", []))
    with pytest.raises(ValueError, match="max_model_len"):
        sched.add_request(req(4, 12))


@pytest.mark.parametrize("seed", range(5))
def test_random_load_under_scarcity(seed):
    rng = random.Random(seed)
    block = rng.choice([4, 16])
    sched, cache = make(num_blocks=rng.choice([12, 30]), block=block, chunk=rng.choice([5, 33, 256]),
                        budget=rng.choice([16, 64, 1000]), limit=rng.choice([2, 4, 8]))
    cap = cache.num_blocks * block
    rs = []
    for i in range(14):
        n = rng.randrange(1, cap // 2)
        r = req(i, n, max_tokens=rng.randrange(1, max(2, min(40, cap - n))), seed=seed)
        rs.append(r)
        sched.add_request(r)
    steps = run(sched, cache)
    for r in rs:
        assert r.finish_reason == "length", (r.id, r.finish_reason)
        assert r.generated_tokens == alone(r.prompt_tokens, r.max_tokens)
    assert cache.num_free_blocks == cache.num_blocks and not cache.live
    for fed in steps:
        assert sum(n for _, _, n, _ in fed) <= sched.max_num_batched_tokens
        assert len(fed) <= sched.max_batch_size_limit


def _golden():
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "ref_scheduler_trace.json")) as fh:
        return json.load(fh)


@pytest.mark.parametrize("name", sorted(_golden()))
def test_same_portions_and_order_as_the_reference_scheduler(name):
    """Where the reference's scheduler is sound (distinct prompts, pages to spare) this one makes
    the same decisions: the recorded run of the reference's own scheduler (tests/golden/) and this
    scheduler feed the same requests the same number of tokens from the same context length, in the
    same order, iteration by iteration.  Pages held are not compared: the reference gives later
    portions of a long prompt too few (one more page a step), this one what the portion needs."""
    g = _golden()[name]
    sched, cache = make(num_blocks=g["pages"], block=16, chunk=g["max_prefill_chunk_size"],
                        limit=g["max_batch_size_limit"])
    rng = random.Random(1)
    for rid, n_prompt, max_tokens in g["requests"]:
        sched.add_request(GenerationRequest(rid, [rng.randrange(V) for _ in range(n_prompt)],
                                            SamplingParams(max_tokens=max_tokens)))
    steps = run(sched, cache)
    assert [[[rid, start, n] for rid, start, n, _ in s] for s in steps] == \
        [[[rid, start, n] for rid, start, n, _pages in s] for s in g["steps"]]
