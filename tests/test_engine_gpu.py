"""Generation through the Python entry point on the GPU, compared with the plain
implementation: greedy tokens, scarcity of pages, captured graphs, sampling."""
import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as U

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg, seed in (("A", P.TINY_A, 0), ("B", P.TINY_B, 1)):
        w = P.random_weights(cfg, seed, dtype=torch.float32, scale=0.05)
        path = str(tmp_path_factory.mktemp(f"gen{name}"))
        U.write_model_dir(path, cfg, w, torch.float32)
        out[name] = (path, cfg, w)
    return out


def _llm(path, **kw):
    from firefly_b200 import LLM
    return LLM(path, **kw)


@pytest.mark.parametrize("name,block,chunk", [("A", 16, 256), ("B", 8, 17)])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_matches_plain(models, name, block, chunk, graphs):
    path, cfg, w = models[name]
    rng = np.random.RandomState(5)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=n))) for n in (1, 2, 40, 23, 9)]
    llm = _llm(path, dtype="float32", kv_block_size=block, max_prefill_chunk_size=chunk,
               num_kv_blocks=64, use_cuda_graphs=graphs)
    got = llm.generate(prompts, max_tokens=12)
    for p, g in zip(prompts, got):
        assert g == P.greedy_generate(cfg, w, p, 12)
    if graphs:
        assert llm.engine.stats["graph_steps"] > 0
    llm.engine.cache.check()
    assert not llm.engine.cache.live


def test_few_pages_preempt_and_still_match(models):
    path, cfg, w = models["B"]
    rng = np.random.RandomState(7)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=n))) for n in (30, 30, 21, 5)]
    llm = _llm(path, dtype="float32", kv_block_size=8, num_kv_blocks=10, max_prefill_chunk_size=16)
    got = llm.generate(prompts, max_tokens=14)
    assert llm.engine.stats["preemptions"] > 0
    for p, g in zip(prompts, got):
        assert g == P.greedy_generate(cfg, w, p, 14)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_more_decoding_requests_than_the_largest_graph(models, dtype):
    """70 requests decode together: more than the largest captured batch (64), so those steps run
    without a graph (one-token sequences, the split-KV attention at a batch of 70)."""
    path, cfg, w = models["B"]
    rng = np.random.RandomState(11)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=int(n)))) for n in rng.randint(1, 12, size=70)]
    llm = _llm(path, dtype=dtype, kv_block_size=8, num_kv_blocks=70 * 4, max_batch_size_limit=80,
               max_prefill_chunk_size=64, max_num_batched_tokens=1024)
    got = llm.generate(prompts, max_tokens=5)
    st = llm.engine.stats
    assert st["steps"] > st["graph_steps"] and len(llm.engine.scheduler.active_requests) == 0
    wd = {k: v.double() for k, v in w.items()}
    for p, g in zip(prompts, got):
        if dtype == "float32":
            assert g == P.greedy_generate(cfg, w, p, 5)
        else:
            rows = P.forward(cfg, wd, list(p) + g[:-1])
            for i, tok in enumerate(g):
                row = rows[len(p) - 1 + i]
                assert float(row.max() - row[tok]) <= U.TOL[dtype] * float(row.abs().max())
    llm.engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_whose_shape_repeats_run_from_graphs_with_the_same_tokens(models, dtype):
    """Long prompts come in in portions of 16 while other requests decode: the same step shapes repeat
    and are captured at their second coming.  Tokens (greedy and sampled) must not depend on it."""
    path, cfg, w = models["B"]
    rng = np.random.RandomState(21)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=n))) for n in (150, 9, 131, 40, 200)]
    from firefly_b200.sampling import SamplingParams
    sp = [SamplingParams(temperature=0.0 if i % 2 == 0 else 0.8, seed=5 + i, max_tokens=10) for i in range(len(prompts))]
    got = {}
    for capture in (False, True):
        llm = _llm(path, dtype=dtype, kv_block_size=8, num_kv_blocks=128, max_prefill_chunk_size=16,
                   max_batch_size_limit=3, capture_repeating_steps=capture)
        got[capture] = llm.generate(prompts, sampling=sp)
        g = llm.engine.graphs
        if capture:
            assert g.shape_captures > 0 and g.shape_replays > g.shape_captures
        else:
            assert g.shape_captures == 0
        llm.engine.cache.check()
        assert not llm.engine.cache.live
    if dtype == "float32":
        assert got[True] == got[False]
        for p, g, s in zip(prompts, got[True], sp):
            if s.temperature == 0:
                assert g == P.greedy_generate(cfg, w, p, 10)
    else:
        same = sum(a == b for a, b in zip(got[True], got[False]))
        assert same >= len(prompts) - 1          # bfloat16: the same kernels and order, so all but a rare near-tie


def test_long_decoding_and_first_tokens(models):
    path, cfg, w = models["A"]
    llm = _llm(path, dtype="float32", num_kv_blocks=16)
    got = llm.generate([[7]], max_tokens=120)[0]          # from one token up to the model's length
    assert len(got) == 120
    assert got == P.greedy_generate(cfg, w, [7], 120)


def test_bfloat16_generation_picks_a_top_token(models):
    """bfloat16 may break a near tie the other way: every token it picks must be
    within rounding of the plain implementation's best at that place."""
    path, cfg, w = models["B"]
    rng = np.random.RandomState(9)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=n))) for n in (12, 33)]
    got = _llm(path, dtype="bfloat16", kv_block_size=8, num_kv_blocks=64).generate(prompts, max_tokens=8)
    for p, g in zip(prompts, got):
        assert len(g) == 8
        ids = list(p)
        for t in g:
            row = P.forward(cfg, w, ids)[-1]
            assert float(row.max() - row[t]) <= U.TOL["bfloat16"] * float(row.abs().max())
            ids.append(t)


@pytest.mark.parametrize("graphs", [False, True])
def test_bfloat16_requests_of_very_different_lengths(models, graphs):
    """One long request beside short ones: the decode attention shares its blocks out by length
    (from a graph of its own when graphs are on); the tokens stay within rounding of the best."""
    from firefly_b200.ops import kernels as K
    path, cfg, w = models["B"]
    rng = np.random.RandomState(21)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=n))) for n in (200, 5, 12)]
    llm = _llm(path, dtype="bfloat16", kv_block_size=8, num_kv_blocks=96, use_cuda_graphs=graphs)
    calls = K.BY_LENGTH_CALLS
    got = llm.generate(prompts, max_tokens=6)
    if graphs:
        assert llm.engine.graphs.replays_by_length > 0
    else:
        assert K.BY_LENGTH_CALLS > calls
    for p, g in zip(prompts, got):
        assert len(g) == 6
        ids = list(p)
        for t in g:
            row = P.forward(cfg, w, ids)[-1]
            assert float(row.max() - row[t]) <= U.TOL["bfloat16"] * float(row.abs().max())
            ids.append(t)
    llm.engine.cache.check()


def test_temperature_sampling_is_seeded_and_follows_softmax(models):
    path, cfg, w = models["A"]
    llm = _llm(path, dtype="float32", num_kv_blocks=32)
    a = llm.generate([[1, 2, 3]] * 2, max_tokens=10, temperature=0.8, seed=11)
    b = llm.generate([[1, 2, 3]] * 2, max_tokens=10, temperature=0.8, seed=11)
    c = llm.generate([[1, 2, 3]], max_tokens=10, temperature=0.8, seed=12)
    assert a == b and a[0] != a[1] and c[0] == a[1]        # request i uses seed + i
    # the kernel alone: frequencies follow softmax(logits / T)
    from firefly_b200.ops import kernels as K
    V, n, T = 37, 20000, 0.7
    logits = torch.randn(V, device="cuda") * 2
    rows = logits[None, :].expand(n, V).contiguous()
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    temp = torch.full((n,), T, device="cuda")
    seeds = torch.full((n,), 5, dtype=torch.int64, device="cuda")
    counters = torch.arange(n, dtype=torch.int64, device="cuda")
    K.sample(rows, out, temp, seeds, counters)
    freq = torch.bincount(out.long(), minlength=V).double().cpu() / n
    want = torch.softmax(logits.double().cpu() / T, dim=0)
    assert float((freq - want).abs().max()) < 0.015
    out2 = torch.empty_like(out)
    K.sample(rows, out2, temp, seeds, counters)
    assert torch.equal(out, out2)
    K.sample(rows, out2)                                   # no temperature: arg-max
    assert int(out2[0]) == int(torch.argmax(logits))


def test_temperature_draws_do_not_depend_on_graphs_or_launching_ahead(models):
    """The sampler inside the captured step draws what the sampler outside it draws: the same
    tokens with graphs and steps launched ahead, with graphs alone and without graphs, for a
    batch that mixes greedy requests with requests of different temperatures and lengths."""
    from firefly_b200 import SamplingParams
    path, cfg, w = models["B"]
    rng = np.random.RandomState(21)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=n))) for n in (4, 21, 9, 2, 30)]
    params = [SamplingParams(temperature=t, seed=s, max_tokens=m)
              for t, s, m in ((0.9, 3, 24), (0.0, 0, 11), (1.3, 4, 17), (0.6, 5, 24), (0.0, 0, 5))]
    got = {}
    for graphs, overlap in ((True, True), (True, False), (False, False)):
        llm = _llm(path, dtype="float32", kv_block_size=8, num_kv_blocks=64, max_prefill_chunk_size=16,
                   use_cuda_graphs=graphs, overlap_decode=overlap)
        got[(graphs, overlap)] = llm.generate(prompts, sampling=params)
        if overlap:
            assert llm.engine.stats["launched_ahead"] > 0
        llm.engine.cache.check()
        assert not llm.engine.cache.live and llm.engine._inflight is None
    assert got[(True, True)] == got[(False, False)] == got[(True, False)]
    assert [len(t) for t in got[(True, True)]] == [p.max_tokens for p in params]
    assert got[(True, True)][1] == P.greedy_generate(cfg, w, prompts[1], 11)     # greedy lanes stay greedy


def test_argmax_ties_go_to_lowest_index():
    from firefly_b200.ops import kernels as K
    V = 151936 + 5
    x = torch.full((3, V), -1.0, device="cuda")
    x[0, 70000] = 2.0
    x[0, 150000] = 2.0
    x[1, V - 1] = 3.0
    x[2, :] = 0.5
    out = torch.empty(3, dtype=torch.int32, device="cuda")
    K.sample(x, out)
    assert out.tolist() == [70000, V - 1, 0]


def test_sampling_waits_for_the_product_that_writes_the_logits():
    """The sampler is launched right behind the output head's product, which lets its dependents
    start early: it must still see the finished logits.  A vocabulary of real size (two sampling
    kernels, a product that runs for a while), fresh activations every round so that stale logits
    would give another token."""
    from firefly_b200.ops import kernels as K
    V, H, T = 151936, 2048, 3
    g = torch.Generator(device="cuda").manual_seed(3)
    w = (torch.randn(V, H, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    logits = torch.zeros(T, V, device="cuda")
    out = torch.empty(T, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(8):
        x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
        K.gemm_tc(x, w, logits, K.EPI_F32, 1, status)
        K.sample(logits, out)
        torch.cuda.synchronize()
        best = logits.max(dim=1).values
        picked = logits[torch.arange(T, device="cuda"), out.long()]
        assert torch.equal(picked, best), (picked - best).tolist()
    assert int(status) == 0


def test_async_engine_interface(models):
    path, cfg, w = models["A"]
    from firefly_b200 import Engine, ResultQueue
    from firefly_b200.engine import load_model
    model, config = load_model(path, dtype="float32")
    q = ResultQueue()
    eng = Engine(model, config, q, max_prefill_chunk_size=8)
    assert eng.options.max_prefill_chunk_size == 8
    eng.start()
    eng.async_generate("x", [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5], 6)
    eng.async_generate("y", [2, 7], 4)
    toks = {"x": [], "y": []}
    finished = set()
    while len(finished) < 2:
        out = q.pop(timeout=30)
        assert out is not None
        toks[out.request_id] += out.new_tokens
        if out.is_finished:
            finished.add(out.request_id)
    eng.stop()
    assert toks["x"] == P.greedy_generate(cfg, w, [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5], 6)
    assert toks["y"] == P.greedy_generate(cfg, w, [2, 7], 4)


def test_decode_steps_launched_ahead_give_the_same_tokens(models):
    """Greedy decode steps are put on the stream before the step before them has been read.
    Requests of different lengths end at different steps, some by an end-of-sequence token
    that the engine learns of one step late: the tokens are those of the plain implementation
    (cut at the end-of-sequence token), with and without the overlap."""
    from firefly_b200 import SamplingParams
    path, cfg, w = models["A"]
    rng = np.random.RandomState(11)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=n))) for n in (5, 19, 3, 33)]
    limits = [25, 9, 17, 25]
    plain = [P.greedy_generate(cfg, w, p, m) for p, m in zip(prompts, limits)]
    first = {}
    for i, t in enumerate(plain[0]):
        first.setdefault(t, i)
    eos = max(first, key=first.get)                     # request 0 ends by end of sequence, some steps in
    assert 3 <= first[eos] < limits[0] - 1

    def cut(toks):
        return toks[:toks.index(eos) + 1] if eos in toks else toks
    want = [cut(t) for t in plain]
    assert len(want[0]) < limits[0]
    results = {}
    for overlap in (True, False):
        llm = _llm(path, dtype="float32", num_kv_blocks=64, overlap_decode=overlap, eos_token_ids=[eos])
        got = llm.generate(prompts, sampling=[SamplingParams(max_tokens=m) for m in limits])
        assert got == want
        st = llm.engine.stats
        if overlap:
            assert st["launched_ahead"] > 0
            # alone, request 0 is ahead by one step when its end-of-sequence token is read
            before = st["dropped_tokens"]
            assert llm.generate([prompts[0]], max_tokens=limits[0]) == [want[0]]
            assert llm.engine.stats["dropped_tokens"] == before + 1
        else:
            assert st["launched_ahead"] == 0
        llm.engine.cache.check()
        assert not llm.engine.cache.live and llm.engine._inflight is None
        results[overlap] = got
    assert results[True] == results[False]


def test_launch_ahead_stops_for_new_requests_and_scarce_pages(models):
    """A waiting request, or a batch whose next pages are not all free, is left to the scheduler."""
    from firefly_b200 import Engine, SamplingParams
    from firefly_b200.engine import load_model
    from firefly_b200.engine.engine import EngineOptions
    from firefly_b200.engine.request import GenerationRequest
    path, cfg, w = models["B"]
    model, config = load_model(path, dtype="float32")
    eng = Engine(model, config, options=EngineOptions(kv_block_size=8, num_kv_blocks=12, max_prefill_chunk_size=16))
    a, b = [3, 1, 4, 1, 5, 9, 2, 6], [2, 7, 1, 8, 2, 8]
    ra = GenerationRequest("a", a, SamplingParams(max_tokens=40))
    eng.add_request(ra)
    for _ in range(4):
        eng.step()
    assert eng.stats["launched_ahead"] > 0
    rb = GenerationRequest("b", b, SamplingParams(max_tokens=30))
    eng.add_request(rb)                                 # arrives while a step of "a" is on the stream
    while eng.has_unfinished_requests():
        eng.step()
    assert ra.generated_tokens == P.greedy_generate(cfg, w, a, 40)
    assert rb.generated_tokens == P.greedy_generate(cfg, w, b, 30)
    eng.cache.check()
    assert not eng.cache.live


@pytest.mark.parametrize("seed", [0, 1])
def test_many_requests_few_pages_random_lengths(models, seed):
    """Two dozen requests of random lengths on a pool that holds a few of them: admission, portions,
    steps launched ahead, ends by length at every step, preemption and recomputation all meet; every
    request still gets the plain implementation's greedy tokens and every page comes back."""
    from firefly_b200 import SamplingParams
    path, cfg, w = models["B"]
    rng = np.random.RandomState(100 + seed)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=int(rng.randint(1, 41))))) for _ in range(24)]
    limits = [int(rng.randint(1, 21)) for _ in prompts]
    llm = _llm(path, dtype="float32", kv_block_size=8, num_kv_blocks=14, max_prefill_chunk_size=16,
               max_batch_size_limit=6, max_num_batched_tokens=48)
    got = llm.generate(prompts, sampling=[SamplingParams(max_tokens=m) for m in limits])
    st = llm.engine.stats
    assert st["preemptions"] > 0 and st["launched_ahead"] > 0
    for p, m, g in zip(prompts, limits, got):
        assert g == P.greedy_generate(cfg, w, p, m)
    llm.engine.cache.check()
    assert not llm.engine.cache.live and llm.engine._inflight is None


def test_sampled_requests_survive_preemption_with_the_same_draws(models):
    """A preempted request recomputes its prompt and the tokens it had drawn, and goes on with the
    counter where it stood: sampled with a temperature on a pool that forces preemptions, every
    request gets the tokens it gets on a pool with room for all."""
    from firefly_b200 import SamplingParams
    path, cfg, w = models["B"]
    rng = np.random.RandomState(33)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=n))) for n in (30, 28, 21, 5, 17, 9)]
    params = [SamplingParams(temperature=0.7 + 0.1 * i, seed=50 + i, max_tokens=16) for i in range(len(prompts))]
    got = {}
    for pages in (10, 96):
        llm = _llm(path, dtype="float32", kv_block_size=8, num_kv_blocks=pages, max_prefill_chunk_size=16)
        got[pages] = llm.generate(prompts, sampling=params)
        assert (llm.engine.stats["preemptions"] > 0) == (pages == 10)
        llm.engine.cache.check()
        assert not llm.engine.cache.live
    assert got[10] == got[96]


def test_host_may_run_steps_ahead_of_the_device(tmp_path):
    """Steps without wanted logits are never waited for, so the host can queue several of them while
    the device is still busy; each must run with its own metadata.  The device is held up by a
    spinning kernel while a prompt is queued in more portions than there are metadata buffers.  A second
    request that holds thousands of pages rides along, so that a step's block tables are tens of
    kilobytes (a copy that is small enough may be taken at the time it is queued and would hide the
    fault)."""
    from firefly_b200.engine.runner import StepEntry
    from firefly_b200.replay import ReplaySession
    cfg = dict(P.TINY_B, max_position_embeddings=65536)
    w = P.random_weights(cfg, 1, dtype=torch.float32, scale=0.05)
    path = U.write_model_dir(str(tmp_path), cfg, w, torch.float32)
    rng = np.random.RandomState(4)
    toks = list(map(int, rng.randint(0, cfg["vocab_size"], size=60)))
    want = P.forward(cfg, w, toks)[-1].numpy()
    for hold in (False, True):
        s = ReplaySession(path, dtype="float32", max_tokens=65536, block_size=8)
        assert s.runner.max_blocks == [8192]
        warm = s.cache.admit("warm")                    # scratch buffers get their sizes before the hold
        assert s.cache.grow(warm, 13)
        s.runner.step([StepEntry(warm, toks[:13], [])])
        torch.cuda.synchronize()
        s.cache.free(warm)
        rc = s.cache.admit("a")
        big = s.cache.admit("big")                      # its table is as wide as 40000 tokens need
        assert s.cache.grow(big, 40000) and len(big.tables[0]) == 5000
        if hold:
            torch.cuda._sleep(int(3e8))                 # some tenths of a second
        p = 0
        for k, n in enumerate((7, 2, 13, 5, 9, 11, 3, 10)):
            assert s.cache.grow(rc, p + n)
            last = s.runner.step([StepEntry(rc, toks[p:p + n], [n - 1] if p + n == len(toks) else []),
                                  StepEntry(big, [toks[k]], [])])
            p += n
        got = last[0].cpu().numpy()
        s.runner.check_status()
        assert U.rel_err(got, want) <= U.TOL["float32"], f"hold={hold}"


def test_serving_benchmark_counts_and_figures(models):
    """The closed-loop load tool on the asynchronous interface: every request is served, with
    the tokens asked for, and the figures are those of the reference's tool."""
    from firefly_b200.engine import load_model
    from firefly_b200.engine.engine import Engine, EngineOptions, ResultQueue
    from firefly_b200.serving_bench import report, run_load
    path, cfg, w = models["A"]
    model, config = load_model(path, dtype="float32")
    q = ResultQueue()
    eng = Engine(model, config, result_queue=q,
                 options=EngineOptions(kv_block_size=16, num_kv_blocks=24, max_prefill_chunk_size=8))
    rng = np.random.RandomState(9)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=n))) for n in (5, 30, 12, 1, 22, 9, 17)]
    res = run_load(eng, q, prompts, concurrency=3, max_tokens=6)
    assert res["successful"] == 7 and res["failed"] == 0 and res["total_tokens"] == 42
    assert res["ttft_s"]["median"] > 0 and res["tpot_s"]["p99"] >= res["tpot_s"]["median"] > 0
    assert "Mean TPOT" in report(res) and "Throughput" in report(res)
    eng.cache.check()
    assert not eng.cache.live
