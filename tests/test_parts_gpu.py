"""The parts alone, and the generality of their assembly: windows, a cache read by
another layer, a layer that runs twice, and a toy mixer with state of its own that
is registered, built and stepped from this file without a change to the package."""
import dataclasses
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as U

pytestmark = pytest.mark.gpu


def _runtime(dtype):
    from firefly_b200.parts import Runtime
    return Runtime(torch.device("cuda:0"), dtype)


def _bound_model(cfg, weights, dtype, spec_edit=None):
    from firefly_b200.models import DecoderModel, config_from_dict, spec_for
    from firefly_b200.ops import kernels as K
    K.set_exact_matmul()
    spec = spec_for(config_from_dict(cfg))
    if spec_edit is not None:
        spec = spec_edit(spec)
    model = DecoderModel(spec, _runtime(dtype))
    model.bind({k: v.to("cuda").to(dtype if v.dim() > 1 else torch.float32) for k, v in weights.items()})
    return model


def _session(model, max_tokens, block):
    from firefly_b200.replay import ReplaySession
    return ReplaySession(model=model, max_tokens=max_tokens, block_size=block)


def _context(model, seqs, block=8):
    """A StepContext for sequences given as (tokens already cached, new tokens)."""
    from firefly_b200.cache import CacheManager
    from firefly_b200.engine.runner import ModelRunner, StepEntry
    cache = CacheManager(model.cache_slot_specs(), block_size=block, num_blocks=64, max_requests=8)
    cache.allocate_storage(model.rt.dtype, model.rt.device)
    runner = ModelRunner(model, cache, max_model_len=256)
    entries = []
    for i, (ctx_len, toks) in enumerate(seqs):
        rc = cache.admit(i)
        assert cache.grow(rc, ctx_len + len(toks))
        rc.num_tokens = ctx_len
        entries.append(StepEntry(rc, toks, [len(toks) - 1]))
    return runner.build_context(entries), runner


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_each_part_alone(dtype):
    cfg = P.TINY_C                    # hidden 72, 3 q heads / 1 kv head, head 48, intermediate 200, vocab 333
    w = P.random_weights(cfg, 4, dtype=dtype, scale=0.08)
    wd = {k: v.double() for k, v in w.items()}
    model = _bound_model(cfg, w, dtype)
    ctx, runner = _context(model, [(0, [5, 9, 200, 7, 1, 300, 17]), (0, [3, 4])])
    T, H = 9, cfg["hidden_size"]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    g = torch.Generator().manual_seed(0)

    def close(got, want):
        want = want.double()
        return float((got.cpu().double() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))

    # embedding
    h = model.embedding.forward(ctx)
    ids = torch.tensor([5, 9, 200, 7, 1, 300, 17, 3, 4])
    assert h.dtype == torch.float32 and torch.equal(h.cpu(), P.embedding(ids, w["model.embed_tokens.weight"]).float())
    # norm (with a pending delta)
    blk = model.blocks[0]
    res = torch.randn(T, H, generator=g)
    delta = torch.randn(T, H, generator=g).to(dtype)
    r = res.cuda()
    x = blk.norms[0].forward(r, delta.cuda(), ctx)
    assert close(r, res.double() + delta.double())
    assert close(x, P.rms_norm(res.double() + delta.double(), wd["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"]))
    # position encoding: the table holds cos and sin of pos * theta^(-2i/d)
    table, rot = blk.position.rotary_table()
    assert rot == cfg["head_dim"] and table.shape == (cfg["max_position_embeddings"], rot // 2, 2)
    pos, i = 301, 5
    ang = pos * cfg["rope_theta"] ** (-2.0 * i / rot)
    assert abs(float(table[pos, i, 0]) - math.cos(ang)) < 1e-6 and abs(float(table[pos, i, 1]) - math.sin(ang)) < 1e-6
    # mixer: whole sequences from position 0, so the plain block sees the same keys
    xin = (torch.randn(T, H, generator=g)).to(dtype)
    got = blk.mixer.forward(xin.cuda(), ctx, 0, True)
    want = torch.cat([P.attention_block(xin[a:b].double(), wd, "model.layers.0.self_attn", cfg,
                                        torch.arange(b - a))[0] for a, b in ((0, 7), (7, 9))])
    assert close(got, want)
    # feed-forward
    got = blk.feed_forward.forward(xin.cuda(), ctx)
    want = P.swiglu_mlp(xin.double(), wd["model.layers.0.mlp.gate_proj.weight"], wd["model.layers.0.mlp.up_proj.weight"],
                        wd["model.layers.0.mlp.down_proj.weight"])
    assert close(got, want)
    # head: 32-bit logits
    rows = xin[:3].cuda()
    got = model.head.forward(rows, ctx)
    assert got.dtype == torch.float32 and close(got, xin[:3].double() @ wd["lm_head.weight"].T)
    runner.check_status()


def _edit_windows_and_schedule(windows, schedule):
    from firefly_b200.config import ScheduleEntry

    def edit(spec):
        layers = []
        for ls, win in zip(spec.layers, windows):
            layers.append(dataclasses.replace(ls, mixer=ls.mixer.with_params(window=win)))
        sched = tuple(ScheduleEntry(l, cache=c, write_cache=wr) for l, c, wr in schedule) if schedule \
            else spec.schedule
        return dataclasses.replace(spec, layers=tuple(layers), schedule=sched)
    return edit


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["windows", "shared_cache", "layer_twice"])
def test_assembly_is_data(dtype, case):
    cfg = P.TINY_B
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    w = P.random_weights(cfg, 6, dtype=tdt, scale=0.05)
    windows = [None, None, None]
    schedule = None
    if case == "windows":
        windows = [None, 21, 5]                    # three groups of pages: all keys, 21 keys, 5 keys
    elif case == "shared_cache":
        schedule = [(0, 0, True), (1, 1, True), (2, 1, False)]
    else:
        schedule = [(0, 0, True), (1, 1, True), (1, 2, True), (2, 3, True)]
    model = _bound_model(cfg, w, tdt, _edit_windows_and_schedule(windows, schedule))
    reqs = U.make_requests(cfg["vocab_size"], [90, 33, 140, 7, 61], 3)
    plain = {rid: P.forward(cfg, w, toks, windows=windows, schedule=schedule).numpy() for rid, toks in reqs.items()}
    for steps in (U.trace_whole(reqs), U.trace_mixed(reqs, seed=2, max_live=3)):
        sess = _session(model, U.peak_tokens(steps), 8)
        if case == "windows":
            assert len(sess.cache.groups) == 3
        got = U.run_trace(sess, steps)
        U.compare(got, plain, U.TOL[dtype], f"{case}/{dtype}")
        sess.cache.check()
        assert not sess.cache.live


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_groups_with_their_own_page_sizes_and_counts_through_the_engine(dtype):
    """Three cache groups: every key in pages of 8, a window of 21 in pages of 4, a window of 5 in pages
    of 16.  The engine gives the windowed groups the pages of their windows only; logits and generated
    tokens are the plain implementation's."""
    from firefly_b200.engine.engine import Engine, EngineOptions
    from firefly_b200.engine.request import GenerationRequest
    from firefly_b200.sampling import SamplingParams
    cfg = P.TINY_B
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    w = P.random_weights(cfg, 6, dtype=tdt, scale=0.05)
    windows, pages = [None, 21, 5], [None, 4, 16]

    def edit(spec):
        layers = [dataclasses.replace(ls, mixer=ls.mixer.with_params(window=win, cache_block_size=bs))
                  for ls, win, bs in zip(spec.layers, windows, pages)]
        return dataclasses.replace(spec, layers=tuple(layers))
    model = _bound_model(cfg, w, tdt, edit)
    # replay: whole, and mixed with pages used again
    reqs = U.make_requests(cfg["vocab_size"], [90, 33, 140, 7, 61], 3)
    plain = {rid: P.forward(cfg, w, toks, windows=windows).numpy() for rid, toks in reqs.items()}
    for steps in (U.trace_whole(reqs), U.trace_mixed(reqs, seed=2, max_live=3)):
        sess = _session(model, U.peak_tokens(steps), 8)
        assert [g.block_size for g in sess.cache.groups] == [8, 4, 16]
        U.compare(U.run_trace(sess, steps), plain, U.TOL[dtype], f"own page sizes/{dtype}")
        sess.cache.check()
    # the engine: sizes per group, generation equal to the plain implementation's
    opts = EngineOptions(num_kv_blocks=128, kv_block_size=8, max_batch_size_limit=4, max_prefill_chunk_size=16)
    eng = Engine(model, options=opts)
    full, w21, w5 = eng.cache.groups
    assert (full.num_blocks, full.block_size) == (128, 8)
    assert (w21.num_blocks, w21.block_size) == (4 * (-(-(21 + 16) // 4) + 2), 4)
    assert (w5.num_blocks, w5.block_size) == (4 * (-(-(5 + 16) // 16) + 2), 16)
    assert w5.num_blocks * w5.block_size < full.num_blocks * full.block_size // 2
    prompts = [reqs["r0"][:50], reqs["r1"][:20], reqs["r2"][:77]]
    rs = [GenerationRequest(f"g{i}", list(p), SamplingParams(max_tokens=12)) for i, p in enumerate(prompts)]
    for r in rs:
        eng.add_request(r)
    while eng.has_unfinished_requests():
        eng.step()
    eng.runner.check_status()
    eng.cache.check()
    for r, prompt in zip(rs, prompts):
        assert len(r.generated_tokens) == 12
        rows = P.forward(cfg, {k: v.double() for k, v in w.items()}, list(prompt) + r.generated_tokens[:-1], windows=windows)
        for i, tok in enumerate(r.generated_tokens):
            row = rows[len(prompt) - 1 + i]
            if dtype == "float32":
                assert tok == P.greedy_pick(row), (r.id, i)
            else:
                assert float(row.max() - row[tok]) <= U.TOL[dtype] * float(row.abs().max())


def test_window_pages_are_given_back_while_the_request_lives():
    cfg = P.TINY_A
    w = P.random_weights(cfg, 8, scale=0.05)
    model = _bound_model(cfg, w, torch.float32, _edit_windows_and_schedule([10, 10], None))
    toks = U.make_requests(cfg["vocab_size"], [128], 1)["r0"]
    plain = P.forward(cfg, w, toks, windows=[10, 10]).numpy()
    sess = _session(model, 64, 8)                 # 8 pages of 8 for a sequence of 128: only a window fits
    got = U.Collected()
    p = 0
    for k, n in enumerate([9, 1, 1, 17, 2, 1, 30, 1, 1, 1, 40, 24]):
        arr = sess.run_step({"step": k, "entries": [{"id": "w", "tokens": toks[p:p + n], "want": list(range(n))}]})
        for i in range(n):
            got.add("r0", p + i, arr[i])
        p += n
        held = sess.cache.groups[0].allocator.num_held
        assert held <= 10 // 8 + 2 + (n + 7) // 8
    assert p == 128
    U.compare(got, {"r0": plain}, U.TOL["float32"], "window, pages reused by the same request")


# ---------------------------------------------------------------- a toy mixer --
class ToyDecayMixer:
    """y_t = s_t W_out, s_t = decay * s_{t-1} + x_t W_in: state of fixed size per
    request, kept in the request's state slot between steps.  Written with torch
    operations; it stands for any mixer a user might add."""

    def __init__(self, spec, rt, position=None):
        from firefly_b200.parts.base import Part
        self._part = Part(spec, rt)
        self.hidden = spec.params["hidden_size"]
        self.state = spec.params["state_size"]
        self.decay = spec.params["decay"]
        self.prefix = spec.prefix

    def weight_specs(self):
        from firefly_b200.weights import WeightSpec
        return [WeightSpec(f"{self.prefix}.in.weight", (self.state, self.hidden)),
                WeightSpec(f"{self.prefix}.out.weight", (self.hidden, self.state))]

    def bind(self, tensors):
        self.w_in = tensors[f"{self.prefix}.in.weight"].float()
        self.w_out = tensors[f"{self.prefix}.out.weight"].float()

    def cache_spec(self):
        from firefly_b200.cache import StateSpec
        return StateSpec((self.state,), torch.float32)

    def forward(self, x, ctx, slot, write_cache):
        st = ctx.state(slot)                                   # [1 + max_requests, state]
        u = x.float() @ self.w_in.T
        out = torch.empty(x.shape[0], self.hidden, device=x.device)
        start = 0
        for i, n in enumerate(ctx.q_lens):
            # the slot is a value on the device: it is used as an index tensor, never read by the host,
            # so that the step can be captured into a CUDA graph
            sl = ctx.state_slots[i:i + 1].long()
            s = st.index_select(0, sl)[0] * (1 - ctx.seq_fresh[i]).float()   # a fresh request starts from zero
            for t in range(start, start + n):
                s = self.decay * s + u[t]
                out[t] = s @ self.w_out.T
            st.index_copy_(0, sl, s[None])
            start += n
        return out.to(ctx.dtype)


def _toy_plain(cfg, w, ids, decay):
    """Whole sequence, float64: attention layer 0, then the toy mixer as layer 1's mixer."""
    wd = {k: v.double() for k, v in w.items()}
    T = len(ids)
    pos = torch.arange(T)
    h = P.embedding(torch.tensor(ids), wd["model.embed_tokens.weight"])
    for layer in range(2):
        p = f"model.layers.{layer}"
        x = P.rms_norm(h, wd[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
        if layer == 0:
            a, _ = P.attention_block(x, wd, f"{p}.self_attn", cfg, pos)
        else:
            s = torch.zeros(wd["toy.in.weight"].shape[0], dtype=torch.float64)
            rows = []
            for t in range(T):
                s = decay * s + wd["toy.in.weight"] @ x[t]
                rows.append(wd["toy.out.weight"] @ s)
            a = torch.stack(rows)
        h = h + a
        x = P.rms_norm(h, wd[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        h = h + P.swiglu_mlp(x, wd[f"{p}.mlp.gate_proj.weight"], wd[f"{p}.mlp.up_proj.weight"], wd[f"{p}.mlp.down_proj.weight"])
    x = P.rms_norm(h, wd["model.norm.weight"], cfg["rms_norm_eps"])
    return (x @ wd["model.embed_tokens.weight"].T).numpy()


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    from firefly_b200.config import PartSpec
    from firefly_b200.models import DecoderModel, config_from_dict, spec_for
    from firefly_b200.parts import register_part
    register_part("mixer", "toy_decay", ToyDecayMixer, replace=True)
    cfg = P.TINY_A
    decay = 0.9
    spec = spec_for(config_from_dict(cfg))
    toy = PartSpec("toy_decay", dict(hidden_size=cfg["hidden_size"], state_size=24, decay=decay), prefix="toy")
    layers = (spec.layers[0], dataclasses.replace(spec.layers[1], mixer=toy, position=None))
    spec = dataclasses.replace(spec, layers=layers)
    model = DecoderModel(spec, _runtime(torch.float32))
    names = {ws.name for ws in model.weight_specs()}
    assert "toy.in.weight" in names and "model.layers.1.self_attn.q_proj.weight" not in names
    w = P.random_weights(cfg, 2, scale=0.05)
    g = torch.Generator().manual_seed(5)
    w["toy.in.weight"] = torch.randn(24, cfg["hidden_size"], generator=g) * 0.1
    w["toy.out.weight"] = torch.randn(cfg["hidden_size"], 24, generator=g) * 0.1
    model.bind({k: v.cuda() for k, v in w.items() if k in names})
    reqs = U.make_requests(cfg["vocab_size"], [50, 3, 77, 20, 31], 9)
    plain = {rid: _toy_plain(cfg, w, toks, decay) for rid, toks in reqs.items()}
    for steps in (U.trace_whole(reqs), U.trace_tail_decode(reqs, tail=8), U.trace_mixed(reqs, seed=4, max_live=3)):
        sess = _session(model, U.peak_tokens(steps), 16)
        assert len(sess.cache.groups) == 1 and list(sess.cache.state_specs) == [1]
        got = U.run_trace(sess, steps)
        U.compare(got, plain, U.TOL["float32"], "toy mixer")
        sess.cache.check()


def _generate(model, prompts, n_new, **options):
    """Greedy generation through the engine's own loop for a model built by hand."""
    from firefly_b200.engine.engine import Engine, EngineOptions
    from firefly_b200.engine.request import GenerationRequest
    from firefly_b200.sampling import SamplingParams
    eng = Engine(model, options=EngineOptions(kv_block_size=8, num_kv_blocks=64, max_batch_size_limit=4,
                                              eos_token_ids=[], **options))
    reqs = [GenerationRequest(f"g{i}", list(p), SamplingParams(max_tokens=n_new, ignore_eos=True)) for i, p in enumerate(prompts)]
    for r in reqs:
        eng.add_request(r)
    while eng.has_unfinished_requests():
        eng.step()
    eng.runner.check_status()
    eng.cache.check()
    return [list(r.generated_tokens) for r in reqs], eng


def test_toy_mixer_with_state_generates_from_cuda_graphs():
    """The toy mixer's state lives in the cache manager's slots, so captured decode steps and captured
    prompt portions find it like any page: tokens with graphs equal tokens without, and the plain ones."""
    from firefly_b200.config import PartSpec
    from firefly_b200.models import DecoderModel, config_from_dict, spec_for
    from firefly_b200.parts import register_part
    register_part("mixer", "toy_decay", ToyDecayMixer, replace=True)
    cfg, decay = P.TINY_A, 0.9
    spec = spec_for(config_from_dict(cfg))
    toy = PartSpec("toy_decay", dict(hidden_size=cfg["hidden_size"], state_size=24, decay=decay), prefix="toy")
    spec = dataclasses.replace(spec, layers=(spec.layers[0], dataclasses.replace(spec.layers[1], mixer=toy, position=None)))
    model = DecoderModel(spec, _runtime(torch.float32))
    assert not model.host_synchronous
    names = {ws.name for ws in model.weight_specs()}
    w = P.random_weights(cfg, 2, scale=0.05)
    g = torch.Generator().manual_seed(5)
    w["toy.in.weight"] = torch.randn(24, cfg["hidden_size"], generator=g) * 0.1
    w["toy.out.weight"] = torch.randn(cfg["hidden_size"], 24, generator=g) * 0.1
    model.bind({k: v.cuda() for k, v in w.items() if k in names})
    rng = np.random.RandomState(3)
    prompts = [list(map(int, rng.randint(0, cfg["vocab_size"], size=n))) for n in (40, 7, 33)]
    with_graphs, eng = _generate(model, prompts, 12, max_prefill_chunk_size=8)
    assert eng.graphs is not None and eng.stats["graph_steps"] > 0 and eng.graphs.shape_replays > 0
    without, eng2 = _generate(model, prompts, 12, max_prefill_chunk_size=8, use_cuda_graphs=False)
    assert eng2.graphs is None
    assert with_graphs == without
    for p, got in zip(prompts, with_graphs):
        toks = list(p)
        for _ in range(12):
            toks.append(int(np.argmax(_toy_plain(cfg, w, toks, decay)[-1])))
        assert got == toks[len(p):]


def test_an_undeclared_host_read_fails_the_capture_with_words():
    """A part that reads the device on the host without declaring it: the first captured step says
    what is wrong and what to do, instead of a bare CUDA error."""
    from firefly_b200.config import PartSpec
    from firefly_b200.engine.runner import StepError
    from firefly_b200.models import DecoderModel, config_from_dict, spec_for
    from firefly_b200.parts import register_part

    class Peeking(ToyDecayMixer):
        def forward(self, x, ctx, slot, write_cache):
            float(x.float().abs().max())                       # a read-back in the middle of the step
            return super().forward(x, ctx, slot, write_cache)
    register_part("mixer", "toy_peeking", Peeking, replace=True)
    cfg = P.TINY_A
    spec = spec_for(config_from_dict(cfg))
    toy = PartSpec("toy_peeking", dict(hidden_size=cfg["hidden_size"], state_size=24, decay=0.5), prefix="toy")
    spec = dataclasses.replace(spec, layers=(spec.layers[0], dataclasses.replace(spec.layers[1], mixer=toy, position=None)))
    model = DecoderModel(spec, _runtime(torch.float32))
    names = {ws.name for ws in model.weight_specs()}
    w = P.random_weights(cfg, 2, scale=0.05)
    w["toy.in.weight"] = torch.zeros(24, cfg["hidden_size"])
    w["toy.out.weight"] = torch.zeros(cfg["hidden_size"], 24)
    model.bind({k: v.cuda() for k, v in w.items() if k in names})
    with pytest.raises(StepError, match="host_synchronous"):
        _generate(model, [[1, 2, 3]], 4)
    torch.cuda.synchronize()                                   # the device is fine afterwards
    Peeking.host_synchronous = True
    model2 = DecoderModel(spec, _runtime(torch.float32))
    model2.bind({k: v.cuda() for k, v in w.items() if k in names})
    out, eng = _generate(model2, [[1, 2, 3]], 4)
    assert eng.graphs is None and len(out[0]) == 4


# ------------------------------------- a toy feed-forward with routing, a toy position encoding --
class ToyRoutedFFN:
    """Two small experts and a router: every token goes to its top-1 expert, whose output is
    scaled by the router's softmax weight.  Written with torch operations in the test."""

    host_synchronous = True      # forward() asks the device which experts have tokens: no CUDA graphs for this model

    def __init__(self, spec, rt):
        self.hidden = spec.params["hidden_size"]
        self.inner = spec.params["inner_size"]
        self.n_experts = spec.params["num_experts"]
        self.prefix = spec.prefix

    def weight_specs(self):
        from firefly_b200.weights import WeightSpec
        out = [WeightSpec(f"{self.prefix}.router.weight", (self.n_experts, self.hidden))]
        for e in range(self.n_experts):
            out += [WeightSpec(f"{self.prefix}.experts.{e}.up.weight", (self.inner, self.hidden)),
                    WeightSpec(f"{self.prefix}.experts.{e}.down.weight", (self.hidden, self.inner))]
        return out

    def bind(self, tensors):
        self.router = tensors[f"{self.prefix}.router.weight"].float()
        self.up = [tensors[f"{self.prefix}.experts.{e}.up.weight"].float() for e in range(self.n_experts)]
        self.down = [tensors[f"{self.prefix}.experts.{e}.down.weight"].float() for e in range(self.n_experts)]

    def forward(self, x, ctx):
        x = x.float()
        probs = torch.softmax(x @ self.router.T, dim=-1)           # router logits in 32-bit
        top = probs.argmax(dim=-1)
        out = torch.zeros_like(x)
        for e in range(self.n_experts):
            sel = top == e
            if bool(sel.any()):
                h = torch.relu(x[sel] @ self.up[e].T) @ self.down[e].T
                out[sel] = h * probs[sel, e:e + 1]
        return out.to(ctx.dtype)


class ToyLearnedPositions:
    """A learned table added to the embedding output: position encoding that is no rotation."""

    def __init__(self, spec, rt):
        self.n, self.hidden, self.prefix = spec.params["max_positions"], spec.params["hidden_size"], spec.prefix

    def weight_specs(self):
        from firefly_b200.weights import WeightSpec
        return [WeightSpec(f"{self.prefix}.weight", (self.n, self.hidden))]

    def bind(self, tensors):
        self.table = tensors[f"{self.prefix}.weight"].float()

    def rotary_table(self):
        return None

    def apply_to_embedding(self, h, ctx):
        h += self.table[ctx.positions.long()]


def _toy2_plain(cfg, w, ids):
    """float64, whole sequence: learned positions, attention without rotation, routed experts."""
    wd = {k: v.double() for k, v in w.items()}
    T = len(ids)
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    h = P.embedding(torch.tensor(ids), wd["model.embed_tokens.weight"]) + wd["pos.weight"][:T]
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}"
        x = P.rms_norm(h, wd[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
        q = P.rms_norm((x @ wd[f"{p}.self_attn.q_proj.weight"].T).view(T, nq, d), wd[f"{p}.self_attn.q_norm.weight"], cfg["rms_norm_eps"])
        k = P.rms_norm((x @ wd[f"{p}.self_attn.k_proj.weight"].T).view(T, nkv, d), wd[f"{p}.self_attn.k_norm.weight"], cfg["rms_norm_eps"])
        v = (x @ wd[f"{p}.self_attn.v_proj.weight"].T).view(T, nkv, d)
        h = h + P.attention(q, k, v).reshape(T, nq * d) @ wd[f"{p}.self_attn.o_proj.weight"].T
        x = P.rms_norm(h, wd[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        probs = torch.softmax(x @ wd[f"{p}.moe.router.weight"].T, dim=-1)
        top = probs.argmax(-1)
        f = torch.zeros_like(x)
        for t in range(T):
            e = int(top[t])
            f[t] = (torch.relu(wd[f"{p}.moe.experts.{e}.up.weight"] @ x[t]) @ wd[f"{p}.moe.experts.{e}.down.weight"].T) * probs[t, e]
        h = h + f
    x = P.rms_norm(h, wd["model.norm.weight"], cfg["rms_norm_eps"])
    return (x @ wd["lm_head.weight"].T).numpy()


def test_toy_routed_feed_forward_and_learned_positions():
    """Other kinds of feed-forward and position encoding plug in the same way as a mixer does."""
    from firefly_b200.config import PartSpec
    from firefly_b200.models import DecoderModel, config_from_dict, spec_for
    from firefly_b200.parts import register_part
    register_part("feed_forward", "toy_routed", ToyRoutedFFN, replace=True)
    register_part("position", "toy_learned", ToyLearnedPositions, replace=True)
    cfg = P.TINY_C
    spec = spec_for(config_from_dict(cfg))
    layers = []
    for i, ls in enumerate(spec.layers):
        moe = PartSpec("toy_routed", dict(hidden_size=cfg["hidden_size"], inner_size=40, num_experts=3),
                       prefix=f"model.layers.{i}.moe")
        layers.append(dataclasses.replace(ls, feed_forward=moe, position=None))
    pos = PartSpec("toy_learned", dict(max_positions=cfg["max_position_embeddings"], hidden_size=cfg["hidden_size"]), prefix="pos")
    spec = dataclasses.replace(spec, layers=tuple(layers), embedding_position=pos)
    model = DecoderModel(spec, _runtime(torch.float32))
    names = {ws.name: ws.shape for ws in model.weight_specs()}
    assert "pos.weight" in names and "model.layers.1.moe.experts.2.down.weight" in names
    assert not any("mlp" in n for n in names)
    g = torch.Generator().manual_seed(11)
    w = {n: (torch.randn(shape, generator=g) * (0.01 if len(shape) == 1 else 0.08) + (1.0 if len(shape) == 1 else 0.0))
         for n, shape in names.items()}
    model.bind({k: v.cuda() for k, v in w.items()})
    reqs = U.make_requests(cfg["vocab_size"], [60, 5, 131, 22], 6)
    plain = {rid: _toy2_plain(cfg, w, toks) for rid, toks in reqs.items()}
    for steps in (U.trace_whole(reqs), U.trace_portions(reqs), U.trace_mixed(reqs, seed=8, max_live=3)):
        sess = _session(model, U.peak_tokens(steps), 16)
        got = U.run_trace(sess, steps)
        # a token whose two best experts are within rounding may be routed differently: not with these weights
        U.compare(got, plain, 2e-4, "toy routed feed-forward and learned positions")
    # the routed part reads the device on the host and says so: the engine then runs launch by launch
    assert model.host_synchronous
    prompts = [reqs["r1"][:20], reqs["r2"]]
    got, eng = _generate(model, prompts, 6)
    assert eng.graphs is None
    for p, out in zip(prompts, got):
        toks = list(p)
        for _ in range(6):
            toks.append(int(np.argmax(_toy2_plain(cfg, w, toks)[-1])))
        assert out == toks[len(p):]


# ------------------------------------- a toy norm, arrangement and architecture --
class ToyMeanAbsNorm:
    """y = v / (mean |v| + eps) * w after the pending delta has been added into the 32-bit residual.
    Written with torch operations; it stands for any norm a user might add."""

    def __init__(self, spec, rt):
        self.size = spec.params["size"]
        self.eps = spec.params["eps"]
        self.prefix = spec.prefix

    def weight_specs(self):
        from firefly_b200.weights import WeightSpec
        return [WeightSpec(f"{self.prefix}.weight", (self.size,), init="norm")]

    def bind(self, tensors):
        self.weight = tensors[f"{self.prefix}.weight"].float()

    def forward(self, residual, delta, ctx, *, tag="normed", row_idx=None, may_defer=False):
        if delta is not None:
            residual += delta.float()
        v = residual if row_idx is None else residual[row_idx.long()]
        return (v / (v.abs().mean(dim=-1, keepdim=True) + self.eps) * self.weight).to(ctx.dtype)


def _toy_parallel_block():
    from firefly_b200.parts.block import Block

    class ToyParallelBlock(Block):
        """h += mixer(norm(h)) + feed_forward(norm(h)): one norm, both parts read the same rows."""
        n_norms = 1

        def forward(self, residual, pending, ctx, slot, write_cache):
            x = self.norms[0].forward(residual, pending, ctx)
            a = self.mixer.forward(x, ctx, slot, write_cache)
            f = self.feed_forward.forward(x, ctx)
            return residual, a.float() + f.float()          # one pending delta for the next norm
    return ToyParallelBlock


def _toy_architecture():
    """A configuration class with keys of its own and a spec builder: what a user writes to add an
    architecture (here: parallel blocks, the toy norm, attention without q/k norms, tied head)."""
    from firefly_b200.config import ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture = "ToyParallelForCausalLM"
        width: int = 0
        depth: int = 0
        heads: int = 0
        kv_heads: int = 0
        head_size: int = 0
        ffn_width: int = 0
        vocab: int = 0
        positions: int = 0
        norm_eps: float = 1e-5
        theta: float = 10000.0

        @classmethod
        def from_dict(cls, raw):
            keys = [f.name for f in dataclasses.fields(cls)]
            cfg = cls(**{k: raw[k] for k in keys if k in raw})
            cfg.validate()
            return cfg

        def validate(self):
            if min(self.width, self.depth, self.heads, self.kv_heads, self.head_size, self.ffn_width, self.vocab) <= 0:
                raise ConfigError("toy config: every size must be positive")

    def toy_spec(cfg):
        rope = PartSpec("rotary", dict(head_dim=cfg.head_size, rotary_dim=cfg.head_size, theta=cfg.theta,
                                       max_positions=cfg.positions))
        layers = []
        for i in range(cfg.depth):
            p = f"blocks.{i}"
            layers.append(LayerSpec(
                arrangement="toy_parallel",
                mixer=PartSpec("gqa_attention", dict(hidden_size=cfg.width, num_heads=cfg.heads,
                                                     num_kv_heads=cfg.kv_heads, head_dim=cfg.head_size, qk_norm=False,
                                                     qk_norm_eps=cfg.norm_eps, window=None, scale=None),
                               prefix=f"{p}.attn"),
                feed_forward=PartSpec("swiglu_mlp", dict(hidden_size=cfg.width, intermediate_size=cfg.ffn_width),
                                      prefix=f"{p}.ffn"),
                norms=(PartSpec("toy_mean_abs", dict(size=cfg.width, eps=cfg.norm_eps), prefix=f"{p}.norm"),),
                position=rope))
        return ModelSpec(
            vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=cfg.positions,
            embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=cfg.width), prefix="embed"),
            layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(cfg.depth)),
            final_norm=PartSpec("toy_mean_abs", dict(size=cfg.width, eps=cfg.norm_eps), prefix="out_norm"),
            head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tied_to="embed.weight"),
                          prefix="head"))
    return ToyConfig, toy_spec


def _toy_parallel_plain(raw, w, ids):
    """The toy architecture on a whole sequence in float64, from the plain implementation's parts."""
    wd = {k: v.double() for k, v in w.items()}
    pos = torch.arange(len(ids))
    nq, nkv, d, T = raw["heads"], raw["kv_heads"], raw["head_size"], len(ids)

    def attn(x, p):                                         # no per-head norms in this architecture
        q = P.rope((x @ wd[f"{p}.q_proj.weight"].T).view(T, nq, d), pos, raw["theta"])
        k = P.rope((x @ wd[f"{p}.k_proj.weight"].T).view(T, nkv, d), pos, raw["theta"])
        v = (x @ wd[f"{p}.v_proj.weight"].T).view(T, nkv, d)
        return P.attention(q, k, v).reshape(T, nq * d) @ wd[f"{p}.o_proj.weight"].T

    def norm(v, weight):
        return v / (v.abs().mean(dim=-1, keepdim=True) + raw["norm_eps"]) * weight
    h = P.embedding(torch.tensor(ids), wd["embed.weight"])
    for i in range(raw["depth"]):
        p = f"blocks.{i}"
        x = norm(h, wd[f"{p}.norm.weight"])
        a = attn(x, f"{p}.attn")
        f = P.swiglu_mlp(x, wd[f"{p}.ffn.gate_proj.weight"], wd[f"{p}.ffn.up_proj.weight"], wd[f"{p}.ffn.down_proj.weight"])
        h = h + a + f
    return (norm(h, wd["out_norm.weight"]) @ wd["embed.weight"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_its_own_config_norm_and_arrangement(dtype, tmp_path):
    """An architecture is added from outside the package: a configuration class with keys of its
    own, a norm and an arrangement defined here, registered, written as a model folder with random
    weights, loaded by name from config.json, replayed and generated from, against a plain version."""
    import json
    from firefly_b200 import LLM
    from firefly_b200.models import config_from_dict, register_architecture
    from firefly_b200.parts import register_part
    from firefly_b200.replay import ReplaySession
    from firefly_b200.weights import write_random_model
    from firefly_b200.weights.safetensors_io import SafetensorsFile
    ToyConfig, toy_spec = _toy_architecture()
    register_part("norm", "toy_mean_abs", ToyMeanAbsNorm, replace=True)
    register_part("arrangement", "toy_parallel", _toy_parallel_block(), replace=True)
    register_architecture("ToyParallelForCausalLM", ToyConfig, toy_spec, replace=True)
    raw = dict(architectures=["ToyParallelForCausalLM"], width=96, depth=3, heads=6, kv_heads=2, head_size=16,
               ffn_width=208, vocab=331, positions=256, norm_eps=1e-4, theta=5000.0)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = str(tmp_path / "toy")
    write_random_model(config_from_dict(raw), seed=3, out_dir=folder, dtype=tdt)
    with open(f"{folder}/config.json") as fh:
        assert json.load(fh)["architectures"] == ["ToyParallelForCausalLM"]
    f = SafetensorsFile(f"{folder}/model.safetensors")
    w = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    assert "blocks.2.norm.weight" in w and "blocks.0.attn.q_norm.weight" not in w and "head.weight" not in w
    reqs = U.make_requests(raw["vocab"], [60, 5, 131, 33], 21)
    plain = {rid: _toy_parallel_plain(raw, w, toks) for rid, toks in reqs.items()}
    for steps in (U.trace_whole(reqs), U.trace_tail_decode(reqs, tail=8), U.trace_mixed(reqs, seed=2, max_live=3)):
        sess = ReplaySession(folder, dtype=dtype, max_tokens=U.peak_tokens(steps), block_size=16)
        got = U.run_trace(sess, steps)
        U.compare(got, plain, U.TOL[dtype], f"toy architecture {dtype}")
        sess.cache.check()
    if dtype == "float32":
        prompt = reqs["r1"]
        got = LLM(folder, dtype="float32", num_kv_blocks=32).generate([prompt], max_tokens=6)[0]
        toks = list(prompt)
        for _ in range(6):
            toks.append(int(np.argmax(_toy_parallel_plain(raw, w, toks)[-1])))
        assert got == toks[len(prompt):]
