"""The engine at the layer sizes of a real model (4096 wide, 32/8 heads of 128, 12288 intermediate,
a vocabulary of 151936; two layers, random weights, bfloat16).  Tiny models leave some faults
unseen: kernels there end before the next one starts, the vocabulary fits one sampling block and the
host is slower than the device.  Here generation through graphs and steps launched ahead is held
against the engine's own replay of the same tokens (whose logits the other tests hold against the
plain implementation): every generated token must be the replay's best, within rounding."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REAL_SIZES = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, intermediate_size=12288,
                  num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                  vocab_size=151936, max_position_embeddings=4096, rms_norm_eps=1e-6, rope_theta=1000000.0,
                  tie_word_embeddings=False)


@pytest.mark.parametrize("options", [dict(), dict(max_prefill_chunk_size=1024), dict(use_cuda_graphs=False)],
                         ids=["portions", "whole-prompts", "no-graphs"])
def test_generated_tokens_are_the_replays_best_at_real_layer_sizes(options):
    from firefly_b200 import LLM
    from firefly_b200.models import config_from_dict
    from firefly_b200.replay import ReplaySession
    cfg = config_from_dict(REAL_SIZES)
    rng = np.random.RandomState(5)
    prompts = [list(map(int, rng.randint(0, cfg.vocab_size, size=n))) for n in (45, 100, 520)]
    llm = LLM(cfg, seed=3, dtype="bfloat16", num_kv_blocks=256, **options)
    outs = llm.generate(prompts, max_tokens=6)
    if options.get("use_cuda_graphs", True):
        assert llm.engine.stats["launched_ahead"] > 0
    llm.engine.runner.check_status()
    for p, g in zip(prompts, outs):
        assert len(g) == 6
        ids = list(p) + list(g)
        sess = ReplaySession(model=llm.model, max_tokens=len(ids) + 64)
        want = list(range(len(p) - 1, len(ids) - 1))
        rows = sess.run_step({"step": 0, "entries": [{"id": "x", "tokens": ids, "want": want}], "end": ["x"]})
        for k, t in enumerate(g):
            gap = float(rows[k].max() - rows[k][t]) / float(np.abs(rows[k]).max())
            assert gap <= 2e-2, f"prompt of {len(p)}: token {k} lies {gap:.3f} of the row's scale below the best"
        del sess


def test_captured_portions_share_out_the_keys_of_long_contexts_like_uncaptured_ones():
    """A prompt of 2700 tokens comes in portions of 128 (twice, so that the shapes repeat and are
    captured at every level of context length).  Captured steps fix over how many blocks a portion's
    keys are shared out; the logits of the last portion and the generated tokens must agree with the
    run that launches every step kernel by kernel."""
    from firefly_b200 import LLM
    from firefly_b200.models import config_from_dict
    cfg = config_from_dict(REAL_SIZES)
    rng = np.random.RandomState(8)
    prompts = [list(map(int, rng.randint(0, cfg.vocab_size, size=2700))) for _ in range(2)]
    outs, captures = {}, {}
    for capture in (True, False):
        llm = LLM(cfg, seed=3, dtype="bfloat16", num_kv_blocks=512, max_prefill_chunk_size=128,
                  capture_repeating_steps=capture)
        got = []
        for p in prompts:                                  # one after the other: the second meets captured shapes
            got.append(llm.generate([p], max_tokens=4)[0])
        llm.engine.runner.check_status()
        outs[capture] = got
        captures[capture] = (llm.engine.graphs.shape_captures, llm.engine.graphs.shape_replays,
                             sorted({k[2] for k in llm.engine.graphs.shapes}))
        del llm
        torch.cuda.empty_cache()
    # every level of context length got a graph of its own (a scratch buffer that grows voids the older ones)
    assert captures[True][0] >= 4 and captures[True][1] >= 10 and captures[True][2][-1] == 8
    assert captures[False][0] == 0
    assert outs[True][0] == outs[False][0]                  # the first prompt ran launch by launch in both
    same = sum(a == b for a, b in zip(outs[True][1], outs[False][1]))
    assert same >= 3, (outs[True][1], outs[False][1])       # bfloat16: the same kernels, a near tie at most


@pytest.fixture(scope="module")
def real_size_case(tmp_path_factory):
    """A model folder at the real layer sizes (bfloat16 values), three requests and the plain
    implementation's logits for them (32-bit, on the CPU), made once for the tests below."""
    import plain_qwen3 as P
    import replay_util as U
    tmp = tmp_path_factory.mktemp("real_sizes")
    cfg = dict(REAL_SIZES, tie_word_embeddings=True)       # one matrix of 151936 x 4096 less to draw on the CPU
    w = P.random_weights(cfg, 3, dtype=torch.bfloat16, scale=0.02)
    U.write_model_dir(str(tmp), cfg, w, torch.bfloat16)
    reqs = U.make_requests(cfg["vocab_size"], [150, 20, 330], 5)
    w32 = {k: v.float() for k, v in w.items()}
    plain = {rid: P.forward(cfg, w32, toks, dtype=torch.float32).numpy() for rid, toks in reqs.items()}
    return str(tmp), reqs, plain


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_replay_matches_the_plain_implementation_at_real_layer_sizes(real_size_case, dtype):
    """The plain implementation against the replay at these sizes, in bfloat16 and in true 32-bit (the
    folder's bfloat16 values widened exactly): a request whole, its last tokens one by one, in portions
    of changing size, and mixed with two others of very different lengths."""
    import replay_util as U
    from firefly_b200.replay import ReplaySession
    path, reqs, plain = real_size_case
    tol = U.TOL[dtype]
    for family in ("whole", "tail", "portions", "mixed"):
        steps = {"whole": U.trace_whole, "tail": U.trace_tail_decode, "portions": U.trace_portions,
                 "mixed": U.trace_mixed}[family](reqs)
        sess = ReplaySession(path, dtype=dtype, max_tokens=U.peak_tokens(steps))
        U.compare(U.run_trace(sess, steps), plain, tol, f"real sizes/{dtype}/{family}")
        sess.cache.check()
        del sess
        torch.cuda.empty_cache()
