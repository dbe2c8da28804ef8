"""Replay on the GPU: the same requests whole, with the last 32 tokens decoded one
by one, in portions of changing size, and mixed with other requests on a pool so
small that pages are used again; in 32-bit and in bfloat16; all compared with the
plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as U

pytestmark = pytest.mark.gpu

# "S": the weights of the per-head q and k norms are three times as large, so the scores have three
# times the spread and a row's attention rests on a few keys, near or far: a key that is lost, read
# from the wrong page or masked by mistake changes the logits far beyond the tolerance.  In 32-bit
# only: scores that sharp multiply the rounding of bfloat16 activations beyond its tolerance at every
# position (the tensor-core attention kernels have their own test with one key that stands out).
CONFIGS = {"A": (P.TINY_A, 0, 16, [40, 100, 1, 77, 128, 33]),
           "S": (P.TINY_D, 5, 16, [130, 47, 333, 16, 65, 700]),
           "B": (P.TINY_B, 1, 8, [70, 3, 200, 45, 256, 129, 17]),
           "C": (P.TINY_C, 2, 32, [150, 64, 65, 300, 2, 97]),
           "D": (P.TINY_D, 3, 16, [300, 129, 640, 70, 1000])}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, seed, block, lengths) in CONFIGS.items():
        for dtype, tdt in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            if name == "S" and dtype != "float32":
                continue
            w = P.random_weights(cfg, seed, dtype=tdt, scale=0.05)
            if name == "S":
                for k in w:
                    if k.endswith("q_norm.weight") or k.endswith("k_norm.weight"):
                        w[k] = (w[k].float() * 3.0).to(tdt)
            path = str(tmp_path_factory.mktemp(f"model{name}_{dtype}"))
            U.write_model_dir(path, cfg, w, tdt)
            reqs = U.make_requests(cfg["vocab_size"], lengths, seed + 10)
            plain = U.plain_all(cfg, w, reqs)     # the plain model sees the stored (rounded) weights
            out[(name, dtype)] = (path, cfg, block, reqs, plain)
    return out


def _session(path, dtype, max_tokens, block):
    from firefly_b200.replay import ReplaySession
    return ReplaySession(path, dtype=dtype, max_tokens=max_tokens, block_size=block)


@pytest.mark.parametrize("name,dtype", [(n, d) for n in CONFIGS for d in ("float32", "bfloat16")
                                        if n != "S" or d == "float32"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_replay_family(folders, name, dtype, family):
    path, cfg, block, reqs, plain = folders[(name, dtype)]
    steps = {"whole": U.trace_whole, "tail": U.trace_tail_decode, "portions": U.trace_portions,
             "mixed": U.trace_mixed}[family](reqs)
    peak = U.peak_tokens(steps)
    sess = _session(path, dtype, peak, block)
    got = U.run_trace(sess, steps)
    assert len(got.rows) == sum(len(t) for t in reqs.values())
    U.compare(got, plain, U.TOL[dtype], f"{name}/{dtype}/{family}")
    sess.cache.check()
    assert not sess.cache.live
    if family == "mixed":
        # the pool held fewer tokens than the requests have: pages were used again
        assert peak < sum(-(-len(t) // 64) * 64 for t in reqs.values())


def test_trace_run_program(folders, tmp_path):
    """The program itself: stdin protocol, files, 'done' lines, exit code."""
    path, cfg, block, reqs, plain = folders[("B", "float32")]
    steps = U.trace_mixed(reqs, seed=3)
    exe = os.path.join(os.path.dirname(__file__), "..", "bin", "trace_run")
    out = tmp_path / "out"
    proc = subprocess.Popen([sys.executable, exe, "--model", path, "--dtype", "float32", "--out", str(out),
                             "--max-tokens", str(U.peak_tokens(steps)), "--block-size", str(block)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    got = U.Collected()
    done = {}
    V = cfg["vocab_size"]
    for rec in steps:
        proc.stdin.write(json.dumps(rec) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()
        assert line == f"done {rec['step']}", line
        arr = np.fromfile(out / f"{rec['step']}.f32", dtype="<f4").reshape(-1, V)
        k = 0
        for ent in rec["entries"]:
            base = done.get(ent["id"], 0)
            for w in ent["want"]:
                got.add(ent["id"], base + w, arr[k])
                k += 1
            done[ent["id"]] = base + len(ent["tokens"])
    proc.stdin.close()
    assert proc.wait(timeout=60) == 0
    U.compare(got, plain, U.TOL["float32"], "trace_run program")


def _odd(h, i, L, nq, nkv, d, v, tied):
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=h, intermediate_size=i, num_hidden_layers=L,
                num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d, vocab_size=v,
                max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=tied)


# sizes at the edges of what the kernels take: a width and an intermediate size that are no multiple of
# 8 (no vector loads, no tensor-core product), head sizes that are no multiple of 16 (plain attention
# kernel also in bfloat16), a head size between the compiled classes, a group of 17 query heads per
# key/value head (more than the decode kernel's 16), many heads of a small size
ODD = {"width100": _odd(100, 150, 2, 5, 5, 16, 257, False),
       "head24": _odd(52, 36, 2, 3, 1, 24, 101, True),
       "head6": _odd(30, 50, 1, 5, 5, 6, 33, False),
       "head144": _odd(64, 128, 1, 2, 2, 144, 300, False),
       "group17": _odd(128, 256, 1, 34, 2, 64, 640, True),
       "heads40": _odd(256, 512, 1, 40, 8, 32, 2048, False)}


@pytest.mark.parametrize("name", sorted(ODD))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_sizes_at_the_kernels_edges(tmp_path, name, dtype):
    cfg = ODD[name]
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    w = P.random_weights(cfg, 7, dtype=tdt, scale=0.05)
    U.write_model_dir(str(tmp_path), cfg, w, tdt)
    reqs = U.make_requests(cfg["vocab_size"], [70, 3, 129, 45], 3)
    plain = U.plain_all(cfg, w, reqs)
    for family, block in (("whole", 16), ("mixed", 8)):
        steps = (U.trace_whole if family == "whole" else U.trace_mixed)(reqs)
        sess = _session(str(tmp_path), dtype, U.peak_tokens(steps), block)
        U.compare(U.run_trace(sess, steps), plain, U.TOL[dtype], f"{name}/{dtype}/{family}")
        sess.cache.check()
        assert not sess.cache.live
