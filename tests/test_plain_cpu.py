"""The plain implementation itself (no GPU): each part against an independent
restatement, and properties that pin down the formulas."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P


def test_rms_norm_formula():
    x = torch.randn(5, 7, dtype=torch.float64)
    w = torch.randn(7, dtype=torch.float64)
    y = P.rms_norm(x, w, 1e-5)
    for r in range(5):
        ms = sum(float(v) ** 2 for v in x[r]) / 7
        for j in range(7):
            assert abs(float(y[r, j]) - float(x[r, j]) / math.sqrt(ms + 1e-5) * float(w[j])) < 1e-12


def test_rope_is_rotate_half_with_theta():
    d, theta = 8, 10000.0
    x = torch.randn(3, 2, d, dtype=torch.float64)
    pos = torch.tensor([0, 5, 131])
    y = P.rope(x, pos, theta)
    assert torch.allclose(y[0], x[0])                            # position 0: identity
    for t in range(3):
        for i in range(d // 2):
            a = float(pos[t]) * theta ** (-2.0 * i / d)
            lo, hi = float(x[t, 1, i]), float(x[t, 1, i + d // 2])
            assert abs(float(y[t, 1, i]) - (lo * math.cos(a) - hi * math.sin(a))) < 1e-12
            assert abs(float(y[t, 1, i + d // 2]) - (hi * math.cos(a) + lo * math.sin(a))) < 1e-12
    # relative: <rope(q,m), rope(k,n)> depends on m-n only
    q, k = torch.randn(1, 1, d, dtype=torch.float64), torch.randn(1, 1, d, dtype=torch.float64)
    s1 = (P.rope(q, torch.tensor([9]), theta) * P.rope(k, torch.tensor([4]), theta)).sum()
    s2 = (P.rope(q, torch.tensor([105]), theta) * P.rope(k, torch.tensor([100]), theta)).sum()
    assert abs(float(s1 - s2)) < 1e-10


def test_attention_against_loops():
    T, nq, nkv, d = 6, 4, 2, 4
    q, k, v = (torch.randn(T, n, d, dtype=torch.float64) for n in (nq, nkv, nkv))
    for window in (None, 3):
        o = P.attention(q, k, v, window=window)
        for t in range(T):
            for h in range(nq):
                kh = h // 2
                lo = 0 if window is None else max(0, t - window + 1)
                s = [float(q[t, h] @ k[j, kh]) / math.sqrt(d) for j in range(lo, t + 1)]
                m = max(s)
                p = [math.exp(x - m) for x in s]
                want = sum(pj * v[lo + j, kh] for j, pj in enumerate(p)) / sum(p)
                assert torch.allclose(o[t, h], want, atol=1e-12)


def test_silu_mul():
    g, u = torch.tensor([-2.0, 0.0, 3.0], dtype=torch.float64), torch.tensor([1.0, 5.0, -2.0], dtype=torch.float64)
    want = [x / (1 + math.exp(-x)) * y for x, y in zip(g.tolist(), u.tolist())]
    assert torch.allclose(P.silu_mul(g, u), torch.tensor(want, dtype=torch.float64))


@pytest.mark.parametrize("cfg", [P.TINY_A, P.TINY_B, P.TINY_C])
def test_forward_is_causal_and_uses_every_option(cfg):
    w = P.random_weights(cfg, 3, scale=0.05)
    ids = list(np.random.RandomState(0).randint(0, cfg["vocab_size"], size=20))
    full = P.forward(cfg, w, ids)
    assert full.shape == (20, cfg["vocab_size"])
    assert torch.allclose(P.forward(cfg, w, ids[:11]), full[:11], atol=1e-9)    # causal
    for key, val in (("rms_norm_eps", 0.1), ("rope_theta", 77.0)):
        other = dict(cfg)
        other[key] = val
        assert not torch.allclose(P.forward(other, w, ids), full, atol=1e-6), key
    # tied / untied heads
    if cfg["tie_word_embeddings"]:
        x = dict(w)
        x["lm_head.weight"] = torch.randn_like(w["model.embed_tokens.weight"])
        assert torch.allclose(P.forward(cfg, x, ids), full)
    else:
        x = dict(w)
        x["lm_head.weight"] = x["lm_head.weight"] * 2
        assert torch.allclose(P.forward(cfg, x, ids), 2 * full, atol=1e-9)
    # the q/k norm acts per head before the rotation: scaling q_proj changes nothing
    x = dict(w)
    x["model.layers.0.self_attn.q_proj.weight"] = w["model.layers.0.self_attn.q_proj.weight"] * 3.0
    assert torch.allclose(P.forward(cfg, x, ids), full, atol=1e-4 * float(full.abs().max()))


def test_window_and_schedule_options():
    cfg = P.TINY_B
    w = P.random_weights(cfg, 5, scale=0.05)
    ids = list(range(30))
    full = P.forward(cfg, w, ids)
    win = P.forward(cfg, w, ids, windows=[None, 4, None])
    assert torch.allclose(win[:4], full[:4], atol=1e-9) and not torch.allclose(win[10:], full[10:], atol=1e-6)
    shared = P.forward(cfg, w, ids, schedule=[(0, 0, True), (1, 1, True), (2, 1, False)])
    assert not torch.allclose(shared, full, atol=1e-6)
    twice = P.forward(cfg, w, ids, schedule=[(0, 0, True), (0, 1, True), (1, 2, True), (2, 3, True)])
    assert twice.shape == full.shape and not torch.allclose(twice, full, atol=1e-6)


def test_greedy_is_argmax_lowest_index():
    cfg = P.TINY_A
    w = P.random_weights(cfg, 1, scale=0.05)
    out = P.greedy_generate(cfg, w, [1, 2, 3], 4)
    ids = [1, 2, 3]
    for t in out:
        assert t == int(torch.argmax(P.forward(cfg, w, ids)[-1]))
        ids.append(t)
