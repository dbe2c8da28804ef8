"""Each kernel alone against a plain 32-bit reference, at sizes other than the
engine's: head sizes in steps of 16, odd widths and vocabularies, groups of 1-8,
contexts that cross page edges, windows, pages in shuffled order."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu


def K():
    from firefly_b200.ops import kernels
    return kernels


def dev(t):
    return t.to("cuda")


@pytest.mark.parametrize("H,V,tdt", [(72, 333, torch.float32), (4096, 1000, torch.bfloat16), (100, 50, torch.bfloat16)])
def test_embedding(H, V, tdt):
    table = torch.randn(V, H).to(tdt)
    ids = torch.randint(0, V, (37,), dtype=torch.int32)
    out = torch.empty(37, H, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    K().embedding(dev(ids), dev(table), out, status)
    assert torch.equal(out.cpu(), P.embedding(ids, table).float()) and int(status) == 0
    bad = ids.clone()
    bad[5] = V
    K().embedding(dev(bad), dev(table), out, status)
    assert int(status) == 1                                     # reported, and the table was not overrun


@pytest.mark.parametrize("H", [64, 72, 1000, 4096, 5120 + 8, 60000])
@pytest.mark.parametrize("adt", [torch.float32, torch.bfloat16])
def test_add_rms_norm(H, adt):
    rows = 11
    res = torch.randn(rows, H) * 3
    delta = (torch.randn(rows, H)).to(adt)
    w = 1 + 0.1 * torch.randn(H)
    eps = 1e-5
    want_res = res.double() + delta.double()
    want = P.rms_norm(want_res, w.double(), eps)
    r = dev(res.clone())
    out = torch.empty(rows, H, dtype=adt, device="cuda")
    K().add_rms_norm(r, dev(delta), dev(w), eps, out)
    tol = 1e-5 if adt == torch.float32 else 1e-2
    assert torch.allclose(r.cpu().double(), want_res, atol=1e-6, rtol=1e-6)     # residual updated in 32-bit
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
    # no delta; and selected rows only (the residual stays)
    r2 = dev(res.clone())
    K().add_rms_norm(r2, None, dev(w), eps, out)
    assert torch.allclose(out.cpu().double(), P.rms_norm(res.double(), w.double(), eps), atol=tol, rtol=tol)
    idx = torch.tensor([7, 0, 3], dtype=torch.int32)
    out3 = torch.empty(3, H, dtype=adt, device="cuda")
    r3 = dev(res.clone())
    K().add_rms_norm(r3, dev(delta), dev(w), eps, out3, dev(idx))
    assert torch.equal(r3.cpu(), res)
    assert torch.allclose(out3.cpu().double(), want[idx.long()], atol=tol, rtol=tol)


@pytest.mark.parametrize("I", [160, 200, 12288])
@pytest.mark.parametrize("adt", [torch.float32, torch.bfloat16])
def test_silu_mul(I, adt):
    gu = (torch.randn(9, 2 * I) * 3).to(adt)
    out = torch.empty(9, I, dtype=adt, device="cuda")
    K().silu_mul(dev(gu), out)
    want = P.silu_mul(gu[:, :I].double(), gu[:, I:].double())
    tol = 1e-6 if adt == torch.float32 else 1e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("I", [48, 160, 12288])
@pytest.mark.parametrize("adt", [torch.float32, torch.bfloat16])
def test_silu_mul_interleaved(I, adt):
    """Gate and up columns alternating in groups of 16, the layout the fused product's weight has."""
    gate, up = (torch.randn(7, I) * 3).to(adt), (torch.randn(7, I) * 3).to(adt)
    gu = torch.stack([gate.view(7, I // 16, 16), up.view(7, I // 16, 16)], dim=2).reshape(7, 2 * I).contiguous()
    out = torch.empty(7, I, dtype=adt, device="cuda")
    K().silu_mul(dev(gu), out, True)
    want = P.silu_mul(gate.double(), up.double())
    tol = 1e-6 if adt == torch.float32 else 1e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)


def _paged(k, v, block, n_extra=3, seed=0):
    """Scatter whole-sequence k, v [T, nkv, d] into shuffled pages.  Returns
    (pages [blocks,2,nkv,block,d], table row)."""
    T, nkv, d = k.shape
    n_pages = -(-T // block)
    total = n_pages + n_extra + 1
    order = np.random.RandomState(seed).permutation(np.arange(1, total))[:n_pages]
    pages = torch.randn(total, 2, nkv, block, d, dtype=k.dtype) * 7.0      # stale data everywhere else
    for t in range(T):
        pg = order[t // block]
        pages[pg, 0, :, t % block, :] = k[t]
        pages[pg, 1, :, t % block, :] = v[t]
    return pages, [int(x) for x in order]


@pytest.mark.parametrize("d,nq,nkv,block,rot", [(16, 4, 2, 16, 16), (48, 3, 1, 8, 32), (128, 8, 2, 16, 128),
                                                (256, 2, 2, 32, 256), (72, 2, 1, 4, 72)])
@pytest.mark.parametrize("adt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [21, 300])          # 300: the form for long portions (a warp per 8 heads of a token)
def test_qk_norm_rope_store(d, nq, nkv, block, rot, adt, T):
    torch.manual_seed(d)
    theta, eps = 12345.0, 1e-5
    ctx_len = 13                                   # tokens already cached: the write starts mid-page
    width = (nq + 2 * nkv) * d
    qkv = torch.randn(T, width).to(adt)
    qw, kw = 1 + 0.1 * torch.randn(d), 1 + 0.1 * torch.randn(d)
    positions = torch.arange(ctx_len, ctx_len + T, dtype=torch.int32)
    n_pages = -(-(ctx_len + T) // block)
    table = torch.full((2, n_pages + 2), -1, dtype=torch.int32)
    table[1, :n_pages] = torch.tensor(np.random.RandomState(1).permutation(np.arange(1, n_pages + 4))[:n_pages])
    pages = torch.zeros(n_pages + 4, 2, nkv, block, d, dtype=adt)
    half = rot // 2
    freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / rot)
    ang = torch.arange(ctx_len + T + 3, dtype=torch.float64)[:, None] * freq[None]
    cs = torch.stack([torch.cos(ang), torch.sin(ang)], -1).float()
    g_qkv, g_pages = dev(qkv.clone()), dev(pages)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    K().qk_norm_rope_store(g_qkv, nq, nkv, d, dev(qw), dev(kw), eps, dev(cs), rot, dev(positions),
                           dev(torch.ones(T, dtype=torch.int32)), dev(table), g_pages, status)
    assert int(status) == 0
    x = qkv.double()
    q = x[:, :nq * d].view(T, nq, d)
    k = x[:, nq * d:(nq + nkv) * d].view(T, nkv, d)
    v = x[:, (nq + nkv) * d:].view(T, nkv, d)

    def rot_part(t):
        y = t.clone()
        y[..., :rot] = P.rope(t[..., :rot], positions, theta)
        return y
    q_want = rot_part(P.rms_norm(q, qw.double(), eps))
    k_want = rot_part(P.rms_norm(k, kw.double(), eps))
    tol = 2e-5 if adt == torch.float32 else 2e-2
    got_q = g_qkv.cpu().double()[:, :nq * d].view(T, nq, d)
    assert torch.allclose(got_q, q_want, atol=tol, rtol=tol)
    assert torch.equal(g_qkv.cpu()[:, nq * d:], qkv[:, nq * d:])           # k, v columns untouched
    gp = g_pages.cpu().double()
    for t in range(T):
        p = ctx_len + t
        pg = int(table[1, p // block])
        assert torch.allclose(gp[pg, 0, :, p % block], k_want[t], atol=tol, rtol=tol)
        assert torch.allclose(gp[pg, 1, :, p % block], v[t], atol=0, rtol=0)
    written = {(int(table[1, (ctx_len + t) // block]), (ctx_len + t) % block) for t in range(T)}
    for pg in range(pages.shape[0]):
        for o in range(block):
            if (pg, o) not in written:
                assert float(gp[pg, :, :, o].abs().max()) == 0.0         # nothing else was written


def _attention_case(d, nq, nkv, block, seqs, window, adt, seed=0, spike=True):
    """seqs: list of (ctx_len, q_len).  Builds whole-sequence q,k,v, pages them and
    returns everything the kernels need plus the plain result for the new tokens."""
    g = torch.Generator().manual_seed(seed)
    G = nq // nkv
    tables, qs, wants, cu, ctxs, token_seq, positions = [], [], [], [0], [], [], []
    page_list = []
    base = 1
    for si, (ctx_len, q_len) in enumerate(seqs):
        T = ctx_len + q_len
        q = torch.randn(T, nq, d, generator=g)
        k = torch.randn(T, nkv, d, generator=g)
        v = torch.randn(T, nkv, d, generator=g)
        if spike and T > 3:
            # one far key stands out for the last query: a lost or misplaced key shows
            k[1] = k[1] * 0.1 + 3.0 * q[T - 1, ::G] / math.sqrt(d) * 4
        q, k, v = q.to(adt), k.to(adt), v.to(adt)
        want = P.attention(q.double(), k.double(), v.double(), window=window)[ctx_len:]
        pages, order = _paged(k, v, block, seed=seed + si)
        page_list.append(pages[1:])
        tables.append([o - 1 + base for o in order])
        base += pages.shape[0] - 1
        qs.append(q[ctx_len:])
        wants.append(want)
        cu.append(cu[-1] + q_len)
        ctxs.append(ctx_len)
        token_seq += [si] * q_len
        positions += list(range(ctx_len, T))
    all_pages = torch.cat([torch.zeros(1, *page_list[0].shape[1:], dtype=adt)] + page_list, 0)
    mb = max(len(t) for t in tables) + 1
    table = torch.full((len(seqs), mb), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    return dict(q=torch.cat(qs, 0).reshape(-1, nq * d).contiguous(), pages=all_pages, table=table,
                cu_q=torch.tensor(cu, dtype=torch.int32), ctx_lens=torch.tensor(ctxs, dtype=torch.int32),
                token_seq=torch.tensor(token_seq, dtype=torch.int32),
                positions=torch.tensor(positions, dtype=torch.int32),
                want=torch.cat(wants, 0).reshape(-1, nq * d), q_lens=[s[1] for s in seqs])


ATT_SHAPES = [(16, 4, 2, 16), (32, 6, 2, 8), (48, 3, 1, 32), (64, 8, 1, 16), (128, 8, 2, 16), (80, 5, 5, 4),
              (256, 4, 2, 64)]
MIXED = [(0, 1), (0, 2), (5, 17), (63, 1), (64, 1), (65, 3), (130, 70), (0, 129), (300, 1)]


@pytest.mark.parametrize("d,nq,nkv,block", ATT_SHAPES)
@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("adt", [torch.float32, torch.bfloat16])
def test_attention_simt(d, nq, nkv, block, window, adt):
    c = _attention_case(d, nq, nkv, block, MIXED, window, adt)
    out = torch.empty(c["q"].shape, dtype=adt, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    K().paged_attention_simt(dev(c["q"]), nq * d, dev(c["pages"]), dev(c["table"]), dev(c["token_seq"]),
                             dev(c["positions"]), out, nq, nkv, d, 1 / math.sqrt(d), window or 0, status)
    assert int(status) == 0
    tol = 2e-5 if adt == torch.float32 else 2e-2
    err = (out.cpu().double() - c["want"]).abs().max() / c["want"].abs().max()
    assert float(err) < tol


@pytest.mark.parametrize("d,nq,nkv,block", ATT_SHAPES)
@pytest.mark.parametrize("window", [None, 37, 200])
def test_attention_tiled_tensor_core(d, nq, nkv, block, window):
    c = _attention_case(d, nq, nkv, block, MIXED, window, torch.bfloat16)
    G = nq // nkv
    out = torch.zeros(c["q"].shape, dtype=torch.bfloat16, device="cuda")
    tiles = sum(-(-(ql * G) // 64) for ql in c["q_lens"])
    K().attn_tiled(dev(c["q"]), nq * d, dev(c["pages"]), dev(c["table"]), dev(c["cu_q"]), dev(c["ctx_lens"]),
                   len(MIXED), tiles, out, nq, nkv, d, 1 / math.sqrt(d), window or 0)
    torch.cuda.synchronize()
    err = (out.cpu().double() - c["want"]).abs().max() / c["want"].abs().max()
    assert float(err) < 2e-2, float(err)


TC_SHAPES = [(64, 8, 1, 16), (128, 8, 2, 16), (256, 4, 2, 64), (128, 32, 8, 16), (64, 6, 2, 8), (128, 4, 4, 32),
             (192, 5, 1, 16)]


@pytest.mark.parametrize("d,nq,nkv,block", TC_SHAPES)
@pytest.mark.parametrize("window", [None, 37, 200])
def test_attention_tcgen05(d, nq, nkv, block, window):
    seqs = MIXED + [(700, 300), (0, 1000)]
    c = _attention_case(d, nq, nkv, block, seqs, window, torch.bfloat16, seed=5)
    G = nq // nkv
    out = torch.zeros(c["q"].shape, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tiles = sum(-(-(ql * G) // 128) for ql in c["q_lens"])
    K().attn_tc(dev(c["q"]), nq * d, dev(c["pages"]), dev(c["table"]), dev(c["cu_q"]), dev(c["ctx_lens"]),
                len(seqs), tiles, out, nq, nkv, d, 1 / math.sqrt(d), window or 0, status)
    torch.cuda.synchronize()
    assert int(status) == 0
    err = (out.cpu().double() - c["want"]).abs().max() / c["want"].abs().max()
    assert float(err) < 2e-2, float(err)


@pytest.mark.parametrize("d,nq,nkv,block", [(64, 8, 1, 16), (128, 8, 2, 16), (128, 4, 4, 32), (192, 5, 1, 8)])
@pytest.mark.parametrize("window", [None, 200])
@pytest.mark.parametrize("count", [2, 3, 8])
def test_attention_tcgen05_keys_shared_out_over_blocks(d, nq, nkv, block, window, count):
    """Every row tile's keys shared out over `count` blocks and joined by the second kernel: the same
    result as one block per row tile.  Sequences with fewer key tiles than shares (empty shares), one
    key, and a far key that stands out are among them; sequences in front of the compared ones shift
    the rows' indices in the scratch memory."""
    seqs = [(0, 1), (5, 17), (700, 300), (0, 1000), (63, 2), (1200, 130)]
    c = _attention_case(d, nq, nkv, block, seqs, window, torch.bfloat16, seed=11)
    G = nq // nkv
    T = sum(c["q_lens"])
    first = 2                                  # the first two sequences are left to another launch
    row0 = sum(c["q_lens"][:first])
    out = torch.zeros(c["q"].shape, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tiles = sum(-(-(ql * G) // 128) for ql in c["q_lens"][first:])
    cells = T * nq * count
    part_o = torch.full((cells * d,), float("nan"), device="cuda")
    part_ml = torch.full((cells * 2,), float("nan"), device="cuda")
    K().attn_tc(dev(c["q"]), nq * d, dev(c["pages"]), dev(c["table"][first:]), dev(c["cu_q"][first:]),
                dev(c["ctx_lens"][first:]), len(seqs) - first, tiles, out, nq, nkv, d, 1 / math.sqrt(d), window or 0,
                status, shares=(count, part_o, part_ml, row0, T - row0))
    torch.cuda.synchronize()
    assert int(status) == 0
    got, want = out.cpu().double()[row0:], c["want"][row0:]
    assert float((got - want).abs().max() / want.abs().max()) < 2e-2
    assert bool((out[:row0] == 0).all())       # rows of the sequences left out are not touched
    from firefly_b200.ops.kernels import attn_tc_shares
    assert attn_tc_shares(64, 8, 32) == 1 and attn_tc_shares(8, 8, 36) >= 2 and attn_tc_shares(8, 8, 5) == 1


@pytest.mark.parametrize("d,nq,nkv,block,page_list", [(64, 4, 1, 16, 16), (128, 8, 2, 8, 16), (128, 4, 4, 64, 16),
                                                      (64, 6, 2, 32, 32)])
@pytest.mark.parametrize("window", [None, 150])
def test_attention_tcgen05_walks_long_block_tables_in_pieces(d, nq, nkv, block, page_list, window):
    """A build whose ring of page ids holds 16 or 32 entries (1024 in the product): contexts of a
    thousand tokens then need it refilled many times, as contexts beyond 16 k tokens do in the
    product.  One far key stands out for the last query of each sequence, so a page read from the wrong
    place of the ring shows."""
    seqs = [(0, 1000), (700, 300), (1100, 2), (64 * 7, 129), (5, 17)]
    c = _attention_case(d, nq, nkv, block, seqs, window, torch.bfloat16, seed=9)
    G = nq // nkv
    out = torch.zeros(c["q"].shape, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tiles = sum(-(-(ql * G) // 128) for ql in c["q_lens"])
    K().attn_tc(dev(c["q"]), nq * d, dev(c["pages"]), dev(c["table"]), dev(c["cu_q"]), dev(c["ctx_lens"]),
                len(seqs), tiles, out, nq, nkv, d, 1 / math.sqrt(d), window or 0, status, page_list=page_list)
    torch.cuda.synchronize()
    assert int(status) == 0
    err = (out.cpu().double() - c["want"]).abs().max() / c["want"].abs().max()
    assert float(err) < 2e-2, float(err)


def test_attention_tcgen05_context_beyond_one_ring_of_page_ids():
    """The product build at a context of 17 000 tokens in pages of 16: 1 066 page ids a block, more than
    its ring of 1 024 holds.  Only the portion's 200 queries are compared (softmax over keys 0..position
    in 64-bit, written out here: the whole-sequence plain function would need the full score matrix)."""
    d, nq, nkv, block, ctx_len, q_len = 128, 4, 1, 16, 17000, 200
    g = torch.Generator().manual_seed(21)
    T = ctx_len + q_len
    q = torch.randn(q_len, nq, d, generator=g)
    k = torch.randn(T, nkv, d, generator=g)
    v = torch.randn(T, nkv, d, generator=g)
    k[3] = k[3] * 0.1 + 3.0 * q[-1, 0] / math.sqrt(d) * 4                 # far keys that stand out for late queries,
    k[16500] = k[16500] * 0.1 + 3.0 * q[-2, 1] / math.sqrt(d) * 4          # one on each side of the ring's refill
    q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    want = torch.empty(q_len, nq, d, dtype=torch.float64)
    kd, vd = k.double()[:, 0], v.double()[:, 0]
    for i in range(q_len):
        n = ctx_len + i + 1
        sc = (q[i].double() @ kd[:n].T) / math.sqrt(d)                     # [nq, n]
        want[i] = torch.softmax(sc, dim=-1) @ vd[:n]
    pages, order = _paged(k, v, block, seed=4)
    table = torch.tensor([order + [-1]], dtype=torch.int32)
    out = torch.zeros(q_len, nq * d, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tiles = -(-(q_len * nq) // 128)
    K().attn_tc(dev(q.reshape(q_len, nq * d).contiguous()), nq * d, dev(pages), dev(table),
                dev(torch.tensor([0, q_len], dtype=torch.int32)), dev(torch.tensor([ctx_len], dtype=torch.int32)), 1,
                tiles, out, nq, nkv, d, 1 / math.sqrt(d), 0, status)
    torch.cuda.synchronize()
    assert int(status) == 0
    err = (out.cpu().double() - want.reshape(q_len, nq * d)).abs().max() / want.abs().max()
    assert float(err) < 2e-2, float(err)


@pytest.mark.parametrize("d", [64, 128])
def test_attention_tcgen05_weights_of_late_large_scores(d):
    """Two heavy keys come late and stand 4.5 and 6 powers of two above everything before them: not
    far enough for the kernel to move its reference maximum (it does so beyond 8), so their softmax
    arguments are large.  The keys are tuned so that rounding those arguments to bfloat16 (spacing
    2^-5 there) would move one weight up and the other down by 0.9 %; their values are opposite, so
    the output is their weighted difference and shows it: 1.7 % against the 64-bit result.  The kernel
    must stay within 5e-3 (rounding of P, V and the output to bfloat16 costs up to about 4e-3)."""
    nq, nkv, block, T = 2, 1, 16, 192
    log2e = 1.4426950408889634
    g = torch.Generator().manual_seed(17)
    u = torch.randn(d, generator=g)
    u = u / u.norm()
    qv = (u * 4.0).to(torch.bfloat16)

    def key_for(target):                 # a key along u whose score, in powers of two, is `target`
        lo, hi, best = 0.0, 40.0, None
        for _ in range(60):
            mid = (lo + hi) / 2
            kv = (u * mid).to(torch.bfloat16)
            x = float(qv.double() @ kv.double()) / math.sqrt(d) * log2e
            if best is None or abs(x - target) < abs(best[1] - target):
                best = (kv, x)
            lo, hi = (mid, hi) if x < target else (lo, mid)
        return best
    h = 2.0 ** -5
    (k1, x1), (k2, x2) = key_for(6.0 + 0.4 * h), key_for(4.5 + 0.6 * h)
    assert abs((x1 - 6.0) / h - 0.4) < 0.05 and abs((x2 - 4.5) / h - 0.6) < 0.05
    q = qv.repeat(T, nq, 1)                                   # every query the same: every other score is 0
    k = torch.zeros(T, nkv, d, dtype=torch.bfloat16)
    v = torch.zeros(T, nkv, d, dtype=torch.bfloat16)
    w = torch.randn(d, generator=g).to(torch.bfloat16)
    k[130, 0], k[150, 0] = k1, k2
    v[130, 0], v[150, 0] = w, -w
    want = P.attention(q.double(), k.double(), v.double()).reshape(T, nq * d)
    pages, order = _paged(k, v, block, seed=2)
    table = torch.tensor([order + [-1]], dtype=torch.int32)
    out = torch.zeros(T, nq * d, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tiles = -(-(T * (nq // nkv)) // 128)
    K().attn_tc(dev(q.reshape(T, nq * d).contiguous()), nq * d, dev(pages), dev(table),
                dev(torch.tensor([0, T], dtype=torch.int32)), dev(torch.tensor([0], dtype=torch.int32)), 1, tiles, out,
                nq, nkv, d, 1 / math.sqrt(d), 0, status)
    torch.cuda.synchronize()
    assert int(status) == 0
    late = slice(160, T)                     # queries that see both heavy keys
    err = (out.cpu().double()[late] - want[late]).abs().max() / want[late].abs().max()
    assert float(err) < 5e-3, float(err)


@pytest.mark.parametrize("d,nq,nkv,block", ATT_SHAPES)
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("splits", [1, 2, 5])
def test_attention_decode_tensor_core(d, nq, nkv, block, window, splits):
    seqs = [(0, 1), (1, 1), (63, 1), (64, 1), (200, 1), (517, 1), (15, 1)]
    c = _attention_case(d, nq, nkv, block, seqs, window, torch.bfloat16, seed=3)
    n = len(seqs)
    out = torch.zeros(c["q"].shape, dtype=torch.bfloat16, device="cuda")
    part_o = torch.full((n * nq * splits * d,), float("nan"), device="cuda")
    part_ml = torch.full((n * nq * splits * 2,), float("nan"), device="cuda")
    K().attn_decode(dev(c["q"]), nq * d, dev(c["pages"]), dev(c["table"]), dev(c["cu_q"]), dev(c["ctx_lens"]),
                    n, out, part_o, part_ml, nq, nkv, d, 1 / math.sqrt(d), window or 0, splits)
    torch.cuda.synchronize()
    err = (out.cpu().double() - c["want"]).abs().max() / c["want"].abs().max()
    assert float(err) < 2e-2, float(err)


@pytest.mark.parametrize("d,nq,nkv,block", ATT_SHAPES)
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("units,max_ranges", [(9, 24), (10, 24), (55, 24), (200, 24), (55, 2), (31, 1)])
def test_attention_decode_ranges_shared_out_by_length(d, nq, nkv, block, window, units, max_ranges):
    """Sequences of very different lengths, and as many units as sequences (one range each, no
    join), one more, many more than there are tiles of keys, and a cap on the ranges."""
    seqs = [(0, 1), (1, 1), (63, 1), (64, 1), (200, 1), (1517, 1), (15, 1), (700, 1), (127, 1)]
    c = _attention_case(d, nq, nkv, block, seqs, window, torch.bfloat16, seed=4)
    n = len(seqs)
    out = torch.zeros(c["q"].shape, dtype=torch.bfloat16, device="cuda")
    part_o = torch.full((n * nq * units * d,), float("nan"), device="cuda")
    part_ml = torch.full((n * nq * units * 2,), float("nan"), device="cuda")
    seq_ranges = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    K().attn_decode_units(dev(c["q"]), nq * d, dev(c["pages"]), dev(c["table"]), dev(c["cu_q"]),
                          dev(c["ctx_lens"]), n, out, part_o, part_ml, seq_ranges, nq, nkv, d, 1 / math.sqrt(d),
                          window or 0, units, max_ranges)
    torch.cuda.synchronize()
    err = (out.cpu().double() - c["want"]).abs().max() / c["want"].abs().max()
    assert float(err) < 2e-2, float(err)
    # every sequence got a range at least, none more than it has tiles or than the cap, all of them within the units
    got = seq_ranges.cpu().tolist()
    tiles = [(cl + 64) // 64 - (max(0, cl - window + 1) // 64 if window else 0) for cl, _ in seqs]
    assert all(1 <= g <= min(t, max_ranges) for g, t in zip(got, tiles)), (got, tiles)
    assert sum(got) <= units
    if units >= 55 and max_ranges >= 24:
        assert window or (got[5] == max(got) and got[5] > got[7] > got[4])       # by length


@pytest.mark.parametrize("ctx_len,n", [(9000, 1), (6100, 2), (70, 1)])
def test_attention_decode_one_or_two_long_sequences_take_all_the_places(ctx_len, n):
    """Few long sequences: as many ranges as there are units (here 55 a kv head), each of a tile and a
    half of keys at least; a short sequence is not cut into crumbs.  One far key carries nearly all the
    weight of a row, so that a range that is lost or joined twice shows.  The plain result is written
    out for the new token alone (the whole-sequence function would need the full score matrix)."""
    d, nq, nkv, block = 128, 8, 2, 16
    G = nq // nkv
    g = torch.Generator().manual_seed(6)
    qs, wants, tables, page_list, ctxs, base = [], [], [], [], [], 1
    for si in range(n):
        cl = ctx_len - 37 * si
        T = cl + 1
        q = torch.randn(nq, d, generator=g)
        k = torch.randn(T, nkv, d, generator=g)
        v = torch.randn(T, nkv, d, generator=g)
        far = min(T - 1, 5 + 700 * si)
        k[far] = k[far] * 0.1 + 3.0 * q[::G] / math.sqrt(d) * 4
        q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
        want = torch.empty(nq, d, dtype=torch.float64)
        for h in range(nq):
            sc = (k.double()[:, h // G] @ q[h].double()) / math.sqrt(d)
            want[h] = torch.softmax(sc, dim=0) @ v.double()[:, h // G]
        pages, order = _paged(k, v, block, seed=30 + si)
        page_list.append(pages[1:])
        tables.append([o - 1 + base for o in order])
        base += pages.shape[0] - 1
        qs.append(q.reshape(1, nq * d))
        wants.append(want.reshape(1, nq * d))
        ctxs.append(cl)
    all_pages = torch.cat([torch.zeros(1, *page_list[0].shape[1:], dtype=torch.bfloat16)] + page_list, 0)
    mb = max(len(t) for t in tables) + 1
    table = torch.full((n, mb), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    want = torch.cat(wants, 0)
    units, max_ranges = 55, 64
    out = torch.zeros(n, nq * d, dtype=torch.bfloat16, device="cuda")
    part_o = torch.full((n * nq * units * d,), float("nan"), device="cuda")
    part_ml = torch.full((n * nq * units * 2,), float("nan"), device="cuda")
    seq_ranges = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    K().attn_decode_units(dev(torch.cat(qs, 0).contiguous()), nq * d, dev(all_pages), dev(table),
                          dev(torch.arange(n + 1, dtype=torch.int32)), dev(torch.tensor(ctxs, dtype=torch.int32)),
                          n, out, part_o, part_ml, seq_ranges, nq, nkv, d, 1 / math.sqrt(d), 0, units, max_ranges)
    torch.cuda.synchronize()
    err = (out.cpu().double() - want).abs().max() / want.abs().max()
    assert float(err) < 2e-2, float(err)
    got = seq_ranges.cpu().tolist()
    for r, cl in zip(got, ctxs):
        tiles = (cl + 64) // 64
        assert 1 <= r <= max(1, tiles * 2 // 3), (got, tiles)
    if ctx_len >= 6000:
        assert sum(got) >= units - n           # the long ones fill the units
    from firefly_b200.ops import kernels as kern
    assert kern.lengths_differ_much([ctx_len] * n) == (ctx_len >= 3072)
    assert not kern.lengths_differ_much([2100] * 8) and kern.lengths_differ_much([200, 6000, 300, 250])


class _Scratch:
    def __init__(self):
        self.bufs = {}

    def get(self, name, shape, dtype):
        key = (name, tuple(shape), dtype)
        if key not in self.bufs:
            fill = float("nan") if dtype.is_floating_point else -7
            self.bufs[key] = torch.full(tuple(shape), fill, dtype=dtype, device="cuda")
        return self.bufs[key]


@pytest.mark.parametrize("d,nq,nkv,block", [(64, 8, 1, 16), (128, 8, 2, 16), (192, 5, 5, 8), (256, 4, 2, 64),
                                            (128, 32, 2, 32), (64, 6, 2, 4)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("splits", [1, 2, 5, 0])                  # 0: ranges shared out by length
@pytest.mark.parametrize("norm,rot", [(True, True), (False, True), (True, False)])
def test_attention_decode_that_finishes_the_heads(d, nq, nkv, block, window, splits, norm, rot):
    """The decode kernel fed with the raw q|k|v projection against the two-kernel route (head kernel,
    then attention), which it equals bit for bit in its output and in the pages where both do the
    same arithmetic, and against the plain attention over the finished heads.  Contexts end on and beside tile and page edges."""
    from types import SimpleNamespace
    ctxs = [0, 1, 15, 63, 64, 65, 127, 128, 200, 517]
    n = len(ctxs)
    seqs = [(c, 1) for c in ctxs]
    theta, eps = 9000.0, 1e-5
    torch.manual_seed(d + nq)
    # history: finished keys and values in the pages; the row of the newest token holds stale data
    c = _attention_case(d, nq, nkv, block, seqs, window, torch.bfloat16, seed=11, spike=False)
    width = (nq + 2 * nkv) * d
    raw = torch.randn(n, width).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(d)) if norm else None
    kw = (1 + 0.1 * torch.randn(d)) if norm else None
    half = d // 2
    freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / d)
    ang = torch.arange(max(ctxs) + 2, dtype=torch.float64)[:, None] * freq[None]
    cs = torch.stack([torch.cos(ang), torch.sin(ang)], -1).float() if rot else None
    pages0 = c["pages"].clone()
    for i, p in enumerate(ctxs):                    # stale rows where the newest token goes
        pages0[int(c["table"][i, p // block]), :, :, p % block] = 77.0
    g = lambda t: None if t is None else dev(t)
    table, cu_q, ctx_lens = dev(c["table"]), dev(c["cu_q"]), dev(c["ctx_lens"])
    scale, win = 1 / math.sqrt(d), window or 0

    # two kernels
    qkv_a, pages_a = dev(raw.clone()), dev(pages0.clone())
    out_a = torch.zeros(n, nq * d, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    K().qk_norm_rope_store(qkv_a, nq, nkv, d, g(qw), g(kw), eps, g(cs), d if rot else 0, ctx_lens,
                           dev(torch.arange(n, dtype=torch.int32)), table, pages_a, status)
    part_o = torch.full((n * nq * max(splits, 1) * d,), float("nan"), device="cuda")
    part_ml = torch.full((n * nq * max(splits, 1) * 2,), float("nan"), device="cuda")
    K().attn_decode(qkv_a, width, pages_a, table, cu_q, ctx_lens, n, out_a, part_o, part_ml, nq, nkv, d, scale,
                    win, max(splits, 1))
    # one kernel
    qkv_b, pages_b = dev(raw.clone()), dev(pages0.clone())
    out_b = torch.zeros(n, nq * d, dtype=torch.bfloat16, device="cuda")
    ctx = SimpleNamespace(num_seqs=n, cu_q=cu_q, ctx_lens=ctx_lens, max_kv_len=max(ctxs) + 1, workspace=_Scratch(),
                          status=status, ranges_by_length=True)
    K().attn_decode_heads(qkv_b, pages_b, table, ctx, out_b, nq, nkv, d, scale, win, g(qw), g(kw), eps, g(cs),
                          num_splits=splits or None)
    torch.cuda.synchronize()
    assert splits or K().decode_units(n, nkv, d, True) > 0
    assert int(status) == 0
    assert torch.equal(qkv_b.cpu(), raw)                           # the projection's output is left as it was
    if d in (128, 256):          # the head kernel's register form does the same arithmetic in the same order
        assert torch.equal(pages_a.cpu(), pages_b.cpu())
    if d in (128, 256) and splits:
        assert torch.equal(out_a.cpu(), out_b.cpu())
    else:
        assert torch.allclose(pages_a.cpu().float(), pages_b.cpu().float(), atol=2e-2, rtol=2e-2)
        assert torch.allclose(out_a.cpu().float(), out_b.cpu().float(), atol=2e-2, rtol=2e-2)
    # and the plain result: heads finished in 64-bit, attention over history + newest token
    x = raw.double()
    q = x[:, :nq * d].view(n, nq, d)
    k = x[:, nq * d:(nq + nkv) * d].view(n, nkv, d)
    v = x[:, (nq + nkv) * d:].view(n, nkv, d)
    pos = torch.tensor(ctxs, dtype=torch.int32)
    if norm:
        q, k = P.rms_norm(q, qw.double(), eps), P.rms_norm(k, kw.double(), eps)
    if rot:
        q, k = P.rope(q, pos, theta), P.rope(k, pos, theta)
    gp = pages_b.cpu().double()
    G = nq // nkv
    for i, p in enumerate(ctxs):
        pg = int(c["table"][i, p // block])
        assert torch.allclose(gp[pg, 0, :, p % block], k[i], atol=2e-2, rtol=2e-2)
        assert torch.equal(gp[pg, 1, :, p % block], v[i])
        ks = torch.stack([gp[int(c["table"][i, t // block]), 0, :, t % block] for t in range(p + 1)])
        vs = torch.stack([gp[int(c["table"][i, t // block]), 1, :, t % block] for t in range(p + 1)])
        qs = torch.zeros(p + 1, nq, d, dtype=torch.float64)
        qs[p] = q[i].to(torch.bfloat16).double()
        want = P.attention(qs, ks, vs, window=window)[p].reshape(-1)
        got = out_b[i].cpu().double()
        assert float((got - want).abs().max() / want.abs().max()) < 2e-2


def test_attention_q_inside_wider_buffer():
    """q read in place from a [T, (nq+2nkv)*d] projection output."""
    d, nq, nkv, block = 64, 4, 2, 16
    c = _attention_case(d, nq, nkv, block, [(10, 20), (40, 1)], None, torch.bfloat16)
    T = c["q"].shape[0]
    width = (nq + 2 * nkv) * d
    buf = torch.randn(T, width).to(torch.bfloat16)
    buf[:, :nq * d] = c["q"]
    out = torch.zeros(T, nq * d, dtype=torch.bfloat16, device="cuda")
    K().attn_tiled(dev(buf), width, dev(c["pages"]), dev(c["table"]), dev(c["cu_q"]), dev(c["ctx_lens"]), 2,
                   2 + 1, out, nq, nkv, d, 1 / math.sqrt(d), 0)
    err = (out.cpu().double() - c["want"]).abs().max() / c["want"].abs().max()
    assert float(err) < 2e-2


def test_kernels_refuse_cpu_tensors_and_bad_sizes():
    k = K()
    with pytest.raises(k.KernelError, match="CUDA device only"):
        k.silu_mul(torch.zeros(2, 8), torch.zeros(2, 4))
    q = torch.zeros(1, 300, device="cuda")
    pages = torch.zeros(2, 2, 1, 16, 300, device="cuda")
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(k.KernelError, match="not supported"):
        k.paged_attention_simt(q, 300, pages, torch.zeros(1, 2, dtype=torch.int32, device="cuda"), z, z,
                               torch.zeros(1, 300, device="cuda"), 1, 1, 300, 1.0, 0, z)
