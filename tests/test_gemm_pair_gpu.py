"""The two-SM matrix product (tcgen05 with cta_group::2) alone against a 64-bit reference: token
counts from one tile's half to several tiles, widths and depths that are no multiple of the tile,
K ranges over the cluster, each epilogue, and the RMSNorm folded into two products."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def K():
    from firefly_b200.ops import kernels
    return kernels


def _run(T, N, Kd, ranges, epilogue, seed=0):
    k = K()
    g = torch.Generator().manual_seed(seed + T + N)
    x = (torch.randn(T, Kd, generator=g)).to(torch.bfloat16)
    w = (torch.randn(N, Kd, generator=g) / Kd ** 0.5).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    xd, wd = x.cuda(), w.cuda()
    if epilogue == k.EPI_BF16:
        out = torch.zeros(T, N, dtype=torch.bfloat16, device="cuda")
        want = ref
    elif epilogue == k.EPI_F32:
        out = torch.zeros(T, N, dtype=torch.float32, device="cuda")
        want = ref
    elif epilogue == k.EPI_RESIDUAL_ADD:
        base = torch.randn(T, N, generator=g)
        out = base.cuda()
        want = base.double() + ref
    else:
        I = N // 2
        gate, up = w[:I], w[I:]
        wd = k.interleave_gate_up(gate.cuda(), up.cuda())
        out = torch.zeros(T, I, dtype=torch.bfloat16, device="cuda")
        gv, uv = x.double() @ gate.double().T, x.double() @ up.double().T
        want = gv / (1 + torch.exp(-gv)) * uv
    for rep in range(2):
        if epilogue == k.EPI_RESIDUAL_ADD and rep:
            out.copy_(base)
        k.gemm_pair(xd, wd, out, epilogue, ranges, status)
        torch.cuda.synchronize()
        assert int(status) == 0
        tol = 2e-2 if out.dtype == torch.bfloat16 else 2e-3
        err = float((out.cpu().double() - want).abs().max()) / (float(want.abs().max()) + 1e-9)
        assert err < tol, (T, N, Kd, ranges, epilogue, err)


@pytest.mark.parametrize("T", [1, 33, 65, 100, 128, 200, 256, 300, 512, 700])
@pytest.mark.parametrize("N,Kd", [(256, 64), (384, 512), (200, 1000), (4096, 4096)])
def test_store_bf16(T, N, Kd):
    _run(T, N, Kd, 1, K().EPI_BF16)


@pytest.mark.parametrize("T", [70, 256, 300])
@pytest.mark.parametrize("ranges", [2, 3, 4, 100])
@pytest.mark.parametrize("N,Kd", [(256, 1024), (72, 200), (1024, 12288)])
def test_k_ranges(T, ranges, N, Kd):
    _run(T, N, Kd, ranges, K().EPI_F32)


@pytest.mark.parametrize("T", [66, 130, 256])
@pytest.mark.parametrize("ranges", [1, 4])
def test_residual_add(T, ranges):
    _run(T, 4096 + 64, 1536, ranges, K().EPI_RESIDUAL_ADD)


@pytest.mark.parametrize("T", [70, 256, 400])
@pytest.mark.parametrize("ranges", [1, 3])
@pytest.mark.parametrize("I", [160, 2048, 12288])
def test_swiglu(T, ranges, I):
    _run(T, 2 * I, 512, ranges, K().EPI_SWIGLU)


@pytest.mark.parametrize("T", [65, 128, 300])
@pytest.mark.parametrize("ranges", [1, 4])
def test_rms_norm_folded_into_two_products(T, ranges):
    """Product A adds into the residual and leaves bfloat16(residual*w) and per-tile sums of squares;
    product B consumes them: together they equal add, RMSNorm, product."""
    k = K()
    g = torch.Generator().manual_seed(T * 10 + ranges)
    H, Ka, Nb, eps = 328, 512, 384, 1e-5                 # a width that is no multiple of 128
    res0 = torch.randn(T, H, generator=g) * 2
    xa = torch.randn(T, Ka, generator=g).to(torch.bfloat16)
    wa = (torch.randn(H, Ka, generator=g) / Ka ** 0.5).to(torch.bfloat16)
    nw = 1 + 0.1 * torch.randn(H, generator=g)
    wb = (torch.randn(Nb, H, generator=g) / H ** 0.5).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = res0.cuda()
    xw = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    parts = -(-H // 128)
    ssq = torch.full((parts, T), float("nan"), device="cuda")
    k.gemm_pair(xa.cuda(), wa.cuda(), res, k.EPI_RESIDUAL_ADD, ranges, status, norm_out=(xw, nw.cuda(), ssq))
    outb = torch.zeros(T, Nb, dtype=torch.float32, device="cuda")
    k.gemm_pair(xw, wb.cuda(), outb, k.EPI_F32, ranges, status, norm_in=(ssq, H, eps))
    torch.cuda.synchronize()
    assert int(status) == 0
    res_want = res0.double() + xa.double() @ wa.double().T
    assert float((res.cpu().double() - res_want).abs().max()) < 2e-2
    assert torch.allclose(ssq.sum(0).cpu().double(), (res.cpu().double() ** 2).sum(-1), rtol=1e-4)
    xn = res_want * torch.rsqrt((res_want ** 2).mean(-1, keepdim=True) + eps) * nw.double()
    want = xn @ wb.double().T
    err = float((outb.cpu().double() - want).abs().max()) / float(want.abs().max())
    assert err < 2e-2, err


@pytest.mark.parametrize("family", ["whole", "portions", "mixed"])
def test_replay_with_the_two_sm_product_switched_on(family, monkeypatch):
    """The engine's products between 65 and 512 tokens routed to the two-SM kernel (off by default):
    replayed logits still match the plain implementation, with the folded norms and fused epilogues."""
    import plain_qwen3 as P
    import replay_util as U
    from firefly_b200.models import DecoderModel, config_from_dict, spec_for
    from firefly_b200.parts import Runtime
    from firefly_b200.replay import ReplaySession
    k = K()
    monkeypatch.setattr(k, "USE_PAIR_GEMM", True)
    k.set_exact_matmul()
    cfg = P.TINY_D
    w = P.random_weights(cfg, 13, dtype=torch.bfloat16, scale=0.05)
    model = DecoderModel(spec_for(config_from_dict(cfg)), Runtime(torch.device("cuda"), torch.bfloat16))
    model.bind({n: v.to("cuda").to(torch.bfloat16 if v.dim() > 1 else torch.float32) for n, v in w.items()})
    reqs = U.make_requests(cfg["vocab_size"], [300, 90, 170], 4)
    plain = {rid: P.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    steps = {"whole": U.trace_whole, "mixed": U.trace_mixed,
             "portions": lambda r: U.trace_portions(r, sizes=(130, 70, 2, 100, 66))}[family](reqs)
    before = k.LAUNCHES
    sess = ReplaySession(model=model, max_tokens=U.peak_tokens(steps), block_size=16)
    U.compare(U.run_trace(sess, steps), plain, U.TOL["bfloat16"], f"two-SM product/{family}")
    sess.runner.check_status()
    assert k.LAUNCHES > before
