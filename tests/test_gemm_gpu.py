"""The tcgen05 matrix product alone against a 32-bit reference: token counts from 1
to several tiles, widths and depths that are no multiple of the tile, splits over
K, and each epilogue."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def K():
    from firefly_b200.ops import kernels
    return kernels


def _run(T, N, Kd, splits, epilogue, seed=0):
    k = K()
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, Kd, generator=g)).to(torch.bfloat16)
    w = (torch.randn(N, Kd, generator=g) / Kd ** 0.5).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    tok, s = k.gemm_tc_plan(T, N, Kd, splits)
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
        k.gemm_tc(xd, wd, out, epilogue, splits, status)
        torch.cuda.synchronize()
        assert int(status) == 0
        tol = 2e-2 if out.dtype == torch.bfloat16 else 2e-3
        err = float((out.cpu().double() - want).abs().max()) / (float(want.abs().max()) + 1e-9)
        assert err < tol, (T, N, Kd, splits, epilogue, s, tok, err)


@pytest.mark.parametrize("T", [1, 8, 16, 17, 64, 100, 256, 300])
@pytest.mark.parametrize("N,Kd", [(128, 64), (384, 512), (200, 1000), (4096, 4096)])
def test_store_bf16(T, N, Kd):
    _run(T, N, Kd, 1, K().EPI_BF16)


@pytest.mark.parametrize("T", [1, 8, 33])
@pytest.mark.parametrize("splits", [2, 3, 4, 5, 6, 7, 8, 100])
@pytest.mark.parametrize("N,Kd", [(256, 1024), (72, 200), (1024, 12288)])
def test_split_k(T, splits, N, Kd):
    _run(T, N, Kd, splits, K().EPI_F32)


@pytest.mark.parametrize("T", [3, 64, 130])
@pytest.mark.parametrize("splits", [1, 4])
def test_residual_add(T, splits):
    _run(T, 4096 + 64, 1536, splits, K().EPI_RESIDUAL_ADD)


@pytest.mark.parametrize("T", [1, 8, 70])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("I", [160, 2048, 12288])
def test_swiglu(T, splits, I):
    _run(T, 2 * I, 512, splits, K().EPI_SWIGLU)


@pytest.mark.parametrize("T", [1, 8, 20, 64])
@pytest.mark.parametrize("splits", [1, 4])
def test_rms_norm_folded_into_two_products(T, splits):
    """Product A adds into the residual and leaves bfloat16(residual*w) and per-tile sums of
    squares; product B consumes them: together they equal add, RMSNorm, product."""
    k = K()
    g = torch.Generator().manual_seed(T * 10 + splits)
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
    k.gemm_tc(xa.cuda(), wa.cuda(), res, k.EPI_RESIDUAL_ADD, splits, status, norm_out=(xw, nw.cuda(), ssq))
    outb = torch.zeros(T, Nb, dtype=torch.float32, device="cuda")
    k.gemm_tc(xw, wb.cuda(), outb, k.EPI_F32, splits, status, norm_in=(ssq, H, eps))
    torch.cuda.synchronize()
    assert int(status) == 0
    res_want = res0.double() + xa.double() @ wa.double().T
    assert float((res.cpu().double() - res_want).abs().max()) < 2e-2
    assert torch.allclose(ssq.sum(0).cpu().double(), (res.cpu().double() ** 2).sum(-1), rtol=1e-4)
    xn = res_want * torch.rsqrt((res_want ** 2).mean(-1, keepdim=True) + eps) * nw.double()
    want = xn @ wb.double().T
    err = float((outb.cpu().double() - want).abs().max()) / float(want.abs().max())
    assert err < 2e-2, err


def test_refuses_what_it_cannot_do():
    k = K()
    x = torch.zeros(4, 20, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(16, 20, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(4, 16, dtype=torch.bfloat16, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(k.KernelError, match="bad argument"):
        k.gemm_tc(x, w, out, k.EPI_BF16, 1, st)      # K not a multiple of 8


def test_a_wait_that_runs_out_ends_the_kernel_with_a_status_and_leaves_the_device_usable():
    """A test build of the product in which the loads of one k block are never issued and waits give
    up after a few milliseconds: the kernel must return, say which wait ran out (102: a loaded stage,
    or 103: the accumulator), store nothing, and the next ordinary launch must be right.  One block,
    no cluster (a block that gives up never leaves a peer waiting at a cluster barrier this way)."""
    import ctypes
    from ctypes import c_float, c_int, c_void_p
    from firefly_b200.ops.build import load_module
    k = K()
    lib = load_module("gemm_tcgen05.cu", {"FF_GEMM_TEST_DROP_KBLOCK": 1, "FF_GEMM_WAIT_LIMIT_CYCLES": "8000000ull"})
    g = torch.Generator().manual_seed(3)
    T, N, Kd = 16, 128, 256                                   # one tile of 128 rows, four k blocks
    x = torch.randn(T, Kd, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, Kd, generator=g) / 16).to(torch.bfloat16).cuda()
    out = torch.full((T, N), 7.0, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    null = c_void_p(0)
    rc = lib.ff_gemm_tc(c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(N), c_int(T),
                        c_int(N), c_int(Kd), c_int(k.EPI_F32), c_int(1), c_int(0), null, null, null, null, c_int(0),
                        c_int(0), c_float(0.0), c_void_p(status.data_ptr()),
                        c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()                                   # the kernel came back
    assert int(status) in (102, 103)
    assert bool((out == 7.0).all())                            # a block that gave up stores nothing
    status.zero_()
    good = torch.zeros(T, N, dtype=torch.float32, device="cuda")
    k.gemm_tc(x, w, good, k.EPI_F32, 1, status)
    torch.cuda.synchronize()
    assert int(status) == 0
    ref = x.double() @ w.double().T
    assert float((good.double() - ref).abs().max()) < 2e-3 * float(ref.abs().max())
