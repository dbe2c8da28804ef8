"""Python faces of the CUDA kernels in ``csrc/``.

Every function takes CUDA tensors, launches on torch's current stream (so the
calls can be captured into a CUDA graph) and writes into buffers the caller
provides; nothing is allocated here.  There is no CPU or library fallback: a
tensor that is not on a CUDA device, or a kernel that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_float, c_int, c_size_t, c_void_p
from typing import Optional

import torch

from .build import compile_many, load_module

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream's handle.  Asked for at every launch: the raw getter costs well under a
    microsecond where ``torch.cuda.current_stream()`` builds an object each time (15 us)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {t.dtype}") from None


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None:
            if not t.is_cuda:
                raise KernelError("firefly_b200 kernels run on a CUDA device only; got a "
                                  f"{t.device} tensor (there is no CPU implementation)")
            if not t.is_contiguous():
                raise KernelError("kernel operand must be contiguous")


LAUNCHES = 0   # launches of this package's own kernels (library products are not counted)


def _check(code: int, what: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        return
    if code == -1:
        raise KernelError(f"{what}: bad argument")
    if code == -2:
        raise KernelError(f"{what}: size not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {code}")


_MODULES = {
    "elementwise": ("elementwise.cu", None),
    "qk_rope_store": ("qk_rope_store.cu", None),
    "attention_simt": ("attention_simt.cu", None),
    "sampling": ("sampling.cu", None),
    "gemm_tcgen05": ("gemm_tcgen05.cu", None),
    "gemm_pair": ("gemm_pair.cu", None),
    "weights": ("weights.cu", None),
}


USE_PDL = True      # programmatic dependent launch: a kernel's prologue overlaps its predecessor's tail
_pdl_state = {}     # id(library) -> flag it was last given


def _configured(lib: ctypes.CDLL) -> ctypes.CDLL:
    if _pdl_state.get(id(lib)) != USE_PDL:
        lib.ff_set_pdl(c_int(1 if USE_PDL else 0))
        _pdl_state[id(lib)] = USE_PDL
    return lib


def set_pdl(on: bool) -> None:
    """Switch programmatic dependent launch on or off for all kernels of this package."""
    global USE_PDL
    USE_PDL = bool(on)


def _lib(name: str) -> ctypes.CDLL:
    src, defs = _MODULES[name]
    return _configured(load_module(src, defs))


DEFAULT_HEAD_DIMS = (128,)


def build_all(head_dims=DEFAULT_HEAD_DIMS) -> None:
    """Compile every module (used by the build check; needs no GPU).  The
    tensor-core attention is compiled per head size; others are built when a
    model with that head size is first run."""
    mods = list(_MODULES.values()) + [("attention_mma.cu", {"FF_HEAD_DIM": int(d)}) for d in head_dims] + \
        [("attention_tc.cu", {"FF_HEAD_DIM": int(d)}) for d in head_dims if int(d) % 64 == 0]
    compile_many(mods)


# --------------------------------------------------------------------------- #
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[t,:] = float(table[ids[t],:]); ids int32 [T], out float32 [T,H]."""
    _need_cuda(ids, table, out, status)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32
    T, H = out.shape
    V = table.shape[0]
    assert table.shape[1] == H and ids.numel() == T
    _check(_lib("elementwise").ff_embedding(_p(ids), _p(table), c_int(_dt(table)), _p(out), c_int(T),
                                           c_int(H), c_int(V), _p(status), _stream()), "embedding")


def scatter_int(buf: torch.Tensor, updates: torch.Tensor, cap: int) -> None:
    """buf[updates[1 + 2i]] = updates[2 + 2i] for i < min(updates[0], cap); all int32."""
    _need_cuda(buf, updates)
    assert buf.dtype == torch.int32 and updates.dtype == torch.int32 and updates.numel() >= 1 + 2 * cap
    _check(_lib("elementwise").ff_scatter_int(_p(buf), _p(updates), c_int(cap), c_int(buf.numel()), _stream()),
           "scatter_int")


def add_rms_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                 eps: float, out: torch.Tensor, row_idx: Optional[torch.Tensor] = None) -> None:
    """residual (+= delta), out = rms_norm(residual) * weight.

    residual float32 [T,H], updated in place when ``delta`` is given and
    ``row_idx`` is not.  With ``row_idx`` (int32 [n]) only those rows are
    normalised, into ``out`` [n,H], and the residual is left as it is.
    """
    _need_cuda(residual, delta, weight, out, row_idx)
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32
    H = residual.shape[-1]
    rows = out.shape[0]
    assert out.shape[-1] == H and weight.numel() == H
    if row_idx is None:
        assert rows == residual.shape[0]
    else:
        assert row_idx.dtype == torch.int32 and row_idx.numel() == rows
    if delta is not None:
        assert delta.shape == residual.shape
    _check(_lib("elementwise").ff_add_rms_norm(
        _p(residual), _p(delta), c_int(_dt(delta) if delta is not None else _dt(out)), _p(row_idx),
        _p(weight), c_float(eps), _p(out), c_int(_dt(out)), c_int(rows), c_int(H),
        c_int(1 if row_idx is None else 0), _stream()), "add_rms_norm")


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    _need_cuda(residual, delta)
    assert residual.dtype == torch.float32 and residual.shape == delta.shape
    _check(_lib("elementwise").ff_residual_add(_p(residual), _p(delta), c_int(_dt(delta)),
                                              c_size_t(residual.numel()), _stream()), "residual_add")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out[t,i] = silu(gate) * up, gate = gate_up[t,i], up = gate_up[t,I+i]; with
    ``interleaved`` the columns hold gate and up in alternating groups of 16."""
    _need_cuda(gate_up, out)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype == out.dtype
    _check(_lib("elementwise").ff_silu_mul(_p(gate_up), _p(out), c_int(_dt(out)), c_int(T), c_int(I),
                                          c_int(1 if interleaved else 0), _stream()), "silu_mul")


def cast(src: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(src, out)
    assert src.numel() == out.numel()
    _check(_lib("elementwise").ff_cast(_p(src), c_int(_dt(src)), _p(out), c_int(_dt(out)),
                                      c_size_t(src.numel()), _stream()), "cast")


def qk_norm_rope_store(qkv: torch.Tensor, nq: int, nkv: int, d: int, q_norm_w, k_norm_w, eps: float,
                       cos_sin: Optional[torch.Tensor], rotary_dim: int, positions: torch.Tensor,
                       token_seq: torch.Tensor, block_table: Optional[torch.Tensor],
                       cache: Optional[torch.Tensor], status: torch.Tensor) -> None:
    """Per-head RMSNorm of q and k, rotation, and the write of k, v into the
    paged cache ``[blocks, 2, nkv, block_size, d]``; q is rewritten in place in
    ``qkv`` [T, (nq+2nkv)*d].  ``nkv == 0``: q only, no cache write."""
    _need_cuda(qkv, q_norm_w, k_norm_w, cos_sin, positions, token_seq, block_table, cache, status)
    T, width = qkv.shape
    if nkv:
        assert cache is not None and block_table is not None and cache.dtype == qkv.dtype
        num_blocks, two, ckv, block_size, cd = cache.shape
        assert two == 2 and ckv == nkv and cd == d
        max_blocks = block_table.shape[1]
    else:
        num_blocks = block_size = max_blocks = 1
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.shape[1] * cos_sin.shape[2] == rotary_dim
    _check(_lib("qk_rope_store").ff_qk_norm_rope_store(
        _p(qkv), c_int(_dt(qkv)), c_int(width), c_int(T), c_int(nq), c_int(nkv), c_int(d),
        _p(q_norm_w), _p(k_norm_w), c_float(eps), _p(cos_sin), c_int(rotary_dim), c_int(max_pos),
        _p(positions), _p(token_seq), _p(block_table), c_int(max_blocks), c_int(block_size),
        c_int(num_blocks), _p(cache), _p(status), _stream()), "qk_norm_rope_store")


def paged_attention_simt(q: torch.Tensor, q_stride: int, cache: torch.Tensor, block_table: torch.Tensor,
                         token_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                         nq: int, nkv: int, d: int, scale: float, window: int,
                         status: torch.Tensor) -> None:
    """Attention of every query token over its sequence's cached keys 0..pos
    (or the last ``window`` of them; 0 = all).  ``q`` is read with row stride
    ``q_stride`` elements (it may be the head of a wider qkv buffer)."""
    _need_cuda(cache, block_table, token_seq, positions, out, status)
    if not q.is_cuda:
        raise KernelError("firefly_b200 kernels run on a CUDA device only")
    T = out.shape[0]
    num_blocks, two, ckv, block_size, cd = cache.shape
    assert two == 2 and ckv == nkv and cd == d and cache.dtype == q.dtype == out.dtype
    _check(_lib("attention_simt").ff_paged_attention_simt(
        _p(q), c_int(_dt(q)), c_int(q_stride), _p(cache), _p(block_table), c_int(block_table.shape[1]),
        _p(token_seq), _p(positions), _p(out), c_int(out.shape[1]), c_int(T), c_int(nq), c_int(nkv),
        c_int(d), c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), _p(status),
        _stream()), "paged_attention_simt")


_sample_scratch = {}


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           seeds: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None) -> None:
    """out[r] = arg-max of logits[r] (lowest index on ties), or, where
    temperature[r] > 0, a draw from softmax(logits[r] / temperature[r]) with the
    random numbers of (seeds[r], counters[r]).

    The one wrapper that keeps memory of its own: the partial results of rows split over several
    blocks live in a scratch pair per device that grows when more rows come.  It never grows while
    the stream is being captured (an error then: the run before the capture sizes it)."""
    global LAUNCHES
    _need_cuda(logits, out, temperature, seeds, counters)
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and logits.dim() == 2
    rows, V = logits.shape
    if temperature is not None:
        assert temperature.dtype == torch.float32 and seeds.dtype == torch.int64 \
            and counters.dtype == torch.int64
    # a row is split over several blocks so that few rows still fill the GPU
    chunks = max(1, min(64, _sm_target_ctas() // 2 // max(rows, 1), V // 2048))
    pv = pi = None
    if chunks > 1:
        key = logits.device
        buf = _sample_scratch.get(key)
        if buf is None or buf[0].numel() < rows * chunks:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("sample: its scratch memory would have to grow while a CUDA graph is being "
                                  "captured; run the same step once before the capture")
            n = max(rows * chunks, 4096)
            buf = (torch.empty(n, dtype=torch.float32, device=key), torch.empty(n, dtype=torch.int32, device=key))
            _sample_scratch[key] = buf
        pv, pi = buf
    _check(_lib("sampling").ff_sample(_p(logits), c_int(rows), c_int(V), c_size_t(logits.stride(0)),
                                     _p(temperature), _p(seeds), _p(counters), _p(out), c_int(chunks),
                                     _p(pv), _p(pi), _stream()), "sample")
    if chunks > 1:
        LAUNCHES += 1


# --------------------------------------------------------------------------- #
# matrix products: a library routine (cuBLAS through torch), as the reference
# uses a library (CUTLASS, src/kernels/linear.cu:15-104) for them.
def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out = x @ weight^T with 32-bit accumulation.  ``weight`` [N,K] row-major
    as stored in checkpoints.  ``out`` may be float32 for bfloat16 operands."""
    _need_cuda(x, weight, out)
    if x.dtype != weight.dtype:
        raise KernelError(f"linear: operand types differ ({x.dtype} vs {weight.dtype})")
    if out.dtype == x.dtype:
        torch.mm(x, weight.t(), out=out)
    elif out.dtype == torch.float32:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
    else:
        raise KernelError(f"linear: cannot write {out.dtype} from {x.dtype}")


def linear_add(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor) -> None:
    """residual (float32) += x @ weight^T through the library, the sum formed in 32-bit: the product
    never exists rounded to the operands' type, and the norm behind it has one tensor less to read."""
    _need_cuda(x, weight, residual)
    if x.dtype != weight.dtype or residual.dtype != torch.float32:
        raise KernelError(f"linear_add: {x.dtype} x {weight.dtype} into {residual.dtype}")
    if x.dtype == torch.float32:
        torch.addmm(residual, x, weight.t(), out=residual)
    else:
        torch.addmm(residual, x, weight.t(), out_dtype=torch.float32, out=residual)


LIBRARY_ADDS_INTO_RESIDUAL = True   # products of more than GEMM_TC_MAX_TOKENS tokens add into the 32-bit residual themselves
EPI_BF16, EPI_F32, EPI_RESIDUAL_ADD, EPI_SWIGLU = 0, 1, 2, 3
GEMM_TC_MAX_TOKENS = 64    # up to here the one-block tcgen05 product runs
# From there to GEMM_PAIR_MAX_TOKENS the two-SM product (cta_group::2, csrc/gemm_pair.cu) can take over,
# with the same fused epilogues.  Off: alone it reaches 0.7 to 1.0 of the library's speed at 128 to 512
# tokens (the gate|up product at 128 tokens: 41 us against 41), but inside a step its blocks, one per SM
# with nearly all of the shared memory, leave no room for the next kernel to move in early, and a
# 256-token step of the 8B shape takes 8.2 ms with it against 5.9 ms with the library's products.
USE_PAIR_GEMM = False
GEMM_PAIR_MAX_TOKENS = 512
USE_TCGEN05_GEMM = True    # tests flip this to compare with the library route
FOLD_NORM = True           # fold the RMSNorm between two tcgen05 products into their epilogues


def gemm_tc_plan(T: int, N: int, K: int, want_splits: int):
    """(tokens per tile, K ranges) the tensor-core product would use."""
    tok, splits = c_int(), c_int()
    _lib("gemm_tcgen05").ff_gemm_tc_plan(c_int(T), c_int(N), c_int(K), c_int(want_splits), ctypes.byref(tok),
                                       ctypes.byref(splits))
    return tok.value, splits.value


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int, want_splits: int,
            status: torch.Tensor, *, norm_out: Optional[tuple] = None, norm_in: Optional[tuple] = None) -> None:
    """out (op)= x @ weight^T on tcgen05 tensor cores; bfloat16 operands, 32-bit accumulation.

    epilogue: EPI_BF16 store bfloat16, EPI_F32 store float32, EPI_RESIDUAL_ADD add into a float32
    ``out``, EPI_SWIGLU store silu(gate)*up as bfloat16 [T, N/2] for a weight whose rows interleave
    gate and up in groups of 16.  ``want_splits`` K ranges (at most 8) share a thread-block cluster.

    An RMSNorm between two products can be folded into them.  Producing side (EPI_RESIDUAL_ADD):
    ``norm_out`` = (xw bfloat16 [T, N], norm weight float32 [N], ssq float32 [ceil(N/128), T]) receives
    bfloat16(out * w) and each row tile's sum of squares per token.  Consuming side: ``norm_in`` =
    (ssq [parts, T], norm_dim, eps) scales token t's result by rsqrt(sum_p ssq[p, t] / norm_dim + eps)."""
    _need_cuda(x, weight, out, status)
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    T, Kd = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == Kd
    if epilogue == EPI_BF16 or epilogue == EPI_SWIGLU:
        assert out.dtype == torch.bfloat16
    else:
        assert out.dtype == torch.float32
    assert out.shape[0] == T and out.shape[1] == (N // 2 if epilogue == EPI_SWIGLU else N)
    xw = xw_w = ssq_out = ssq_in = None
    parts = dim = 0
    eps = 0.0
    if norm_out is not None:
        xw, xw_w, ssq_out = norm_out
        _need_cuda(xw, xw_w, ssq_out)
        assert epilogue == EPI_RESIDUAL_ADD and xw.dtype == torch.bfloat16 and xw.shape == (T, N)
        assert xw_w.dtype == torch.float32 and xw_w.numel() == N
        assert ssq_out.dtype == torch.float32 and ssq_out.numel() >= -(-N // 128) * T
    if norm_in is not None:
        ssq_in, dim, eps = norm_in
        _need_cuda(ssq_in)
        assert ssq_in.dtype == torch.float32 and ssq_in.dim() == 2 and ssq_in.shape[1] == T
        parts = ssq_in.shape[0]
    _check(_lib("gemm_tcgen05").ff_gemm_tc(
        _p(x), _p(weight), _p(out), c_int(out.stride(0)), c_int(T), c_int(N), c_int(Kd), c_int(epilogue),
        c_int(want_splits), c_int(1 if USE_PDL else 0), _p(xw), _p(xw_w), _p(ssq_out), _p(ssq_in),
        c_int(parts), c_int(dim), c_float(eps), _p(status), _stream()), "gemm_tc")


def gemm_pair_plan(T: int, N: int, K: int, want_ranges: int):
    """(tokens per tile, K ranges) the two-SM product would use."""
    tok, ranges = c_int(), c_int()
    _lib("gemm_pair").ff_gemm_pair_plan(c_int(T), c_int(N), c_int(K), c_int(want_ranges), ctypes.byref(tok),
                                        ctypes.byref(ranges))
    return tok.value, ranges.value


def gemm_pair(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int, want_ranges: int,
              status: torch.Tensor, *, norm_out: Optional[tuple] = None, norm_in: Optional[tuple] = None) -> None:
    """out (op)= x @ weight^T on pairs of SMs (tcgen05 with cta_group::2), for steps of about a hundred to
    a few hundred tokens.  Arguments as `gemm_tc`; ``want_ranges`` K ranges (at most 4)."""
    _need_cuda(x, weight, status)
    if not out.is_cuda or out.dim() != 2 or out.stride(1) != 1:
        raise KernelError("gemm_pair: the output must be a CUDA matrix with contiguous rows")
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    T, Kd = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == Kd
    assert out.dtype == (torch.bfloat16 if epilogue in (EPI_BF16, EPI_SWIGLU) else torch.float32)
    assert out.shape[0] == T and out.shape[1] == (N // 2 if epilogue == EPI_SWIGLU else N)
    xw = xw_w = ssq_out = ssq_in = None
    parts = dim = 0
    eps = 0.0
    if norm_out is not None:
        xw, xw_w, ssq_out = norm_out
        _need_cuda(xw, xw_w, ssq_out)
        assert epilogue == EPI_RESIDUAL_ADD and xw.dtype == torch.bfloat16 and xw.shape == (T, N)
        assert xw_w.dtype == torch.float32 and xw_w.numel() == N
        assert ssq_out.dtype == torch.float32 and ssq_out.numel() >= -(-N // 128) * T
    if norm_in is not None:
        ssq_in, dim, eps = norm_in
        _need_cuda(ssq_in)
        assert ssq_in.dtype == torch.float32 and ssq_in.dim() == 2 and ssq_in.shape[1] == T
        parts = ssq_in.shape[0]
    _check(_lib("gemm_pair").ff_gemm_pair(
        _p(x), _p(weight), _p(out), c_int(out.stride(0)), c_int(T), c_int(N), c_int(Kd), c_int(epilogue),
        c_int(want_ranges), c_int(1 if USE_PDL else 0), _p(xw), _p(xw_w), _p(ssq_out), _p(ssq_in),
        c_int(parts), c_int(dim), c_float(eps), _p(status), _stream()), "gemm_pair")


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stack gate and up rows in groups of 16: rows [32g, 32g+16) are gate rows [16g, 16g+16),
    rows [32g+16, 32g+32) the up rows of the same columns.  Needs I % 16 == 0."""
    I, H = gate.shape
    assert I % 16 == 0 and up.shape == gate.shape
    return torch.stack([gate.view(I // 16, 16, H), up.view(I // 16, 16, H)], dim=1).reshape(2 * I, H).contiguous()


def set_exact_matmul() -> None:
    """No reduced-precision matrix mode anywhere: 32-bit products are true
    32-bit (no TF32), 16-bit products accumulate and reduce in 32-bit."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    try:
        torch.set_float32_matmul_precision("highest")
    except Exception:  # noqa: BLE001
        pass


_ATTN_FORCE_SIMT = False      # tests flip this to compare the two kernels


@functools.lru_cache(maxsize=None)
def sm_count(device_index: Optional[int] = None) -> int:
    """Streaming multiprocessors of the device (the current one by default), asked of the driver
    once.  Grid sizes, K splits and scratch extents are derived from it; no file holds the figure."""
    if device_index is None:
        device_index = torch.cuda.current_device()
    return int(torch.cuda.get_device_properties(device_index).multi_processor_count)


def _sm_target_ctas() -> int:
    """Blocks that the decode attention's scratch memory is sized for: four per SM."""
    return 4 * sm_count()


def _attn_lib(d: int) -> ctypes.CDLL:
    return _configured(load_module("attention_mma.cu", {"FF_HEAD_DIM": d}))


def mma_attention_supported(dtype: torch.dtype, d: int) -> bool:
    return dtype == torch.bfloat16 and d % 16 == 0 and 16 <= d <= 256


def attn_tiled(q, q_stride, pages, table, cu_q, ctx_lens, n_seqs, total_tiles, out, nq, nkv, d, scale,
               window, status: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention for any mix of sequences (bfloat16).  ``status`` (int32 [1]) is set to 4
    when a key that must be read has no valid page in the block table."""
    _need_cuda(pages, table, cu_q, ctx_lens, out, status)
    num_blocks, _, _, block_size, _ = pages.shape
    _check(_attn_lib(d).ff_attn_tiled(
        _p(q), c_int(q_stride), _p(pages), _p(table), c_int(table.shape[1]), _p(cu_q), _p(ctx_lens),
        c_int(n_seqs), c_int(total_tiles), _p(out), c_int(out.shape[1]), c_int(nq), c_int(nkv),
        c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), _p(status), _stream()), "attn_tiled")


def attn_decode(q, q_stride, pages, table, cu_q, ctx_lens, n_seqs, out, part_o, part_ml, nq, nkv, d,
                scale, window, num_splits, status: Optional[torch.Tensor] = None) -> None:
    """Split-KV tensor-core attention when every sequence has one token (bfloat16).  ``status`` as
    for `attn_tiled`."""
    _need_cuda(pages, table, cu_q, ctx_lens, out, part_o, part_ml, status)
    num_blocks, _, _, block_size, _ = pages.shape
    _check(_attn_lib(d).ff_attn_decode(
        _p(q), c_int(q_stride), _p(pages), _p(table), c_int(table.shape[1]), _p(cu_q), _p(ctx_lens),
        c_int(n_seqs), _p(out), c_int(out.shape[1]), _p(part_o), _p(part_ml), c_int(nq), c_int(nkv),
        c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), c_int(num_splits),
        _p(status), _stream()), "attn_decode")
    global LAUNCHES
    if num_splits > 1:
        LAUNCHES += 1     # the kernel that joins the splits


DECODE_FINISHES_HEADS = True    # pure decode steps: per-head norm, rotation and cache write inside the attention kernel


def decode_finishes_heads(ctx, dtype: torch.dtype, nq: int, nkv: int, d: int, rotary_dim: int) -> bool:
    """True if this step's attention kernel can take the raw q|k|v projection: every sequence
    decodes one token, bfloat16, a head size in steps of 64 that is rotated whole or not at all,
    and at most 16 query heads per kv head."""
    return (DECODE_FINISHES_HEADS and not _ATTN_FORCE_SIMT and ctx.num_seqs > 0
            and ctx.num_decode_seqs == ctx.num_seqs and dtype == torch.bfloat16 and d % 64 == 0 and d <= 256
            and nkv > 0 and nq // nkv <= 16 and rotary_dim in (0, d))


def attn_decode_heads(qkv, pages, table, ctx, out, nq, nkv, d, scale, window, q_norm_w, k_norm_w, eps,
                      cos_sin, num_splits: Optional[int] = None) -> None:
    """The split-KV decode attention fed with the raw q|k|v projection ``[T, (nq + 2 nkv) d]``:
    it finishes the heads itself (per-head RMSNorm, rotation, cache write of the newest key and
    value) and replaces `qk_norm_rope_store` + `attn_decode` in steps that only decode."""
    _need_cuda(qkv, pages, table, out, q_norm_w, k_norm_w, cos_sin)
    num_blocks, _, _, block_size, _ = pages.shape
    n = ctx.num_seqs
    global LAUNCHES
    units = 0 if num_splits else decode_units(n, nkv, d, ctx.ranges_by_length)
    splits = num_splits or decode_splits(n, nkv, ctx.max_kv_len)
    part_o, part_ml, seq_ranges = _decode_scratch(ctx.workspace, n, nq, nkv, d, splits)
    if units:
        attn_decode_units(qkv, qkv.shape[1], pages, table, ctx.cu_q, ctx.ctx_lens, n, out, part_o, part_ml,
                          seq_ranges, nq, nkv, d, scale, window, units, DECODE_MAX_RANGES,
                          heads=(q_norm_w, k_norm_w, eps, cos_sin), status=ctx.status)
        return
    _check(_attn_lib(d).ff_attn_decode_heads(
        _p(qkv), c_int(qkv.shape[1]), _p(pages), _p(table), c_int(table.shape[1]), _p(ctx.cu_q), _p(ctx.ctx_lens),
        c_int(n), _p(out), c_int(out.shape[1]), _p(part_o), _p(part_ml), c_int(nq), c_int(nkv),
        c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), c_int(splits),
        _p(q_norm_w), _p(k_norm_w), c_float(eps), _p(cos_sin), c_int(cos_sin.shape[0] if cos_sin is not None else 0),
        _p(ctx.status), _stream()), "attn_decode_heads")
    if splits > 1:
        LAUNCHES += 1     # the kernel that joins the splits


USE_TC_ATTENTION = True     # tcgen05 attention for prompt portions where the sizes allow


def _attn_tc_lib(d: int, page_list: Optional[int] = None) -> ctypes.CDLL:
    defs = {"FF_HEAD_DIM": d}
    if page_list is not None:
        defs["FF_ATC_PAGE_LIST"] = int(page_list)       # a test build with a tiny ring of page ids
    return _configured(load_module("attention_tc.cu", defs))


def tc_attention_supported(dtype: torch.dtype, d: int, block_size: int, max_kv_len: int = 0) -> bool:
    """The tcgen05 attention kernel takes head sizes 64..256 in steps of 64 and pages of 8..64 tokens
    that divide 64; contexts of any length (it walks the block table in pieces)."""
    return dtype == torch.bfloat16 and d % 64 == 0 and 64 <= d <= 256 and block_size in (8, 16, 32, 64)


def attn_tc(q, q_stride, pages, table, cu_q, ctx_lens, n_seqs, total_tiles, out, nq, nkv, d, scale, window,
            status, page_list: Optional[int] = None, shares=None) -> None:
    """tcgen05 flash attention over the paged cache (bfloat16); total_tiles counts row tiles of 128.
    ``shares`` = (count, part_o, part_ml, first row, rows): every row tile's keys are shared out over
    ``count`` blocks and a second kernel joins their partial results (for prompts so short that their
    row tiles alone would leave most SMs idle); the scratch tensors are float32 with at least
    (first row + rows) * nq * count * d and ... * 2 elements."""
    _need_cuda(pages, table, cu_q, ctx_lens, out, status)
    num_blocks, _, _, block_size, _ = pages.shape
    count, part_o, part_ml, row0, rows = shares if shares is not None else (1, None, None, 0, 0)
    if count > 1:
        _need_cuda(part_o, part_ml)
        need = (row0 + rows) * nq * count
        assert part_o.dtype == part_ml.dtype == torch.float32 and part_o.numel() >= need * d and part_ml.numel() >= need * 2
    _check(_attn_tc_lib(d, page_list).ff_attn_tc(
        _p(q), c_int(q_stride), _p(pages), _p(table), c_int(table.shape[1]), _p(cu_q), _p(ctx_lens),
        c_int(n_seqs), c_int(total_tiles), _p(out), c_int(out.shape[1]), c_int(nq), c_int(nkv),
        c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), _p(status), c_int(count), _p(part_o),
        _p(part_ml), c_int(row0), c_int(rows), _stream()), "attn_tc")
    if count > 1:
        global LAUNCHES
        LAUNCHES += 1     # the kernel that joins the shares


USE_TC_SHARES = True       # short portions behind long contexts share their keys out over several blocks


def attn_tc_shares(total_tiles: int, nkv: int, max_key_tiles: int) -> int:
    """Over how many blocks a row tile's keys are shared out: 1 unless the row tiles alone would fill
    less than three quarters of the places (two per SM) and each would walk at least eight tiles of
    keys; then as many as fill the places once, each share at least four key tiles long, at most 8."""
    places = 2 * sm_count()
    units = total_tiles * nkv
    if not USE_TC_SHARES or units * 4 >= places * 3 or max_key_tiles < 8:
        return 1
    return max(1, min(8, places // units, max_key_tiles // 4))


def decode_splits(n_seqs: int, nkv: int, max_kv_len: int) -> int:
    """Ranges of keys per (sequence, kv head).  Three blocks of the decode kernel fit an SM: few
    sequences get as many ranges as fill those places once (at most 20), many sequences three.
    Measured on the 8B shape at context 2100 (ms per step, ranges): batch 1 3.29 (24), 4 3.51 (13),
    8 3.70 (6) against 3.83 (8), 16 4.18 (3) against 4.39 (8), 32 5.43 (3) against 5.70 (8),
    64 8.08 (3) against 8.34 (8)."""
    tiles = max(1, -(-max_kv_len // 64))
    places = 3 * sm_count()
    want = max(3, min(places // max(1, n_seqs * nkv), 20))
    return max(1, min(want, tiles, 64))


DECODE_BY_UNITS = True      # few sequences: ranges of keys shared out by length so that the blocks fill the SMs once
DECODE_MAX_RANGES = 64      # a sequence is cut into at most this many ranges (and a range holds 1.5 tiles of keys at least)


@functools.lru_cache(maxsize=None)
def _decode_places_per_kv_head(nkv: int, d: int) -> int:
    return sm_count() * int(_attn_lib(d).ff_attn_decode_blocks_per_sm()) // nkv


def lengths_differ_much(ctx_lens) -> bool:
    """True if the longest of these decoding sequences has a quarter more tiles of keys than the
    average: then a fixed number of ranges per sequence makes blocks of very different length, and
    the attention shares its blocks out by length instead (`decode_units`).  Also true for one or
    two sequences of 3000 tokens or more."""
    tiles = [c // 64 + 1 for c in ctx_lens]
    if len(tiles) <= 2:
        # one or two long sequences: the fixed 20 ranges leave two thirds of the SMs' places empty and every
        # block waits for its own tiles one after the other (batch 1 behind 32 000 tokens: 2.3 TB/s);
        # shared out by length a sequence gets as many ranges as there are places
        return bool(tiles) and max(tiles) >= 48
    return max(tiles) >= 4 and max(tiles) * len(tiles) >= 1.25 * sum(tiles)


BY_LENGTH_CALLS = 0         # how often the kernel that shares its blocks out by length was chosen


def decode_units(n_seqs: int, nkv: int, d: int, by_length: bool) -> int:
    """Blocks per kv head when the ranges of keys are shared out by length (as many as fill every
    SM's places once, at most `DECODE_MAX_RANGES` a sequence), or 0 for the fixed number of ranges
    of `decode_splits`.  Measured on the 8B shape, kernel and join alone, us: eight sequences of
    200 to 6000 tokens 18.6 against 31.4 (six ranges each); seven of 100 and one of 16000 28 against
    70; eight of 2100 17.7 against 17.2 (the share-out costs every block a scan of the lengths), so
    equal lengths keep the fixed ranges.  Each sequence should get two units at least."""
    if not (DECODE_BY_UNITS and by_length):
        return 0
    units = min(_decode_places_per_kv_head(nkv, d), n_seqs * DECODE_MAX_RANGES)
    return units if 2 * n_seqs <= units and n_seqs <= 128 else 0


def _decode_scratch(ws, n: int, nq: int, nkv: int, d: int, splits: int):
    """Scratch memory of the decode attention: partial outputs, their (max, sum) pairs and the
    number of ranges per sequence.  The extent never shrinks as the batch grows (captured graphs
    of every batch size share the buffers that the largest one sized)."""
    units = _decode_places_per_kv_head(nkv, d) if DECODE_BY_UNITS else 0
    cap = max(n * nq * splits, (nq // nkv) * _sm_target_ctas() + n * nq, nq * units * (units // 2))
    return (ws.get("attn.part_o", (cap * d,), torch.float32), ws.get("attn.part_ml", (cap * 2,), torch.float32),
            ws.get("attn.seq_ranges", (max(n, 128),), torch.int32))


def attn_decode_units(q, q_stride, pages, table, cu_q, ctx_lens, n_seqs, out, part_o, part_ml, seq_ranges,
                      nq, nkv, d, scale, window, units, max_ranges, heads=None, status=None) -> None:
    """Split-KV decode attention with `units` blocks per kv head shared out among the sequences
    in proportion to their lengths.  ``heads = (q_norm_w, k_norm_w, eps, cos_sin)``: q is the raw
    q|k|v projection and the kernel finishes the heads itself."""
    _need_cuda(q, pages, table, cu_q, ctx_lens, out, part_o, part_ml, seq_ranges)
    num_blocks, _, _, block_size, _ = pages.shape
    assert part_o.numel() >= n_seqs * nq * units * d and part_ml.numel() >= n_seqs * nq * units * 2
    qw, kw, eps, cos_sin = heads if heads is not None else (None, None, 0.0, None)
    _need_cuda(qw, kw, cos_sin, status)
    _check(_attn_lib(d).ff_attn_decode_units(
        _p(q), c_int(q_stride), _p(pages), _p(table), c_int(table.shape[1]), _p(cu_q), _p(ctx_lens),
        c_int(n_seqs), _p(out), c_int(out.shape[1]), _p(part_o), _p(part_ml), _p(seq_ranges), c_int(nq),
        c_int(nkv), c_int(block_size), c_int(num_blocks), c_float(scale), c_int(window), c_int(units),
        c_int(max_ranges), c_int(1 if heads is not None else 0), _p(qw), _p(kw), c_float(eps), _p(cos_sin),
        c_int(cos_sin.shape[0] if cos_sin is not None else 0), _p(status), _stream()), "attn_decode_units")
    global LAUNCHES, BY_LENGTH_CALLS
    BY_LENGTH_CALLS += 1
    if units > n_seqs and max_ranges > 1:
        LAUNCHES += 1     # the kernel that joins the ranges


def paged_attention(q: torch.Tensor, q_stride: int, pages: torch.Tensor, table: torch.Tensor, ctx,
                    out: torch.Tensor, nq: int, nkv: int, d: int, scale: float, window: int) -> None:
    """Attention of a step's tokens over the paged cache; picks the kernel: the
    tensor-core kernels for bfloat16 and head sizes in steps of 16, the plain
    kernel for 32-bit and every other head size up to 256."""
    if _ATTN_FORCE_SIMT or not mma_attention_supported(q.dtype, d):
        paged_attention_simt(q, q_stride, pages, table, ctx.token_seq, ctx.positions, out, nq, nkv, d,
                             scale, window, ctx.status)
        return
    G = nq // nkv
    n = ctx.num_seqs
    n_dec = ctx.num_decode_seqs if G <= 16 else 0      # these come first in the step's arrays
    if n_dec:
        # one-token sequences: split-KV kernel
        splits = decode_splits(n_dec, nkv, ctx.max_kv_len)
        units = decode_units(n_dec, nkv, d, ctx.ranges_by_length)
        part_o, part_ml, seq_ranges = _decode_scratch(ctx.workspace, n_dec, nq, nkv, d, splits)
        if units:
            attn_decode_units(q, q_stride, pages, table, ctx.cu_q, ctx.ctx_lens, n_dec, out, part_o, part_ml,
                              seq_ranges, nq, nkv, d, scale, window, units, DECODE_MAX_RANGES, status=ctx.status)
        else:
            attn_decode(q, q_stride, pages, table, ctx.cu_q, ctx.ctx_lens, n_dec, out, part_o, part_ml, nq, nkv,
                        d, scale, window, splits, ctx.status)
    if n_dec < n:
        # portions of prompts: tiled kernel over the remaining sequences (token offsets in cu_q are absolute)
        # every layer of a step asks the same of the step's arrays: worked out once and kept with the step
        memo = getattr(ctx, "memo", None)
        tail = memo.get(("attn_tail", id(table), n_dec)) if memo is not None else None
        if tail is None:
            tail = (table[n_dec:], ctx.cu_q[n_dec:], ctx.ctx_lens[n_dec:])
            if memo is not None:
                memo[("attn_tail", id(table), n_dec)] = tail
        table_t, cu_q_t, ctx_lens_t = tail
        if USE_TC_ATTENTION and tc_attention_supported(q.dtype, d, pages.shape[3], ctx.max_kv_len):
            plan = memo.get(("attn_tc_plan", G, nkv, n_dec, ctx.captured)) if memo is not None else None
            if plan is None:
                tiles = sum(-(-(ql * G) // 128) for ql in ctx.q_lens[n_dec:])
                # a captured step does not know its requests' lengths: the level it was captured for stands in
                key_tiles = 4 * getattr(ctx, "key_share_level", 0) if ctx.captured else \
                    max(-(-(c + ql) // 64) for c, ql in zip(ctx.ctx_lens_host[n_dec:], ctx.q_lens[n_dec:]))
                count = attn_tc_shares(tiles, nkv, key_tiles)
                plan = (tiles, count, sum(ctx.q_lens[:n_dec]), sum(ctx.q_lens[n_dec:]))
                if memo is not None:
                    memo[("attn_tc_plan", G, nkv, n_dec, ctx.captured)] = plan
            tiles, count, row0, rows = plan
            shares = None
            if count > 1:
                cells = (row0 + rows) * nq * count
                shares = (count, ctx.workspace.get("attn.tc_part_o", (cells * d,), torch.float32),
                          ctx.workspace.get("attn.tc_part_ml", (cells * 2,), torch.float32), row0, rows)
            attn_tc(q, q_stride, pages, table_t, cu_q_t, ctx_lens_t, n - n_dec, tiles,
                    out, nq, nkv, d, scale, window, ctx.status, shares=shares)
        else:
            tiles = sum(-(-(ql * G) // 64) for ql in ctx.q_lens[n_dec:])
            attn_tiled(q, q_stride, pages, table_t, cu_q_t, ctx_lens_t, n - n_dec,
                       tiles, out, nq, nkv, d, scale, window, ctx.status)
