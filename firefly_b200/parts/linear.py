"""Matrix products y = x W^T with the weight as stored ([out, in], row-major), and
the fused forms the layers use.

Two routes.  For few tokens (decode steps, short portions) bfloat16 products run
on this package's own tcgen05 kernel, whose epilogue can add into the 32-bit
residual or apply SiLU(gate)*up, so those steps need no further launch.  Larger
token counts, 32-bit weights and shapes the kernel does not take go to the
library routine (cuBLAS), followed by the separate kernels.  The product runs in
the weight's type: bfloat16 operands with 32-bit accumulation, or true 32-bit;
when a 32-bit weight meets 16-bit activations (a tensor stored in 32-bit inside a
bfloat16 engine) the activations are widened and the result narrowed again, so the
weight is never rounded.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import kernels as K



def tc_usable(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """True if one of the package's tcgen05 products takes this size: the one-block kernel up to
    `GEMM_TC_MAX_TOKENS` tokens, the two-SM kernel from there to `GEMM_PAIR_MAX_TOKENS`."""
    if not (K.USE_TCGEN05_GEMM and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and weight.shape[1] % 8 == 0):
        return False
    return x.shape[0] <= K.GEMM_TC_MAX_TOKENS or (K.USE_PAIR_GEMM and x.shape[0] <= K.GEMM_PAIR_MAX_TOKENS)


def _pair_ranges(T: int, N: int, Kd: int) -> int:
    """K ranges of the two-SM product.  A tile of 256 rows x up to 256 tokens is one pair of blocks; the
    K range is cut in two or three while that still leaves the blocks fewer than the SMs (clusters of
    four pack the GPU well, clusters of six only when they are few; clusters of eight were slower)."""
    tok, _ = K.gemm_pair_plan(T, N, Kd, 1)
    pairs = -(-N // 256) * -(-T // tok)
    sms = K.sm_count()
    kb = -(-Kd // 64)
    if 6 * pairs <= 0.7 * sms and kb >= 12:
        return 3
    if 4 * pairs <= sms and kb >= 8:
        return 2
    return 1


def _splits(N: int, Kd: int) -> int:
    """K ranges (blocks of a cluster) of a product with few row tiles.  About 1.3 blocks per SM
    measured best for the decode step (192 blocks on 148 SMs: 3.83 ms against 3.95 ms with one block
    per SM and 3.90 ms with more): half of each SM's shared memory stays free for the blocks of the
    product that follows, which request their first weight tiles while this one still runs, and the
    SMs that hold two blocks of this product make up for the ones that finish early."""
    tiles = -(-N // 128)
    kb = -(-Kd // 64)
    want = (13 * K.sm_count() + 5 * tiles) // (10 * tiles)       # round(1.3 * SMs / tiles)
    return max(1, min(want, 8, kb // 4))


def _resolve(x, weight):
    """A folded norm stays folded only if the product that consumes it can finish it."""
    from .norm import FoldedNorm
    if isinstance(x, FoldedNorm) and not tc_usable(x, weight):
        return x.materialize()
    return x


def _tc(x, weight, out, epilogue, ctx, norm_out=None) -> None:
    from .norm import FoldedNorm
    N, Kd = weight.shape
    kw = {}
    if isinstance(x, FoldedNorm):
        kw["norm_in"] = (x.ssq, x.norm.size, x.norm.eps)
        x = x.xw
    if x.shape[0] > K.GEMM_TC_MAX_TOKENS:
        K.gemm_pair(x, weight, out, epilogue, _pair_ranges(x.shape[0], N, Kd), ctx.status, norm_out=norm_out, **kw)
    else:
        K.gemm_tc(x, weight, out, epilogue, _splits(N, Kd), ctx.status, norm_out=norm_out, **kw)


def apply_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, ctx, tag: str) -> torch.Tensor:
    """out = x W^T (out in the activation type, or float32)."""
    ws = ctx.workspace
    x = _resolve(x, weight)
    if tc_usable(x, weight):
        _tc(x, weight, out, K.EPI_F32 if out.dtype == torch.float32 else K.EPI_BF16, ctx)
        return out
    if x.dtype == weight.dtype:
        K.linear(x, weight, out)
        return out
    if weight.dtype == torch.float32 and x.dtype == torch.bfloat16:
        x32 = ws.get(tag + ".x32", x.shape, torch.float32)
        K.cast(x, x32)
        if out.dtype == torch.float32:
            K.linear(x32, weight, out)
        else:
            y32 = ws.get(tag + ".y32", out.shape, torch.float32)
            K.linear(x32, weight, y32)
            K.cast(y32, out)
        return out
    if weight.dtype == torch.bfloat16 and x.dtype == torch.float32:
        raise K.KernelError("a 32-bit engine holds 32-bit matrices only")
    raise K.KernelError(f"linear: no product for {x.dtype} x {weight.dtype}")


def linear_into_residual(x: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor], ctx,
                         tag: str, then_norm=None):
    """The product as a delta for the residual stream.  When it can be fused it is
    added into ``residual`` (float32) in the product's epilogue; then None is
    returned, or, when the norm that follows is given as ``then_norm`` and can be
    folded, a FoldedNorm that the norm's consumer finishes.  Larger bfloat16 products
    let the library add into the residual (32-bit sum), None again.  Else the delta
    is returned for the next norm to add."""
    x = _resolve(x, weight)
    if residual is not None and tc_usable(x, weight):
        if then_norm is not None and K.FOLD_NORM and getattr(then_norm, "foldable", False) \
                and then_norm.size == weight.shape[0]:
            from .norm import FoldedNorm
            xw, nw, ssq = then_norm.fold_buffers(x.shape[0], ctx)
            _tc(x, weight, residual, K.EPI_RESIDUAL_ADD, ctx, norm_out=(xw, nw, ssq))
            return FoldedNorm(then_norm, residual, xw, ssq, ctx)
        _tc(x, weight, residual, K.EPI_RESIDUAL_ADD, ctx)
        return None
    if residual is not None and K.LIBRARY_ADDS_INTO_RESIDUAL and x.dtype == weight.dtype == torch.bfloat16 \
            and residual.dtype == torch.float32 and residual.is_contiguous():
        K.linear_add(x, weight, residual)
        return None
    out = ctx.workspace.get(tag, (x.shape[0], weight.shape[0]), ctx.dtype)
    return apply_linear(x, weight, out, ctx, tag)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, inter: int, interleaved: bool, ctx) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for the stacked weight [2I, H] (``interleaved``: gate
    and up rows alternate in groups of 16)."""
    ws = ctx.workspace
    x = _resolve(x, w_gate_up)
    if not interleaved and not isinstance(x, torch.Tensor):
        x = x.materialize()
    T = x.shape[0]
    act = ws.get("mlp.act", (T, inter), ctx.dtype)
    if interleaved and tc_usable(x, w_gate_up):
        _tc(x, w_gate_up, act, K.EPI_SWIGLU, ctx)
        return act
    gu = ws.get("mlp.gate_up", (T, 2 * inter), ctx.dtype)
    apply_linear(x, w_gate_up, gu, ctx, "mlp.gate_up")
    K.silu_mul(gu, act, interleaved)
    return act
