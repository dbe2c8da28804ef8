"""A matrix product y = x W^T with the weight as stored ([out, in], row-major).

The product runs in the weight's type: bfloat16 operands with 32-bit
accumulation, or true 32-bit.  When a 32-bit weight meets 16-bit activations
(a tensor stored in 32-bit inside a bfloat16 engine) the activations are widened
and the result narrowed again, so the weight is never rounded.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K


def apply_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, ws, tag: str) -> torch.Tensor:
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
