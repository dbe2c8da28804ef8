"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, statistics in 32-bit, the weight a
plain multiplier (src/kernels/norm.cu:73-131 of the reference).  The residual add
that the reference does in a launch of its own (src/kernels/add.cu) is folded in:
the residual stream is 32-bit and the norm adds the pending delta on its way."""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..ops import kernels as K
from ..weights.loader import WeightSpec
from .base import Part, register_part


class FoldedNorm:
    """The output of an RMSNorm that was never materialised: the product in front of the norm
    left ``xw`` = bfloat16(residual * weight) and the per-tile sums of squares ``ssq`` [tiles, T];
    the product behind it multiplies its result by 1/rms per token (parts/linear.py).  A
    consumer that cannot do that calls ``materialize()``, which runs the norm kernel on the
    (already updated) residual."""

    def __init__(self, norm: "RMSNorm", residual: torch.Tensor, xw: torch.Tensor, ssq: torch.Tensor, ctx):
        self.norm, self.residual, self.xw, self.ssq, self.ctx = norm, residual, xw, ssq, ctx
        self.shape = xw.shape
        self.dtype = xw.dtype

    def materialize(self) -> torch.Tensor:
        out = self.ctx.workspace.get("normed", self.shape, self.ctx.dtype)
        K.add_rms_norm(self.residual, None, self.norm.weight, self.norm.eps, out, None)
        return out


class RMSNorm(Part):
    foldable = True                      # fold_buffers / size / eps: the products around it can take it in

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.size = int(self.p("size"))
        self.eps = float(self.p("eps"))
        self.weight: Optional[torch.Tensor] = None
        self.fold_tag = "fold.0"          # scratch of the folded form; a block gives its norms different tags

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name("weight"), (self.size,), init="norm", as_float32=True)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = self._vector32(tensors[self.name("weight")])

    def fold_buffers(self, T: int, ctx):
        """(xw [T, size] bfloat16, norm weight, ssq [tiles, T] float32) for a product that folds this
        norm into its residual-adding epilogue."""
        tiles = -(-self.size // 128)
        xw = ctx.workspace.get(self.fold_tag + ".xw", (T, self.size), torch.bfloat16)
        ssq = ctx.workspace.get(self.fold_tag + ".ssq", (tiles, T), torch.float32)
        return xw, self.weight, ssq

    def forward(self, residual: torch.Tensor, delta, ctx, *, tag: str = "normed",
                row_idx: Optional[torch.Tensor] = None, may_defer: bool = False):
        """Adds ``delta`` (a tensor, None, or a FoldedNorm: then the residual is already updated) into
        the residual and returns the normalised rows.  With ``may_defer`` a FoldedNorm made for this
        very norm is handed on as it is, for the consumer's first product to finish."""
        if isinstance(delta, FoldedNorm):
            if may_defer and delta.norm is self and row_idx is None:
                return delta
            delta = None
        rows = residual.shape[0] if row_idx is None else row_idx.numel()
        out = ctx.workspace.get(tag, (rows, self.size), ctx.dtype)
        K.add_rms_norm(residual, delta, self.weight, self.eps, out, row_idx)
        return out


register_part("norm", "rms_norm", RMSNorm)
