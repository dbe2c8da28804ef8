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


class RMSNorm(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.size = int(self.p("size"))
        self.eps = float(self.p("eps"))
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name("weight"), (self.size,), init="norm")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = self._vector32(tensors[self.name("weight")])

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx, *,
                tag: str = "normed", row_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        rows = residual.shape[0] if row_idx is None else row_idx.numel()
        out = ctx.workspace.get(tag, (rows, self.size), ctx.dtype)
        K.add_rms_norm(residual, delta, self.weight, self.eps, out, row_idx)
        return out


register_part("norm", "rms_norm", RMSNorm)
