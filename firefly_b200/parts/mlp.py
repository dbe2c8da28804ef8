"""SwiGLU feed-forward: (silu(x Wg^T) * (x Wu^T)) Wd^T, silu(g) = g / (1 + exp(-g))
in 32-bit (src/model/qwen_model.cu:164-174, src/kernels/activation.cu:15-19 of the
reference, which runs gate and up as two products and the activation as a third
launch).  Gate and up are one product against the stacked matrix [2I, H].

Parameters: hidden_size, intermediate_size.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..ops import kernels as K
from ..weights.arena import FusedSpec, Piece
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import linear_into_residual, linear_swiglu


class SwiGLUMLP(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    folds_next_norm = True           # forward(then_norm=...)
    accepts_folded_norm = True       # its first operation is a product that can finish a folded norm

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.inter = int(self.p("intermediate_size"))
        self.w_gate_up = self.w_down = None
        self.interleaved = False

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name("gate_proj.weight"), (self.inter, self.hidden)),
                WeightSpec(self.name("up_proj.weight"), (self.inter, self.hidden)),
                WeightSpec(self.name("down_proj.weight"), (self.hidden, self.inter))]

    def _interleaves(self, gate_dtype, up_dtype) -> bool:
        """bfloat16: rows of gate and up alternate in groups of 16, the layout the fused product's
        epilogue pairs up; else gate rows first, then up rows."""
        return gate_dtype == up_dtype == torch.bfloat16 and self.rt.dtype == torch.bfloat16 and self.inter % 16 == 0

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        g, u = self.name("gate_proj.weight"), self.name("up_proj.weight")
        if self._interleaves(dtype_of(g), dtype_of(u)):
            pieces = (Piece(g, 0, 16, 32), Piece(u, 16, 16, 32))
        else:
            pieces = (Piece(g, 0), Piece(u, self.inter))
        return [FusedSpec(self.name("gate_up_proj.weight"), (2 * self.inter, self.hidden), pieces)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        fused = self.name("gate_up_proj.weight")
        if fused in tensors:
            self.w_gate_up = self._matrix(tensors[fused])
            self.interleaved = self._interleaves(self.w_gate_up.dtype, self.w_gate_up.dtype)
        else:
            g = self._matrix(tensors[self.name("gate_proj.weight")])
            u = self._matrix(tensors[self.name("up_proj.weight")])
            if g.dtype != u.dtype:
                g, u = g.to(torch.float32), u.to(torch.float32)
            self.interleaved = self._interleaves(g.dtype, u.dtype)
            self.w_gate_up = K.interleave_gate_up(g, u) if self.interleaved else torch.cat([g, u], dim=0).contiguous()
        self.w_down = self._matrix(tensors[self.name("down_proj.weight")])

    def forward(self, x, ctx, accumulate_into=None, then_norm=None):
        """Returns the delta [T, hidden]; or None when it was added into ``accumulate_into`` (the
        32-bit residual) by the last product's epilogue; or a FoldedNorm when that epilogue also
        prepared the norm that follows (``then_norm``)."""
        act = linear_swiglu(x, self.w_gate_up, self.inter, self.interleaved, ctx)
        return linear_into_residual(act, self.w_down, accumulate_into, ctx, "mlp.down", then_norm)


register_part("feed_forward", "swiglu_mlp", SwiGLUMLP)
