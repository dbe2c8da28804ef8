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
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear


class SwiGLUMLP(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.inter = int(self.p("intermediate_size"))
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name("gate_proj.weight"), (self.inter, self.hidden)),
                WeightSpec(self.name("up_proj.weight"), (self.inter, self.hidden)),
                WeightSpec(self.name("down_proj.weight"), (self.hidden, self.inter))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        g = self._matrix(tensors[self.name("gate_proj.weight")])
        u = self._matrix(tensors[self.name("up_proj.weight")])
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = self._matrix(tensors[self.name("down_proj.weight")])

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        T = x.shape[0]
        ws = ctx.workspace
        gu = ws.get("mlp.gate_up", (T, 2 * self.inter), ctx.dtype)
        apply_linear(x, self.w_gate_up, gu, ws, "mlp.gate_up")
        act = ws.get("mlp.act", (T, self.inter), ctx.dtype)
        K.silu_mul(gu, act)
        out = ws.get("mlp.down", (T, self.hidden), ctx.dtype)
        apply_linear(act, self.w_down, out, ws, "mlp.down")
        return out


register_part("feed_forward", "swiglu_mlp", SwiGLUMLP)
