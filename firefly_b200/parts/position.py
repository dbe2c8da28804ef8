"""Position encodings.

``rotary``: rotate-half rotary encoding, f_i = theta^(-2i/r) for i in [0, r/2),
angle = position * f_i, pairs (i, i + r/2) of the first ``rotary_dim`` = r
elements of a head (the reference rotates the whole head: src/kernels/rope.cu:68-95).
The reference evaluates powf/cosf/sinf per element under --use_fast_math; here
cosines and sines come from a table computed once on the host in double
precision and stored in 32-bit, one row per position up to ``max_positions``.

``none``: no position information (a mixer that needs none).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import Part, register_part


class PositionEncoding(Part):
    def rotary_table(self) -> Optional[Tuple[torch.Tensor, int]]:
        return None

    def apply_to_embedding(self, h: torch.Tensor, ctx) -> None:
        return None


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.head_dim = int(self.p("head_dim"))
        self.rotary_dim = int(self.p("rotary_dim", self.head_dim))
        self.theta = float(self.p("theta"))
        self.max_positions = int(self.p("max_positions"))
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within the head "
                             f"({self.head_dim})")

    def rotary_table(self):
        key = ("rotary", self.rotary_dim, self.theta, self.max_positions)
        table = self.rt.shared.get(key)
        if table is None:
            half = self.rotary_dim // 2
            i = torch.arange(half, dtype=torch.float64)
            freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rotary_dim)
            ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * freq[None, :]
            table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32)
            table = table.contiguous().to(self.rt.device)
            self.rt.shared[key] = table
        return table, self.rotary_dim


class NoPosition(PositionEncoding):
    pass


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPosition)
