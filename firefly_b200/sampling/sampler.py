"""Turns a step's logits into next tokens on the device."""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..ops import kernels as K
from .params import SamplingParams


class Sampler:
    def __init__(self, device, max_rows: int = 256):
        self.device = torch.device(device)
        self._cap = 0
        self._grow(max_rows)

    def _grow(self, rows: int) -> None:
        if rows <= self._cap:
            return
        self._cap = rows
        self.out = torch.empty(rows, dtype=torch.int32, device=self.device)
        self.temp = torch.empty(rows, dtype=torch.float32, device=self.device)
        self.seeds = torch.empty(rows, dtype=torch.int64, device=self.device)
        self.counters = torch.empty(rows, dtype=torch.int64, device=self.device)
        self.h_temp = torch.empty(rows, dtype=torch.float32).pin_memory()
        self.h_seeds = torch.empty(rows, dtype=torch.int64).pin_memory()
        self.h_counters = torch.empty(rows, dtype=torch.int64).pin_memory()
        self.h_out = torch.empty(rows, dtype=torch.int32).pin_memory()

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               counters: Sequence[int]) -> List[int]:
        """One token per row of ``logits``; ``counters[r]`` is how many tokens row
        r's request has generated so far (it selects the random numbers)."""
        n = logits.shape[0]
        if n == 0:
            return []
        self._grow(n)
        out = self.out[:n]
        if all(p.temperature <= 0 for p in params):
            K.sample(logits, out)
        else:
            for i, (p, c) in enumerate(zip(params, counters)):
                self.h_temp[i] = p.temperature
                self.h_seeds[i] = p.seed
                self.h_counters[i] = c
            self.temp[:n].copy_(self.h_temp[:n], non_blocking=True)
            self.seeds[:n].copy_(self.h_seeds[:n], non_blocking=True)
            self.counters[:n].copy_(self.h_counters[:n], non_blocking=True)
            K.sample(logits, out, self.temp[:n], self.seeds[:n], self.counters[:n])
        self.h_out[:n].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.h_out[:n].tolist()
