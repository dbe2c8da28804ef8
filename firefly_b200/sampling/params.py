"""Per-request sampling options."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    """``temperature`` 0 means greedy (arg-max, the reference's only mode,
    src/kernels/sampling.cu:12-44); > 0 draws from softmax(logits / temperature)
    with random numbers fixed by ``seed`` and the number of tokens generated so
    far.  ``max_tokens`` defaults to the reference's 512 (src/server.cu:189)."""

    temperature: float = 0.0
    seed: int = 0
    max_tokens: int = 512
    ignore_eos: bool = False

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
