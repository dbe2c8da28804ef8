"""Seeded random weights: on the device for benchmarks, or as a model folder.

Laws: matrices and embedding tables N(0, 0.02), norm weights 1 + N(0, 0.01).  The generator is
counter-based: an element's value depends only on (seed, its tensor's name, its index in that
tensor), so it does not depend on which other tensors exist, on their order, on how tensors are
fused on the device, or on where it is computed.  ``draw_cpu`` here and the kernel in
``csrc/weights.cu`` produce the same bits: both use 64-bit integer arithmetic up to a
fixed-point normal deviate (a table of 65537 quantiles of N(0,1), linear interpolation between
knots) and then one correctly rounded conversion, product and sum in 32-bit floating point.
The reference has no such mode; it only loads checkpoints.
"""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

from ..config.base import ModelConfig
from .loader import WeightSpec
from .safetensors_io import save_safetensors

_GOLDEN = 0x9E3779B97F4A7C15
_MASK = (1 << 64) - 1
FIXED_ONE = 1 << 24            # the table holds quantiles in units of 2^-24


def _mix64_int(z: int) -> int:
    z = (z + _GOLDEN) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def _mix64(z: np.ndarray) -> np.ndarray:
    """The splitmix64 finaliser of csrc/common.cuh on uint64 arrays (wrapping arithmetic)."""
    z = z + np.uint64(_GOLDEN)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def tensor_key(seed: int, name: str) -> int:
    """64-bit key of a tensor: the seed mixed with an FNV-1a hash of the name."""
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _MASK
    return _mix64_int((int(seed) & _MASK) ^ h)


@functools.lru_cache(maxsize=1)
def normal_table() -> torch.Tensor:
    """int32 [65537]: round(2^24 * Phi^-1(i / 65536)), the ends clamped to +-Phi^-1(2^-17)."""
    p = torch.arange(65537, dtype=torch.float64) / 65536.0
    p = p.clamp(2.0 ** -17, 1.0 - 2.0 ** -17)
    q = torch.special.ndtri(p) * FIXED_ONE
    # make the table exactly antisymmetric, so that it does not depend on the library's last bit
    q = (q - q.flip(0)) / 2
    return torch.round(q).to(torch.int32)


def law(spec: WeightSpec) -> Tuple[float, float]:
    """(scale, shift) of ``spec``'s law as 32-bit floats; the scale is in units of the table."""
    if spec.init == "norm":
        std, mean = 0.01, 1.0
    elif spec.init == "zeros":
        std, mean = 0.0, 0.0
    elif spec.init == "ones":
        std, mean = 0.0, 1.0
    else:
        std, mean = 0.02, 0.0
    return float(np.float32(std / FIXED_ONE)), float(np.float32(mean))


def int_high(spec: WeightSpec) -> int:
    return int(spec.init.split(":", 1)[1]) if spec.init.startswith("int:") else 2


def draw_cpu(spec: WeightSpec, seed: int, *, dtype: torch.dtype) -> torch.Tensor:
    """One tensor of ``spec``'s law on the CPU, the same bits as the device kernel gives."""
    numel = 1
    for s in spec.shape:
        numel *= s
    key = np.uint64(tensor_key(seed, spec.name))
    if spec.kind == "int":
        out = np.empty(numel, dtype=np.int32)
    else:
        out = np.empty(numel, dtype=np.float32)
        scale, shift = (np.float32(v) for v in law(spec))
        table = normal_table().numpy().astype(np.int64)
    piece = 1 << 22
    with np.errstate(over="ignore"):
        for lo in range(0, numel, piece):
            idx = np.arange(lo, min(lo + piece, numel), dtype=np.uint64)
            h = _mix64(key + idx * np.uint64(_GOLDEN))
            if spec.kind == "int":
                out[lo: lo + idx.size] = (h % np.uint64(int_high(spec))).astype(np.int32)
                continue
            u = (h >> np.uint64(32)).astype(np.int64)
            knot, frac = u >> 16, u & 0xFFFF
            t0, t1 = table[knot], table[knot + 1]
            fixed = t0 + (((t1 - t0) * frac) >> 16)
            out[lo: lo + idx.size] = fixed.astype(np.float32) * scale + shift
    t = torch.from_numpy(out).view(spec.shape if spec.shape else ())
    return t if spec.kind == "int" else t.to(dtype)


def random_weights_cpu(expected: Iterable[WeightSpec], seed: int, *, dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    """All tensors of a model on the CPU, floating ones rounded once to ``dtype``."""
    return {w.name: draw_cpu(w, seed, dtype=dtype) for w in expected if not w.optional}


def write_random_model(config: ModelConfig, seed: int, out_dir: str, *,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded
    random weights stored as ``dtype``.  Returns ``out_dir``."""
    from ..models.decoder import expected_weights
    from ..models.registry import spec_for

    os.makedirs(out_dir, exist_ok=True)
    tensors = random_weights_cpu(expected_weights(spec_for(config)), seed, dtype=dtype)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                          torch.float16: "float16"}.get(dtype, str(dtype))
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(raw, fh, indent=1)
    save_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                     metadata={"format": "pt", "seed": str(seed)})
    return out_dir
