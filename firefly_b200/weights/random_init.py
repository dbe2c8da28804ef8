"""Seeded random weights: on the device for benchmarks, or as a model folder.

Laws: matrices and embedding tables N(0, 0.02), norm weights 1 + N(0, 0.01).
Each tensor has a generator of its own, seeded from (seed, tensor name), so a
tensor's values do not depend on which other tensors exist or on their order.
The reference has no such mode; it only loads checkpoints.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterable

import torch

from ..config.base import ModelConfig
from .loader import WeightSpec, storage_dtype
from .safetensors_io import save_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def draw(spec: WeightSpec, seed: int, *, dtype: torch.dtype, device) -> torch.Tensor:
    """One tensor of ``spec``'s law, drawn in 32-bit and rounded once to ``dtype``."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(_seed_for(seed, spec.name))
    if spec.kind == "int":
        high = int(spec.init.split(":", 1)[1]) if spec.init.startswith("int:") else 2
        return torch.randint(0, high, spec.shape, generator=gen, device=dev, dtype=torch.int32)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=dev)
    if spec.init == "ones":
        return torch.ones(spec.shape, dtype=dtype, device=dev)
    numel = 1
    for s in spec.shape:
        numel *= s
    out = torch.empty(spec.shape, dtype=dtype, device=dev)
    flat = out.view(-1)
    # in pieces, so that a large matrix never needs a 32-bit copy of itself
    piece = 1 << 26
    for lo in range(0, numel, piece):
        n = min(piece, numel - lo)
        x = torch.randn(n, generator=gen, device=dev, dtype=torch.float32)
        if spec.init == "norm":
            x.mul_(0.01).add_(1.0)
        else:
            x.mul_(0.02)
        flat[lo:lo + n] = x.to(dtype)
    return out


def random_weights(expected: Iterable[WeightSpec], seed: int, *, dtype: torch.dtype,
                   device) -> Dict[str, torch.Tensor]:
    """All tensors of a model, drawn on ``device`` (no file involved)."""
    out = {}
    for w in expected:
        if w.optional:
            continue
        out[w.name] = draw(w, seed, dtype=storage_dtype(dtype, dtype) if w.kind == "float" else dtype,
                           device=device)
    return out


def write_random_model(config: ModelConfig, seed: int, out_dir: str, *,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded
    random weights stored as ``dtype``.  Returns ``out_dir``."""
    from ..models.decoder import expected_weights
    from ..models.registry import spec_for

    os.makedirs(out_dir, exist_ok=True)
    spec = spec_for(config)
    tensors = {}
    for w in expected_weights(spec):
        if w.optional:
            continue
        tensors[w.name] = draw(w, seed, dtype=dtype if w.kind == "float" else torch.int32, device="cpu")
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                          torch.float16: "float16"}.get(dtype, str(dtype))
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(raw, fh, indent=1)
    save_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                     metadata={"format": "pt", "seed": str(seed)})
    return out_dir
