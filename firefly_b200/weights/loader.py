"""Binding weights by tensor name, with one error that says everything wrong.

A model states what it expects as a list of ``WeightSpec`` (full tensor name,
shape, kind).  ``load_weights`` reads the folder's safetensors, checks names and
shapes against that list and returns ``{name: tensor}`` on the device.

Storage policy.  16-bit floating tensors are kept in bfloat16 (a BF16 tensor is
copied bit for bit; the reference instead converts BF16 to FP16 element by
element on the host, include/firefly/model_loader.h:79-92).  A tensor stored in
32-bit floating point stays 32-bit.  Integer tensors of any width become int32.
With ``dtype=float32`` every floating tensor is widened to 32-bit (exact).
The reference binds with ``unordered_map::at`` (src/model/qwen_model.cu:58-92),
so a missing tensor surfaces as a bare ``std::out_of_range``; here all missing,
unexpected and mis-shaped tensors are listed in one ``WeightError``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsError, open_model_files


class WeightError(ValueError):
    """Names every missing, unexpected and wrongly shaped tensor at once."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_kind: Sequence[Tuple[str, str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)
        lines = [f"weights in '{where}' do not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file has {list(got)}, model needs {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_kind:
            lines.append(f"  wrong element kinds ({len(self.wrong_kind)}): " + "; ".join(
                f"{n}: file has {got}, model needs {want}" for n, got, want in self.wrong_kind))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part expects.

    ``kind``  "float" or "int".
    ``init``  how the random-weights mode draws it: "linear" (N(0, 0.02)),
              "norm" (1 + N(0, 0.01)), "zeros", "ones", or "int:<high>" for a
              table of integers in [0, high).
    ``optional``  may be absent from the file (e.g. a tied head stored anyway).
    """

    name: str
    shape: Tuple[int, ...]
    kind: str = "float"
    init: str = "linear"
    optional: bool = False


def storage_dtype(stored: torch.dtype, mode: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor has on the device under engine dtype ``mode``."""
    if stored.is_floating_point:
        if mode == torch.float32:
            return torch.float32
        if stored in (torch.float32, torch.float64):
            return torch.float32
        return torch.bfloat16
    return torch.int32


def check_and_collect(where: str, available: Dict[str, Tuple[Tuple[int, ...], torch.dtype]],
                      expected: Iterable[WeightSpec], ignore: Iterable[str] = ()) -> None:
    expected = list(expected)
    names = {w.name for w in expected}
    ignore = set(ignore)
    missing = [w.name for w in expected if w.name not in available and not w.optional]
    unexpected = sorted(n for n in available if n not in names and n not in ignore)
    wrong_shape, wrong_kind = [], []
    for w in expected:
        if w.name in available:
            shape, dt = available[w.name]
            if tuple(shape) != tuple(w.shape):
                wrong_shape.append((w.name, tuple(shape), tuple(w.shape)))
            got_kind = "float" if dt.is_floating_point else "int"
            if got_kind != w.kind:
                wrong_kind.append((w.name, got_kind, w.kind))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightError(where, missing, unexpected, wrong_shape, wrong_kind)


def load_weights(model_dir: str, expected: Iterable[WeightSpec], *, dtype: torch.dtype,
                 device: torch.device | str, ignore: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    expected = list(expected)
    files = open_model_files(model_dir)
    try:
        where: Dict[str, object] = {}
        available: Dict[str, Tuple[Tuple[int, ...], torch.dtype]] = {}
        for f in files:
            for name, ent in f.entries.items():
                if name in available:
                    raise SafetensorsError(f"tensor '{name}' appears in more than one shard")
                available[name] = (ent.shape, ent.dtype)
                where[name] = f
        check_and_collect(model_dir, available, expected, ignore)
        out: Dict[str, torch.Tensor] = {}
        for w in expected:
            if w.name not in available:
                continue
            t = where[w.name].tensor(w.name)
            target = storage_dtype(t.dtype, dtype)
            # one copy to the device in the stored dtype, conversion there
            if t.dtype == torch.float64:
                t = t.to(torch.float32)
            if not t.dtype.is_floating_point and t.dtype != torch.int32:
                t = t.to(torch.int32)
            out[w.name] = t.to(device=device).to(target).contiguous()
        return out
    finally:
        for f in files:
            f.close()
