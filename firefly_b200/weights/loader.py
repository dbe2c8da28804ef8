"""Binding weights by tensor name, with one error that says everything wrong.

A model states what it expects as a list of ``WeightSpec`` (full tensor name,
shape, kind).  ``load_weights`` reads the folder's safetensors, checks names and
shapes against that list and returns ``{name: tensor}`` on the device.

Storage policy.  16-bit floating tensors are kept in bfloat16 (a BF16 tensor is
copied bit for bit; the reference instead converts BF16 to FP16 element by
element on the host, include/firefly/model_loader.h:79-92).  A tensor stored in
32-bit floating point stays 32-bit (``weight_dtype="keep"``, the default: its
products then run in true 32-bit also inside a bfloat16 engine) or is narrowed
to the engine's type on the device (``weight_dtype="engine"``).  Integer tensors
of any width become int32.  With ``dtype=float32`` every floating tensor is
widened to 32-bit (exact).  Tensors that a part reads in 32-bit arithmetic
(norm weights) are declared ``as_float32`` and converted once, on the way in.

All tensors lie in one device arena (``weights/arena.py``) and are copied from a
pinned mapping of the file straight into their final places; tensors that parts
want fused (q|k|v, gate|up) exist only in their fused form.
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
    ``as_float32``  kept in 32-bit on the device whatever the file and the engine use.
    """

    name: str
    shape: Tuple[int, ...]
    kind: str = "float"
    init: str = "linear"
    optional: bool = False
    as_float32: bool = False


WEIGHT_DTYPES = ("keep", "engine")


def storage_dtype(stored: torch.dtype, mode: torch.dtype, weight_dtype: str = "keep") -> torch.dtype:
    """The dtype a stored tensor has on the device under engine dtype ``mode``."""
    if weight_dtype not in WEIGHT_DTYPES:
        raise ValueError(f"weight_dtype must be one of {WEIGHT_DTYPES}, got {weight_dtype!r}")
    if stored.is_floating_point:
        if mode == torch.float32:
            return torch.float32
        if stored in (torch.float32, torch.float64) and weight_dtype == "keep":
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


def read_weights(model_dir: str, expected: Iterable[WeightSpec], *, dtype: torch.dtype,
                 ignore: Iterable[str] = (), weight_dtype: str = "keep") -> Dict[str, torch.Tensor]:
    """The folder's tensors in host memory, checked and converted by the same rules as the device
    loader (for tools and tests; the engine itself loads through ``load_weights``)."""
    from .arena import FileSource
    expected = list(expected)
    source = FileSource(model_dir, register=False)
    try:
        check_and_collect(model_dir, source.available, expected, ignore)
        out: Dict[str, torch.Tensor] = {}
        for w in expected:
            if w.name in source.available:
                t = source.where[w.name].tensor(w.name)
                target = torch.float32 if (w.as_float32 and w.kind == "float") \
                    else storage_dtype(t.dtype, dtype, weight_dtype)
                out[w.name] = t.to(target).clone()
        return out
    finally:
        source.close()


def plan_arena(model, available: Dict[str, Tuple[Tuple[int, ...], torch.dtype]], *, dtype: torch.dtype,
               weight_dtype: str = "keep"):
    """The arena plan of ``model`` for tensors stored as ``available`` says, and the names to load."""
    from .arena import ArenaPlan
    sources = {}
    for w in model.weight_specs():
        if w.name not in available:
            continue
        _, stored = available[w.name]
        dev_dt = torch.float32 if (w.as_float32 and w.kind == "float") else storage_dtype(stored, dtype, weight_dtype)
        sources[w.name] = (tuple(w.shape), dev_dt)
    fused = model.fused_specs(lambda name: sources[name][1]) if hasattr(model, "fused_specs") else []
    fused = [f for f in fused if all(p.source in sources for p in f.pieces)]
    return ArenaPlan(sources, fused), list(sources)


def load_weights(model_dir: str, model, *, dtype: torch.dtype, device: torch.device | str,
                 ignore: Iterable[str] = (), weight_dtype: str = "keep", register: bool = True):
    """Check the folder's tensors against what ``model`` expects (one error for everything wrong),
    make the arena and fill it.  Returns (name -> tensor for ``model.bind``, the arena, load facts)."""
    from .arena import FileSource, WeightArena
    source = FileSource(model_dir, register=register)
    try:
        check_and_collect(model_dir, source.available, model.weight_specs(), ignore)
        plan, names = plan_arena(model, source.available, dtype=dtype, weight_dtype=weight_dtype)
        arena = WeightArena(plan, device)
        source.fill(arena, names)
        facts = {"arena_bytes": plan.total_bytes, "file_bytes": source.bytes_copied,
                 "pinned_files": source.pinned_files, "files": len(source.files)}
        return arena.tensors(), arena, facts
    finally:
        source.close()
