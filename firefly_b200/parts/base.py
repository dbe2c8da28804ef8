"""Interfaces of the parts a model is put together from, and their registry.

A *part* knows its own sizes and constants (they arrive as parameters), the
names and shapes of its tensors, and how to run on a step's tokens.  It does not
know which model it is in, which layer it is, or what the other parts are.

Categories and what each must offer (beyond ``weight_specs`` and ``bind``):

* ``norm``          ``forward(residual, delta, out_rows=None) -> normed``:
                    adds ``delta`` (may be None) into the 32-bit residual and
                    returns the normalised rows in the activation type.
* ``position``      ``rotary_table()`` -> (cos/sin table [P, r/2, 2] float32,
                    rotary_dim) or None, and ``apply_to_embedding(h, ctx)``
                    (default: nothing) for encodings added to the embedding.
* ``mixer``         ``cache_spec()`` -> PagedKVSpec | StateSpec | None and
                    ``forward(x, ctx, slot, write_cache) -> delta`` [T, hidden].
* ``feed_forward``  ``forward(x, ctx) -> delta`` [T, hidden].
* ``arrangement``   built from a layer's parts;
                    ``forward(residual, pending, ctx, slot, write_cache)``
                    -> (residual, pending): ``pending`` is a delta that has not
                    been added to the residual yet (the next norm folds it in).
* ``embedding``     ``forward(ctx) -> residual`` float32 [T, hidden].
* ``head``          ``forward(x_rows) -> logits`` float32 [rows, vocab].

Registering a new kind: ``register_part("mixer", "my_mixer", MyMixer)``; a
``PartSpec("my_mixer", {...})`` in a layer then builds it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping

import torch

from ..config.base import ConfigError, PartSpec
from ..weights.loader import WeightSpec

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "arrangement", "embedding", "head")
_REGISTRY: Dict[str, Dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: type, *, replace: bool = False) -> None:
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category '{category}'; one of {CATEGORIES}")
    if kind in _REGISTRY[category] and not replace:
        raise ValueError(f"{category} '{kind}' is already registered")
    _REGISTRY[category][kind] = cls


def part_class(category: str, kind: str) -> type:
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        raise ConfigError(f"unknown {category} '{kind}'; known: "
                          f"{', '.join(sorted(_REGISTRY.get(category, {}))) or '(none)'}") from None


@dataclass
class Runtime:
    """The surroundings a part may use: where it runs and in which type."""

    device: torch.device
    dtype: torch.dtype                      # activation / matrix type: bfloat16 or float32
    shared: Dict[Any, Any] = field(default_factory=dict)   # tables shared between equal parts


def build_part(category: str, spec: PartSpec, rt: Runtime, **extra):
    return part_class(category, spec.kind)(spec, rt, **extra)


class Part:
    """Base: parameters from the spec, tensors bound by full name."""

    def __init__(self, spec: PartSpec, rt: Runtime):
        self.spec = spec
        self.params = dict(spec.params)
        self.prefix = spec.prefix
        self.rt = rt

    def p(self, key: str, default=...):
        if key in self.params:
            return self.params[key]
        if default is ...:
            raise ConfigError(f"part '{self.spec.kind}' ({self.prefix}) needs parameter '{key}'")
        return default

    def name(self, leaf: str) -> str:
        return f"{self.prefix}.{leaf}" if self.prefix else leaf

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        pass

    # helpers ---------------------------------------------------------------
    def _matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A matrix operand in the type its product runs in.  Matrices stored in
        16-bit run in bfloat16; a matrix stored in 32-bit stays 32-bit and its
        product runs in true 32-bit, also inside a bfloat16 engine."""
        if self.rt.dtype == torch.float32:
            return t.to(torch.float32).contiguous()
        return t.contiguous()

    @staticmethod
    def _vector32(t: torch.Tensor) -> torch.Tensor:
        return t.to(torch.float32).contiguous()
