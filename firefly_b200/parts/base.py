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

Optional abilities are *declared* as class attributes and checked when a block or a model is
built (``declared``): a flag without its keyword, or a keyword without its flag, is an error then,
not a fusion that is silently lost.

=====================  ==========================  ==============================================
flag (class attribute)  keyword / method it needs   meaning
=====================  ==========================  ==============================================
adds_into_residual      forward(accumulate_into=)   mixer / feed_forward may add its output into the
                                                    32-bit residual itself and return None
folds_next_norm         forward(then_norm=)         ... and, told which norm follows, may leave that
                                                    norm folded (a ``FoldedNorm``) for its consumer
accepts_folded_norm     (none)                      its first operation can finish a ``FoldedNorm``
takes_next_norm         forward(next_norm=)         arrangement: hands the next block's first norm
                                                    to its last part
foldable                fold_buffers, size, eps     norm: can be folded into the products around it
host_synchronous        (none)                      any part: its forward() reads device values on the
                                                    host (``.item()``, ``bool(t.any())``, shapes that
                                                    depend on data), so the steps of a model that holds
                                                    it cannot be captured into CUDA graphs and run
                                                    launch by launch
=====================  ==========================  ==============================================
A part that declares nothing simply runs unfused; it need not derive from ``Part``.  A part that
holds other parts (an arrangement) lists them in ``parts()``.
"""
from __future__ import annotations

import inspect
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


_FLAG_KEYWORD = {"adds_into_residual": "accumulate_into", "folds_next_norm": "then_norm",
                 "takes_next_norm": "next_norm"}
_FLAG_MEMBERS = {"foldable": ("fold_buffers", "size", "eps")}


def declared(part, flag: str) -> bool:
    """Does ``part`` declare the optional ability ``flag``?  Checks the declaration against what the
    part really offers, both ways, and raises ``ConfigError`` when they disagree."""
    has = bool(getattr(part, flag, False))
    who = type(part).__name__
    kw = _FLAG_KEYWORD.get(flag)
    if kw is not None:
        takes = kw in inspect.signature(part.forward).parameters
        if has and not takes:
            raise ConfigError(f"{who} declares {flag} = True but its forward() has no '{kw}' keyword")
        if takes and not has:
            raise ConfigError(f"{who}.forward() takes '{kw}' but the class does not declare {flag} = True")
    for member in _FLAG_MEMBERS.get(flag, ()):
        if has and not hasattr(part, member):
            raise ConfigError(f"{who} declares {flag} = True but has no '{member}'")
    if flag == "folds_next_norm" and has and not getattr(part, "adds_into_residual", False):
        raise ConfigError(f"{who} declares folds_next_norm without adds_into_residual")
    return has


def host_synchronous(part) -> bool:
    """True if ``part`` or a part it holds (``parts()``) declares that it synchronises with the host."""
    if bool(getattr(part, "host_synchronous", False)):
        return True
    inner = getattr(part, "parts", None)
    return any(host_synchronous(p) for p in inner()) if callable(inner) else False


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

    # optional abilities (see the module's table); a subclass that has one sets it to True
    adds_into_residual = False
    folds_next_norm = False
    accepts_folded_norm = False
    foldable = False

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

    def fused_layout(self, dtype_of) -> list:
        """Tensors this part wants put together from several of its source tensors when the weights
        are loaded: a list of ``weights.arena.FusedSpec``.  ``dtype_of(source name)`` is the element
        type that source will have on the device.  The loader then keeps only the fused tensor and
        hands it to ``bind`` under its name; a part must still be able to bind from the plain
        sources (tensors made by hand)."""
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
