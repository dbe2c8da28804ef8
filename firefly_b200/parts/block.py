"""Arrangements: how a layer's parts are joined into a block.

``pre_norm`` is the reference's (src/model/qwen_model.cu:106-175):
    h += mixer(norm_0(h));  h += feed_forward(norm_1(h))
The residual stream ``h`` is 32-bit.  A part's output is not added at once: it is
handed on as ``pending`` and the next norm adds it while it reads the row, so
each sum is done once, in 32-bit, without a pass of its own.
"""
from __future__ import annotations

import inspect
from typing import List, Mapping

import torch

from ..weights.loader import WeightSpec
from .base import Part, Runtime, build_part, register_part


class Block:
    """Base of arrangements: owns the built parts of one layer."""

    n_norms = 2

    def __init__(self, layer_spec, rt: Runtime):
        self.layer_spec = layer_spec
        self.position = build_part("position", layer_spec.position, rt) \
            if layer_spec.position is not None else None
        self.mixer = build_part("mixer", layer_spec.mixer, rt, position=self.position)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, rt)
        if len(layer_spec.norms) != self.n_norms:
            raise ValueError(f"arrangement '{layer_spec.arrangement}' needs {self.n_norms} norms, "
                             f"got {len(layer_spec.norms)}")
        self.norms = [build_part("norm", n, rt) for n in layer_spec.norms]
        # a part whose forward takes ``accumulate_into`` may add its output into the 32-bit
        # residual itself (and return None); others return a delta
        self._mixer_fuses = "accumulate_into" in inspect.signature(self.mixer.forward).parameters
        self._ffn_fuses = "accumulate_into" in inspect.signature(self.feed_forward.forward).parameters
        # ... and, told which norm follows (``then_norm``), may fold that norm into its last product
        self._mixer_folds = "then_norm" in inspect.signature(self.mixer.forward).parameters
        self._ffn_folds = "then_norm" in inspect.signature(self.feed_forward.forward).parameters
        # a part that declares ``accepts_folded_norm`` may be handed a FoldedNorm as its input
        self._mixer_defers = bool(getattr(self.mixer, "accepts_folded_norm", False))
        self._ffn_defers = bool(getattr(self.feed_forward, "accepts_folded_norm", False))
        for k, nrm in enumerate(self.norms):
            if hasattr(nrm, "fold_tag"):
                nrm.fold_tag = f"fold.{k}"

    def parts(self) -> List[Part]:
        out = [self.mixer, self.feed_forward, *self.norms]
        if self.position is not None:
            out.append(self.position)
        return out

    def weight_specs(self) -> List[WeightSpec]:
        return [w for p in self.parts() for w in p.weight_specs()]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.bind(tensors)

    def cache_spec(self):
        return self.mixer.cache_spec()


class PreNormBlock(Block):
    def first_norm(self):
        """The norm a block in front of this one may fold into its last product."""
        return self.norms[0]

    def forward(self, residual: torch.Tensor, pending, ctx, slot: int, write_cache: bool, next_norm=None):
        x = self.norms[0].forward(residual, pending, ctx, may_defer=self._mixer_defers)
        kw = {}
        if self._mixer_fuses:
            kw["accumulate_into"] = residual
            if self._mixer_folds:
                kw["then_norm"] = self.norms[1]
        a = self.mixer.forward(x, ctx, slot, write_cache, **kw)
        x = self.norms[1].forward(residual, a, ctx, may_defer=self._ffn_defers)
        kw = {}
        if self._ffn_fuses:
            kw["accumulate_into"] = residual
            if self._ffn_folds:
                kw["then_norm"] = next_norm
        f = self.feed_forward.forward(x, ctx, **kw)
        return residual, f


register_part("arrangement", "pre_norm", PreNormBlock)
