"""Arrangements: how a layer's parts are joined into a block.

``pre_norm`` is the reference's (src/model/qwen_model.cu:106-175):
    h += mixer(norm_0(h));  h += feed_forward(norm_1(h))
The residual stream ``h`` is 32-bit.  A part's output is not added at once: it is
handed on as ``pending`` and the next norm adds it while it reads the row, so
each sum is done once, in 32-bit, without a pass of its own.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..weights.loader import WeightSpec
from .base import Part, Runtime, build_part, declared, register_part


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
        # the parts' declared abilities (parts/base.py), checked here against their signatures:
        # adding into the 32-bit residual themselves, folding the norm that follows into their last
        # product, taking a folded norm as input
        self._mixer_fuses = declared(self.mixer, "adds_into_residual")
        self._ffn_fuses = declared(self.feed_forward, "adds_into_residual")
        self._mixer_folds = declared(self.mixer, "folds_next_norm")
        self._ffn_folds = declared(self.feed_forward, "folds_next_norm")
        self._mixer_defers = declared(self.mixer, "accepts_folded_norm")
        self._ffn_defers = declared(self.feed_forward, "accepts_folded_norm")
        self._norm_folds = [declared(nrm, "foldable") for nrm in self.norms]
        for k, nrm in enumerate(self.norms):
            if self._norm_folds[k]:
                nrm.fold_tag = f"fold.{k}"      # scratch of the folded form, one per norm of the block

    def parts(self) -> List[Part]:
        out = [self.mixer, self.feed_forward, *self.norms]
        if self.position is not None:
            out.append(self.position)
        return out

    def weight_specs(self) -> List[WeightSpec]:
        return [w for p in self.parts() for w in p.weight_specs()]

    takes_next_norm = False      # an arrangement whose forward takes ``next_norm`` sets this

    def first_norm(self):
        """The norm a block in front of this one may fold into its last product (None: none)."""
        return None

    def fused_layout(self, dtype_of) -> list:
        # a part need not derive from ``Part``: one without the method wants nothing fused
        return [f for p in self.parts() if hasattr(p, "fused_layout") for f in p.fused_layout(dtype_of)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.bind(tensors)

    def cache_spec(self):
        return self.mixer.cache_spec()


class PreNormBlock(Block):
    takes_next_norm = True

    def first_norm(self):
        """The norm a block in front of this one may fold into its last product."""
        return self.norms[0]

    def parts(self) -> list:
        """The parts this block holds."""
        return [p for p in (self.mixer, self.feed_forward, *self.norms, getattr(self, "position", None)) if p is not None]

    def forward(self, residual: torch.Tensor, pending, ctx, slot: int, write_cache: bool, next_norm=None):
        # only a foldable norm knows ``may_defer`` (hand a folded norm on to a consumer that finishes it)
        defer0 = {"may_defer": True} if self._norm_folds[0] and self._mixer_defers else {}
        defer1 = {"may_defer": True} if self._norm_folds[1] and self._ffn_defers else {}
        x = self.norms[0].forward(residual, pending, ctx, **defer0)
        kw = {}
        if self._mixer_fuses:
            kw["accumulate_into"] = residual
            if self._mixer_folds:
                kw["then_norm"] = self.norms[1]
        a = self.mixer.forward(x, ctx, slot, write_cache, **kw)
        x = self.norms[1].forward(residual, a, ctx, **defer1)
        kw = {}
        if self._ffn_fuses:
            kw["accumulate_into"] = residual
            if self._ffn_folds:
                kw["then_norm"] = next_norm
        f = self.feed_forward.forward(x, ctx, **kw)
        return residual, f


register_part("arrangement", "pre_norm", PreNormBlock)
