"""The generic decoder: builds any ``ModelSpec`` from registered parts and runs a
step's tokens through the schedule.

Nothing here is specific to an architecture: the layers, their parts and the
order of the runs are all data in the spec.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..config.base import ModelSpec
from ..parts import Runtime, build_part, part_class
from ..parts.base import declared, host_synchronous
from ..weights.loader import WeightSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.embedding = build_part("embedding", spec.embedding, rt)
        self.embedding_position = build_part("position", spec.embedding_position, rt) \
            if spec.embedding_position is not None else None
        self.blocks = [part_class("arrangement", ls.arrangement)(ls, rt) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, rt)
        self.head = build_part("head", spec.head, rt)
        self.schedule = spec.resolved_schedule()
        self._takes_next_norm = [declared(b, "takes_next_norm") for b in self.blocks]
        # a part that reads device values on the host keeps the whole model's steps out of CUDA graphs
        self.host_synchronous = any(host_synchronous(p) for p in (
            self.embedding, self.embedding_position, *self.blocks, self.final_norm, self.head) if p is not None)
        self.bound = False

    # -- weights ------------------------------------------------------------------
    def weight_specs(self) -> List[WeightSpec]:
        seen: Dict[str, WeightSpec] = {}
        parts = [self.embedding, *self.blocks, self.final_norm, self.head]
        if self.embedding_position is not None:
            parts.append(self.embedding_position)
        for p in parts:
            for w in p.weight_specs():
                if w.name in seen and seen[w.name].shape != w.shape:
                    raise ValueError(f"tensor '{w.name}' is declared twice with different shapes")
                seen.setdefault(w.name, w)
        return list(seen.values())

    def fused_specs(self, dtype_of) -> list:
        """The fused tensors the parts want (``Part.fused_layout``), each once."""
        parts = [self.embedding, *self.blocks, self.final_norm, self.head]
        if self.embedding_position is not None:
            parts.append(self.embedding_position)
        seen = {}
        for p in parts:
            for f in (p.fused_layout(dtype_of) if hasattr(p, "fused_layout") else ()):
                seen.setdefault(f.name, f)
        return list(seen.values())

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.embedding.bind(tensors)
        if self.embedding_position is not None:
            self.embedding_position.bind(tensors)
        for b in self.blocks:
            b.bind(tensors)
        self.final_norm.bind(tensors)
        self.head.bind(tensors)
        self.bound = True

    # -- caches ------------------------------------------------------------------
    def cache_slot_specs(self) -> Dict[int, object]:
        """What each written cache slot needs (slot id -> spec)."""
        out: Dict[int, object] = {}
        for layer, slot, write in self.schedule:
            if write:
                out[slot] = self.blocks[layer].cache_spec()
        for layer, slot, write in self.schedule:
            if not write:
                want = self.blocks[layer].cache_spec()
                if out.get(slot) != want:
                    raise ValueError(f"layer {layer} reads cache slot {slot}, whose shape "
                                     f"{out.get(slot)} is not what it needs ({want})")
        return out

    # -- run ------------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        """Logits float32 [len(ctx.logits_rows), vocab] for this step's tokens."""
        if not self.bound:
            raise RuntimeError("model has no weights bound")
        residual = self.embedding.forward(ctx)
        if self.embedding_position is not None:
            self.embedding_position.apply_to_embedding(residual, ctx)
        pending: Optional[torch.Tensor] = None
        runs = self.schedule
        for i, (layer, slot, write) in enumerate(runs):
            block = self.blocks[layer]
            # the norm that follows this run, for a last product that can fold it in
            nxt = self.blocks[runs[i + 1][0]] if i + 1 < len(runs) else None
            if self._takes_next_norm[layer]:
                next_norm = nxt.first_norm() if nxt is not None and hasattr(nxt, "first_norm") else None
                residual, pending = block.forward(residual, pending, ctx, slot, write, next_norm=next_norm)
            else:
                residual, pending = block.forward(residual, pending, ctx, slot, write)
        x = self.final_norm.forward(residual, pending, ctx, tag="final_normed", row_idx=ctx.logits_rows)
        return self.head.forward(x, ctx)


def expected_weights(spec: ModelSpec) -> List[WeightSpec]:
    """Tensor names and shapes of ``spec`` (no device needed)."""
    rt = Runtime(torch.device("cpu"), torch.float32)
    return DecoderModel(spec, rt).weight_specs()
