"""Grouped-query attention over the paged cache.

Order of operations as in the reference's layer (src/model/qwen_model.cu:113-160):
q, k, v projections; RMSNorm of each q and k head over its ``head_dim`` elements
(weight [head_dim] shared by the heads, before the rotation, :124-128); rotary
encoding of q and k at the tokens' absolute positions (:136); k and v into the
cache (:139-143); attention with scale 1/sqrt(head_dim) where q head h reads kv
head h // (num_heads/num_kv_heads) (src/kernels/attention.cu:44,304,458);
output projection.  The three projections are one product against the
concatenated matrix; norm, rotation and cache write are one kernel.

Unlike the reference, whose prefill attends only inside the portion it is given
(src/model/qwen_model.cu:147-151), every query attends the cache from position 0
(or the start of its window) to itself, so a prompt may be cut anywhere.

Parameters: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm (bool),
qk_norm_eps, window (None = all keys, W = the last W keys including the query's
own), scale (None = 1/sqrt(head_dim)), has_kv (False: the layer has no k/v
projections and only ever reads another run's cache), cache_block_size (tokens per
cache page if this layer wants a page size of its own; None: the engine's).
"""
from __future__ import annotations

import math
from typing import List, Mapping

import torch

from ..cache.spec import PagedKVSpec
from ..ops import kernels as K
from ..weights.arena import FusedSpec, Piece
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear, linear_into_residual


class GQAttention(Part):
    adds_into_residual = True        # forward(accumulate_into=...)
    folds_next_norm = True           # forward(then_norm=...)
    accepts_folded_norm = True       # its first operation is a product that can finish a folded norm

    def __init__(self, spec, rt, position=None):
        super().__init__(spec, rt)
        self.hidden = int(self.p("hidden_size"))
        self.nq = int(self.p("num_heads"))
        self.nkv = int(self.p("num_kv_heads"))
        self.d = int(self.p("head_dim"))
        self.qk_norm = bool(self.p("qk_norm", False))
        self.eps = float(self.p("qk_norm_eps", 1e-6))
        self.window = self.p("window", None)
        scale = self.p("scale", None)
        self.scale = 1.0 / math.sqrt(self.d) if scale is None else float(scale)
        self.has_kv = bool(self.p("has_kv", True))
        self.cache_block_size = self.p("cache_block_size", None)
        self.position = position
        if self.nq % self.nkv:
            raise ValueError(f"num_heads {self.nq} is not a multiple of num_kv_heads {self.nkv}")
        if self.d > 256:
            raise ValueError(f"head_dim {self.d} > 256 is not supported by the attention kernels")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("window must be positive")
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    # -- cache ------------------------------------------------------------------
    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.d, None if self.window is None else int(self.window),
                           None if self.cache_block_size is None else int(self.cache_block_size))

    # -- weights ------------------------------------------------------------------
    def weight_specs(self) -> List[WeightSpec]:
        out = [WeightSpec(self.name("q_proj.weight"), (self.nq * self.d, self.hidden))]
        if self.has_kv:
            out += [WeightSpec(self.name("k_proj.weight"), (self.nkv * self.d, self.hidden)),
                    WeightSpec(self.name("v_proj.weight"), (self.nkv * self.d, self.hidden))]
        out.append(WeightSpec(self.name("o_proj.weight"), (self.hidden, self.nq * self.d)))
        if self.qk_norm:
            out.append(WeightSpec(self.name("q_norm.weight"), (self.d,), init="norm", as_float32=True))
            if self.has_kv:
                out.append(WeightSpec(self.name("k_norm.weight"), (self.d,), init="norm", as_float32=True))
        return out

    def fused_layout(self, dtype_of) -> List[FusedSpec]:
        """q, k and v stacked into one matrix [(nq + 2 nkv) d, hidden], the three projections' rows
        in this order."""
        if not self.has_kv:
            return []
        q_rows, kv_rows = self.nq * self.d, self.nkv * self.d
        return [FusedSpec(self.name("qkv_proj.weight"), (q_rows + 2 * kv_rows, self.hidden),
                          (Piece(self.name("q_proj.weight"), 0), Piece(self.name("k_proj.weight"), q_rows),
                           Piece(self.name("v_proj.weight"), q_rows + kv_rows)))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        fused = self.name("qkv_proj.weight")
        if fused in tensors:
            self.w_qkv = self._matrix(tensors[fused])
        else:
            mats = [self._matrix(tensors[self.name("q_proj.weight")])]
            if self.has_kv:
                mats += [self._matrix(tensors[self.name("k_proj.weight")]),
                         self._matrix(tensors[self.name("v_proj.weight")])]
            if len({m.dtype for m in mats}) != 1:
                mats = [m.to(torch.float32) for m in mats]
            self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.w_o = self._matrix(tensors[self.name("o_proj.weight")])
        if self.qk_norm:
            self.q_norm_w = self._vector32(tensors[self.name("q_norm.weight")])
            if self.has_kv:
                self.k_norm_w = self._vector32(tensors[self.name("k_norm.weight")])

    # -- run ------------------------------------------------------------------
    def forward(self, x, ctx, slot: int, write_cache: bool, accumulate_into=None, then_norm=None):
        T = x.shape[0]
        ws = ctx.workspace
        if write_cache and not self.has_kv:
            raise RuntimeError(f"{self.prefix}: a layer without k/v projections cannot write a cache")
        nkv_w = self.nkv if write_cache else 0
        width = (self.nq + 2 * nkv_w) * self.d
        w = self.w_qkv if (write_cache or not self.has_kv) else self.w_qkv[: self.nq * self.d]
        qkv = ws.get("attn.qkv", (T, width), ctx.dtype)
        apply_linear(x, w, qkv, ctx, "attn.qkv")
        pages, table = ctx.kv(slot)
        rot = self.position.rotary_table() if self.position is not None else None
        cos_sin, rotary_dim = rot if rot is not None else (None, 0)
        att = ws.get("attn.out", (T, self.nq * self.d), ctx.dtype)
        if write_cache and K.decode_finishes_heads(ctx, ctx.dtype, self.nq, self.nkv, self.d, rotary_dim):
            # a step of single tokens: the attention kernel finishes the heads itself
            K.attn_decode_heads(qkv, pages, table, ctx, att, self.nq, self.nkv, self.d, self.scale,
                                0 if self.window is None else int(self.window), self.q_norm_w,
                                self.k_norm_w, self.eps, cos_sin)
        else:
            K.qk_norm_rope_store(qkv, self.nq, nkv_w, self.d, self.q_norm_w,
                                 self.k_norm_w if write_cache else None, self.eps, cos_sin, rotary_dim,
                                 ctx.positions, ctx.token_seq, table if write_cache else None,
                                 pages if write_cache else None, ctx.status)
            self._attend(qkv, width, pages, table, ctx, att)
        return linear_into_residual(att, self.w_o, accumulate_into, ctx, "attn.proj", then_norm)

    def _attend(self, qkv, width, pages, table, ctx, att) -> None:
        window = 0 if self.window is None else int(self.window)
        K.paged_attention(qkv, width, pages, table, ctx, att, self.nq, self.nkv, self.d, self.scale,
                          window)


register_part("mixer", "gqa_attention", GQAttention)
