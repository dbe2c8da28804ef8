"""Token embedding and output head.

Embedding: h[t,:] = E[id[t],:] (src/kernels/embedding.cu:19-37), written into the
32-bit residual stream.  The reference maps an id outside the vocabulary to row 0
without a word; here ids are checked on the host before a step and the kernel
raises a status flag should one slip through.

Head: logits = x W^T in 32-bit for the rows that are asked for
(src/model/qwen_model.cu:177-188 computes the last position only).  ``tied_to``
names the embedding tensor when the head shares it; the reference requires
``lm_head.weight`` (src/model/qwen_model.cu:92) and cannot run tied checkpoints.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..ops import kernels as K
from ..weights.loader import WeightSpec
from .base import Part, register_part
from .linear import apply_linear


class TokenEmbedding(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(self.p("vocab_size"))
        self.hidden = int(self.p("hidden_size"))
        self.table = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name("weight"), (self.vocab, self.hidden))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = self._matrix(tensors[self.name("weight")])

    def forward(self, ctx) -> torch.Tensor:
        out = ctx.workspace.get("residual", (ctx.num_tokens, self.hidden), torch.float32)
        K.embedding(ctx.token_ids, self.table, out, ctx.status)
        return out


class LMHead(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(self.p("vocab_size"))
        self.hidden = int(self.p("hidden_size"))
        self.tied_to = self.p("tied_to", None)
        self.weight = None

    def weight_specs(self) -> List[WeightSpec]:
        # a tied head has no tensor of its own; one stored anyway is ignored
        return [WeightSpec(self.name("weight"), (self.vocab, self.hidden),
                           optional=self.tied_to is not None)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        src = self.tied_to if self.tied_to is not None else self.name("weight")
        self.weight = self._matrix(tensors[src])

    def forward(self, x_rows: torch.Tensor, ctx) -> torch.Tensor:
        out = ctx.workspace.get("logits", (x_rows.shape[0], self.vocab), torch.float32)
        if x_rows.shape[0]:
            apply_linear(x_rows, self.weight, out, ctx, "logits")
        return out


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
