"""Token embedding and output head.

``x[t] = E[token[t]]`` widened to 32-bit, no scaling (cleanroom-transformer/src/cpu_backend.c:236);
``logit[v] = dot(h, W[v])`` with ``W = E`` when the embeddings are tied, else ``lm_head.weight``,
which carries no decoder prefix (model.c:399-406).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import EMBEDDINGS, HEADS, ParamSpec, Part


@EMBEDDINGS.register("embedding")
class TokenEmbedding(Part):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.weight = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec("weight", (self.vocab, self.hidden))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def share(self, stored) -> None:
        """Reads the table from ``stored`` from now on (the same values in the layout a tied head
        keeps them in), so that one copy serves both; the row-major copy is let go."""
        self.weight = stored

    def forward(self, tokens, out) -> None:
        self.ctx.ops.embed(tokens, self.weight, out)


@HEADS.register("lm_head")
class LMHead(Part):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied = bool(spec.get("tied", False))
        self.weight = None

    def params(self) -> List[ParamSpec]:
        # a tied checkpoint may still carry a copy of the head; it is then not read
        return [ParamSpec("weight", (self.vocab, self.hidden), absolute=True, optional=self.tied)]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = self.ctx.ops.pack_weight(tensors["weight"].contiguous())

    def tie(self, embedding_weight: torch.Tensor):
        """The head reads the embedding table; returns the form it keeps it in (tiles, where the
        tensor-core product can read them), which the embedding can gather from as well."""
        self.weight = self.ctx.ops.pack_weight(embedding_weight)
        return self.weight

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, hn, logits) -> None:
        """``logits[n, vocab]`` (32-bit) from normalised rows ``hn[n, hidden]``."""
        self.ctx.ops.linear(hn, self.weight, logits)
