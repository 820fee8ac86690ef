"""Token embedding (rows of the table into the float32 residual, no scaling:
``decoder.pas:3292-3309`` of the reference) and the head (logits = h · Headᵀ in float32, the
head being the embedding when tied: ``model.qwen3.pas:555-579``)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from .base import EMBEDDINGS, HEADS, Part, TensorNeed
from .linear import Linear


class TokenEmbedding(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.name = spec.params["name"]
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])

    def tensors(self) -> List[TensorNeed]:
        return [TensorNeed(self.name, (self.vocab, self.hidden), "table")]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.table = weights[self.name]

    def forward(self, ids: torch.Tensor, x: torch.Tensor) -> None:
        K.embed(self.table, ids, x)


class LmHead(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.tied = bool(p["tied"])
        self.name = p["tied_to"] if self.tied else p["name"]
        self.stored_name = p["name"]
        self.vocab, self.hidden = int(p["vocab_size"]), int(p["hidden_size"])

    def tensors(self) -> List[TensorNeed]:
        if self.tied:
            # a stored copy of a tied head is tolerated when it equals the embedding
            return [TensorNeed(self.stored_name, (self.vocab, self.hidden), "table", optional=True,
                               must_equal=self.name)]
        return [TensorNeed(self.name, (self.vocab, self.hidden), "matrix")]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.linear = Linear(weights[self.name], rt)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.linear(h, out_dtype=torch.float32)


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("lm_head", LmHead)
