"""Token embedding and output head.

Embedding: ``h0[t, :] = E[id_t, :]`` with no scale and no position term
(reference: kernels/src/embedding.cu:12-26, models/llama/llama_model.cpp:424-425);
the rows are widened into the 32-bit residual stream.

Head: final norm, then ``logits = x W^T`` with no bias, scale or soft cap; with
tied embeddings ``W`` is the embedding table (llama_model.cpp:257-261,658-666).
The reference multiplies every token's row by the vocabulary matrix and copies
one row out (llama_model.cpp:663-698); here only the rows whose logits are
wanted are gathered, before the norm, so the large product has as many rows as
answers.  Logits are 32-bit.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import NORMS, ParamSpec, Part


class Embedding(Part):
    graph_safe = True
    kernels = ("embedding",)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.vocab_size, spec.hidden_size), role="table")}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = self.rt.empty(token_ids.shape[0], self.spec.hidden_size, dtype=torch.float32)
        self.rt.ops.embedding(self.weight, token_ids, out)
        return out


class LMHead(Part):
    graph_safe = True
    kernels = ("gemm", "norm")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.norm = NORMS.build(spec.norm, rt)
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        if spec.tied:
            return {}
        return {"weight": ParamSpec((spec.vocab_size, spec.hidden_size))}

    def children(self) -> Dict[str, Part]:
        return {"norm": self.norm}

    def load(self, tensors):
        if not self.spec.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, embedding: Embedding) -> None:
        self.weight = embedding.weight

    def forward(self, residual: torch.Tensor, pending: Optional[torch.Tensor],
                rows: torch.Tensor) -> torch.Tensor:
        h = self.norm.gather_add_norm(residual, pending, rows)
        return self.rt.ops.linear(h, self.weight, out_dtype=torch.float32)
