"""RMSNorm, fused with the residual addition that precedes it.

``y = x * rsqrt(mean(x^2) + eps) * w`` with eps inside the square root and the
weight applied after normalisation (reference: kernels/src/rmsnorm.cu:42-72, used
at models/llama/llama_model.cpp:506-508,629-631,658-660).  The residual stream is
32-bit; sum of squares, rsqrt and the product are 32-bit; the result is rounded
to the compute dtype only on the way out.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import ParamSpec, Part, register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    graph_safe = True
    replayable = True
    foldable = True
    kernels = ("norm",)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((spec.size,), role="vector", init="ones")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def fold(self):
        """What a product needs to take this norm upon itself: the weight and eps."""
        return self.weight, self.spec.eps

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        out = self.rt.empty(*residual.shape)
        self.rt.ops.add_rmsnorm(residual, delta, self.weight, self.spec.eps, out)
        return out

    def gather_add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor],
                        rows: torch.Tensor) -> torch.Tensor:
        out = self.rt.empty(rows.shape[0], residual.shape[1])
        self.rt.ops.gather_add_rmsnorm(residual, delta, rows, self.weight, self.spec.eps, out)
        return out
