"""Dense gated feed-forward: ``down( act(gate(x)) * up(x) )``, no bias; ``act`` is named by
the spec (silu in this architecture; the tanh form of gelu and none are there for others).

Reference: two products, ``silu(g) * u`` with ``silu(g) = g / (1 + exp(-g))``,
then the down product (models/llama/llama_model.cpp:634-649;
kernels/src/activations.cu:11-21).  Here gate and up are one product against a
matrix whose rows alternate ``Wgate[i], Wup[i]``, so that a gate and its up value
come out side by side and the activation is applied in the product's epilogue
(evaluated in 32-bit); the gate/up values themselves never go to memory.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import ParamSpec, Part, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(Part):
    graph_safe = True
    replayable = True
    folds_norm = True
    takes_unnormed = True
    kernels = ("gemm", "activation")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        known = getattr(rt.ops, "ACTIVATIONS", None)
        if known is not None and spec.activation not in known:
            raise ValueError(f"activation '{spec.activation}' is not implemented "
                             f"(known: {', '.join(sorted(known))})")

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        H, I = spec.hidden_size, spec.intermediate_size
        return {"gate_proj": ParamSpec((I, H)), "up_proj": ParamSpec((I, H)),
                "down_proj": ParamSpec((H, I))}

    def load(self, tensors):
        # rows 2i, 2i + 1 = gate_i, up_i
        self.w_gate_up = torch.stack([tensors["gate_proj"], tensors["up_proj"]], dim=1).reshape(
            2 * self.spec.intermediate_size, self.spec.hidden_size).contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    def forward(self, x, ctx, into=None):
        ops = self.rt.ops
        act = ops.linear(x, self.w_gate_up, gated=True, activation=self.spec.activation)   # [T, I]
        if into is not None:
            return ops.linear(act, self.w_down, into=into)
        return ops.linear(act, self.w_down)
