"""Block arrangements: how norms, mixer and feed-forward sit on the residual stream.

``pre_norm`` is the reference's order (models/llama/llama_model.cpp:502-655):
``x += mixer(norm1(x)); x += ffn(norm2(x))``.  The residual stream is a 32-bit
tensor updated in place.  Each addition is fused with the norm that follows it,
so a block hands its feed-forward output back as ``pending`` (not yet added) and
the next block's first norm, or the head's final norm, adds it.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FEED_FORWARDS, MIXERS, NORMS, Part, register_block


@register_block("pre_norm")
class PreNormBlock(Part):
    graph_safe = True
    replayable = True
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer_norm = NORMS.build(spec.mixer_norm, rt)
        self.mixer = MIXERS.build(spec.mixer, rt)
        self.ffn_norm = NORMS.build(spec.ffn_norm, rt)
        self.ffn = FEED_FORWARDS.build(spec.ffn, rt)

    def children(self) -> Dict[str, Part]:
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def forward(self, residual: torch.Tensor, pending: Optional[torch.Tensor], ctx, cache,
                writes_cache: bool = True) -> torch.Tensor:
        h = self.mixer_norm.add_norm(residual, pending)
        a = self.mixer.forward(h, ctx, cache, writes_cache)
        h = self.ffn_norm.add_norm(residual, a)
        return self.ffn.forward(h, ctx)
