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
    folds_next = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.mixer_norm = NORMS.build(spec.mixer_norm, rt)
        self.mixer = MIXERS.build(spec.mixer, rt)
        self.ffn_norm = NORMS.build(spec.ffn_norm, rt)
        self.ffn = FEED_FORWARDS.build(spec.ffn, rt)

    def children(self) -> Dict[str, Part]:
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def first_norm(self):
        """The norm this block's input meets first, if the block before may fold it into its last
        product."""
        return self.mixer_norm if self.mixer_norm.foldable else None

    def _input(self, h, part):
        """``h`` as ``part`` can take it: a norm's output with the rows' scale still owed only if the
        part says so."""
        if isinstance(h, torch.Tensor) or part.takes_unnormed:
            return h
        return self.rt.ops.finish_norm(h)

    def forward(self, residual: torch.Tensor, pending, ctx, cache, writes_cache: bool = True,
                next_norm=None):
        """``pending`` is the output of the block before, not yet added to the residual stream; or,
        if that block was given this block's ``first_norm()`` as its ``next_norm`` and folded it,
        an ``ops.NormOut``: added already, and what the mixer takes.  What comes back is the one or
        the other in the same way."""
        ops = self.rt.ops
        fold = getattr(ops, "folds_norm", None)
        fold = fold is not None and fold(residual.shape[0], self.rt.dtype)
        if isinstance(pending, getattr(ops, "NormOut", ())):
            h = pending
        else:
            h = self.mixer_norm.add_norm(residual, pending)
        if fold and self.mixer.folds_norm and self.ffn_norm.foldable:
            h = self.mixer.forward(self._input(h, self.mixer), ctx, cache, writes_cache,
                                   into=(residual, *self.ffn_norm.fold()))
        else:
            a = self.mixer.forward(self._input(h, self.mixer), ctx, cache, writes_cache)
            h = self.ffn_norm.add_norm(residual, a)
        if fold and next_norm is not None and self.ffn.folds_norm:
            return self.ffn.forward(self._input(h, self.ffn), ctx, into=(residual, *next_norm.fold()))
        return self.ffn.forward(self._input(h, self.ffn), ctx)
