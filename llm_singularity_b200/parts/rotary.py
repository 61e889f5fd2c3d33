"""Rotary position encoding (split-half pairing) with optional llama3 scaling.

For i in [0, rotary_dim/2): ``f_i = theta ** (-2i / rotary_dim)``, angle
``a = pos * f_i`` and the pair ``(x_i, x_{i+rotary_dim/2})`` is rotated by ``a``
(reference: kernels/src/rope.cu:13-26; pairing per CLAUDE.md:63,87).  The
reference recomputes ``powf`` per element and has no scaling; here the
frequencies are a table computed once in 64-bit and stored in 32-bit, and the
angle ``pos * f_i`` is formed in 32-bit inside the kernel.

llama3 scaling (position independent, applied to the table): with wavelength
``l_i = 2*pi / f_i``, ``l_high = original_max / high_freq_factor`` and ``l_low =
original_max / low_freq_factor``: ``l_i < l_high`` keeps ``f_i``; ``l_i > l_low``
gives ``f_i / factor``; in between ``s = (original_max / l_i - low) / (high - low)``
and ``f_i' = (1 - s) * f_i / factor + s * f_i``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .base import Part, register_position


def rotary_inv_freq(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """The frequency table ``[rotary_dim/2]`` in float64."""
    i = torch.arange(0, rotary_dim // 2, dtype=torch.float64)
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * i / rotary_dim)
    if scaling is None:
        return inv
    orig = float(scaling.original_max_position_embeddings)
    low, high, factor = scaling.low_freq_factor, scaling.high_freq_factor, scaling.factor
    wavelen = 2.0 * math.pi / inv
    smooth = (orig / wavelen - low) / (high - low)
    blended = (1.0 - smooth) * inv / factor + smooth * inv
    out = torch.where(wavelen > orig / low, inv / factor, blended)
    out = torch.where(wavelen < orig / high, inv, out)
    return out


@register_position("rotary")
class RotaryEncoding(Part):
    graph_safe = True
    replayable = True
    kernels = ("rope_cache",)

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and at most "
                             f"head_dim {spec.head_dim}")
        self.inv_freq = rotary_inv_freq(spec.rotary_dim, spec.theta, spec.scaling).to(
            dtype=torch.float32, device=rt.device)

    def rotary_table(self) -> Optional[Tuple[torch.Tensor, int]]:
        return self.inv_freq, self.spec.rotary_dim


@register_position("none")
class NoPosition(Part):
    graph_safe = True
    def rotary_table(self):
        return None

    def apply(self, q, k, ctx):
        return None
