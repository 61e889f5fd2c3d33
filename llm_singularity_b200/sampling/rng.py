"""The uniform draws of temperature sampling: a counter-based generator.

``uniform(seed, n)`` is the n-th draw of the stream keyed by ``seed``: one
splitmix64 scramble of ``seed + (n + 1) * golden``, its top 24 bits centred in
their cell, so the value lies strictly inside (0, 1) and is exact in float32.  A
request's n-th generated token always uses its own n-th draw, whatever else is
in the batch and however its prompt was cut, so sampled generations can be
replayed.  (The reference draws from one process-wide mt19937 seeded from the
system, core/src/sampling.cpp:9,106-107, and cannot be replayed.)
"""
from __future__ import annotations

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


def splitmix64(x: int) -> int:
    z = x & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, n: int) -> float:
    z = splitmix64((seed + (n + 1) * _GOLDEN) & _MASK)
    return ((z >> 40) + 0.5) / float(1 << 24)
