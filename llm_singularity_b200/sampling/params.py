"""SamplingParams: the reference's fields and defaults (core/include/core/sampling.h:6-12).

``temperature == 0`` is greedy (first maximum).  ``top_k == 0`` and ``top_p == 1``
switch those filters off, ``repetition_penalty == 1`` the penalty.  ``seed`` is
never read by the reference (core/src/sampling.cpp:9 seeds from the system);
here it keys the request's own stream of uniform draws.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be positive, got {self.repetition_penalty}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


GREEDY = SamplingParams(temperature=0.0)
