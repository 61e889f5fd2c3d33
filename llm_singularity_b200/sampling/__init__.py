"""Sampling: parameters, the counter-based uniform generator, the device sampler."""
from .params import GREEDY, SamplingParams
from .rng import uniform
from .sampler import Sampler

__all__ = ["GREEDY", "SamplingParams", "uniform", "Sampler"]
