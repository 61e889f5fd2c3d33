"""Sampler: one token per row of logits, on the device.

Greedy, temperature, top-k, top-p and repetition penalty in the reference's
order (core/src/sampling.cpp:11-118), done by the ``sampling`` kernel library; the
host only packs the per-row parameters and the uniform draws.  The reference
never passes previous tokens to its sampler (app/main.cpp:308-310), which leaves
its penalty without effect; here the request's generated tokens are passed.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .params import SamplingParams
from .rng import uniform


class StagedSampling:
    """Per-row sampling parameters already on the device, in arrays that keep their addresses from
    step to step (one set per number of rows), and the launch that uses them.  Calling it is the
    same work every time, so a decode step captured in a CUDA graph can hold it."""

    def __init__(self, ops, params: torch.Tensor, top_k: torch.Tensor, out: torch.Tensor):
        self.ops, self.params, self.top_k, self.out = ops, params, top_k, out
        self.key = ("sample", out.shape[0])

    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        self.ops.sample(logits, self.params, self.top_k, None, None, self.out)
        return self.out


class Sampler:
    def __init__(self, rt):
        self.rt = rt
        self._greedy = {}               # batch size -> device arrays for all-greedy batches
        self._staged = {}               # batch size -> StagedSampling
        prepare = getattr(rt.ops, "prepare", None)
        if prepare is not None:
            prepare(["sampling"])

    def stage(self, params: Sequence[SamplingParams], draw_index: Sequence[int]) -> Optional[StagedSampling]:
        """Put this step's per-row parameters and uniform draws into the persistent device arrays
        of their batch size and return the launch that samples with them; None where a repetition
        penalty is in use (it needs the generated tokens, packed per step by :meth:`sample`)."""
        R = len(params)
        if R == 0 or any(p.repetition_penalty != 1.0 for p in params):
            return None
        st = self._staged.get(R)
        dev = self.rt.device
        if st is None:
            st = self._staged[R] = StagedSampling(
                self.rt.ops, torch.tensor([[0.0, 1.0, 1.0, 0.5]] * R, dtype=torch.float32, device=dev),
                torch.zeros(R, dtype=torch.int32, device=dev), torch.empty(R, dtype=torch.int32, device=dev))
            st.greedy = True
        if all(p.greedy for p in params):
            if not st.greedy:                        # back to the constant rows of an all-greedy batch
                st.params.copy_(torch.tensor([[0.0, 1.0, 1.0, 0.5]] * R, dtype=torch.float32))
                st.top_k.zero_()
                st.greedy = True
            return st
        fl = np.empty((R, 4), dtype=np.float32)
        tk = np.empty(R, dtype=np.int32)
        for r, (p, n) in enumerate(zip(params, draw_index)):
            fl[r] = (p.temperature, p.top_p, 1.0, 0.5 if p.greedy else uniform(p.seed, n))
            tk[r] = p.top_k
        # (pageable host arrays: the copies have left them when these calls return; on the device
        # they run in stream order, after the sampling of the step before)
        st.params.copy_(torch.from_numpy(fl), non_blocking=True)
        st.top_k.copy_(torch.from_numpy(tk), non_blocking=True)
        st.greedy = False
        return st

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               draw_index: Sequence[int],
               previous: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """``logits`` [R, V] float32 on the device; ``draw_index[r]`` is how many tokens request
        r has generated so far (selects its uniform draw); ``previous[r]`` its generated tokens
        (used only where a repetition penalty is set).  Returns int32 [R] on the device."""
        R = logits.shape[0]
        if len(params) != R or len(draw_index) != R:
            raise ValueError("one SamplingParams and one draw index per row of logits")
        dev = self.rt.device
        if all(p.greedy and p.repetition_penalty == 1.0 for p in params):
            # nothing varies from step to step: keep the per-row arrays on the device
            cached = self._greedy.get(R)
            if cached is None:
                fl = torch.tensor([[0.0, 1.0, 1.0, 0.5]] * R, dtype=torch.float32, device=dev)
                cached = self._greedy[R] = (fl, torch.zeros(R, dtype=torch.int32, device=dev),
                                            torch.empty(R, dtype=torch.int32, device=dev))
            d_fl, d_tk, out = cached
            self.rt.ops.sample(logits, d_fl, d_tk, None, None, out)
            return out
        fl = np.empty((R, 4), dtype=np.float32)
        tk = np.empty(R, dtype=np.int32)
        penal = False
        for r, (p, n) in enumerate(zip(params, draw_index)):
            fl[r] = (p.temperature, p.top_p, p.repetition_penalty,
                     0.5 if p.greedy else uniform(p.seed, n))
            tk[r] = p.top_k
            penal |= p.repetition_penalty != 1.0
        d_fl = torch.from_numpy(fl).to(dev, non_blocking=True)
        d_tk = torch.from_numpy(tk).to(dev, non_blocking=True)
        d_start = d_prev = None
        if penal and previous is not None:
            start = np.zeros(R + 1, dtype=np.int32)
            flat: List[int] = []
            for r, prev in enumerate(previous):
                if params[r].repetition_penalty != 1.0:
                    flat.extend(prev)
                start[r + 1] = len(flat)
            d_start = torch.from_numpy(start).to(dev)
            d_prev = torch.from_numpy(np.asarray(flat if flat else [0], dtype=np.int32)).to(dev)
        out = torch.empty(R, dtype=torch.int32, device=dev)
        self.rt.ops.sample(logits, d_fl, d_tk, d_start, d_prev, out)
        return out
