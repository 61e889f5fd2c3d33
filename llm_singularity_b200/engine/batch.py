"""StepEntry and StepContext: one step's batch, flattened for the kernels.

A step is a list of entries ``(request, its next tokens, wanted places)``:
portions of prompts beside single decoded tokens, cut anywhere.  All entries are
flattened into one token stream ``[T]``; per token the context carries its
position and its request's index, per request where its tokens start in the
stream, how long its sequence is after this step, and which block-table row is
its own.  The reference builds the same arrays per forward, in separate passes
for prompts and decode tokens, with five ``cudaMalloc`` and a per-token copy of
the block table (models/llama/llama_model.cpp:306-400,434-500); here it is one
packed int32 buffer and one host-to-device copy per step.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import native


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # places among ``tokens``


class StepContext:
    """Device arrays (int32) and host mirrors describing one step's batch."""

    # device
    token_ids: torch.Tensor      # [T]
    positions: torch.Tensor      # [T]  absolute position of each token in its sequence
    token_req: torch.Tensor      # [T]  index of the token's request within this step
    q_start: torch.Tensor        # [R+1] first token of each request in the stream
    kv_len: torch.Tensor         # [R]  sequence length after this step
    table_rows: torch.Tensor     # [R]  the request's row in block tables and state
    want_rows: torch.Tensor      # [W]  stream indices whose logits are wanted
    # host
    n_tokens: int
    n_requests: int
    n_wanted: int
    h_q_len: np.ndarray
    h_q_start: np.ndarray        # [R+1]
    h_kv_len: np.ndarray
    h_table_rows: np.ndarray
    max_q_len: int
    max_kv_len: int


class ContextBuilder:
    """Packs step metadata into one pinned buffer and copies it to the device once."""

    RING = 4

    def __init__(self, device, max_tokens: int, max_requests: int, max_table_updates: int = 0):
        self.device = torch.device(device)
        self.max_tokens = max_tokens
        self.max_requests = max_requests
        cap = 4 * max_tokens + 3 * max_requests + 1 + 2 * max(max_table_updates, 1024) + 64
        self._cap = cap
        self._cuda = self.device.type == "cuda"
        self._host = [torch.empty(cap, dtype=torch.int32, pin_memory=self._cuda)
                      for _ in range(self.RING)]
        self._dev = [torch.empty(cap, dtype=torch.int32, device=self.device)
                     for _ in range(self.RING)]
        self._host_np = [h.numpy() for h in self._host]
        self._events = [None] * self.RING
        self._turn = 0
        self._offsets = np.zeros(8, dtype=np.int64)
        self._summary = np.zeros(4, dtype=np.int64)

    def _grow(self, n: int) -> None:
        cap = max(n, 2 * self._cap)
        self._cap = cap
        if self._cuda:
            torch.cuda.synchronize(self.device)
        self._host = [torch.empty(cap, dtype=torch.int32, pin_memory=self._cuda)
                      for _ in range(self.RING)]
        self._dev = [torch.empty(cap, dtype=torch.int32, device=self.device)
                     for _ in range(self.RING)]
        self._host_np = [h.numpy() for h in self._host]
        self._events = [None] * self.RING

    def build(self, tokens: List[Sequence[int]], starts: List[int], rows: List[int],
              wants: List[Sequence[int]], extra: Optional[List[np.ndarray]] = None,
              static: Optional[torch.Tensor] = None):
        """``tokens[r]`` are request r's new tokens, ``starts[r]`` how many it already
        holds, ``rows[r]`` its block-table row, ``wants[r]`` places among its tokens.
        ``extra`` are further int32 arrays to ride along; returns (ctx, extra on device).
        ``static``: a persistent device buffer to fill instead of the ring's (so that the
        arrays keep their addresses from step to step, as a captured graph needs)."""
        R = len(tokens)
        if R == 0:
            raise ValueError("a step needs at least one entry, and every entry at least one token")
        arrays = [t if isinstance(t, np.ndarray) and t.dtype == np.int32 else np.asarray(t, dtype=np.int32)
                  for t in tokens]
        q_len = np.fromiter(map(len, arrays), dtype=np.int32, count=R)
        flat = np.ascontiguousarray(arrays[0]) if R == 1 else np.concatenate(arrays)
        starts_a = np.asarray(starts, dtype=np.int32)
        rows_a = np.asarray(rows, dtype=np.int32)
        want_count = np.fromiter(map(len, wants), dtype=np.int32, count=R)
        W = int(want_count.sum())
        wants_a = np.fromiter(itertools.chain.from_iterable(wants), dtype=np.int32, count=W)
        T = int(flat.shape[0])
        extra = extra or []
        n = 3 * T + (R + 1) + 2 * R + W + sum(len(e) for e in extra)
        if n > self._cap:
            self._grow(n)

        i = self._turn
        self._turn = (self._turn + 1) % self.RING
        if self._events[i] is not None:
            self._events[i].synchronize()
        host = self._host_np[i]
        # one pass in the host library writes tokens, positions, each token's entry, where each
        # entry starts, its length after the step, its block-table row and the wanted rows
        o = native.lib().lsbh_pack_step(R, q_len.ctypes.data, starts_a.ctypes.data, rows_a.ctypes.data,
                                        flat.ctypes.data, want_count.ctypes.data, wants_a.ctypes.data,
                                        host.ctypes.data, self._cap, self._offsets.ctypes.data,
                                        self._summary.ctypes.data)
        if o < 0:
            r = -o - 2
            if o == -1 or q_len[r] <= 0:
                raise ValueError("a step needs at least one entry, and every entry at least one token")
            bad = next(w for w in wants[r] if not 0 <= w < q_len[r])
            raise ValueError(f"entry {r}: wanted place {bad} outside its {q_len[r]} tokens")
        s_tok, s_pos, s_req, s_qs, s_kv, s_rows, s_want, end = (int(x) for x in self._offsets)
        s_extra = []
        for e in extra:
            host[o:o + len(e)] = e
            s_extra.append((o, o + len(e)))
            o += len(e)

        dev = self._dev[i] if static is None else static
        if dev.numel() < o:
            raise ValueError(f"static metadata buffer holds {dev.numel()} ints, step needs {o}")
        dev[:o].copy_(self._host[i][:o], non_blocking=True)
        if self._cuda:
            if self._events[i] is None:
                self._events[i] = torch.cuda.Event()
            self._events[i].record()

        ctx = StepContext()
        ctx.token_ids = dev[s_tok:s_pos]
        ctx.positions = dev[s_pos:s_req]
        ctx.token_req = dev[s_req:s_qs]
        ctx.q_start = dev[s_qs:s_kv]
        ctx.kv_len = dev[s_kv:s_rows]
        ctx.table_rows = dev[s_rows:s_want]
        ctx.want_rows = dev[s_want:end]
        ctx.n_tokens, ctx.n_requests, ctx.n_wanted = T, R, W
        ctx.h_q_len = q_len
        ctx.h_q_start = host[s_qs:s_kv].copy()
        ctx.h_kv_len = host[s_kv:s_rows].copy()
        ctx.h_table_rows = rows_a
        ctx.max_q_len, ctx.max_kv_len = int(self._summary[2]), int(self._summary[3])
        return ctx, [dev[a:b] for a, b in s_extra]
