"""Scheduler: admits requests, cuts prompts into portions, decodes, finishes, frees.

Each call of :meth:`Scheduler.schedule` plans one step under a token budget and
a limit of live requests:

1. every running request whose prompt is done gets its one decode token;
2. running requests still in their prompt get the next portion, at most
   ``max_prefill_chunk`` tokens and at most what is left of the budget;
3. waiting requests are admitted first come, first served (no overtaking), as long
   as a slot is free and the pools can hold their whole prompt plus one token
   (pages the prefix cache could give up count as free), and get a first portion.

Pages are reserved here, before the step, for exactly the tokens the step
brings.  When a reservation fails the prefix cache is asked to evict; if that is
not enough the most recently admitted running request is preempted: its pages and
slot are freed and it goes back to the front of the queue with everything it has
produced so far appended to its prompt, to be recomputed later.  Its sampling
stream continues where it stopped, so the tokens it yields are the same.  A
request that could never fit (its prompt plus one token needs more pages than the
pool has, or exceeds ``max_model_len``) finishes at once with an error status.
Nothing here is random, so a run can be replayed.

Accounting has two halves.  Planning a step advances its requests at once: the tokens it runs
count as computed, and a request whose logits it samples gets a place-holder (``PENDING``) at
the end of its tokens.  :meth:`Scheduler.update` fills the place-holders in when the sampled
tokens have come back, and finishes requests.  Between the two the next step can already be
planned (:meth:`Scheduler.schedule_ahead`): a request with a place-holder decodes on, its input
token being fed on the device, so the device never waits for the host.

The rules are applied by native code (``csrc/host_scheduler.cpp``, in one library with the memory
layer it works on); this module is its Python face.  The library reports what it did as a list of
events (admitted, preempted, failed, item, token, finished), which are replayed here onto the
``Request`` records that the engine and its users read: their tokens, their generated tokens,
their status.  ``tests/plain_scheduler.py`` states the same rules in plain Python and the tests
hold the two to each other.

The reference schedules prompts before decode tokens, iterates an unordered map,
allocates whole prompts at admission, samples after every portion and, when pages
run out during decoding, silently carries on into page 0
(core/src/scheduler.cpp:67-272; app/main.cpp:295-337); its stop rules (eos, stop
ids, max_new_tokens, output includes the stop token; scheduler.cpp:238-266) are
kept.
"""
from __future__ import annotations

import ctypes
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Tuple

from ..cache import native
from ..cache.manager import CacheManager
from ..cache.pages import PageError
from ..sampling.params import SamplingParams


@dataclass
class SchedulerConfig:
    max_batch_size: int = 64            # live requests (reference default, scheduler.h:23)
    max_tokens_per_batch: int = 512     # tokens per step (scheduler.h:24)
    max_prefill_chunk: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()
    max_model_len: int = 1 << 30


@dataclass(eq=False)            # a request is itself: compared and looked up by identity
class Request:
    id: Hashable
    prompt: List[int]
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    ignore_eos: bool = False
    # progress (a record of what the native scheduler has decided)
    tokens: List[int] = field(default_factory=list)      # prompt + generated so far (+ place-holders)
    generated: List[int] = field(default_factory=list)
    computed: int = 0               # tokens whose keys/values are cached once the planned steps have run
    pending: int = 0                # place-holders at the end of ``tokens``: sampled, not yet known
    status: str = "waiting"          # waiting | running | finished | error
    error: str = ""
    preemptions: int = 0
    handle: int = -1                # its name inside the native scheduler

    def __post_init__(self):
        if not self.tokens:
            self.tokens = list(self.prompt)


@dataclass
class ScheduledItem:
    request: Request
    start: int                 # position of the first token of the portion
    tokens: List[int]
    sample: bool               # the portion ends the known tokens: logits of its last token wanted
    decode: bool = False       # one token after a sampled one (the rest is prompt work)


_ADMIT, _PREEMPT, _FAIL, _ITEM, _TOKEN, _FINISH = 1, 2, 3, 4, 5, 6
_STATS = ("steps", "preemptions", "prefill_tokens", "decode_tokens", "prefix_hit_tokens",
          "evicted_pages", "admitted", "errors", "ahead_steps")


class Scheduler:
    PENDING = -1        # stands for a token that a step in flight has yet to produce

    def __init__(self, config: SchedulerConfig, cache: CacheManager, prefix_cache=None):
        self.cfg = config
        self.cache = cache
        self.prefix = prefix_cache
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # admission order
        self.finished: List[Request] = []
        self._lib = native.lib()
        stops = self._stops = [int(t) for t in config.stop_token_ids]
        self._ptr = self._lib.lsbs_create(
            cache._ptr, 1 if prefix_cache is not None else 0, config.max_batch_size,
            config.max_tokens_per_batch, config.max_prefill_chunk or 0, native.ints(stops), len(stops),
            config.max_model_len)
        if not self._ptr:
            raise ValueError("max_batch_size and max_tokens_per_batch must be positive")
        self._by_handle: Dict[int, Request] = {}
        self._by_id: Dict[Hashable, Request] = {}
        self._stat_buf = (ctypes.c_longlong * len(_STATS))()
        self._event_buf = (ctypes.c_longlong * (5 * 256))()
        self._token_buf = (ctypes.c_int * (2 * config.max_batch_size))()   # handles, then tokens

    def __del__(self):
        if getattr(self, "_ptr", None):
            self._lib.lsbs_destroy(self._ptr)
            self._ptr = None

    @property
    def stats(self) -> Dict[str, int]:
        self._lib.lsbs_stats(self._ptr, self._stat_buf)
        return dict(zip(_STATS, self._stat_buf))

    # ----------------------------------------------------------------- intake
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if request.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if request.id in self._by_id:
            raise KeyError(f"request id {request.id!r} is in use")
        keep, ptr = native.token_array(request.tokens)
        h = self._lib.lsbs_add(self._ptr, ptr, len(keep), request.max_new_tokens,
                               1 if request.ignore_eos else 0,
                               1 if request.sampling.repetition_penalty != 1.0 else 0)
        if h == native.ERR:
            raise ValueError(self._error())
        request.handle = h
        self._by_handle[h] = request
        self._by_id[request.id] = request
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _error(self) -> str:
        return self._lib.lsbs_last_error(self._ptr).decode()

    # --------------------------------------------------------------- schedule
    def schedule(self) -> List[ScheduledItem]:
        """Plan the next step; the step before it has been accounted (:meth:`update`)."""
        if self._lib.lsbs_plans_in_flight(self._ptr):
            raise RuntimeError("a step is in flight: account it first, or plan with schedule_ahead")
        if self._lib.lsbs_plan(self._ptr, 0) == native.ERR:
            raise PageError(self._error())
        return self._replay()

    def schedule_ahead(self) -> Optional[List[ScheduledItem]]:
        """Plan the step after the one in flight before that one's tokens are known.  A request
        whose next token is in flight brings ``[PENDING]``; the caller feeds it from the device.
        Left out of such a step: a request that the token in flight finishes (``max_new_tokens``
        or the model's length; its pages come back when it is accounted) and anything that
        needs preemption.  A request that turns out to have stopped on the token in flight (a stop
        token) is skipped when the step planned here is accounted.  Returns None when there is
        nothing to run, when two steps would be ahead, or when a request samples with a repetition
        penalty (which needs the token in flight on the host): plan with :meth:`schedule` after
        :meth:`update` then."""
        if self._lib.lsbs_plan(self._ptr, 1) == native.ERR:
            raise PageError(self._error())
        return self._replay() or None

    def _replay(self) -> List[ScheduledItem]:
        """Apply the events of the last native call to the request records; returns the items."""
        n = self._lib.lsbs_num_events(self._ptr)
        if n == 0:
            return []
        if 5 * n > len(self._event_buf):
            self._event_buf = (ctypes.c_longlong * (10 * n))()
        self._lib.lsbs_events(self._ptr, self._event_buf, len(self._event_buf) // 5)
        ev = self._event_buf[:5 * n]
        items: List[ScheduledItem] = []
        for k in range(0, 5 * n, 5):
            kind, h, a, b, c = ev[k:k + 5]
            req = self._by_handle[h]
            if kind == _ITEM:
                items.append(ScheduledItem(req, a, req.tokens[a:a + b], bool(c & 1), bool(c & 2)))
                req.computed = a + b                 # the first half of the accounting
                if c & 1:
                    req.tokens.append(self.PENDING)
                    req.pending += 1
            elif kind == _TOKEN:
                req.tokens[b] = a
                req.pending -= 1
                req.generated.append(a)
            elif kind == _ADMIT:
                self.waiting.remove(req)             # it stood at the front
                req.computed, req.status = a, "running"
                self.running.append(req)
                self.cache.bind(req.id, self._lib.lsbs_request_slot(self._ptr, h))
            elif kind == _FINISH:
                del req.tokens[a + 1:]               # a place-holder of a step planned ahead
                req.pending, req.computed, req.status = 0, a, "finished"
                self._leave_running(req)
            elif kind == _PREEMPT:
                self._leave_running(req)
                req.computed, req.status = 0, "waiting"
                req.preemptions += 1
                self.waiting.appendleft(req)
            elif kind == _FAIL:
                if req.status == "running":
                    self._leave_running(req)
                else:
                    self.waiting.remove(req)
                req.status = "error"
                req.error = self._lib.lsbs_request_error(self._ptr, h).decode()
            if kind in (_FINISH, _FAIL):
                self.finished.append(req)
        return items

    def _leave_running(self, req: Request) -> None:
        self.running.remove(req)
        self.cache.unbind(req.id)                    # its slot is closed in the memory layer already

    # ----------------------------------------------------------------- update
    def update(self, sampled: Dict[Hashable, int]) -> List[Request]:
        """The oldest step still unaccounted has run: ``sampled`` maps the ids of requests whose
        logits were wanted to their new token, which takes its place among the request's tokens.
        Returns requests that finished."""
        stops = [int(t) for t in self.cfg.stop_token_ids]
        if stops != self._stops:                     # the configuration was changed under way
            self._lib.lsbs_set_stop_ids(self._ptr, native.ints(stops), len(stops))
            self._stops = stops
        by_id, buf, cap, k = self._by_id, self._token_buf, len(self._token_buf) // 2, 0
        if len(sampled) > cap:
            buf = self._token_buf = (ctypes.c_int * (2 * len(sampled)))()
            cap = len(sampled)
        for rid, tok in sampled.items():
            req = by_id.get(rid)
            if req is not None:                      # else: finished and forgotten, a stray token
                buf[k], buf[cap + k] = req.handle, tok
                k += 1
        tokens = ctypes.cast(ctypes.byref(buf, cap * ctypes.sizeof(ctypes.c_int)), ctypes.POINTER(ctypes.c_int))
        if self._lib.lsbs_update(self._ptr, buf, tokens, k) == native.ERR:
            raise RuntimeError(self._error())
        before = len(self.finished)
        self._replay()
        return [r for r in self.finished[before:] if r.status == "finished"]

    def take_finished(self) -> List[Request]:
        """Finished and failed requests since the last call; the scheduler forgets them."""
        out, self.finished = self.finished, []
        for req in out:
            self._lib.lsbs_forget(self._ptr, req.handle)
            del self._by_handle[req.handle]
            del self._by_id[req.id]
        return out
