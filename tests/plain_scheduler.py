"""A plain scheduler in Python over the plain memory layer (tests/plain_memory.py): lists, a deque
and the rules in the order the engine's scheduler applies them.  The engine's scheduler is native
code (``llm_singularity_b200/csrc/host_scheduler.cpp``); the tests drive both with the same random
loads and compare every planned step, every preemption and every finished request.

Rules: decode tokens first (oldest request first; when pages run out the youngest running request
is preempted, or, while a step is in flight, the request waits), then the next portions of prompts
already running (they wait for pages, never preempt), then admission first come, first served.
Planning a step counts it as run and leaves a place-holder for each token it samples; ``update``
fills the place-holders in and finishes requests; ``schedule_ahead`` plans the step after the one in
flight.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Tuple

from llm_singularity_b200.sampling.params import SamplingParams


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
    # progress
    tokens: List[int] = field(default_factory=list)      # prompt + generated so far (+ place-holders)
    generated: List[int] = field(default_factory=list)
    computed: int = 0               # tokens whose keys/values are cached once the planned steps have run
    pending: int = 0                # place-holders at the end of ``tokens``: sampled, not yet known
    status: str = "waiting"          # waiting | running | finished | error
    error: str = ""
    preemptions: int = 0
    prefix_path: list = field(default_factory=list)

    def __post_init__(self):
        if not self.tokens:
            self.tokens = list(self.prompt)


@dataclass
class ScheduledItem:
    request: Request
    start: int                 # == request.computed: position of the first token of the portion
    tokens: List[int]
    sample: bool               # the portion ends the known tokens: logits of its last token wanted
    decode: bool = False       # one token after a sampled one (the rest is prompt work)


class PlainScheduler:
    def __init__(self, config: SchedulerConfig, cache, prefix_cache=None):
        self.cfg = config
        self.cache = cache
        self.prefix = prefix_cache
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # admission order
        self.finished: List[Request] = []
        self.stats = {"steps": 0, "preemptions": 0, "prefill_tokens": 0, "decode_tokens": 0,
                      "prefix_hit_tokens": 0, "evicted_pages": 0, "admitted": 0, "errors": 0}
        # plans of steps whose results have not come back yet, oldest first: one in the plain
        # loop (schedule, run, update), two while a step is planned ahead of the previous one's
        # tokens (schedule_ahead)
        self._plans: Deque[List[ScheduledItem]] = deque()

    # ----------------------------------------------------------------- intake
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if request.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------------- helpers
    def _free_pages(self) -> int:
        n = self.cache.free_pages()
        if self.prefix is not None:
            n += self.prefix.evictable_pages()
        return n

    def _reserve(self, req: Request, new_len: int) -> bool:
        """Pages for ``new_len`` tokens of ``req``, evicting cached prefixes if needed."""
        if self.cache.reserve(req.id, new_len):
            return True
        if self.prefix is not None:
            need = self.cache.pages_needed(req.id, new_len) - self.cache.free_pages()
            self.stats["evicted_pages"] += self.prefix.evict(need)
            return self.cache.reserve(req.id, new_len)
        return False

    def _release(self, req: Request) -> None:
        if self.prefix is not None and req.prefix_path:
            self.prefix.release(req.prefix_path)
            req.prefix_path = []
        self.cache.close(req.id)

    def _preempt(self, req: Request) -> None:
        """Free everything ``req`` holds; it will be recomputed from its tokens so far."""
        self._release(req)
        self.running.remove(req)
        req.computed = 0
        req.status = "waiting"
        req.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(req)

    def _fail(self, req: Request, why: str) -> None:
        req.status, req.error = "error", why
        self.stats["errors"] += 1
        self.finished.append(req)

    def _never_fits(self, req: Request) -> Optional[str]:
        n = len(req.tokens) + 1
        pool = min(g.pool.num_pages for g in self.cache.groups) if self.cache.groups else 1 << 30
        if n > self.cfg.max_model_len:
            return f"{len(req.tokens)} tokens plus one exceed max_model_len {self.cfg.max_model_len}"
        if self.cache.pages_for(n) > min(pool, self.cache.max_pages):
            return (f"{len(req.tokens)} tokens plus one need {self.cache.pages_for(n)} pages, "
                    f"the pool has {pool}")
        return None

    # --------------------------------------------------------------- schedule
    PENDING = -1        # stands for a token that a step in flight has yet to produce

    def schedule(self) -> List[ScheduledItem]:
        """Plan the next step; the step before it has been accounted (:meth:`update`)."""
        if self._plans:
            raise RuntimeError("a step is in flight: account it first, or plan with schedule_ahead")
        return self._plan(ahead=False)

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
        if len(self._plans) != 1:
            return None
        if any(r.pending and r.sampling.repetition_penalty != 1.0 for r in self.running):
            return None
        items = self._plan(ahead=True)
        if items:
            self.stats["ahead_steps"] = self.stats.get("ahead_steps", 0) + 1
        return items or None

    def _ends_with_token_in_flight(self, req: Request) -> bool:
        return len(req.generated) + req.pending >= req.max_new_tokens \
            or len(req.tokens) + 1 > self.cfg.max_model_len

    def _plan(self, ahead: bool) -> List[ScheduledItem]:
        cfg = self.cfg
        items: List[ScheduledItem] = []
        chunk_cap = cfg.max_prefill_chunk or cfg.max_tokens_per_batch

        # 1. decode tokens (requests with exactly one token left to run), oldest first; when
        #    pages run out the youngest running request is preempted (possibly the one asking),
        #    or, while a step is in flight, the request waits
        for req in list(self.running):
            if req.status != "running" or len(req.tokens) - req.computed != 1:
                continue                             # preempted a moment ago, or still in its prompt
            if req.pending and self._ends_with_token_in_flight(req):
                continue
            if len(items) >= cfg.max_tokens_per_batch:
                break
            placed = False
            while req.status == "running":
                if self._reserve(req, len(req.tokens)):
                    placed = True
                    break
                if ahead:
                    break
                victim = self.running[-1]
                items = [it for it in items if it.request is not victim]
                self._preempt(victim)
            if placed:
                items.append(ScheduledItem(req, req.computed, [req.tokens[-1]], True))
        budget = cfg.max_tokens_per_batch - len(items)

        # 2. next portions of prompts already running (they wait for pages, never preempt)
        for req in self.running:
            remaining = len(req.tokens) - req.computed
            if remaining <= 1 or budget <= 0:
                continue
            n = self._fit_portion(req, min(remaining, budget, chunk_cap))
            if n > 0:
                items.append(self._portion(req, n))
                budget -= n

        # 3. admission, first come first served
        while self.waiting and budget > 0 and len(self.running) < cfg.max_batch_size:
            req = self.waiting[0]
            why = self._never_fits(req)
            if why:
                self.waiting.popleft()
                self._fail(req, why)
                continue
            path = self.prefix.match(req.tokens) if self.prefix is not None else []
            need = self.cache.pages_for(len(req.tokens) + 1) - len(path)
            # pages on the matched path are in use by this request, not evictable for it
            evictable_on_path = sum(1 for n in path if n.users == 0)
            if need > self._free_pages() - evictable_on_path:
                break
            if self.cache.open(req.id) is None:
                break
            self.waiting.popleft()
            if path:
                req.computed = self.prefix.adopt(req.id, path)
                req.prefix_path = path
                self.stats["prefix_hit_tokens"] += req.computed
            req.status = "running"
            self.running.append(req)
            self.stats["admitted"] += 1
            n = self._fit_portion(req, min(len(req.tokens) - req.computed, budget, chunk_cap))
            if n > 0:
                items.append(self._portion(req, n))
                budget -= n

        # nothing could move although requests are live: the youngest gives way
        if not items and self.running and not ahead:
            if len(self.running) == 1:
                req = self.running[0]
                self._release(req)
                self.running.remove(req)
                self._fail(req, "the cache pool cannot hold this request")
            else:
                self._preempt(self.running[-1])
            return self._plan(ahead)

        # the first half of the accounting: the step counts as run
        for it in items:
            req = it.request
            req.computed += len(it.tokens)
            it.decode = len(it.tokens) == 1 and it.start > 0 and bool(req.generated or req.pending)
            if it.sample:
                if self.prefix is not None and not it.decode:
                    # The prompt is whole with this step: later prompts may share its full pages
                    # from now on (a step that reads them is queued behind this one).
                    req.prefix_path = req.prefix_path + self.prefix.share(
                        req.tokens[:req.computed], req.id, req.prefix_path)
                req.tokens.append(self.PENDING)
                req.pending += 1
        if items:
            self._plans.append(items)
            self.stats["steps"] += 1
        return items

    def _fit_portion(self, req: Request, n: int) -> int:
        """Largest portion <= n whose pages can be had now (prompts wait rather than preempt)."""
        if n <= 0:
            return 0
        if self._reserve(req, req.computed + n):
            return n
        ps = self.cache.page_size
        have = self.cache.pages_for(req.computed) * ps      # tokens its held pages cover
        room = have + self._free_pages() * ps - req.computed
        n = min(n, room)
        if n > 0 and self._reserve(req, req.computed + n):
            return n
        return 0

    def _portion(self, req: Request, n: int) -> ScheduledItem:
        toks = req.tokens[req.computed:req.computed + n]
        return ScheduledItem(req, req.computed, toks, req.computed + n == len(req.tokens))

    # ----------------------------------------------------------------- update
    def update(self, sampled: Dict[Hashable, int]) -> List[Request]:
        """The oldest step still unaccounted has run: ``sampled`` maps the ids of requests whose
        logits were wanted to their new token, which takes its place among the request's tokens.
        Returns requests that finished."""
        done: List[Tuple[Request, int]] = []
        for it in (self._plans.popleft() if self._plans else []):
            req = it.request
            if req.status != "running":
                continue         # planned ahead, but it stopped on the token that was in flight
            end = it.start + len(it.tokens)               # tokens cached now that this step has run
            if self.cache.length(req.id) < end:           # the step function has done it already,
                self.cache.commit(req.id, end)            # and a step planned ahead may be further
            if it.sample:
                if it.decode:
                    self.stats["decode_tokens"] += 1
                else:
                    self.stats["prefill_tokens"] += len(it.tokens)
                tok = int(sampled[req.id])
                if req.tokens[end] != self.PENDING:
                    raise RuntimeError(f"request {req.id!r}: no token is outstanding at place {end}")
                req.tokens[end] = tok
                req.pending -= 1
                req.generated.append(tok)
                stop = (not req.ignore_eos and tok in self.cfg.stop_token_ids) \
                    or len(req.generated) >= req.max_new_tokens \
                    or end + 2 > self.cfg.max_model_len
                if stop:
                    done.append((req, end))
            else:
                self.stats["prefill_tokens"] += len(it.tokens)
        for req, end in done:
            del req.tokens[end + 1:]                      # a place-holder of a step planned ahead
            req.pending, req.computed = 0, end
            if self.prefix is not None:
                self.prefix.insert(req.tokens[:end], req.id)
            self._release(req)
            self.running.remove(req)
            req.status = "finished"
            self.finished.append(req)
        return [req for req, _ in done]

    def take_finished(self) -> List[Request]:
        out, self.finished = self.finished, []
        return out
