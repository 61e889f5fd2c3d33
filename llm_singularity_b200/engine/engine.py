"""Engine: the Python entry point — requests in, tokens out.

``Engine`` wires the pieces the reference's ``main`` wires (app/main.cpp:177-344:
model, block pool, prefix cache, scheduler, sampler, inference loop) without the
HTTP server and tokenizer around them: token ids in, token ids out.

    eng = Engine(model_dir, dtype="bfloat16")
    outs = eng.generate([[1, 2, 3], [4, 5]], max_new_tokens=16, temperature=0.0)

One ``step()`` plans a batch (scheduler), runs it (the model's step function),
samples on the device, reads the new tokens back and updates the requests.
"""
from __future__ import annotations

import itertools
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.prefix import RadixPrefixCache
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduler, SchedulerConfig


class _Launched:
    """A step that is queued on the device and not accounted yet."""

    def __init__(self, wanted: List[Request]):
        self.wanted = wanted                 # requests whose next token the step samples
        self.dev_tokens: Optional[torch.Tensor] = None
        self.host_tokens: Optional[torch.Tensor] = None
        self.event = None


class Engine:
    def __init__(self, model_dir: Optional[str] = None, *, random_weights: bool = False,
                 seed: int = 0, dtype="bfloat16", device="cuda:0", kv_block_size: int = 16,
                 num_kv_blocks: int = 1024, max_batch_size: int = 64,
                 max_tokens_per_batch: int = 2048, prefill_chunk: Optional[int] = None,
                 max_model_len: Optional[int] = None, prefix_cache: bool = True,
                 config=None, ops=None, verbose: bool = False, run_ahead: bool = True):
        """``model_dir`` holds config.json and, unless ``random_weights``, the safetensors
        files.  Defaults follow the reference's hints: pages of 16 tokens, 1024 pages, 2048
        tokens per batch (models/llama/llama_model.cpp:111-120)."""
        tensors = None
        if random_weights:
            from ..registry import load_config
            from ..weights.random_init import random_tensors
            from .runner import expected_tensors_of, parse_dtype
            if config is None:
                config = load_config(model_dir)
            tensors = random_tensors(expected_tensors_of(config.to_model_spec()), seed,
                                     dtype=parse_dtype(dtype),
                                     device=device if ops is None else "cpu")
        self.runner = ModelRunner(model_dir, config=config, tensors=tensors, dtype=dtype,
                                  device=device, page_size=kv_block_size, num_pages=num_kv_blocks,
                                  max_requests=max_batch_size,
                                  max_tokens_per_step=max_tokens_per_batch,
                                  max_model_len=max_model_len, ops=ops, verbose=verbose)
        cache = self.runner.cache
        shareable = prefix_cache and cache.groups and all(g.window is None for g in cache.groups) \
            and all(s is not None and s.shareable for s in self.runner.model.cache_specs())
        self.prefix = RadixPrefixCache(cache) if shareable else None
        self.scheduler = Scheduler(
            SchedulerConfig(max_batch_size=max_batch_size,
                            max_tokens_per_batch=max_tokens_per_batch,
                            max_prefill_chunk=prefill_chunk,
                            stop_token_ids=tuple(self.runner.spec.stop_token_ids),
                            max_model_len=self.runner.max_model_len),
            cache, self.prefix)
        self.sampler = Sampler(self.runner.rt)
        self._ids = itertools.count()
        self._requests: Dict[Hashable, Request] = {}       # live requests (and those generate() waits for)
        self._kept: set = set()                            # ids that generate() collects itself
        self.run_ahead = run_ahead
        self._inflight: Optional[_Launched] = None
        pin = torch.device(device).type == "cuda" and ops is None
        self._host_tokens = [torch.empty(max_batch_size, dtype=torch.int32, pin_memory=pin)
                             for _ in range(2)]
        self._host_turn = 0

    # ------------------------------------------------------------------ intake
    def add_request(self, token_ids: Sequence[int], max_new_tokens: int = 16,
                    temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                    repetition_penalty: float = 1.0, seed: int = 0, ignore_eos: bool = False,
                    request_id: Optional[Hashable] = None) -> Hashable:
        rid = next(self._ids) if request_id is None else request_id
        if rid in self._requests:
            raise KeyError(f"request id {rid!r} is in use")
        V = self.runner.vocab_size
        toks = [int(t) for t in token_ids]
        if any(t < 0 or t >= V for t in toks):
            raise ValueError(f"token id outside [0, {V})")
        req = Request(rid, toks, max_new_tokens,
                      SamplingParams(temperature, top_k, top_p, repetition_penalty, seed),
                      ignore_eos)
        self._requests[rid] = req
        self.scheduler.add(req)
        return rid

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    # -------------------------------------------------------------------- step
    def step(self) -> List[Tuple[Hashable, int, bool]]:
        """Run one scheduled batch; returns (request id, new token, finished) for every request
        that produced a token, and (id, -1, True) for requests that ended with an error.

        With ``run_ahead`` the step after this one is planned and queued on the device before
        this one's tokens are read back (Scheduler.schedule_ahead): decoding requests take their
        input token from the device, where the sampler left it, prompt portions and admissions
        are known anyway, and the host's work for the step happens while the device is busy.
        Each call still returns the tokens of exactly one step."""
        out = self._step()
        for rid, _, finished in out:         # a finished request is forgotten: its id is free again
            if finished and rid not in self._kept:
                self._requests.pop(rid, None)
        return out

    def _step(self) -> List[Tuple[Hashable, int, bool]]:
        out: List[Tuple[Hashable, int, bool]] = []
        cur = self._inflight
        if cur is None:
            items = self.scheduler.schedule()
            for req in self.scheduler.take_finished():         # errors found while scheduling
                out.append((req.id, -1, True))
            if not items:
                return out
            cur = self._launch(items, None)
        nxt = None
        if self.run_ahead:
            items = self.scheduler.schedule_ahead()
            for req in self.scheduler.take_finished():
                out.append((req.id, -1, True))
            if items is not None:
                nxt = self._launch(items, cur)
        self._inflight = nxt
        out.extend(self._complete(cur))
        return out

    def _launch(self, items, after: Optional["_Launched"]) -> "_Launched":
        """Queue one planned step on the device: the model step, sampling, and the copy of the
        new tokens to the host.  ``after``: the step in flight, whose sampled tokens are the
        input of the entries that bring a place-holder."""
        pending = self.scheduler.PENDING
        entries, places, which = [], [], []
        place_of = {r.id: i for i, r in enumerate(after.wanted)} if after is not None else {}
        for k, it in enumerate(items):
            tokens = it.tokens
            if tokens[-1] == pending:                          # a single token, still on the device
                places.append(place_of[it.request.id])
                which.append(k)
                tokens = [0]
            entries.append(StepEntry(it.request.id, tokens, [len(tokens) - 1] if it.sample else []))
        feed = (after.dev_tokens, places, which) if which else None
        wanted = [it.request for it in items if it.sample]
        # a request's tokens still in flight count towards its place in the sampling stream
        draws = [len(r.generated) + r.pending - 1 for r in wanted]
        # sampling rides behind the model on the device (inside the captured graph of a decode
        # step) wherever its parameters can be staged ahead: everything but a repetition penalty
        staged = self.sampler.stage([r.sampling for r in wanted], draws) if wanted else None
        logits = self.runner.step(entries, feed=feed, after=staged)
        launched = _Launched(wanted)
        if wanted:
            if staged is not None:
                launched.dev_tokens = self.runner.after_result
            else:
                launched.dev_tokens = self.sampler.sample(
                    logits, [r.sampling for r in wanted], draws, [r.generated for r in wanted])
            if launched.dev_tokens.is_cuda:
                host = self._host_tokens[self._host_turn][:len(wanted)]
                self._host_turn ^= 1
                host.copy_(launched.dev_tokens, non_blocking=True)
                launched.event = torch.cuda.Event()
                launched.event.record()
                launched.host_tokens = host
            else:
                launched.host_tokens = launched.dev_tokens.clone()
        return launched

    def _complete(self, launched: "_Launched") -> List[Tuple[Hashable, int, bool]]:
        """Wait for a queued step's tokens and account it."""
        sampled: Dict[Hashable, int] = {}
        if launched.wanted:
            if launched.event is not None:
                launched.event.synchronize()
            host = launched.host_tokens.tolist()
            sampled = {r.id: t for r, t in zip(launched.wanted, host)}
        live = [r for r in launched.wanted if r.status == "running"]
        done = {r.id for r in self.scheduler.update(sampled)}
        self.scheduler.take_finished()
        return [(r.id, sampled[r.id], r.id in done) for r in live]

    # ---------------------------------------------------------------- generate
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16,
                 temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                 repetition_penalty: float = 1.0, seed: int = 0,
                 ignore_eos: bool = False) -> List[List[int]]:
        """Generate for every prompt; request i samples with seed ``seed + i``.  Returns the
        generated tokens (stop token included), in the order of the prompts."""
        ids = [self.add_request(p, max_new_tokens, temperature, top_k, top_p, repetition_penalty,
                                seed + i, ignore_eos) for i, p in enumerate(prompts)]
        self._kept.update(ids)
        try:
            while self.has_work():
                self.step()
        finally:
            self._kept.difference_update(ids)
        outs = []
        for rid in ids:
            req = self._requests.pop(rid)
            if req.status == "error":
                raise RuntimeError(f"request {rid!r}: {req.error}")
            outs.append(list(req.generated))
        return outs

    def request(self, rid: Hashable) -> Request:
        """The record of a live request (one that ``step()`` has reported finished is forgotten)."""
        return self._requests[rid]

    def forward_logits(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """The raw step function (see ModelRunner.step), for tests and trace replay."""
        return self.runner.step(entries)

    def stats(self) -> dict:
        s = dict(self.scheduler.stats)
        s.update(model_steps=self.runner.steps, tokens_run=self.runner.tokens_run,
                 pages_free=self.runner.cache.free_pages(),
                 prefix_nodes=self.prefix.num_nodes if self.prefix else 0,
                 prefix_hit_pages=self.prefix.hits if self.prefix else 0)
        return s
