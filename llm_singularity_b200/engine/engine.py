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
from ..parts.base import PagedKVSpec
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduler, SchedulerConfig


class Engine:
    def __init__(self, model_dir: Optional[str] = None, *, random_weights: bool = False,
                 seed: int = 0, dtype="bfloat16", device="cuda:0", kv_block_size: int = 16,
                 num_kv_blocks: int = 1024, max_batch_size: int = 64,
                 max_tokens_per_batch: int = 2048, prefill_chunk: Optional[int] = None,
                 max_model_len: Optional[int] = None, prefix_cache: bool = True,
                 config=None, ops=None, verbose: bool = False):
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
            and all(isinstance(s, PagedKVSpec) for s in self.runner.model.cache_specs())
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
        self._requests: Dict[Hashable, Request] = {}

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
        return self.scheduler.has_work()

    # -------------------------------------------------------------------- step
    def step(self) -> List[Tuple[Hashable, int, bool]]:
        """Run one scheduled batch; returns (request id, new token, finished) for every request
        that produced a token, and (id, -1, True) for requests that ended with an error."""
        sch = self.scheduler
        items = sch.schedule()
        out: List[Tuple[Hashable, int, bool]] = []
        for req in sch.take_finished():            # errors found while scheduling
            out.append((req.id, -1, True))
        if not items:
            return out
        entries = [StepEntry(it.request.id, it.tokens, [len(it.tokens) - 1] if it.sample else [])
                   for it in items]
        logits = self.runner.step(entries)
        wanted = [it.request for it in items if it.sample]
        sampled: Dict[Hashable, int] = {}
        if wanted:
            toks = self.sampler.sample(
                logits, [r.sampling for r in wanted], [len(r.generated) for r in wanted],
                [r.generated for r in wanted])
            host = toks.to("cpu").tolist()
            sampled = {r.id: t for r, t in zip(wanted, host)}
        done = {r.id for r in sch.update(sampled)}
        sch.take_finished()
        for r in wanted:
            out.append((r.id, sampled[r.id], r.id in done))
        return out

    # ---------------------------------------------------------------- generate
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16,
                 temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                 repetition_penalty: float = 1.0, seed: int = 0,
                 ignore_eos: bool = False) -> List[List[int]]:
        """Generate for every prompt; request i samples with seed ``seed + i``.  Returns the
        generated tokens (stop token included), in the order of the prompts."""
        ids = [self.add_request(p, max_new_tokens, temperature, top_k, top_p, repetition_penalty,
                                seed + i, ignore_eos) for i, p in enumerate(prompts)]
        while self.has_work():
            self.step()
        outs = []
        for rid in ids:
            req = self._requests.pop(rid)
            if req.status == "error":
                raise RuntimeError(f"request {rid!r}: {req.error}")
            outs.append(list(req.generated))
        return outs

    def request(self, rid: Hashable) -> Request:
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
