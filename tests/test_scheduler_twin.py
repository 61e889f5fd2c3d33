"""The native scheduler (csrc/host_scheduler.cpp behind engine/scheduler.py) against the plain one
in Python (tests/plain_scheduler.py over tests/plain_memory.py): the same random load on both, with
and without prefix sharing, with steps planned ahead at random, few pages so that requests are
preempted, stop tokens and requests that can never fit.  Every planned step, every finished or
failed request, every counter and every page id must be the same."""
import random

import pytest

import plain_memory
import plain_scheduler
from llm_singularity_b200.cache import CacheManager
from llm_singularity_b200.cache.prefix import RadixPrefixCache
from llm_singularity_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
from llm_singularity_b200.parts.base import PagedKVSpec
from llm_singularity_b200.sampling.params import SamplingParams

STOP = 7


def _pair(rng, sharing):
    page = rng.choice([4, 8])
    pages = rng.choice([10, 16, 40])
    slots = rng.choice([2, 4])
    max_pages = rng.choice([6, 12])
    cfg = dict(max_batch_size=slots, max_tokens_per_batch=rng.choice([8, 24, 64]),
               max_prefill_chunk=rng.choice([None, 5, 16]), stop_token_ids=(STOP,),
               max_model_len=min(rng.choice([40, 1 << 30]), max_pages * page))   # as the engine sets it
    specs = [PagedKVSpec(2, 16), PagedKVSpec(1, 32)]          # one group: both keep all keys
    ca = CacheManager(specs, page, pages, slots, max_pages)
    cb = plain_memory.PlainCacheManager(specs, page, pages, slots, max_pages)
    a = Scheduler(SchedulerConfig(**cfg), ca, RadixPrefixCache(ca) if sharing else None)
    b = plain_scheduler.PlainScheduler(plain_scheduler.SchedulerConfig(**cfg), cb,
                                       plain_memory.PlainPrefixCache(cb) if sharing else None)
    return a, b


def _view(items):
    return None if items is None else [(it.request.id, it.start, list(it.tokens), it.sample, it.decode)
                                       for it in items]


def _same(a, b):
    assert [r.id for r in a.waiting] == [r.id for r in b.waiting]
    assert [r.id for r in a.running] == [r.id for r in b.running]
    for ra, rb in zip(list(a.waiting) + a.running, list(b.waiting) + b.running):
        assert (ra.tokens, ra.generated, ra.computed, ra.pending, ra.status, ra.preemptions) == \
               (rb.tokens, rb.generated, rb.computed, rb.pending, rb.status, rb.preemptions)
    for r in a.running:
        assert a.cache.pages_of(r.id) == b.cache.pages_of(r.id)
    sa, sb = a.stats, b.stats
    assert all(sa[k] == sb.get(k, 0) for k in sa)
    assert a.cache.free_pages() == b.cache.free_pages()
    if a.prefix is not None:
        assert a.prefix.num_nodes == b.prefix.num_nodes and a.prefix.hits == b.prefix.hits


@pytest.mark.parametrize("sharing", [False, True])
@pytest.mark.parametrize("seed", range(8))
def test_native_and_plain_scheduler_decide_alike(seed, sharing):
    rng = random.Random(1000 * sharing + seed)
    a, b = _pair(rng, sharing)
    stems = [[rng.randrange(3, 6) for _ in range(48)] for _ in range(2)]
    names = iter(range(10 ** 6))
    in_flight = []                  # plans not yet accounted, oldest first: (items of a, items of b)
    finished = []

    def token(req_id, n_generated):
        return STOP if (req_id * 31 + n_generated * 17) % 11 == 0 else 10 + (req_id + n_generated) % 5

    def account():
        items_a, _ = in_flight.pop(0)
        sampled = {it.request.id: token(it.request.id, len(it.request.generated))
                   for it in items_a if it.sample and it.request.status == "running"}
        da, db = a.update(dict(sampled)), b.update(dict(sampled))
        assert [r.id for r in da] == [r.id for r in db]

    for _ in range(300):
        if rng.random() < 0.3:
            n = next(names)
            toks = rng.choice(stems)[:rng.randrange(1, 48)] + [rng.randrange(3, 6) for _ in range(rng.randrange(0, 4))]
            kw = dict(max_new_tokens=rng.randrange(1, 12), ignore_eos=rng.random() < 0.3,
                      sampling=SamplingParams(repetition_penalty=rng.choice([1.0, 1.0, 1.0, 1.3])))
            a.add(Request(n, list(toks), **kw))
            b.add(plain_scheduler.Request(n, list(toks), **kw))
        if not in_flight:
            ia, ib = a.schedule(), b.schedule()
            assert _view(ia) == _view(ib)
            if ia:
                in_flight.append((ia, ib))
        if in_flight and rng.random() < 0.7:               # plan the step after the one in flight
            ia, ib = a.schedule_ahead(), b.schedule_ahead()
            assert _view(ia) == _view(ib)
            if ia:
                in_flight.append((ia, ib))
        if in_flight:
            account()
        fa, fb = a.take_finished(), b.take_finished()
        assert [(r.id, r.status, r.generated, r.error) for r in fa] == \
               [(r.id, r.status, r.generated, r.error) for r in fb]
        finished += fa
        _same(a, b)
        a.cache.check_invariants()
    while in_flight:
        account()
    assert finished and any(r.status == "finished" for r in finished)


def test_a_handle_used_again_is_not_mistaken_for_the_request_that_had_it():
    ca = CacheManager([PagedKVSpec(2, 16)], 4, 16, 2, 8)
    sch = Scheduler(SchedulerConfig(max_batch_size=2, max_tokens_per_batch=32, stop_token_ids=(STOP,)), ca)
    sch.add(Request("a", [1, 2, 3], 8))
    sch.schedule()
    assert sch.schedule_ahead() is not None               # a's first decode token, planned ahead
    assert [r.id for r in sch.update({"a": STOP})] == ["a"]  # ... but a stops on the token in flight
    sch.take_finished()                                   # its handle is free again
    sch.add(Request("b", [4, 5, 6, 7, 8], 8))             # and goes to b
    items = sch.schedule_ahead()                          # b's prompt, behind a's stray step
    assert [(it.request.id, it.start, it.tokens) for it in items] == [("b", 0, [4, 5, 6, 7, 8])]
    b = sch.running[0]
    assert b.handle == items[0].request.handle == 0       # the handle a had
    assert sch.update({"a": 3}) == []                     # the stray step of a: nothing of b's is touched
    assert b.generated == [] and b.tokens == [4, 5, 6, 7, 8, Scheduler.PENDING] and b.pending == 1
    assert sch.update({"b": 9}) == [] and b.generated == [9] and b.tokens[-1] == 9
    ca.check_invariants()
