"""The scheduler's decisions, driven without a model (no GPU): sampled tokens are handed in,
as the reference's scheduler tests do (tests/test_scheduler.cpp:24-216)."""
import pytest

from llm_singularity_b200.cache import CacheManager
from llm_singularity_b200.cache.prefix import RadixPrefixCache
from llm_singularity_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
from llm_singularity_b200.parts.base import PagedKVSpec
from llm_singularity_b200.sampling import SamplingParams

EOS = 2


def make(pages=100, page=16, slots=8, budget=512, chunk=None, prefix=False, max_len=1 << 20):
    cache = CacheManager([PagedKVSpec(1, 16)], page, pages, slots, 4096)
    pc = RadixPrefixCache(cache) if prefix else None
    sch = Scheduler(SchedulerConfig(max_batch_size=slots, max_tokens_per_batch=budget,
                                    max_prefill_chunk=chunk, stop_token_ids=(EOS,),
                                    max_model_len=max_len), cache, pc)
    return sch, cache


def req(rid, n, max_new=4, first=10, **kw):
    return Request(rid, list(range(first, first + n)), max_new, SamplingParams(0.0), **kw)


def run_step(sch, token=7):
    """One schedule + update in which every sampling request gets ``token`` (or token[rid])."""
    items = sch.schedule()
    sampled = {it.request.id: (token[it.request.id] if isinstance(token, dict) else token)
               for it in items if it.sample}
    done = sch.update(sampled)
    return items, done


def test_two_prompts_prefill_in_one_step():
    sch, cache = make()
    sch.add(req("a", 32)); sch.add(req("b", 20))
    items = sch.schedule()
    assert [(it.request.id, it.start, len(it.tokens), it.sample) for it in items] == \
        [("a", 0, 32, True), ("b", 0, 20, True)]
    assert cache.pages_of("a") == [0, 1] and cache.pages_of("b") == [2, 3]


def test_eos_completes_and_frees_pages_output_includes_stop_token():
    sch, cache = make()
    sch.add(req("a", 32, max_new=10))
    run_step(sch, 7)
    assert 100 - cache.free_pages() == 2          # 32 tokens; the next page comes with the decode step
    items, done = run_step(sch, EOS)
    assert [it.tokens for it in items] == [[7]] and items[0].start == 32
    assert [r.id for r in done] == ["a"] and done[0].generated == [7, EOS] and done[0].status == "finished"
    assert cache.free_pages() == 100 and not sch.has_work()


def test_ignore_eos_and_max_new_tokens():
    sch, _ = make()
    sch.add(req("a", 5, max_new=3, ignore_eos=True))
    outs = [run_step(sch, EOS) for _ in range(3)]
    assert [len(d) for _, d in outs] == [0, 0, 1] and outs[2][1][0].generated == [EOS] * 3


def test_long_prompt_is_cut_under_the_token_budget_and_sampled_only_at_its_end():
    sch, _ = make(budget=128)
    sch.add(req("a", 300))
    seen = []
    for _ in range(3):
        items, _ = run_step(sch)
        seen.append([(it.start, len(it.tokens), it.sample) for it in items])
    assert seen == [[(0, 128, False)], [(128, 128, False)], [(256, 44, True)]]
    assert sch.running[0].generated == [7]       # exactly one token, after the last portion


def test_decode_tokens_come_first_then_portions_fill_the_budget():
    sch, _ = make(budget=64, chunk=24)
    sch.add(req("a", 10))
    run_step(sch)                                # a: prompt done, one token sampled
    sch.add(req("b", 100)); sch.add(req("c", 30))
    items, _ = run_step(sch)
    assert [(it.request.id, it.start, len(it.tokens)) for it in items] == \
        [("a", 10, 1), ("b", 0, 24), ("c", 0, 24)]
    items, _ = run_step(sch)
    assert [(it.request.id, it.start, len(it.tokens), it.sample) for it in items] == \
        [("a", 11, 1, True), ("b", 24, 24, False), ("c", 24, 6, True)]
    items, _ = run_step(sch)                     # c decodes now; b continues
    assert [(it.request.id, len(it.tokens)) for it in items] == [("a", 1), ("c", 1), ("b", 24)]


def test_admission_is_first_come_first_served_without_overtaking():
    sch, cache = make(pages=6, page=16)
    sch.add(req("big", 90))                      # needs 6 pages (91 tokens)
    sch.add(req("huge", 80)); sch.add(req("small", 5))
    items, _ = run_step(sch)
    assert [it.request.id for it in items] == ["big"]
    assert [r.id for r in sch.waiting] == ["huge", "small"]     # small does not jump the queue


def test_a_request_that_can_never_fit_ends_with_an_error():
    sch, _ = make(pages=4, page=16)
    sch.add(req("x", 64)); sch.add(req("ok", 10))
    items, _ = run_step(sch)
    assert [it.request.id for it in items] == ["ok"]
    bad = [r for r in sch.take_finished() if r.status == "error"]
    assert [r.id for r in bad] == ["x"] and "pages" in bad[0].error
    sch2, _ = make(pages=4, page=16)
    sch2.add(req("x", 64))
    assert sch2.schedule() == []
    (x,) = sch2.take_finished()
    assert x.status == "error" and "pages" in x.error
    sch3, _ = make(max_len=32)
    sch3.add(req("y", 32))
    sch3.schedule()
    assert "max_model_len" in sch3.take_finished()[0].error


def test_pages_run_out_while_decoding_youngest_is_preempted_and_recomputed():
    sch, cache = make(pages=4, page=4, budget=64)
    sch.add(req("old", 7, max_new=8)); sch.add(req("young", 6, max_new=8))
    run_step(sch, {"old": 50, "young": 60})      # 2 pages each: pool full
    assert cache.free_pages() == 0
    items, _ = run_step(sch, {"old": 51, "young": 61})          # old at 8 -> fits page 2; young 7 -> fits
    assert [it.request.id for it in items] == ["old", "young"]
    # now old holds 9 tokens -> needs a third page: young (most recently admitted) gives way
    items, _ = run_step(sch, {"old": 52, "young": 62})
    assert [it.request.id for it in items] == ["old"]
    assert sch.stats["preemptions"] == 1 and [r.id for r in sch.waiting] == ["young"]
    young = sch.waiting[0]
    assert young.tokens == list(range(10, 16)) + [60, 61] and young.computed == 0
    assert not cache.has("young")
    cache.check_invariants()
    # old finishes; young comes back, recomputes prompt + its two tokens, then goes on
    while sch.running and sch.running[0].id == "old":
        run_step(sch, {"old": 53, "young": 63})
    items, _ = run_step(sch, {"young": 63})
    assert [(it.request.id, it.start, len(it.tokens), it.sample) for it in items] == [("young", 0, 8, True)]
    assert young.generated == [60, 61, 63]       # its stream continued where it stopped
    cache.check_invariants()


def test_prefill_waits_for_pages_instead_of_preempting():
    sch, cache = make(pages=6, page=4, budget=64)
    sch.add(req("a", 11, max_new=20))
    run_step(sch)                                # a holds 3 pages (12 tokens)
    sch.add(req("b", 7))                         # needs 2 pages (8 tokens): fits
    items, _ = run_step(sch)
    assert [it.request.id for it in items] == ["a", "b"]
    sch.add(req("c", 3))                         # a and b now hold 4 + 2 pages: none left, c waits
    items, _ = run_step(sch)
    assert cache.free_pages() == 0
    assert "c" not in [it.request.id for it in items] and sch.stats["preemptions"] == 0


def test_same_prompt_again_starts_after_the_cached_pages():
    sch, cache = make(prefix=True)
    sch.add(req("a", 40, max_new=1))
    _, done = run_step(sch)
    assert done and cache.free_pages() == 98     # two full pages stay in the prefix cache
    sch.add(req("b", 40, max_new=1))
    items = sch.schedule()
    assert [(it.start, len(it.tokens), it.sample) for it in items] == [(32, 8, True)]
    assert sch.stats["prefix_hit_tokens"] == 32
    sch.update({"b": 7})
    # a prompt that is exactly the cached pages still runs its last page
    sch.add(req("c", 32, max_new=1))
    items = sch.schedule()
    assert [(it.start, len(it.tokens)) for it in items] == [(16, 16)]
    cache.check_invariants()


def test_cached_prefixes_are_evicted_before_anyone_is_preempted():
    sch, cache = make(pages=4, page=4, prefix=True)
    sch.add(req("a", 9, max_new=1))
    run_step(sch)
    assert cache.free_pages() == 2               # two full pages kept for later prompts
    sch.add(req("b", 13, max_new=1, first=500))  # needs 4 pages (14 tokens)
    items, done = run_step(sch)
    assert [it.request.id for it in items] == ["b"] and sch.stats["evicted_pages"] == 2
    assert sch.stats["preemptions"] == 0 and done
    cache.check_invariants()


# ------------------------------------------------------------- planning ahead
P = Scheduler.PENDING


def plan_of(items):
    return [(it.request.id, it.start, it.tokens if len(it.tokens) == 1 else len(it.tokens), it.sample)
            for it in items]


def test_the_next_step_is_planned_while_one_is_in_flight():
    sch, cache = make()
    sch.add(req("a", 20, max_new=6, ignore_eos=True)); sch.add(req("b", 5, max_new=6, ignore_eos=True))
    first = sch.schedule()                                   # both prompts whole, both sample
    # the first half of the accounting: the prompts count as run, place-holders stand for the tokens
    assert [(r.computed, r.pending, r.tokens[-1]) for r in sch.running] == [(20, 1, P), (5, 1, P)]
    ahead = sch.schedule_ahead()                             # their first decode step, token unknown
    assert plan_of(ahead) == [("a", 20, [P], True), ("b", 5, [P], True)]
    assert cache.pages_of("a") == [0, 1] and len(cache.pages_of("b")) == 1
    assert sch.schedule_ahead() is None                      # never two steps ahead
    with pytest.raises(RuntimeError):
        sch.schedule()                                       # plain planning wants every step accounted
    assert sch.update({"a": 7, "b": 8}) == []                # accounts the first step
    assert [r.tokens[-2:] for r in sch.running] == [[7, P], [8, P]]
    assert [r.computed for r in sch.running] == [21, 6]
    again = sch.schedule_ahead()                             # the step after the one planned ahead
    assert [(it.request.id, it.start) for it in again] == [("a", 21), ("b", 6)]
    sch.update({"a": 9, "b": 9})
    assert [r.generated for r in sch.running] == [[7, 9], [8, 9]]
    sch.update({"a": 1, "b": 1})
    assert [(r.computed, r.pending, r.tokens[-3:]) for r in sch.running] == [(22, 0, [7, 9, 1]), (7, 0, [8, 9, 1])]
    assert first and sch.stats["ahead_steps"] == 2
    cache.check_invariants()


def test_prompt_portions_and_admissions_are_planned_ahead_too():
    sch, cache = make(budget=16, slots=2)
    sch.add(req("a", 40, max_new=3, ignore_eos=True))
    assert plan_of(sch.schedule()) == [("a", 0, 16, False)]
    assert plan_of(sch.schedule_ahead()) == [("a", 16, 16, False)]       # nothing of it is unknown
    sch.update({})
    sch.add(req("b", 30, max_new=3, ignore_eos=True))
    assert plan_of(sch.schedule_ahead()) == [("a", 32, 8, True), ("b", 0, 8, False)]   # b is admitted
    sch.update({})
    assert plan_of(sch.schedule_ahead()) == [("a", 40, [P], True), ("b", 8, 15, False)]
    sch.update({"a": 7})
    sch.add(req("c", 4))
    ahead = sch.schedule_ahead()                             # c waits for a slot; the others go on
    assert plan_of(ahead) == [("a", 41, [P], True), ("b", 23, 7, True)]
    sch.update({"a": 8})
    assert plan_of(sch.schedule_ahead()) == [("b", 30, [P], True)]       # a's third token is in flight: its last
    assert [r.id for r in sch.update({"a": 9, "b": 5})] == ["a"]
    assert plan_of(sch.schedule_ahead()) == [("b", 31, [P], True), ("c", 0, 4, True)]
    assert sch.stats["ahead_steps"] == 6 and sch.stats["preemptions"] == 0
    cache.check_invariants()


def test_what_is_not_planned_ahead():
    sch, _ = make()
    sch.add(req("a", 8, max_new=2, ignore_eos=True))
    sch.schedule()
    assert sch.schedule_ahead() is not None                  # one more token to come after this one
    sch.update({"a": 5})
    assert sch.schedule_ahead() is None                      # the token in flight is its last
    assert [r.id for r in sch.update({"a": 5})] == ["a"] and not sch.has_work()
    sch, _ = make(max_len=10)
    sch.add(req("a", 8, max_new=8, ignore_eos=True))
    sch.schedule()
    assert sch.schedule_ahead() is not None                  # position 8, the sequence grows to 10
    sch.update({"a": 5})
    assert sch.schedule_ahead() is None                      # the model's length ends it
    assert [r.id for r in sch.update({"a": 5})] == ["a"] and sch.finished[0].generated == [5, 5]
    sch, _ = make()
    sch.add(Request("p", [1, 2, 3], 8, SamplingParams(0.7, repetition_penalty=1.3), True))
    sch.add(req("a", 8))
    sch.schedule()
    assert sch.schedule_ahead() is None                      # the penalty needs the token on the host


def test_a_step_planned_ahead_waits_for_pages_and_never_preempts():
    sch, cache = make(pages=3, page=16)
    sch.add(req("a", 31, max_new=8, ignore_eos=True)); sch.add(req("b", 10, max_new=8, ignore_eos=True))
    sch.schedule()
    assert plan_of(sch.schedule_ahead()) == [("a", 31, [P], True), ("b", 10, [P], True)]
    sch.update({"a": 5, "b": 5})
    assert plan_of(sch.schedule_ahead()) == [("b", 11, [P], True)]       # a's position 32 finds no page: a waits
    sch.update({"a": 5, "b": 5})
    assert sch.stats["preemptions"] == 0
    sch.update({"b": 5})
    items = sch.schedule()                                   # the plain plan decides: the youngest gives way
    assert plan_of(items) == [("a", 32, [5], True)] and sch.stats["preemptions"] == 1
    cache.check_invariants()


def test_a_request_that_stops_on_the_token_in_flight_is_skipped_in_the_step_planned_ahead():
    sch, cache = make()
    sch.add(req("a", 8, max_new=8)); sch.add(req("b", 8, max_new=8))
    sch.schedule()
    assert sch.schedule_ahead() is not None
    done = sch.update({"a": EOS, "b": 7})                    # a stops; the step ahead already holds it
    assert [r.id for r in done] == ["a"]
    with pytest.raises(KeyError):
        cache.pages_of("a")                                  # everything it held is given back
    a = next(r for r in sch.take_finished() if r.id == "a")
    assert a.generated == [EOS] and a.tokens == list(range(10, 18)) + [EOS] and a.pending == 0
    assert plan_of(sch.schedule_ahead()) == [("b", 9, [P], True)]
    done = sch.update({"a": 3, "b": 9})                      # a's token from the step ahead is dropped
    assert done == [] and sch.running[0].generated == [7, 9]
    sch.update({"b": 4})
    assert sch.running[0].tokens[-3:] == [7, 9, 4] and sch.running[0].pending == 0
    cache.check_invariants()


def test_a_running_requests_prompt_pages_are_shared_with_a_later_prompt():
    sch, cache = make(pages=12, page=16, prefix=True)
    a = req("a", 48, max_new=3, ignore_eos=True)
    sch.add(a)
    run_step(sch, 7)                                         # a's prompt has run; a goes on decoding
    assert a.status == "running" and sch.prefix.num_nodes == 3
    b = Request("b", a.prompt[:32] + list(range(500, 520)), 3, SamplingParams(0.0), True)
    sch.add(b)
    items = sch.schedule()
    by = {it.request.id: it for it in items}
    assert by["b"].start == 32 and len(by["b"].tokens) == 20 and by["a"].tokens == [7]
    assert cache.pages_of("b")[:2] == cache.pages_of("a")[:2] and sch.stats["prefix_hit_tokens"] == 32
    cache.check_invariants(); sch.prefix.check_invariants()
    sch.update({"a": 8, "b": 9})
    # a's shared pages are in use twice over: not offered for eviction, and evicting frees nothing
    assert sch.prefix.evictable_pages() == 0 and sch.prefix.evict(4) == 0
    run_step(sch, 5)                                         # a reaches max_new_tokens and ends
    assert a.status == "finished" and b.status == "running"
    assert cache.pages_of("b")[:2] == [n.pages[0] for n in sch.prefix.match(b.tokens)[:2]]
    cache.check_invariants()
    run_step(sch, 5)
    assert b.status == "finished" and not sch.has_work()
    cache.check_invariants(); sch.prefix.check_invariants()
    sch.prefix.evict(100)
    sch.prefix.check_invariants()
    assert cache.free_pages() == 12 and sch.prefix.num_nodes == 0
