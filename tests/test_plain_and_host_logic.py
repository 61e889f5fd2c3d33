"""The plain implementation, and the engine's host logic against it (no GPU).

The second half drives the real ModelRunner / Engine (cache manager, block tables, step
metadata, scheduler) with dense-tensor stand-ins for the kernels (tests/standin_ops.py), so
that a fault of the cache or the batch shows here, where no GPU exists.
"""
import math

import pytest
import torch

import cuttings
import plain_llama
import replay_util
import standin_ops
import tiny_models
from llm_singularity_b200.engine import ModelRunner
from llm_singularity_b200.engine.engine import Engine
from llm_singularity_b200.parts.rotary import rotary_inv_freq
from llm_singularity_b200.config.specs import Llama3RopeScaling


# ------------------------------------------------------------------ plain parts
def test_rms_norm_by_hand():
    # tests/test_kernels.cpp:33-95: 2x4 rows against sqrt(mean) by hand
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0], [0.5, -0.5, 0.5, -0.5]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 0.5, 1.0], dtype=torch.float64)
    y = plain_llama.rms_norm(x, w, 1e-5)
    r0 = math.sqrt((1 + 4 + 9 + 16) / 4 + 1e-5)
    assert torch.allclose(y[0], torch.tensor([1 / r0, 4 / r0, 1.5 / r0, 4 / r0], dtype=torch.float64))
    assert torch.allclose(y[1].abs(), torch.tensor([1, 2, .5, 1], dtype=torch.float64) * 0.5 / math.sqrt(0.25 + 1e-5))


def test_rope_pairs_split_halves_and_position_zero_is_identity():
    # kernels/src/rope.cu:20-21 rotates (i, i + hd/2); CLAUDE.md:87: position 0 hides a wrong pairing
    x = torch.arange(1.0, 9.0, dtype=torch.float64).view(1, 2, 4).repeat(2, 1, 1)
    inv = plain_llama.rope_inv_freq(4, 10000.0)
    assert torch.allclose(inv, torch.tensor([1.0, 0.01], dtype=torch.float64))
    y = plain_llama.apply_rope(x, [0, 1], inv)
    assert torch.equal(y[0], x[0])
    c, s = math.cos(1.0), math.sin(1.0)
    assert abs(y[1, 0, 0] - (1 * c - 3 * s)) < 1e-6 and abs(y[1, 0, 2] - (1 * s + 3 * c)) < 1e-6
    c2, s2 = math.cos(0.01), math.sin(0.01)
    assert abs(y[1, 0, 1] - (2 * c2 - 4 * s2)) < 1e-6 and abs(y[1, 0, 3] - (2 * s2 + 4 * c2)) < 1e-6


def test_llama3_scaling_two_restatements_agree():
    sc = dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=64)
    for hd, theta in ((32, 500000.0), (64, 500000.0), (16, 10000.0)):
        plain = plain_llama.rope_inv_freq(hd, theta, sc)
        ours = rotary_inv_freq(hd, theta, Llama3RopeScaling(32.0, 1.0, 4.0, 64))
        assert torch.allclose(plain, ours, rtol=1e-12, atol=0)
        base = plain_llama.rope_inv_freq(hd, theta)
        assert torch.equal(plain[0], base[0])                        # shortest wavelength kept
        assert torch.allclose(plain[-1], base[-1] / 32.0)            # longest stretched by factor
        assert ((plain <= base) & (plain >= base / 32.0 * (1 - 1e-12))).all()


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8, dtype=torch.float64), torch.randn(6, 2, 8, dtype=torch.float64), \
        torch.randn(6, 2, 8, dtype=torch.float64)
    full = plain_llama.causal_attention(q, k, v, 0.3)
    assert torch.allclose(full[0, 1], v[0, 0]) and torch.allclose(full[0, 3], v[0, 1])   # one key
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, 9.0
    assert torch.allclose(plain_llama.causal_attention(q, k2, v2, 0.3)[:4], full[:4])     # no future
    w1 = plain_llama.causal_attention(q, k, v, 0.3, window=1)
    assert torch.allclose(w1[:, 0], v[:, 0])                                              # only itself


def test_plain_sampler_follows_the_reference_cases():
    # tests/test_sampling.cpp:6-47
    logits = [1.0, 5.0, 2.0, 5.0, -1.0]
    assert plain_llama.sample_plain(logits, temperature=0.0) == 1                  # first maximum
    assert plain_llama.sample_plain([0.1, 0.2, 10.0, 0.3], temperature=0.001, u=0.7) == 2
    seen = {plain_llama.sample_plain([1.0, 2.0, 3.0, 4.0], top_k=2, u=u / 20 + 0.01) for u in range(20)}
    assert seen == {2, 3}
    assert plain_llama.sample_plain([5.0, 1.0, 0.5], temperature=0.0, repetition_penalty=100.0,
                                    prev_tokens=[0]) != 0
    # top-p keeps the smallest set whose mass exceeds p
    seen = {plain_llama.sample_plain([2.0, 1.0, 0.0, -1.0], top_p=0.6, u=u / 50 + 0.001) for u in range(50)}
    assert seen == {0}                                                             # p0 = 0.64 > 0.6
    seen = {plain_llama.sample_plain([2.0, 1.0, 0.0, -1.0], top_p=0.7, u=u / 50 + 0.001) for u in range(50)}
    assert seen == {0, 1}


def test_plain_decode_equals_plain_prefix(model_dirs):
    cfg, w = plain_llama.load_model_dir(model_dirs["tiny_a"])
    toks = tiny_models.random_tokens(256, 12, 3)
    full = plain_llama.forward_logits(cfg, w, toks)
    assert torch.allclose(plain_llama.forward_logits(cfg, w, toks[:7]), full[:7], atol=1e-12)


# ------------------------------------------------- host logic with stand-in kernels
def _requests(name, lengths, seed=0):
    vocab = tiny_models.CONFIGS[name]["vocab_size"]
    return {f"r{i}": tiny_models.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def plain_refs(model_dirs):
    out = {}
    for name, lengths in (("tiny_a", (5, 17, 33, 70, 100, 64, 20)), ("tiny_b", (1, 9, 40, 70, 50, 23))):
        cfg, w = plain_llama.load_model_dir(model_dirs[name])
        seqs = _requests(name, lengths)
        out[name] = (seqs, {rid: plain_llama.forward_logits(cfg, w, t) for rid, t in seqs.items()})
    return out


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_host_logic_matches_plain_under_every_cutting(model_dirs, plain_refs, tmp_path, name, cut):
    seqs, refs = plain_refs[name]
    steps, max_tokens = getattr(cuttings, cut)(seqs)
    ps = tiny_models.PAGE_SIZE[name]
    runner = ModelRunner(model_dirs[name], dtype="float32", device="cpu", page_size=ps,
                         num_pages=max_tokens // ps, max_requests=4, max_model_len=max_tokens,
                         ops=standin_ops)
    held = replay_util.track_pages(runner)
    replay_util.replay_in_process(runner, steps, str(tmp_path))
    rows = replay_util.collect(steps, str(tmp_path), tiny_models.CONFIGS[name]["vocab_size"])
    replay_util.compare(rows, refs, 2e-5, f"{name}/{cut}")
    if cut == "mixed":
        replay_util.assert_pages_were_used_again(held, seqs, max_tokens, name)
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == max_tokens // ps          # everything was given back


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_mixed_cutting_really_reuses_pages_and_mixes(plain_refs, name):
    seqs, _ = plain_refs[name]
    steps, max_tokens = cuttings.mixed(seqs)
    assert max_tokens < sum(-(-len(t) // 64) * 64 for t in seqs.values())      # pool < total
    assert any(len(s["entries"]) >= 3 for s in steps)
    assert any(len({len(e["tokens"]) for e in s["entries"]}) > 1 and
               min(len(e["tokens"]) for e in s["entries"]) == 1 for s in steps)


def test_engine_greedy_matches_plain_even_with_few_pages_and_preemption(model_dirs):
    cfg, w = plain_llama.load_model_dir(model_dirs["tiny_a"])
    prompts = [tiny_models.random_tokens(256, n, 40 + n) for n in (5, 17, 33)]
    ref = [plain_llama.greedy_generate(cfg, w, p, 8) for p in prompts]
    for pages, chunk, ahead in ((64, None, True), (5, 7, False), (5, 7, True)):
        eng = Engine(model_dirs["tiny_a"], dtype="float32", device="cpu", kv_block_size=16,
                     num_kv_blocks=pages, max_batch_size=4, max_tokens_per_batch=24,
                     prefill_chunk=chunk, ops=standin_ops, prefix_cache=False, run_ahead=ahead)
        assert eng.generate(prompts, max_new_tokens=8, ignore_eos=True) == ref
        eng.runner.cache.check_invariants()
        assert eng.runner.cache.free_pages() == pages
        if pages == 5 and not ahead:
            # (a step planned ahead never preempts: a request that finds no page waits a step)
            assert eng.stats()["preemptions"] > 0


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_engine_running_ahead_yields_the_same_tokens(model_dirs, temperature):
    """Steps planned before the previous step's tokens are read (the tokens stay on the device
    side) against the plain loop: same tokens, also across a stop token found one step late."""
    prompts = [tiny_models.random_tokens(512, n, 90 + n) for n in (3, 12, 30)]
    outs, stats = [], []
    for ahead in (False, True):
        eng = Engine(model_dirs["tiny_b"], dtype="float32", device="cpu", kv_block_size=8,
                     num_kv_blocks=40, max_batch_size=4, max_tokens_per_batch=64,
                     ops=standin_ops, run_ahead=ahead)
        first = eng.generate(prompts, max_new_tokens=12, temperature=temperature, seed=5, ignore_eos=True)
        eng.scheduler.cfg.stop_token_ids = (first[1][4],)       # request 1 now stops at its fifth token
        second = eng.generate(prompts, max_new_tokens=12, temperature=temperature, seed=5)
        outs.append((first, second))
        stats.append(eng.stats())
        eng.runner.cache.check_invariants()
        assert not eng.has_work()
    assert outs[0] == outs[1]
    first, second = outs[1]
    stop = first[1][4]
    assert second[1] == first[1][:first[1].index(stop) + 1]
    assert stats[0].get("ahead_steps", 0) == 0 and stats[1]["ahead_steps"] >= 10


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_engine_under_a_random_load_yields_each_requests_own_tokens(model_dirs, seed):
    """Requests arrive while others run, with prompts that share beginnings, few pages, small
    budgets, stop tokens and sampled streams: whatever the scheduler makes of it (steps planned
    ahead, portions, waits for pages, preemption, shared pages), every request ends with the
    tokens it yields when it runs alone, and every page comes back."""
    import random
    rng = random.Random(seed)
    heads = [tiny_models.random_tokens(512, 16, 300 + i) for i in range(3)]
    jobs = []
    for i in range(14):
        prompt = (rng.choice(heads) if rng.random() < 0.6 else []) + \
            tiny_models.random_tokens(512, rng.randrange(1, 30), 400 + 17 * seed + i)
        jobs.append(dict(token_ids=prompt, max_new_tokens=rng.randrange(1, 14),
                         temperature=rng.choice([0.0, 0.9]), top_k=rng.choice([0, 5]), seed=i,
                         ignore_eos=rng.random() < 0.5))

    def engine(**kw):
        return Engine(model_dirs["tiny_b"], dtype="float32", device="cpu", kv_block_size=8,
                      ops=standin_ops, **kw)

    alone = engine(num_kv_blocks=64, max_batch_size=1, prefix_cache=False, run_ahead=False)
    stops = tuple(range(3, 512, 6))                              # every sixth token stops a request
    want = []
    alone.scheduler.cfg.stop_token_ids = stops
    for j in jobs:
        rid = alone.add_request(**j)
        rec, seen = alone.request(rid), []
        while alone.has_work():
            seen += [tok for r, tok, _ in alone.step() if r == rid]
        want.append(rec.generated)
        assert seen == rec.generated                # what step() reported is what the record holds
        with pytest.raises(KeyError):               # a finished request is forgotten ...
            alone.request(rid)
    again = alone.add_request(**dict(jobs[0], request_id=0))   # ... and its id can be used again
    while alone.has_work():
        alone.step()
    assert again == 0
    assert any(w[-1] in stops and len(w) < j["max_new_tokens"] for w, j in zip(want, jobs))

    for ahead, prefix, pages in ((True, True, 20), (True, False, 14), (False, True, 14)):
        eng = engine(num_kv_blocks=pages, max_batch_size=5, max_tokens_per_batch=24, prefill_chunk=9,
                     prefix_cache=prefix, run_ahead=ahead)
        eng.scheduler.cfg.stop_token_ids = stops
        ids, recs, todo, order = [], [], list(jobs), random.Random(seed + 100)
        while todo or eng.has_work():
            for _ in range(order.randrange(0, 3)):
                if todo:
                    ids.append(eng.add_request(**todo.pop(0)))
                    recs.append(eng.request(ids[-1]))
            eng.step()
        got = [r.generated for r in recs]
        assert got == want, (ahead, prefix, pages)
        assert all(r.status == "finished" and r.pending == 0 for r in recs)
        assert not eng._requests
        eng.runner.cache.check_invariants()
        if prefix:
            eng.prefix.check_invariants()
            eng.prefix.evict(10 ** 6)
        assert eng.runner.cache.free_pages() == pages
        if ahead:
            assert eng.stats()["ahead_steps"] > 10


def test_engine_shares_prompt_pages_between_live_requests_and_yields_the_same_tokens(model_dirs):
    """Prompts with a common beginning, admitted a few per step under a small token budget: the
    later ones adopt pages of the earlier ones while those still decode.  Tokens must be the same
    as without the prefix cache."""
    common = tiny_models.random_tokens(512, 24, 7)
    prompts = []
    for i in range(8):
        head = common if i % 2 == 0 else tiny_models.random_tokens(512, 24, 100 + i)
        prompts.append(head + tiny_models.random_tokens(512, 5 + i, 200 + i))
    outs, stats = [], []
    for sharing in (False, True):
        eng = Engine(model_dirs["tiny_b"], dtype="float32", device="cpu", kv_block_size=8,
                     num_kv_blocks=64, max_batch_size=8, max_tokens_per_batch=40,
                     ops=standin_ops, prefix_cache=sharing)
        outs.append(eng.generate(prompts, max_new_tokens=10, ignore_eos=True))
        stats.append(eng.stats())
        eng.runner.cache.check_invariants()
        if sharing:
            eng.prefix.check_invariants()
    assert outs[0] == outs[1]
    assert stats[1]["prefix_hit_pages"] >= 3 * 3 and stats[0]["prefix_hit_pages"] == 0


@pytest.mark.parametrize("seed", range(4))
def test_step_metadata_is_packed_like_the_plain_arrays(seed):
    """ContextBuilder (one pass in the host library) against the arrays written out in numpy, for
    random entries; lists and arrays of tokens alike; bad entries are refused by name."""
    import numpy as np
    import torch
    from llm_singularity_b200.engine.batch import ContextBuilder
    rng = np.random.default_rng(seed)
    b = ContextBuilder("cpu", 64, 4)                     # small: the buffers have to grow
    for _ in range(6):
        R = int(rng.integers(1, 7))
        q_len = rng.integers(1, 40, R)
        starts = rng.integers(0, 500, R)
        rows = rng.permutation(16)[:R]
        tokens = [rng.integers(0, 1000, n).astype(np.int32) for n in q_len]
        as_given = [t.tolist() if i % 2 else t for i, t in enumerate(tokens)]
        wants = [sorted(set(rng.integers(0, n, int(rng.integers(0, 4))).tolist())) for n in q_len]
        more = [rng.integers(0, 99, 5).astype(np.int32), np.empty(0, dtype=np.int32)]
        ctx, extra = b.build(as_given, starts.tolist(), rows.tolist(), wants, more)
        q_start = np.concatenate([[0], np.cumsum(q_len)])
        assert ctx.token_ids.tolist() == np.concatenate(tokens).tolist()
        assert ctx.positions.tolist() == [s + i for s, n in zip(starts, q_len) for i in range(n)]
        assert ctx.token_req.tolist() == [r for r, n in enumerate(q_len) for _ in range(n)]
        assert ctx.q_start.tolist() == q_start.tolist() == ctx.h_q_start.tolist()
        assert ctx.kv_len.tolist() == (starts + q_len).tolist() == ctx.h_kv_len.tolist()
        assert ctx.table_rows.tolist() == rows.tolist() == ctx.h_table_rows.tolist()
        assert ctx.want_rows.tolist() == [int(q_start[r]) + w for r in range(R) for w in wants[r]]
        assert (ctx.n_tokens, ctx.n_requests, ctx.n_wanted) == (int(q_len.sum()), R, sum(map(len, wants)))
        assert ctx.max_q_len == q_len.max() and ctx.max_kv_len == (starts + q_len).max()
        assert ctx.h_q_len.tolist() == q_len.tolist()
        assert [e.tolist() for e in extra] == [m.tolist() for m in more]
        assert all(t.dtype == torch.int32 for t in (ctx.token_ids, ctx.positions, ctx.want_rows))
    with pytest.raises(ValueError, match="entry 1: wanted place 3 outside its 3 tokens"):
        b.build([[1, 2], [3, 4, 5]], [0, 0], [0, 1], [[1], [0, 3]])
    with pytest.raises(ValueError, match="entry 0: wanted place -1"):
        b.build([[1, 2]], [0], [0], [[-1]])
    with pytest.raises(ValueError, match="every entry at least one token"):
        b.build([[1, 2], []], [0, 0], [0, 1], [[], []])
    with pytest.raises(ValueError, match="at least one entry"):
        b.build([], [], [], [])


def test_token_lists_become_arrays_or_are_refused(model_dirs):
    """Tokens come as lists, as arrays of any integer type or as any sequence; an id that does not
    fit 32 bits is refused like any id outside the vocabulary, by the request's name."""
    import numpy as np
    from llm_singularity_b200.engine import StepEntry
    from llm_singularity_b200.engine.runner import _token_array
    assert _token_array([1, 2, 3]).tolist() == [1, 2, 3] and _token_array([1, 2, 3]).dtype == np.int32
    assert _token_array(np.array([4, 5], dtype=np.int64)).dtype == np.int32
    assert _token_array(range(3)).tolist() == [0, 1, 2]
    assert _token_array([1, 2 ** 40]) is None and _token_array(np.array([2 ** 40])) is None
    with pytest.raises(TypeError):
        _token_array([1.5, 2])
    runner = ModelRunner(model_dirs["tiny_a"], dtype="float32", device="cpu", page_size=16, num_pages=4,
                         max_requests=2, max_model_len=64, ops=standin_ops)
    runner.open("a")
    for bad in ([1, 2 ** 40], [1, -1], [runner.vocab_size]):
        with pytest.raises(ValueError, match="request 'a': token id outside"):
            runner.step([StepEntry("a", bad, [])])
    assert runner.cache.free_pages() == 4
    out = runner.step([StepEntry("a", np.array([1, 2, 3], dtype=np.int64), [2])])
    assert out.shape == (1, runner.vocab_size)


def test_which_steps_get_a_graph(model_dirs):
    """The runner's decision alone (no device needed): single tokens that are all wanted share a
    graph per batch size; a step of one entry with prompt tokens gets one from its second
    occurrence on; steps of more entries only if asked for; the least recently used shape goes when
    there are more than ``max_shape_graphs``."""
    import numpy as np
    from llm_singularity_b200.engine import StepEntry
    runner = ModelRunner(model_dirs["tiny_a"], dtype="float32", device="cpu", page_size=16, num_pages=4,
                         max_requests=2, max_model_len=64, ops=standin_ops)
    assert not runner.cuda_graphs                      # (no device here: nothing is ever captured)

    def key(*entries):
        es = [StepEntry(f"r{i}", list(range(n)), list(want)) for i, (n, want) in enumerate(entries)]
        return runner._graph_key(es, [np.zeros(n, dtype=np.int32) for n, _ in entries], None)

    assert key((1, [0]), (1, [0]), (1, [0])) == (3, None)
    assert key((1, [])) is None and key((1, [])) == ((1,), ((),), None)     # a token nobody wants: a shape
    portion = (40, [39])
    assert key(portion) is None                        # first seen
    k = key(portion)
    assert k == ((40,), ((39,),), None)
    runner._graphs[k] = object()                       # (what capturing it would leave)
    assert key(portion) == k and key(portion) == k
    assert key((40, [39]), (1, [0])) is None and key((40, [39]), (1, [0])) is None      # two entries: never
    runner.shape_graph_entries = 2
    assert key((40, [39]), (1, [0])) is None and key((40, [39]), (1, [0])) is not None
    runner.shape_graph_entries = 1
    runner.max_shape_graphs = 2
    runner._shape_order[:] = [k]
    for n in (50, 60):
        key((n, [0])); kn = key((n, [0]))
        runner._graphs[kn] = object()
    assert k not in runner._graphs and len(runner._shape_order) == 2           # the oldest went
    assert key(portion) is None                        # and starts again from nothing
    runner.shape_graphs = False
    assert key(portion) is None and key(portion) is None


def test_a_step_that_does_not_fit_reserves_nothing(model_dirs):
    """Pages are taken for all entries of a step or for none: a step whose second entry finds no
    room leaves the first entry's request as it was (no page held back, no table update queued),
    and the first entry can then run alone."""
    from llm_singularity_b200.engine import OutOfPages, StepEntry
    runner = ModelRunner(model_dirs["tiny_a"], dtype="float32", device="cpu", page_size=16, num_pages=4,
                         max_requests=2, max_model_len=64, ops=standin_ops)
    runner.open("a"); runner.open("b")
    toks = tiny_models.random_tokens(256, 40, 3)
    with pytest.raises(OutOfPages, match="needs 5 more pages"):
        runner.step([StepEntry("a", toks[:30], []), StepEntry("b", toks[:40], [])])
    assert runner.cache.free_pages() == 4 and runner.cache.pages_of("a") == []
    assert runner.cache.take_updates(0) == []
    runner.step([StepEntry("a", toks[:30], [])])
    assert runner.cache.free_pages() == 2
    runner.cache.check_invariants()
