"""Schedules that the tiny replay traces do not reach, on the GPU against the plain implementation:

* pages taken from the prefix tree, eviction and preemption-and-recompute through ``Engine`` at
  the head sizes of the tensor-core attention kernels (64 and 128), in bfloat16 and in 32-bit;
* the shapes the benchmark runs, at the flagship widths with two of the sixteen layers: a
  2,048-token prompt whole and as four portions of 512, and 64 requests decoding at some 4,090
  cached tokens;
* a block table with two cells swapped between two live requests, which the comparison has to
  catch at the tolerance the other tests use.
"""
import tempfile

import numpy as np
import pytest
import torch

import plain_llama
import tiny_models
from greedy_util import check_greedy

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4
BF16_REL = 4e-2          # of the largest plain logit; see test_replay_gpu.py for the reasoning


def _tol(dtype, ref_rows):
    if dtype == "float32":
        return F32_TOL
    return BF16_REL * float(ref_rows.abs().max())


def _plain(cfg, w, tokens, dtype, **kw):
    return plain_llama.forward_logits(cfg, w, tokens,
                                      act_round="bfloat16" if dtype == "bfloat16" else None, **kw)


# ------------------------------------------------- shared pages, eviction, preemption
SHARED = 128
POOL = {"tiny_d": 44, "tiny_e": 18}      # pages: too few for four live requests of these lengths


def _prompts(name):
    """Six prompts of 256 to 300 tokens; every other one begins with the same 128 tokens."""
    vocab = tiny_models.CONFIGS[name]["vocab_size"]
    shared = tiny_models.random_tokens(vocab, SHARED, 901)
    out = []
    for i, n in enumerate((150, 272, 131, 300, 165, 257)):
        own = tiny_models.random_tokens(vocab, n, 910 + i)
        out.append(shared + own if i % 2 == 0 else own)
    return out


def _engine(model_dir, name, dtype, **kw):
    from llm_singularity_b200 import Engine
    opts = dict(dtype=dtype, kv_block_size=tiny_models.PAGE_SIZE[name], num_kv_blocks=256,
                max_batch_size=4, max_tokens_per_batch=192, prefill_chunk=160)
    opts.update(kw)
    return Engine(model_dir, **opts)


def _common(a, b):
    n = 0
    while n < min(len(a), len(b)) and a[n] == b[n]:
        n += 1
    return n


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", ["tiny_d", "tiny_e"])
def test_adopted_pages_eviction_and_preemption_give_the_cold_run_tokens(model_dirs, name, dtype):
    """Prompts of 256 tokens and more in portions of 160 (the tcgen05 kernel takes those of 128
    and more, the mma.sync kernel the rest, the split-KV kernel the decode tokens), half of them
    sharing their first 128 tokens, through a pool so small that prefix pages are evicted and
    requests are preempted and recomputed: the tokens of a roomy engine without prefix cache."""
    from llm_singularity_b200 import kernels
    cfg, w = plain_llama.load_model_dir(model_dirs[name])
    prompts = _prompts(name)
    cold = _engine(model_dirs[name], name, dtype, prefix_cache=False)
    want = cold.generate(prompts, max_new_tokens=24, ignore_eos=True)
    assert cold.stats()["preemptions"] == 0 and cold.stats()["prefix_hit_tokens"] == 0
    margin = 1e-3 if dtype == "float32" else 0.08
    cold_held = sum(check_greedy(cfg, w, p, c, margin, f"{name}/{dtype}/cold") for p, c in zip(prompts, want))
    assert cold_held >= 6 * 24 // 2
    for ahead in (False, True):
        tight = _engine(model_dirs[name], name, dtype, num_kv_blocks=POOL[name], run_ahead=ahead)
        got = tight.generate(prompts, max_new_tokens=24, ignore_eos=True)
        s = tight.stats()
        assert s["preemptions"] > 0 and s["evicted_pages"] > 0 and s["prefix_hit_tokens"] >= 2 * SHARED, s
        held = sum(check_greedy(cfg, w, p, g, margin, f"{name}/{dtype}/ahead={ahead}")
                   for p, g in zip(prompts, got))
        assert held >= 6 * 24 // 2, f"only {held} tokens could be compared"
        # the same tokens as the cold run, up to the first near-tie of each request
        same = sum(_common(g, c) for g, c in zip(got, want))
        assert same >= 6 * 24 // 2, (got, want)
        if dtype == "float32":
            assert got == want
        kernels.check_status()
        tight.runner.cache.check_invariants()
        assert tight.runner.cache.free_pages() + tight.prefix.evictable_pages() == POOL[name]


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", ["tiny_d", "tiny_e"])
def test_logits_over_adopted_pages_match_plain(model_dirs, name, dtype):
    """A request that starts on another request's pages (its first 128 tokens come from the
    prefix tree): the logits of its own portion, run as one step of 130 and more tokens over the
    adopted pages, and of three further tokens decoded one by one, against the plain rows."""
    from llm_singularity_b200 import kernels
    from llm_singularity_b200.engine import StepEntry
    cfg, w = plain_llama.load_model_dir(model_dirs[name])
    prompts = _prompts(name)
    donor, taker = prompts[0], prompts[2]
    eng = _engine(model_dirs[name], name, dtype)
    eng.generate([donor], max_new_tokens=2, ignore_eos=True)
    runner, prefix = eng.runner, eng.prefix
    assert runner.open("probe")
    path = prefix.match(taker)
    n = prefix.adopt("probe", path)
    assert n == SHARED
    pages = set(runner.cache.pages_of("probe"))
    ref = _plain(cfg, w, taker, dtype)
    tol = _tol(dtype, ref)
    cut = len(taker) - 3
    got = eng.forward_logits([StepEntry("probe", taker[n:cut], list(range(cut - n)))]).cpu()
    assert float((got.double() - ref[n:cut]).abs().max()) <= tol
    for pos in range(cut, len(taker)):
        row = eng.forward_logits([StepEntry("probe", [taker[pos]], [0])]).cpu()
        assert float((row[0].double() - ref[pos]).abs().max()) <= tol, pos
    assert pages <= set(runner.cache.pages_of("probe"))          # it still reads the adopted pages
    kernels.check_status()
    runner.close("probe")
    prefix.release(path)
    runner.cache.check_invariants()


# ------------------------------------------------------------- the benchmark's shapes
WIDE = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=2048,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192,
    vocab_size=128256, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072)
FLAGSHIP_LAYERS = 16      # the benchmark's model has sixteen layers of these sizes; two are run here


@pytest.fixture(scope="module")
def wide_model():
    """The flagship's layer sizes with 2 of its 16 layers, random weights N(0, 0.02), query and
    key projections doubled so that attention is peaked and a wrong key shows."""
    from llm_singularity_b200.config.llama import LlamaConfig
    from llm_singularity_b200.weights import write_random_model
    from llm_singularity_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    import json, os
    with tempfile.TemporaryDirectory() as d:
        write_random_model(d, LlamaConfig.from_dict(WIDE), seed=3, dtype=torch.bfloat16, std=0.02,
                           device="cuda")
        f = SafetensorsFile(os.path.join(d, "model.safetensors"))
        tensors = {n: f.tensor(n).clone() for n in f.names()}
        f.close()
        for n in tensors:
            if n.endswith("q_proj.weight") or n.endswith("k_proj.weight"):
                tensors[n] = (tensors[n].float() * 2.0).to(torch.bfloat16)
        write_safetensors(os.path.join(d, "model.safetensors"), tensors)
        with open(os.path.join(d, "config.json"), "w") as fh:
            json.dump(WIDE, fh)
        cfg, w = plain_llama.load_model_dir(d)
        yield d, cfg, w


def _tokens(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, WIDE["vocab_size"], (n,), generator=g).tolist()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_a_2048_token_prompt_whole_and_in_four_portions(wide_model, dtype):
    """The benchmark's prompt: 2,048 tokens in one step (sixteen 128-row tiles, the persistent
    matrix products, the tcgen05 attention) and as 4 x 512; logits at 64 places spread over the
    prompt against the plain implementation (run on the device in 64-bit: it is dense tensor
    arithmetic and shares nothing with the engine)."""
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    d, cfg, w = wide_model
    toks = _tokens(2048, 1)
    places = sorted(set(list(range(0, 2048, 37)) + [127, 128, 511, 512, 1535, 1536, 2046, 2047]))
    ref = _plain(cfg, w, toks, dtype, rows=places, device="cuda")
    tol = _tol(dtype, ref)
    runner = ModelRunner(d, dtype=dtype, page_size=16, num_pages=2 * 2048 // 16, max_requests=2,
                         max_tokens_per_step=2048, max_model_len=2048)
    runner.open("whole")
    got = runner.step([StepEntry("whole", toks, places)]).cpu().double()
    worst = float((got - ref).abs().max())
    assert worst <= tol, f"whole: {worst:.3e} > {tol:.1e}"
    runner.open("cut")
    rows = []
    for s in range(0, 2048, 512):
        want = [p - s for p in places if s <= p < s + 512]
        rows.append(runner.step([StepEntry("cut", toks[s:s + 512], want)]).cpu().double())
    cut = torch.cat(rows)
    worst = float((cut - ref).abs().max())
    assert worst <= tol, f"4 x 512: {worst:.3e} > {tol:.1e}"
    if dtype == "float32":
        assert (got.argmax(-1) == ref.argmax(-1)).all() and (cut.argmax(-1) == ref.argmax(-1)).all()
    runner.check_kernels()
    runner.close("whole"); runner.close("cut")
    runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_64_requests_decoding_at_4090_cached_tokens(wide_model, dtype):
    """The benchmark's largest decode step: 64 live requests with some 4,090 cached tokens each
    (eight different sequences, each held by eight requests with pages of their own), prompts
    run in portions of 2,048 tokens with several requests in a step, then four steps of 64
    single tokens (the captured graph in bfloat16).  Every decoded row against the plain row."""
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    d, cfg, w = wide_model
    n_seq, copies, total, decoded = 8, 8, 4094, 4
    head = total - decoded
    seqs = [_tokens(total, 20 + i) for i in range(n_seq)]
    places = list(range(head - 1, total))
    ref = [_plain(cfg, w, t, dtype, rows=places, device="cuda") for t in seqs]
    tol = max(_tol(dtype, r) for r in ref)
    R = n_seq * copies
    runner = ModelRunner(d, dtype=dtype, page_size=16, num_pages=R * 4096 // 16, max_requests=R,
                         max_tokens_per_step=4096, max_model_len=4096)
    ids = [(i, c) for c in range(copies) for i in range(n_seq)]
    for rid in ids:
        assert runner.open(rid)
    # prompts: portions of 2048 and of what is left, two requests to a step
    for k in range(0, R, 2):
        pair = ids[k:k + 2]
        runner.step([StepEntry(r, seqs[r[0]][:2048], []) for r in pair])
        last = runner.step([StepEntry(r, seqs[r[0]][2048:head], [head - 2048 - 1]) for r in pair])
        for j, r in enumerate(pair):
            worst = float((last[j].cpu().double() - ref[r[0]][0]).abs().max())
            assert worst <= tol, f"prompt end of {r}: {worst:.3e} > {tol:.1e}"
    for step in range(decoded):
        pos = head + step
        logits = runner.step([StepEntry(r, [seqs[r[0]][pos]], [0]) for r in ids]).cpu().double()
        for j, r in enumerate(ids):
            worst = float((logits[j] - ref[r[0]][1 + step]).abs().max())
            assert worst <= tol, f"step {step}, request {r}: {worst:.3e} > {tol:.1e}"
    if dtype == "bfloat16":
        assert runner.graph_replays >= decoded - 2
    runner.check_kernels()
    for rid in ids:
        runner.close(rid)
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == R * 4096 // 16


# ------------------------------------------------------------------------ mutation
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", ["tiny_b", "tiny_d", "tiny_e"])
def test_a_swapped_block_table_cell_is_caught_at_the_tolerance_in_use(model_dirs, name, dtype):
    """Two live requests; before a decode step the device block tables get one cell of each
    swapped with the other's (the second page of each: valid page ids, held by the wrong request).
    The comparison with the plain rows, at the tolerance the replay tests use, has to fail for
    both requests; the step before, with the tables as they should be, passes.  This is what the bfloat16 bound must be
    tight enough for."""
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    cfg, w = plain_llama.load_model_dir(model_dirs[name])
    ps = tiny_models.PAGE_SIZE[name]
    vocab = tiny_models.CONFIGS[name]["vocab_size"]
    n = 3 * ps + 5
    seqs = {"a": tiny_models.random_tokens(vocab, n + 2, 61), "b": tiny_models.random_tokens(vocab, n + 2, 62)}
    ref = {r: _plain(cfg, w, t, dtype) for r, t in seqs.items()}
    tol = max(_tol(dtype, r) for r in ref.values())
    runner = ModelRunner(model_dirs[name], dtype=dtype, page_size=ps, num_pages=16, max_requests=2,
                         max_model_len=8 * ps)
    for r in seqs:
        runner.open(r)
    runner.step([StepEntry(r, seqs[r][:n], []) for r in seqs])

    def diffs(pos):
        out = runner.step([StepEntry(r, [seqs[r][pos]], [0]) for r in seqs]).cpu().double()
        return [float((out[j] - ref[r][pos]).abs().max()) for j, r in enumerate(seqs)]

    def swap():
        for g in runner.cache.groups:
            t = g.dev_table
            sa, sb = runner.cache.slot("a"), runner.cache.slot("b")
            va, vb = int(t[sa, 1]), int(t[sb, 1])
            assert va != vb and va >= 0 and vb >= 0
            t[sa, 1], t[sb, 1] = vb, va

    right = diffs(n)             # first the sound step: a wrong step leaves wrong keys behind
    swap()
    wrong = diffs(n + 1)
    runner.check_kernels()
    assert all(d > tol for d in wrong), f"swapped pages went unseen: {wrong} within {tol:.2e}"
    assert all(d <= tol for d in right), f"{right} > {tol:.2e}"


# ------------------------------------------------- steps with prompt portions, replayed from a graph
@pytest.mark.parametrize("name", ["tiny_d", "tiny_e"])
def test_steps_of_a_shape_that_comes_again_are_replayed_from_a_graph(model_dirs, name):
    """A step whose entries have the same token counts and wanted places as one before is captured
    at its third occurrence and replayed from then on, wherever its requests stand in their
    sequences and whatever their pages: the same bits as a runner that launches every such step
    kernel by kernel (whole prompts and later portions of them), and rows within rounding of it
    where single tokens ride along (their attention is split otherwise in a captured step).  At
    most ``max_shape_graphs`` are kept; a shape that was dropped is captured again.  (Steps of up
    to three entries here; by default only a portion alone in its step is captured.)"""
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    d = model_dirs[name]
    kw = dict(dtype="bfloat16", page_size=8, num_pages=400, max_requests=8, max_tokens_per_step=512,
              max_model_len=400)
    graphs, plain = ModelRunner(d, **kw), ModelRunner(d, **kw)
    plain.shape_graphs = False
    graphs.max_shape_graphs = 2
    graphs.shape_graph_entries = 3                         # the default is 1: a portion alone in its step
    V = graphs.vocab_size
    assert graphs.cuda_graphs

    def both(entries):
        a = graphs.step([StepEntry(*e) for e in entries]).float().cpu()
        b = plain.step([StepEntry(*e) for e in entries]).float().cpu()
        return a, b

    for r in range(8):
        assert graphs.open(r) and plain.open(r)
    # three shapes by turns, six turns: a whole portion of 150 tokens with two places wanted, two
    # portions side by side, and a portion beside two single tokens
    seqs = {r: tiny_models.random_tokens(V, 400, 50 + r) for r in range(8)}
    pos = {r: 0 for r in range(8)}

    def take(r, n):
        t = seqs[r][pos[r]:pos[r] + n]
        pos[r] += n
        return t

    for r in (4, 5):                                       # the two that will bring single tokens
        both([(r, take(r, 33), [])])
    replays = []
    for turn in range(6):
        a, b = both([(turn % 4, take(turn % 4, 150), [3, 149])])
        assert torch.equal(a, b), f"turn {turn}: a whole portion"
        a, b = both([(6, take(6, 40), [39]), (7, take(7, 24), [])])
        assert torch.equal(a, b), f"turn {turn}: two portions"
        a, b = both([(4, take(4, 1), [0]), (5, take(5, 1), [0]), (turn % 4, take(turn % 4, 30), [29])])
        assert (a - b).abs().max() <= 2e-2 * b.abs().max(), f"turn {turn}: single tokens beside a portion"
        replays.append(graphs.graph_replays)
    # with room for two shapes and three by turns every shape is captured again and again:
    # seen, run once, captured and replayed; with room for all of them they stay
    assert replays[-1] >= 4 and plain.graph_replays == 0
    assert len(graphs._shape_order) <= 2
    graphs.max_shape_graphs = 4
    before = graphs.graph_replays
    for turn in range(5):
        a, b = both([(turn % 4, take(turn % 4, 9), [8])])
        assert torch.equal(a, b)
    assert graphs.graph_replays - before == 3              # turns 2, 3 and 4
    graphs.check_kernels(); plain.check_kernels()
    for r in range(8):
        graphs.close(r); plain.close(r)
    graphs.cache.check_invariants()
