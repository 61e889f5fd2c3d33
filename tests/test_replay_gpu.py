"""Trace replay on the GPU against the plain implementation, in 32-bit and in bfloat16:
each request alone and whole; most of it in one step and the last 32 tokens one by one; in
portions of changing size, down to two tokens; and mixed, up to four live requests with so
few pages that they are used again.  Also long decoding and the first tokens of a sequence."""
import os

import numpy as np
import pytest
import torch

import cuttings
import plain_llama
import replay_util
import tiny_models

pytestmark = pytest.mark.gpu

# more requests than the mixed cutting keeps live (four), so that pages are handed out again
LENGTHS = {"tiny_a": (5, 17, 33, 70, 100, 64, 20), "tiny_b": (1, 9, 40, 70, 50, 23),
           "tiny_c": (3, 64, 65, 47, 2), "tiny_d": (130, 64, 7, 65, 200),
           "tiny_e": (150, 3, 129, 66, 200, 40)}
F32_TOL = 1e-4            # float32 logits against float64 plain logits (observed ~1e-6)
# bfloat16 is held to the plain implementation with activations rounded to bfloat16 at the same
# places; what is left is summation order and single-ulp (2^-8) flips, which the sharpened
# attention of these models amplifies.  Measured floor: the plain implementation against itself
# with 32-bit instead of 64-bit sums before each rounding differs by up to 1.1 % of the largest
# logit (tiny_b, 301 tokens), while rounding itself moves logits by up to 9 %; a wrong or missing
# key moves them by more than that.  The bound is a few times the floor.
BF16_REL = 4e-2           # fraction of the largest plain logit


def _seqs(name):
    vocab = tiny_models.CONFIGS[name]["vocab_size"]
    return {f"r{i}": tiny_models.random_tokens(vocab, n, 100 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def refs(model_dirs):
    out = {}
    for name in LENGTHS:
        cfg, w = plain_llama.load_model_dir(model_dirs[name])
        seqs = _seqs(name)
        out[name] = (seqs, {rid: plain_llama.forward_logits(cfg, w, t) for rid, t in seqs.items()},
                     {rid: plain_llama.forward_logits(cfg, w, t, act_round="bfloat16")
                      for rid, t in seqs.items()})
    return out


def _pick(refs, name, dtype):
    seqs, exact, rounded = refs[name]
    return seqs, exact if dtype == "float32" else rounded


def _tol(dtype, ref):
    if dtype == "float32":
        return F32_TOL
    return BF16_REL * max(float(r.abs().max()) for r in ref.values())


def _runner(model_dir, name, dtype, max_tokens):
    from llm_singularity_b200.engine import ModelRunner
    ps = tiny_models.PAGE_SIZE[name]
    return ModelRunner(model_dir, dtype=dtype, page_size=ps, num_pages=max_tokens // ps,
                       max_requests=4, max_model_len=max_tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(LENGTHS))
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_replay_matches_plain(model_dirs, refs, tmp_path, name, dtype, cut):
    seqs, ref = _pick(refs, name, dtype)
    steps, max_tokens = getattr(cuttings, cut)(seqs)
    runner = _runner(model_dirs[name], name, dtype, max_tokens)
    held = replay_util.track_pages(runner)
    replay_util.replay_in_process(runner, steps, str(tmp_path))
    rows = replay_util.collect(steps, str(tmp_path), tiny_models.CONFIGS[name]["vocab_size"])
    replay_util.compare(rows, ref, _tol(dtype, ref), f"{name}/{dtype}/{cut}")
    if cut == "mixed":
        replay_util.assert_pages_were_used_again(held, seqs, max_tokens, f"{name}/{dtype}")
        assert any(len(s["entries"]) >= 3 for s in steps)
        assert any(min(len(e["tokens"]) for e in s["entries"]) == 1 <
                   max(len(e["tokens"]) for e in s["entries"]) for s in steps)
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == max_tokens // tiny_models.PAGE_SIZE[name]


@pytest.mark.parametrize("dtype, fold", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_cuttings_agree_with_each_other(model_dirs, refs, tmp_path, dtype, fold):
    """The logits at a position do not depend on how the tokens were cut, on what else is in the
    batch or on which pages were used, beyond rounding: all four cuttings against the first.

    With the same arithmetic for every step size (32-bit; bfloat16 with each norm in a kernel of
    its own) the cuttings round at the same places and must agree far closer than they agree with
    the exact logits.  Steps of a few bfloat16 rows fold their norms into the neighbouring products
    (``fold``): other places of rounding, so there the bound is rounding itself, measured: no
    position further from the whole prompt's logits than the tolerance against the exact ones,
    and on average closer to them than those are to the exact ones."""
    from llm_singularity_b200 import kernels
    name = "tiny_b"
    seqs, ref = _pick(refs, name, dtype)
    exact = refs[name][1]
    got = {}
    kernels.FOLD_NORMS = fold
    try:
        for cut in ("whole", "tail_decode", "portions", "mixed"):
            steps, max_tokens = getattr(cuttings, cut)(seqs)
            d = tmp_path / cut
            replay_util.replay_in_process(_runner(model_dirs[name], name, dtype, max_tokens), steps, str(d))
            got[cut] = replay_util.collect(steps, str(d), 512)
    finally:
        kernels.FOLD_NORMS = True
    scale = max(float(r.abs().max()) for r in ref.values())
    tol = 2e-5 if dtype == "float32" else (BF16_REL if fold else 1.5e-2) * scale
    rounding = np.sqrt(np.mean([np.square(row - exact[key[0]][key[1]].numpy()).mean()
                                for key, row in got["whole"].items()]))
    for cut in ("tail_decode", "portions", "mixed"):
        sq = []
        for key, row in got["whole"].items():
            d = float(np.abs(row - got[cut][key]).max())
            assert d <= tol, f"{cut} differs from whole at {key}: {d:.3e}"
            sq.append(np.square(row - got[cut][key]).mean())
        if dtype == "bfloat16":
            assert np.sqrt(np.mean(sq)) <= (0.6 if fold else 0.2) * rounding, (cut, np.sqrt(np.mean(sq)), rounding)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program_as_a_user_runs_it(model_dirs, refs, tmp_path, dtype):
    """bin/trace_run in a process of its own, one step at a time over its standard input."""
    name = "tiny_b"
    seqs, ref = _pick(refs, name, dtype)
    steps, max_tokens = cuttings.mixed(seqs, seed=5)
    replay_util.replay_subprocess(model_dirs[name], dtype, steps, str(tmp_path), max_tokens,
                                  page_size=tiny_models.PAGE_SIZE[name])
    rows = replay_util.collect(steps, str(tmp_path), 512)
    replay_util.compare(rows, ref, _tol(dtype, ref), f"trace_run/{dtype}")
    # steps without wanted places write no file
    assert sorted(int(f[:-4]) for f in os.listdir(tmp_path)) == [s["step"] for s in steps]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_without_wanted_places_and_requests_left_out(model_dirs, refs, tmp_path, dtype):
    name = "tiny_a"
    seqs, ref = _pick(refs, name, dtype)
    a, b = seqs["r2"], seqs["r3"]
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:9], "want": [8]}], "end": []},      # a sits out
        {"step": 2, "entries": [{"id": "b", "tokens": b[9:11], "want": [1, 0]},
                                {"id": "a", "tokens": a[20:], "want": [len(a) - 21]}], "end": ["a"]},
        {"step": 3, "entries": [{"id": "b", "tokens": b[11:], "want": [0, len(b) - 12]}], "end": ["b"]},
    ]
    runner = _runner(model_dirs[name], name, dtype, 192)
    replay_util.replay_in_process(runner, steps, str(tmp_path))
    assert not os.path.exists(tmp_path / "0.f32")
    tol = _tol(dtype, ref)

    def rows(step, n):
        return np.fromfile(tmp_path / f"{step}.f32", dtype="<f4").reshape(n, 256)
    r1, r2, r3 = rows(1, 1), rows(2, 3), rows(3, 2)
    want = [(r1[0], "r3", 8), (r2[0], "r3", 10), (r2[1], "r3", 9), (r2[2], "r2", len(a) - 1),
            (r3[0], "r3", 11), (r3[1], "r3", len(b) - 1)]
    for got, rid, pos in want:
        assert np.abs(got - ref[rid][pos].numpy()).max() <= tol, (rid, pos)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(model_dirs, tmp_path, dtype):
    """Position 0 alone, then 300 tokens decoded one by one (19 pages of 16), with a llama3-scaled
    rope whose original length (64) lies far inside the sequence."""
    name = "tiny_b"
    cfg, w = plain_llama.load_model_dir(model_dirs[name])
    toks = tiny_models.random_tokens(512, 301, 77)
    ref = {"x": plain_llama.forward_logits(cfg, w, toks,
                                           act_round="bfloat16" if dtype == "bfloat16" else None)}
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}],
              "end": ["x"] if i == len(toks) - 1 else []} for i, t in enumerate(toks)]
    runner = _runner(model_dirs[name], name, dtype, 320)
    replay_util.replay_in_process(runner, steps, str(tmp_path))
    rows = replay_util.collect(steps, str(tmp_path), 512)
    replay_util.compare(rows, ref, _tol(dtype, ref), f"long decode/{dtype}")


def test_out_of_pages_is_an_error_not_a_wrong_result(model_dirs):
    from llm_singularity_b200.engine import OutOfPages, StepEntry
    runner = _runner(model_dirs["tiny_a"], "tiny_a", "float32", 64)
    runner.open("a"); runner.open("b")
    runner.step([StepEntry("a", list(range(60)), [])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("b", list(range(20)), [])])
    with pytest.raises(OutOfPages, match="max_model_len"):
        runner.step([StepEntry("a", list(range(10)), [])])
    with pytest.raises(ValueError, match="token id"):
        runner.step([StepEntry("a", [256], [])])
