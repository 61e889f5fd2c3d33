"""Generation through the entry point and the command line on the GPU."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_llama
import tiny_models
from greedy_util import check_greedy

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _engine(model_dir, name, dtype, **kw):
    from llm_singularity_b200 import Engine
    opts = dict(dtype=dtype, kv_block_size=tiny_models.PAGE_SIZE[name], num_kv_blocks=64,
                max_batch_size=4, max_tokens_per_batch=64)
    opts.update(kw)
    return Engine(model_dir, **opts)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_greedy_generation_matches_plain(model_dirs, name, dtype):
    cfg, w = plain_llama.load_model_dir(model_dirs[name])
    vocab = tiny_models.CONFIGS[name]["vocab_size"]
    lengths = (5, 17, 33) if name == "tiny_a" else (1, 9, 40, 70)
    prompts = [tiny_models.random_tokens(vocab, n, 300 + n) for n in lengths]
    margin = 1e-4 if dtype == "float32" else 0.05
    eng = _engine(model_dirs[name], name, dtype, prefill_chunk=24)
    outs = eng.generate(prompts, max_new_tokens=8, ignore_eos=True)
    assert all(len(o) == 8 for o in outs)
    # every token is checked; those at a step where the plain top-2 margin is inside the dtype's
    # rounding may legitimately fall either way and are not counted
    compared = sum(check_greedy(cfg, w, p, o, margin, f"{name}/{dtype}") for p, o in zip(prompts, outs))
    assert compared >= 4 * len(prompts)
    eng.runner.cache.check_invariants()


@pytest.mark.parametrize("name", ["tiny_b", "tiny_d"])
def test_prompts_of_one_length_one_after_another_are_replayed_and_right(model_dirs, name):
    """Six prompts of the same length, each generated alone: from the third on the prompt step is
    replayed from a graph (with the sampler behind the model inside it), other tokens and other
    pages every time; every continuation is held to the plain implementation."""
    cfg, w = plain_llama.load_model_dir(model_dirs[name])
    vocab = tiny_models.CONFIGS[name]["vocab_size"]
    eng = _engine(model_dirs[name], name, "bfloat16", max_batch_size=1, prefix_cache=False)
    compared = 0
    for i in range(6):
        prompt = tiny_models.random_tokens(vocab, 37, 700 + i)
        out = eng.generate([prompt], max_new_tokens=6, ignore_eos=True)[0]
        compared += check_greedy(cfg, w, prompt, out, 0.05, f"{name}, prompt {i}")
    assert compared >= 12
    if eng.runner.cuda_graphs:
        # four replays of the prompt's shape, and the decode steps of batch size 1
        assert eng.runner.graph_replays >= 4 + 6 * 3
        assert any(len(k) == 3 for k in eng.runner._graphs)
    eng.runner.check_kernels()
    eng.runner.cache.check_invariants()


def test_few_pages_preempt_and_still_give_the_same_tokens(model_dirs):
    name = "tiny_a"
    prompts = [tiny_models.random_tokens(256, n, 400 + n) for n in (30, 25, 28)]
    roomy = _engine(model_dirs[name], name, "float32", prefix_cache=False)
    want = roomy.generate(prompts, max_new_tokens=20, ignore_eos=True)
    tight = _engine(model_dirs[name], name, "float32", num_kv_blocks=7, prefix_cache=False)
    got = tight.generate(prompts, max_new_tokens=20, ignore_eos=True)
    assert tight.stats()["preemptions"] > 0 and got == want
    tight.runner.cache.check_invariants()
    assert tight.runner.cache.free_pages() == 7


def test_prefix_cache_hits_give_the_same_tokens(model_dirs):
    name = "tiny_a"
    shared = tiny_models.random_tokens(256, 48, 9)
    prompts = [shared + tiny_models.random_tokens(256, 5, i) for i in range(3)]
    cold = _engine(model_dirs[name], name, "float32", prefix_cache=False)
    want = [cold.generate([p], max_new_tokens=6, ignore_eos=True)[0] for p in prompts]
    warm = _engine(model_dirs[name], name, "float32")
    got = [warm.generate([p], max_new_tokens=6, ignore_eos=True)[0] for p in prompts]
    assert got == want and warm.stats()["prefix_hit_tokens"] == 2 * 48
    warm.runner.cache.check_invariants()


def test_temperature_sampling_is_reproducible_and_seeded(model_dirs):
    name = "tiny_b"
    prompts = [tiny_models.random_tokens(512, n, 500 + n) for n in (1, 9, 40, 70)]
    kw = dict(max_new_tokens=12, temperature=0.8, ignore_eos=True)
    a = _engine(model_dirs[name], name, "float32", prefill_chunk=24).generate(prompts, seed=3, **kw)
    # alone, in another batch composition and with other portions: same tokens per request
    eng = _engine(model_dirs[name], name, "float32")
    b = [eng.generate([p], seed=3 + i, **kw)[0] for i, p in enumerate(prompts)]
    c = _engine(model_dirs[name], name, "float32").generate(prompts, seed=4, **kw)
    assert a == b and a != c
    assert len({tuple(x) for x in a}) == 4


def test_stop_token_ends_a_request_and_is_part_of_the_output(model_dirs):
    name = "tiny_a"
    cfg, w = plain_llama.load_model_dir(model_dirs[name])
    prompt = tiny_models.random_tokens(256, 12, 1)
    free = plain_llama.greedy_generate(cfg, w, prompt, 6)
    # make the third generated token the stop token
    from llm_singularity_b200 import Engine
    eng = _engine(model_dirs[name], name, "float32")
    eng.scheduler.cfg.stop_token_ids = (free[2],)
    out = eng.generate([prompt], max_new_tokens=6)[0]
    assert out == free[:free.index(free[2]) + 1]


def test_command_line(model_dirs, tmp_path):
    name = "tiny_a"
    cfg, w = plain_llama.load_model_dir(model_dirs[name])
    prompts = [tiny_models.random_tokens(256, n, 600 + n) for n in (4, 11)]
    (tmp_path / "p.json").write_text(json.dumps(prompts))
    cmd = [sys.executable, os.path.join(ROOT, "bin", "llm-serve-llama"), "--model-dir", model_dirs[name],
           "--dtype", "fp32", "--prompt-ids", str(tmp_path / "p.json"), "--max-new-tokens", "5",
           "--ignore-eos", "--num-kv-blocks", "32", "--max-batch-size", "4", "--stats"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    lines = [json.loads(l) for l in res.stdout.splitlines()]
    assert [l["tokens"] for l in lines] == [plain_llama.greedy_generate(cfg, w, p, 5) for p in prompts]
    assert '"stats"' in res.stderr


@pytest.mark.parametrize("dtype, margin", [("fp32", 1e-5), ("bf16", 2e-3)])
def test_command_line_random_weights_can_be_rebuilt_from_the_seed(tmp_path, dtype, margin):
    """--random-weights needs only config.json, makes the weights on the device from --seed, and
    the same weights made on the CPU from that seed give, in the plain implementation, the tokens
    the command printed."""
    from llm_singularity_b200.config.llama import LlamaConfig
    from llm_singularity_b200.weights import write_random_model
    only_cfg = tmp_path / "cfg"
    only_cfg.mkdir()
    (only_cfg / "config.json").write_text(json.dumps(tiny_models.CONFIGS["tiny_b"]))
    prompts = [tiny_models.random_tokens(512, n, 800 + n) for n in (9, 3, 30)]
    (tmp_path / "p.json").write_text(json.dumps(prompts))
    cmd = [sys.executable, os.path.join(ROOT, "bin", "llm-serve-llama"), "--model-dir", str(only_cfg),
           "--random-weights", "--seed", "7", "--dtype", dtype, "--prompt-ids", str(tmp_path / "p.json"),
           "--max-new-tokens", "6", "--ignore-eos", "--kv-block-size", "8", "--num-kv-blocks", "32",
           "--max-batch-size", "4"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    got = [json.loads(l)["tokens"] for l in res.stdout.splitlines()]
    rebuilt = str(tmp_path / "rebuilt")
    write_random_model(rebuilt, LlamaConfig.from_dict(tiny_models.CONFIGS["tiny_b"]), seed=7,
                       dtype=torch.float32 if dtype == "fp32" else torch.bfloat16)
    cfg, w = plain_llama.load_model_dir(rebuilt)
    assert all(len(o) == 6 for o in got)
    compared = sum(check_greedy(cfg, w, p, o, margin, dtype) for p, o in zip(prompts, got))
    assert compared >= 9, f"only {compared} tokens could be compared"


@pytest.mark.parametrize("mode", ["decode", "prefill", "serve"])
def test_command_line_bench_modes(model_dirs, mode):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "llm-serve-llama"), "--model-dir", model_dirs["tiny_b"],
           "--bench", mode, "--prompt-len", "40", "--num-requests", "4" if mode == "decode" else "5",
           "--max-new-tokens", "12",
           "--ignore-eos", "--kv-block-size", "8", "--num-kv-blocks", "40" if mode == "decode" else "24",
           "--max-batch-size", "4"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    line = json.loads(res.stdout.splitlines()[-1])
    assert line["bench"] == mode and line["seconds"] > 0
    stats = line["stats"]
    if mode == "serve":
        # five requests of twelve new tokens each, every prompt token run exactly once or taken
        # from the prefix tree, every page given back
        assert line["generated_tokens"] == 5 * 12
        # a token comes from a decode step or from the end of a prompt (again after a preemption)
        assert stats["decode_tokens"] <= 5 * 11 and stats["decode_tokens"] + stats["admitted"] >= 5 * 12
        assert 5 <= line["prompt_tokens"] <= 5 * 40
        assert stats["prefill_tokens"] + stats["prefix_hit_tokens"] >= line["prompt_tokens"]
        assert stats["admitted"] >= 5 and stats["errors"] == 0
        assert line["total_tokens_per_s"] == pytest.approx(
            (line["generated_tokens"] + line["prompt_tokens"]) / line["seconds"], rel=1e-3)
    if mode == "decode":
        # four requests fit the batch; the timed region is eight steps of four tokens
        assert line["num_requests"] == 4 and line["decode_steps"] == 12 - 4
        assert line["generated_tokens"] == line["decode_steps"] * 4
        assert line["generated_tokens_per_s"] == pytest.approx(line["generated_tokens"] / line["seconds"], rel=1e-3)
        assert stats["prefill_tokens"] == 4 * 40
    if mode == "prefill":
        assert line["prompt_tokens"] == 40 and line["runs"] == 4
        assert line["prompt_tokens_per_s"] == pytest.approx(40 / line["seconds"], rel=1e-3)
        assert stats["prefill_tokens"] == 4 * 40 and stats["admitted"] == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_running_ahead_gives_the_same_tokens_as_the_plain_loop(model_dirs, dtype, temperature):
    """Steps queued before the previous step's tokens reach the host (the next step reads them on
    the device, decode graphs included) against one step at a time: identical tokens, also when a
    stop token is found one step late."""
    name = "tiny_b"
    prompts = [tiny_models.random_tokens(512, n, 700 + n) for n in (2, 21, 40)]
    outs = []
    for ahead in (False, True):
        eng = _engine(model_dirs[name], name, dtype, run_ahead=ahead)
        first = eng.generate(prompts, max_new_tokens=24, temperature=temperature, seed=11, ignore_eos=True)
        eng.scheduler.cfg.stop_token_ids = (first[2][6],)
        second = eng.generate(prompts, max_new_tokens=24, temperature=temperature, seed=11)
        outs.append((first, second))
        eng.runner.check_kernels()
        eng.runner.cache.check_invariants()
        assert eng.stats().get("ahead_steps", 0) == (0 if not ahead else eng.stats()["ahead_steps"])
        if ahead:
            assert eng.stats()["ahead_steps"] >= 20
    assert outs[0] == outs[1]
    stop = outs[1][0][2][6]
    assert outs[1][1][2] == outs[1][0][2][:outs[1][0][2].index(stop) + 1]
