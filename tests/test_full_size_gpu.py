"""The flagship sizes (Llama 3.2 1B: 16 layers, width 2048, 32 heads in 8 groups of 64, feed-forward
8192, 128,256 tokens, llama3 rope scaling, tied head) with random weights N(0, 0.02) and norms of 1:
trace replay under every cutting against the plain implementation, in 32-bit and in bfloat16, and
greedy generation through the entry point.  The tiny configurations never reach the tile shapes, the
split products or the 128,256-row head that these sizes run."""
import tempfile

import pytest
import torch

import cuttings
import plain_llama
import replay_util

pytestmark = pytest.mark.gpu

SIZES = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=16, hidden_size=2048,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192,
    vocab_size=128256, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072)
LENGTHS = (150, 70, 33, 140, 90, 129)     # six for four live places: pages are used again
PAGE = 16
F32_TOL = 2e-4       # observed 4.1e-5 on logits of up to 5.4 (float32 sums against float64 ones)
BF16_REL = 4e-2      # of the largest plain logit, as for the tiny models; observed 1.9e-2


@pytest.fixture(scope="module")
def full_size():
    from llm_singularity_b200.config.llama import LlamaConfig
    from llm_singularity_b200.weights import write_random_model
    g = torch.Generator().manual_seed(5)
    seqs = {f"r{i}": torch.randint(0, SIZES["vocab_size"], (n,), generator=g).tolist()
            for i, n in enumerate(LENGTHS)}
    with tempfile.TemporaryDirectory() as d:          # 2.5 GB, gone when the module is done
        write_random_model(d, LlamaConfig.from_dict(SIZES), seed=1, dtype=torch.bfloat16, std=0.02,
                           norm_noise=0.0, device="cuda")
        cfg, w = plain_llama.load_model_dir(d)
        ref = {"float32": {r: plain_llama.forward_logits(cfg, w, t) for r, t in seqs.items()},
               "bfloat16": {r: plain_llama.forward_logits(cfg, w, t, act_round="bfloat16")
                            for r, t in seqs.items()}}
        yield d, cfg, w, seqs, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_replay_at_full_size_matches_plain(full_size, tmp_path, dtype, cut):
    from llm_singularity_b200.engine import ModelRunner
    d, _, _, seqs, ref = full_size
    steps, max_tokens = getattr(cuttings, cut)(seqs)
    runner = ModelRunner(d, dtype=dtype, page_size=PAGE, num_pages=max_tokens // PAGE, max_requests=4,
                         max_model_len=max_tokens)
    held = replay_util.track_pages(runner)
    replay_util.replay_in_process(runner, steps, str(tmp_path))
    if cut == "mixed":
        replay_util.assert_pages_were_used_again(held, seqs, max_tokens, f"full size/{dtype}")
    rows = replay_util.collect(steps, str(tmp_path), SIZES["vocab_size"])
    largest = max(float(r.abs().max()) for r in ref[dtype].values())
    tol = F32_TOL if dtype == "float32" else BF16_REL * largest
    replay_util.compare(rows, ref[dtype], tol, f"full size/{dtype}/{cut}")
    if dtype == "float32":
        for (rid, pos), row in rows.items():
            assert int(row.argmax()) == int(ref[dtype][rid][pos].argmax()), (rid, pos)
    runner.check_kernels()
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == max_tokens // PAGE


@pytest.mark.parametrize("dtype, margin", [("float32", 1e-3), ("bfloat16", 0.05)])
def test_greedy_generation_at_full_size_matches_plain(full_size, dtype, margin):
    from llm_singularity_b200 import Engine, kernels
    d, cfg, w, seqs, _ = full_size
    eng = Engine(d, dtype=dtype, device="cuda:0", kv_block_size=PAGE, num_kv_blocks=64, max_batch_size=4,
                 max_tokens_per_batch=96)
    prompts = [seqs["r1"], seqs["r2"]]
    outs = eng.generate(prompts, max_new_tokens=4, ignore_eos=True)
    from greedy_util import check_greedy
    compared = sum(check_greedy(cfg, w, p, o, margin, dtype) for p, o in zip(prompts, outs))
    kernels.check_status()
    assert compared >= 4, f"only {compared} tokens could be compared"
