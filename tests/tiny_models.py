"""Tiny configurations for the tests, differing in every size and option.

tiny_a / tiny_b are the two small configurations the engine is specified on
(tied vs untied head, no rope scaling vs llama3 scaling, eps 1e-5 vs 1e-6, two vs
one kv head, page 16 vs 8); tiny_c has sizes that are no power of two anywhere
(hidden 72, six heads of 48 in three groups, 100 wide feed-forward, 301 tokens); tiny_d has
heads of 64 and tiny_e heads of 128, the sizes the bfloat16 tensor-core attention kernels take.
Weights are random; query and key projections are scaled up so that attention is
peaked: a wrong, missing or stale key then changes the logits visibly instead of
drowning in a near-uniform average.
"""
import json
import os

import torch

CONFIGS = {
    "tiny_a": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=64,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                   intermediate_size=176, vocab_size=256, rope_theta=10000.0, rope_scaling=None,
                   rms_norm_eps=1e-5, tie_word_embeddings=True, eos_token_id=255),
    "tiny_b": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=3, hidden_size=128,
                   num_attention_heads=4, num_key_value_heads=1, head_dim=32,
                   intermediate_size=320, vocab_size=512, rope_theta=500000.0,
                   rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0,
                                     high_freq_factor=4.0, original_max_position_embeddings=64),
                   rms_norm_eps=1e-6, tie_word_embeddings=False, eos_token_id=[510, 511]),
    "tiny_c": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=72,
                   num_attention_heads=6, num_key_value_heads=3, head_dim=48,
                   intermediate_size=100, vocab_size=301, rope_theta=25000.0, rope_scaling=None,
                   rms_norm_eps=3e-6, tie_word_embeddings=False),
    # head size 64: the size the tensor-core attention kernels take in bfloat16
    "tiny_d": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=96,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                   intermediate_size=144, vocab_size=200, rope_theta=10000.0, rope_scaling=None,
                   rms_norm_eps=1e-5, tie_word_embeddings=True),
    # head size 128 in groups of three (the other size of the tensor-core kernels), pages of 32,
    # llama3 scaling, head_dim not hidden / heads
    "tiny_e": dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=160,
                   num_attention_heads=3, num_key_value_heads=1, head_dim=128,
                   intermediate_size=232, vocab_size=333, rope_theta=500000.0,
                   rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                     original_max_position_embeddings=128),
                   rms_norm_eps=2e-6, tie_word_embeddings=False),
}
PAGE_SIZE = {"tiny_a": 16, "tiny_b": 8, "tiny_c": 16, "tiny_d": 16, "tiny_e": 32}
SEEDS = {"tiny_a": 11, "tiny_b": 22, "tiny_c": 33, "tiny_d": 44, "tiny_e": 55}


def make_model_dir(path, name, sharpen=4.0, dtype=torch.bfloat16):
    """Write a random model of configuration ``name`` to ``path`` through the engine's own
    random-weights mode, then scale q and k projections by ``sharpen``."""
    from llm_singularity_b200.config.llama import LlamaConfig
    from llm_singularity_b200.weights import write_random_model
    from llm_singularity_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    cfg = LlamaConfig.from_dict(CONFIGS[name])
    write_random_model(path, cfg, seed=SEEDS[name], dtype=dtype, std=0.05, norm_noise=0.1)
    if sharpen != 1.0:
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        tensors = {n: f.tensor(n).clone() for n in f.names()}
        for n in tensors:
            if n.endswith("q_proj.weight") or n.endswith("k_proj.weight"):
                tensors[n] = (tensors[n].float() * sharpen).to(dtype)
        f.close()
        write_safetensors(os.path.join(path, "model.safetensors"), tensors)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(CONFIGS[name] | {"hidden_act": "silu", "model_type": "llama"}, fh)
    return path


def random_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
