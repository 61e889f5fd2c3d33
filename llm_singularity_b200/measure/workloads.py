"""Two serving workloads at larger sizes than the headline benchmark, run through ``Engine``.

``mixed_3b``: Llama 3.2 3B sizes, 32 requests with prompts of 128 to 2,048 random tokens, admitted
together, prompts cut into portions of 512 beside the decode tokens of the requests already
running (continuous batching), 128 new tokens each.

``shared_prefix_8b``: Llama 3.1 8B sizes (untied head), 64 streams with 1,024-token prompts, every
other one beginning with the same 512 tokens (32 full pages, taken from the prefix tree instead of
being recomputed), context limit 8,192, 128 new tokens each.

Weights are random (N(0, 0.02), norms 1), made on the device from a seed; prompts are seeded
uniform-random token ids.  Each function returns a flat dict: seconds for the whole run (wall clock,
synchronised on both sides, host tokens in and out), tokens per second, and the engine's counters
(pages in use at the peak, preemptions, pages taken from the prefix tree).  The reference's fixed
limits that these sizes pass are 1,024 pages, 256 sequences and 2,048 tokens a batch
(models/llama/llama_model.cpp:111-120), with 32-bit weights only.
"""
from __future__ import annotations

import time
from typing import Dict, List

import torch


def _scaling(factor: float) -> dict:
    return {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
            "original_max_position_embeddings": 8192}


LLAMA_3_2_3B = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=28, hidden_size=3072, num_attention_heads=24,
    num_key_value_heads=8, head_dim=128, intermediate_size=8192, vocab_size=128256, rope_theta=500000.0,
    rope_scaling=_scaling(32.0), rms_norm_eps=1e-5, tie_word_embeddings=True,
    max_position_embeddings=131072)
LLAMA_3_1_8B = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
    num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256, rope_theta=500000.0,
    rope_scaling=_scaling(8.0), rms_norm_eps=1e-5, tie_word_embeddings=False,
    max_position_embeddings=131072)


def _serve(eng, prompts: List[List[int]], new_tokens: int) -> Dict[str, float]:
    """All prompts added at once; steps until nothing is left.  Tracks the most pages in use."""
    cache = eng.runner.cache
    total_pages = cache.free_pages() + (eng.prefix.evictable_pages() if eng.prefix else 0)
    for i, p in enumerate(prompts):
        eng.add_request(p, new_tokens, ignore_eos=True, seed=i)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    made = steps = 0
    least_free = total_pages
    while eng.has_work():
        made += sum(1 for _, tok, _ in eng.step() if tok >= 0)
        steps += 1
        least_free = min(least_free, cache.free_pages())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    eng.runner.check_kernels()
    cache.check_invariants()
    st = eng.stats()
    n_prompt = sum(map(len, prompts))
    return {"seconds": round(dt, 4), "requests": len(prompts), "prompt_tokens": n_prompt,
            "new_tokens": made, "total_tokens_per_s": round((n_prompt + made) / dt, 1),
            "new_tokens_per_s": round(made / dt, 1), "steps": steps,
            "pages": total_pages, "pages_in_use_peak": total_pages - least_free,
            "preemptions": int(st["preemptions"]), "prefix_hit_pages": int(st["prefix_hit_pages"]),
            "prefix_hit_tokens": int(st["prefix_hit_tokens"]), "evicted_pages": int(st["evicted_pages"]),
            "device_gb_peak": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)}


def _runs(make_engine, prompts, new_tokens, repeats):
    """The first run compiles, captures decode graphs and is dropped; the best of the others."""
    eng = make_engine()
    _serve(eng, prompts, new_tokens)
    best = None
    for _ in range(repeats):
        if eng.prefix is not None:
            eng.prefix.evict(1 << 30)               # every run starts with an empty prefix tree
        r = _serve(eng, prompts, new_tokens)
        if best is None or r["seconds"] < best["seconds"]:
            best = r
    del eng
    torch.cuda.empty_cache()
    return best


def mixed_3b(repeats: int = 2, layers: int = 0, device: str = "cuda:0") -> Dict[str, float]:
    from ..config.llama import LlamaConfig
    from ..engine.engine import Engine
    d = dict(LLAMA_3_2_3B)
    if layers:
        d["num_hidden_layers"] = layers
    cfg = LlamaConfig.from_dict(d)
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(128, 2049, (32,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    out = _runs(lambda: Engine(None, config=cfg, random_weights=True, dtype="bfloat16", device=device,
                               num_kv_blocks=6144, max_batch_size=32, max_tokens_per_batch=2048,
                               prefill_chunk=512, max_model_len=4096), prompts, 128, repeats)
    out.update(model="llama-3.2-3b-sizes", layers=cfg.num_hidden_layers, layers_full_model=28,
               prompt_lengths="128-2048", portion=512)
    return out


def shared_prefix_8b(repeats: int = 2, layers: int = 0, device: str = "cuda:0") -> Dict[str, float]:
    from ..config.llama import LlamaConfig
    from ..engine.engine import Engine
    d = dict(LLAMA_3_1_8B)
    if layers:
        d["num_hidden_layers"] = layers
    cfg = LlamaConfig.from_dict(d)
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(0, cfg.vocab_size, (512,), generator=g).tolist()
    prompts = []
    for i in range(64):
        tail = torch.randint(0, cfg.vocab_size, (512,), generator=g).tolist()
        head = shared if i % 2 == 0 else torch.randint(0, cfg.vocab_size, (512,), generator=g).tolist()
        prompts.append(head + tail)
    out = _runs(lambda: Engine(None, config=cfg, random_weights=True, dtype="bfloat16", device=device,
                               num_kv_blocks=64 * 80 + 64, max_batch_size=64, max_tokens_per_batch=2048,
                               prefill_chunk=1024, max_model_len=8192), prompts, 128, repeats)
    out.update(model="llama-3.1-8b-sizes", layers=cfg.num_hidden_layers, layers_full_model=32,
               shared_prefix_tokens=512, streams_sharing=32, context_limit=8192)
    return out


if __name__ == "__main__":
    import json
    import sys
    which = sys.argv[1:] or ["mixed_3b", "shared_prefix_8b"]
    for name in which:
        print(json.dumps({name: globals()[name]()}))
