#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Llama 3.2 1B sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096]
                    [--layers L] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at the default batch (8) with
every request's context ending at ``--context`` tokens, timed on the device (CUDA events)
over exactly K decode steps after W warm-up steps.  ``e2e`` is the same through the Python
entry point (``Engine.step``): host token ids in (pinned memory, one host-to-device copy of
the step's metadata), sampled token ids out (device-to-host) every step.  ``prefill`` times a
2,048-token prompt in one step; ``roofline`` sets the bytes a decode step must read (every
weight once and the cache of the live requests) against the measured copy bandwidth;
``points`` gives decode tokens per second at batch 1 and 64; ``more`` two larger serving runs
(3B sizes with mixed prompts, 8B sizes with a shared prefix; ``--no-more`` leaves them out).  The
headline is the median of ``--windows`` timed windows of K steps each, with the clocks sampled
over all of them.  Weights are random (N(0, 0.02),
norms 1), prompts are uniform random token ids: synthetic data throughout.  Every decode step
reads more than 2.4 GB of weights, far more than the 126 MB L2, so no L2 flush is needed
between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_3_2_1B = dict(                      # the sizes of Llama 3.2 1B
    architectures=["LlamaForCausalLM"], num_hidden_layers=16, hidden_size=2048,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192,
    vocab_size=128256, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072)
FULL_LAYERS = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            flat = {}

            def walk(x):
                if isinstance(x, dict):
                    for k, v in x.items():
                        if isinstance(v, (int, float)):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(d)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                flat.setdefault("bf16_tflops_sustained", flat["bf16_tflops"])
                return flat, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index=0):
        self.samples = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for p in self.samples:
            try:
                sm.append(float(p[0])); mx.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(self.NAMES, p[2:]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def model_numbers(cfg, layers):
    """Bytes of weights a decode step reads, cache bytes per token, matmul flops per token."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * I * H
    weight_bytes = 2 * (layers * per_layer + V * H)              # bf16; head tied to the table
    kv_bytes_per_token = layers * 2 * nkv * hd * 2
    flops_per_token = 2 * layers * per_layer
    return weight_bytes, kv_bytes_per_token, flops_per_token, 2 * V * H


def run_ours(args):
    import numpy as np
    import torch
    from llm_singularity_b200 import kernels
    from llm_singularity_b200.config.llama import LlamaConfig
    from llm_singularity_b200.engine import StepEntry
    from llm_singularity_b200.engine.engine import Engine

    torch.cuda.init()
    cfg_dict = dict(LLAMA_3_2_1B, num_hidden_layers=args.layers)
    cfg = LlamaConfig.from_dict(cfg_dict)
    V = cfg.vocab_size
    page = 16
    ctx_len = args.context
    batches = sorted({1, args.batch, 64})
    max_b = max(batches)
    pages = max_b * (-(-(ctx_len + 8) // page)) + 64
    eng = Engine(None, config=cfg, random_weights=True, seed=0, dtype="bfloat16",
                 kv_block_size=page, num_kv_blocks=pages, max_batch_size=max_b,
                 max_tokens_per_batch=max(PREFILL_TOKENS, max_b), prefill_chunk=PREFILL_TOKENS,
                 max_model_len=ctx_len + 8, prefix_cache=False, verbose=True)
    runner = eng.runner
    g = torch.Generator().manual_seed(0)
    peaks, peak_src = load_peaks()
    weight_bytes, kv_per_tok, flops_tok, head_flops = model_numbers(cfg_dict, args.layers)

    def fill(batch, upto):
        """Open `batch` requests and prefill each with `upto` random tokens."""
        ids = [f"b{batch}_{i}" for i in range(batch)]
        for rid in ids:
            assert runner.open(rid)
            toks = torch.randint(0, V, (upto,), generator=g).tolist()
            for s in range(0, upto, PREFILL_TOKENS):
                runner.step([StepEntry(rid, toks[s:s + PREFILL_TOKENS], [])])
        return ids

    def decode_steps(ids, n, feed):
        """n decode steps with device-side greedy sampling (inside the step's captured graph, as in
        Engine.step); tokens fed are `feed` (host list)."""
        from llm_singularity_b200.sampling import SamplingParams
        greedy = eng.sampler.stage([SamplingParams(temperature=0.0)] * len(ids), [0] * len(ids))
        for _ in range(n):
            runner.step([StepEntry(rid, [t], [0]) for rid, t in zip(ids, feed)], after=greedy)
        return runner.after_result

    SETTLE = 96

    def time_decode(batch, steps, warmup, windows=1):
        """``windows`` timed windows of exactly ``steps`` decode steps each (the requests are
        refilled to the same lengths before each), after ``warmup`` steps; returns the median
        window's milliseconds per step, every window's, the launches of one window and the mean
        context length inside a window.

        Filling the requests is a burst of prompt steps, and the first sixty-odd decode steps
        after one run 4 - 8 % slower than the steady state (8 x 4096: 0.82 - 0.85 ms a step in the
        first 64 steps, 0.79 from then on): ``SETTLE`` untimed decode steps follow every fill,
        before the warm-up steps, so that a window measures decoding and not the fill before it."""
        start = ctx_len - (steps + warmup + SETTLE + 2)
        ids = fill(batch, start)
        feed = torch.randint(0, V, (batch,), generator=g).tolist()
        runner.cuda_graphs, keep = False, runner.cuda_graphs
        n0 = kernels.launch_count()
        decode_steps(ids, 1, feed)                  # one step launched kernel by kernel: counted
        per_step = kernels.launch_count() - n0
        runner.cuda_graphs = keep
        decode_steps(ids, SETTLE + max(warmup - 1, 2), feed)
        all_ms = []
        for w in range(windows):
            if w:                                   # same lengths again: close, refill, warm up
                for rid in ids:
                    runner.close(rid)
                ids = fill(batch, start)
                decode_steps(ids, SETTLE + warmup, feed)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            launches0 = kernels.launch_count()
            e0.record()
            decode_steps(ids, steps, feed)
            e1.record()
            torch.cuda.synchronize()
            all_ms.append(e0.elapsed_time(e1) / steps)
        # replayed graphs launch the same kernels as the counted step did, without the wrappers
        launches = per_step * steps if runner.graph_replays else kernels.launch_count() - launches0
        kernels.check_status()
        for rid in ids:
            runner.close(rid)
        mean_ctx = ctx_len - steps / 2
        return statistics.median(all_ms), all_ms, launches, mean_ctx

    # ---- prefill: one 2,048-token prompt in one step, logits for its last token
    def time_prefill(reps=5, warm=3):
        toks = torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist()
        times = []
        for i in range(warm + reps):
            rid = f"p{i}"
            runner.open(rid)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step([StepEntry(rid, toks, [PREFILL_TOKENS - 1])])
            e1.record()
            torch.cuda.synchronize()
            runner.close(rid)
            if i >= warm:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times)

    results = {}
    sampler = ClockSampler()
    prefill_ms = time_prefill()
    points = {}
    for b in batches:
        if b == args.batch:
            continue
        ms, _, _, _ = time_decode(b, min(args.steps, 32), args.warmup, windows=3)
        points[f"decode_b{b}"] = round(b / ms * 1e3, 1)

    # ---- the headline: decode at --batch, device-timed, clocks sampled meanwhile
    sampler.start()
    time.sleep(0.3)
    ms, window_ms, launches, mean_ctx = time_decode(args.batch, args.steps, args.warmup, windows=args.windows)
    clocks = sampler.stop()
    value = args.batch / ms * 1e3

    # ---- end to end through Engine.step: host tokens in, host tokens out, every step
    # requests finish their prompts one after another, so the first ones decode a few tokens
    # while the last still prefill: leave room for that, and let none finish inside the timed
    # region (the batch must stay at --batch requests throughout)
    slack = 4 * args.batch + 8
    prompts = [torch.randint(0, V, (ctx_len - (args.steps + args.warmup + SETTLE) - slack,), generator=g).tolist()
               for _ in range(args.batch)]
    for p in prompts:
        eng.add_request(p, max_new_tokens=args.steps + args.warmup + SETTLE + slack, temperature=0.0,
                        ignore_eos=True)
    while any(not r.generated for r in eng._requests.values()):
        eng.step()                                   # prefill until every request decodes
    for _ in range(SETTLE + args.warmup - 1):        # (the same settling after the prompts as above)
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_e2e = 0
    for _ in range(args.steps):
        n_e2e += len(eng.step())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_value = n_e2e / e2e_s
    assert n_e2e == args.steps * args.batch, "the batch changed inside the timed region"
    while eng.has_work():
        eng.step()
    h2d = 4 * (3 * args.batch + (args.batch + 1) + 2 * args.batch + args.batch) + 4 * 5 * args.batch
    d2h = 4 * args.batch

    prefill_flops = PREFILL_TOKENS * flops_tok + head_flops \
        + args.layers * 4 * cfg.num_attention_heads * cfg.head_dim * PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2
    bytes_step = weight_bytes + args.batch * mean_ctx * kv_per_tok
    achieved = bytes_step / (ms * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s at batch 8 (Llama 3.2 1B sizes, context 4096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "llama-3.2-1b-sizes-random-weights", "global_batch": args.batch,
                   "seq_len": ctx_len, "parallelism": "single-gpu", "layers": args.layers,
                   "layers_full_model": FULL_LAYERS, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
                   "vocab": V, "tied_embeddings": True, "kv_page_tokens": page,
                   "prefill_tokens": PREFILL_TOKENS, "settle_steps_after_fill": SETTLE,
                   "l2": "inputs larger than L2, no flush",
                   "peaks": peak_src},
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "windows": {"n": len(window_ms), "ms_per_step": [round(x, 4) for x in window_ms]},
    }
    if not args.no_more:
        # the two larger configurations, through the entry point (host tokens in and out)
        from llm_singularity_b200.measure import workloads
        import gc
        del eng, runner
        gc.collect()
        torch.cuda.empty_cache()
        line["more"] = {"mixed_3b": workloads.mixed_3b(), "shared_prefix_8b": workloads.shared_prefix_8b()}
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS,
                    help=f"decoder layers (the full model has {FULL_LAYERS})")
    ap.add_argument("--windows", type=int, default=5, help="timed windows of K steps; the median is reported")
    ap.add_argument("--no-more", action="store_true", help="leave out the 3B and 8B serving runs")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a CMake C++/CUDA project with no Python packaging "
                          "(pip install of its source tree fails: no setup.py or pyproject.toml) "
                          "and its CMake build fetches dependencies from the network"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus N > 1 is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
