"""Run one kernel on a given size, a few times, and print its time and achieved rate.

    python -m llm_singularity_b200.measure.probe gemm --m 8 --n 16384 --k 2048 [--gated] [--f32-out] [--tile-kernel]
    python -m llm_singularity_b200.measure.probe decode_attention --batch 8 --context 4096
    python -m llm_singularity_b200.measure.probe prefill_attention --tokens 2048
    python -m llm_singularity_b200.measure.probe add_rmsnorm --tokens 2048 --hidden 2048
    python -m llm_singularity_b200.measure.probe rope --tokens 2048
    python -m llm_singularity_b200.measure.probe decode_step --batch 8 --context 4096
    python -m llm_singularity_b200.measure.probe prefill_step --tokens 2048

``decode_step`` runs whole decode steps of a model of the given sizes (random weights) through the
captured graph and prints where one step's time goes: for every kernel of one layer in the middle
of the model, the time from the previous kernel's end to its own end (kernels overlap: each starts
under its predecessor), and the step's total by kernel.  ``prefill_step`` does the same for one
prompt of ``--tokens`` tokens run as one step (a shape that comes again: from its third time on the
runner replays it from a graph, as it would a portion of a long prompt).  ``tc_latency`` builds and
runs ``tc_latency.cu``: the cost of single tcgen05 operations that the attention kernel's loop is
made of.

Times are CUDA-event times on the launching stream after warm-up, with a buffer larger than the
L2 cache read between iterations (``--no-flush`` to keep it warm).  The same command line is
what the profiler summaries under ``profiles/`` were captured from.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch


class _Ctx:
    pass


def _ctx(q_lens, kv_lens):
    from ..engine.batch import ContextBuilder
    b = ContextBuilder("cuda", max(sum(q_lens), 16), len(q_lens))
    ctx, _ = b.build([[0] * n for n in q_lens], [k - q for k, q in zip(kv_lens, q_lens)],
                     list(range(len(q_lens))), [[] for _ in q_lens])
    ctx._builder = b
    return ctx


def _cache(R, max_kv, nkv, hd, page):
    from ..cache.manager import KVCacheView
    per = -(-max_kv // page)
    n_pages = R * per
    table = torch.randperm(n_pages)[:R * per].view(R, per).to(torch.int32).cuda()
    k = torch.randn(n_pages, nkv, page, hd, device="cuda").to(torch.bfloat16)
    v = torch.randn(n_pages, nkv, page, hd, device="cuda").to(torch.bfloat16)
    return KVCacheView(k, v, table, page, None, 0)


def _time(fn, iters, warmup, flush):
    # L2 is flushed by READING a buffer larger than it: a write would leave L2 full of dirty
    # lines whose write-back then competes with the timed kernel for HBM (that cost a memory-bound
    # kernel 20 % here)
    buf = torch.zeros(512 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if buf is not None:
            buf.view(torch.int32).sum()          # no sync: the host queues the timed launch behind it
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters * 1e3          # microseconds


def _decode_step(a) -> None:
    from ..config.llama import LlamaConfig
    from ..engine import StepEntry
    from ..engine.engine import Engine
    cfg = LlamaConfig.from_dict(dict(
        architectures=["LlamaForCausalLM"], num_hidden_layers=a.layers, hidden_size=a.hidden,
        num_attention_heads=a.heads, num_key_value_heads=a.kv_heads, head_dim=a.head_dim,
        intermediate_size=a.intermediate, vocab_size=a.vocab, rope_theta=500000.0, rope_scaling=None,
        rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072))
    B, ctx_len = a.batch, a.context
    grow = 6 * a.iters + 16                           # steps run below: every one adds a token a request
    eng = Engine(None, config=cfg, random_weights=True, dtype="bfloat16", kv_block_size=a.page,
                 num_kv_blocks=B * ((ctx_len + grow) // a.page + 2) + 8, max_batch_size=B,
                 max_tokens_per_batch=2048, max_model_len=ctx_len + grow + 64, prefix_cache=False)
    r = eng.runner
    g = torch.Generator().manual_seed(0)
    ids = [f"r{i}" for i in range(B)]
    for rid in ids:                                   # fill the contexts, 2,048 tokens a step
        r.open(rid)
        toks = torch.randint(0, cfg.vocab_size, (ctx_len - 16,), generator=g).tolist()
        for s0 in range(0, len(toks), 2048):
            r.step([StepEntry(rid, toks[s0:s0 + 2048], [])])

    staged = None
    if a.sample:                                      # greedy sampling behind the model, inside the graph
        from ..sampling import SamplingParams
        staged = eng.sampler.stage([SamplingParams(temperature=0.0)] * B, [0] * B)

    def step():
        return r.step([StepEntry(rid, [5], [0]) for rid in ids], after=staged)

    for _ in range(3):                                # eager once, capture, replay
        step()
    windows = []
    for _ in range(5):                                # (a step's time moves by a per cent or two from
        torch.cuda.synchronize()                      # window to window: the median of five)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            step()
        e1.record()
        torch.cuda.synchronize()
        windows.append(e0.elapsed_time(e1) / a.iters * 1e3)
    windows.sort()
    print(f"decode step B={B} context={ctx_len} layers={a.layers} hidden={a.hidden}: "
          f"{windows[2]:.1f} us per step (CUDA events, graph replay; median of five windows of {a.iters} steps, "
          f"{windows[0]:.1f} .. {windows[-1]:.1f})")
    if not a.no_timeline:
        _timeline(step, "step")


def _model(a, batch, max_len):
    from ..config.llama import LlamaConfig
    from ..engine.engine import Engine
    cfg = LlamaConfig.from_dict(dict(
        architectures=["LlamaForCausalLM"], num_hidden_layers=a.layers, hidden_size=a.hidden,
        num_attention_heads=a.heads, num_key_value_heads=a.kv_heads, head_dim=a.head_dim,
        intermediate_size=a.intermediate, vocab_size=a.vocab, rope_theta=500000.0, rope_scaling=None,
        rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072))
    eng = Engine(None, config=cfg, random_weights=True, dtype="bfloat16", kv_block_size=a.page,
                 num_kv_blocks=batch * (max_len // a.page + 2) + 8, max_batch_size=batch,
                 max_tokens_per_batch=max(2048, a.tokens), max_model_len=max_len + 64, prefix_cache=False)
    return cfg, eng


def _timeline(step, what):
    """Profile one call of ``step`` and print one layer's kernels and the step's total by kernel."""
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                 key=lambda e: e.time_range.end)
    names = [e.name.split("(")[0].replace("void ", "") for e in evs]
    marks = [i for i, n in enumerate(names) if "attention" in n]    # one attention kernel a layer
    if len(marks) >= 4:
        mid, last = marks[len(marks) // 2], marks[len(marks) // 2 + 1]
        print("one layer in the middle, time from the previous kernel's end to this kernel's end:")
        for i in range(mid + 1, last + 1):
            print(f"  {evs[i].time_range.end - evs[i - 1].time_range.end:7.1f} us  {names[i][:70]}")
        print(f"  {evs[last].time_range.end - evs[mid].time_range.end:7.1f} us  the layer")
    total = {}
    for i in range(1, len(evs)):
        total[names[i]] = total.get(names[i], 0.0) + evs[i].time_range.end - max(evs[i - 1].time_range.end,
                                                                               evs[i].time_range.start)
    span = evs[-1].time_range.end - evs[0].time_range.start if evs else 0.0
    print(f"the {what} by kernel (time not hidden under the previous kernel), under the profiler; "
          f"first start to last end {span:.1f} us, {len(evs)} kernels:")
    for n, t in sorted(total.items(), key=lambda kv: -kv[1]):
        print(f"  {t:8.1f} us  {n[:70]}")


def _prefill_step(a) -> None:
    from ..engine import StepEntry
    cfg, eng = _model(a, 2, a.tokens)
    r = eng.runner
    toks = torch.randint(0, cfg.vocab_size, (a.tokens,), generator=torch.Generator().manual_seed(0)).tolist()
    n = [0]

    def step():
        rid = f"p{n[0]}"
        n[0] += 1
        r.open(rid)
        out = r.step([StepEntry(rid, toks, [a.tokens - 1])])
        r.close(rid)
        return out

    for _ in range(max(a.warmup, 2)):
        step()
    times = []
    for _ in range(a.iters):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    print(f"prefill step T={a.tokens} layers={a.layers} hidden={a.hidden}: median {times[len(times) // 2] * 1e3:.1f} us, "
          f"best {times[0] * 1e3:.1f} us (CUDA events around ModelRunner.step; the step's shape has come "
          f"before, so it is replayed from its graph: {r.graph_replays} replays so far)")
    _timeline(step, "step")


def _tc_latency() -> int:
    """Compile ``tc_latency.cu`` (beside this file) into a temporary folder and run it: what a
    ``tcgen05.mma`` costs its issuing thread, and what a warp waits for a barrier test, a load from
    tensor memory and a store to it to answer."""
    import os
    import subprocess
    import tempfile
    from ..kernels.build import find_nvcc
    src = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tc_latency.cu")
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "tc_latency")
        subprocess.run([find_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
                        "-o", exe, src], check=True)
        return subprocess.run([exe], timeout=120).returncode


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="probe", description=__doc__.split("\n\n")[0])
    ap.add_argument("op", choices=["gemm", "decode_attention", "prefill_attention", "add_rmsnorm", "rope",
                                   "decode_step", "prefill_step", "tc_latency"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--gated", action="store_true")
    ap.add_argument("--f32-out", action="store_true")
    ap.add_argument("--scaled", action="store_true", help="gemm: x is a NormOut (the row scale owed)")
    ap.add_argument("--adds", action="store_true", help="gemm: the product is added to a residual (into=)")
    ap.add_argument("--tile-kernel", action="store_true",
                    help="gemm: the tcgen05 tile kernel also where the small or streaming kernel would run")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--intermediate", type=int, default=8192)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-timeline", action="store_true", help="decode_step: the step's time only")
    ap.add_argument("--sample", action="store_true", help="decode_step: with greedy sampling inside the graph")
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args(argv)
    if a.op == "tc_latency":
        return _tc_latency()
    from .. import kernels as K
    torch.manual_seed(0)
    nh, nkv, hd = a.heads, a.kv_heads, a.head_dim

    if a.op == "decode_step":
        _decode_step(a)
    elif a.op == "prefill_step":
        _prefill_step(a)
    elif a.op == "gemm":
        if a.tile_kernel:
            K.SMALL_PRODUCTS = K.STREAM_PRODUCTS = False
        x = torch.randn(a.m, a.k, device="cuda").to(torch.bfloat16)
        w = torch.randn(a.n, a.k, device="cuda").to(torch.bfloat16)
        od = torch.float32 if a.f32_out else torch.bfloat16
        xin, into = x, None
        if a.scaled:        # x as the product before left it: the norm's row scale still owed
            xin = K.NormOut(x, torch.rand(148, 16, device="cuda") * a.k / 148, 1e-5)
        if a.adds:          # the product added to the residual, the next norm half done
            into = (torch.randn(a.m, a.n, device="cuda"), torch.ones(a.n, device="cuda"), 1e-5)
        us = _time(lambda: K.linear(xin, w, out_dtype=od, gated=a.gated, into=into), a.iters, a.warmup,
                   not a.no_flush)
        flop, byt = 2.0 * a.m * a.n * a.k, 2.0 * (a.n * a.k + a.m * a.k) + a.m * a.n * (4 if a.f32_out else 2)
        print(f"gemm M={a.m} N={a.n} K={a.k} gated={a.gated}: {us:.1f} us  {flop / us / 1e6:.1f} TFLOP/s  "
              f"{byt / us / 1e3:.0f} GB/s")
    elif a.op in ("decode_attention", "prefill_attention"):
        if a.op == "decode_attention":
            q_lens, kv_lens = [1] * a.batch, [a.context] * a.batch
        else:
            q_lens, kv_lens = [a.tokens], [a.tokens]
        ctx = _ctx(q_lens, kv_lens)
        cache = _cache(len(q_lens), max(kv_lens), nkv, hd, a.page)
        T = sum(q_lens)
        qkv = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda").to(torch.bfloat16)
        out = torch.empty(T, nh * hd, dtype=torch.bfloat16, device="cuda")
        us = _time(lambda: K.paged_attention(qkv, nh, nkv, hd, ctx, cache, 1 / math.sqrt(hd), 0, out),
                   a.iters, a.warmup, not a.no_flush)
        if a.op == "decode_attention":
            byt = 2.0 * a.batch * a.context * nkv * hd * 2
            print(f"decode attention B={a.batch} context={a.context} heads={nh}/{nkv}x{hd}: {us:.1f} us  "
                  f"{byt / us / 1e3:.0f} GB/s of cache")
        else:
            flop = 4.0 * nh * hd * a.tokens * (a.tokens + 1) / 2
            print(f"prefill attention T={a.tokens} heads={nh}/{nkv}x{hd}: {us:.1f} us  {flop / us / 1e6:.1f} TFLOP/s (causal)")
    elif a.op == "add_rmsnorm":
        res = torch.randn(a.tokens, a.hidden, device="cuda")
        delta = torch.randn(a.tokens, a.hidden, device="cuda").to(torch.bfloat16)
        w = torch.ones(a.hidden, device="cuda")
        out = torch.empty(a.tokens, a.hidden, dtype=torch.bfloat16, device="cuda")
        us = _time(lambda: K.add_rmsnorm(res, delta, w, 1e-5, out), a.iters, a.warmup, not a.no_flush)
        byt = a.tokens * a.hidden * (4 + 2 + 4 + 2.0)
        print(f"add_rmsnorm T={a.tokens} H={a.hidden}: {us:.1f} us  {byt / us / 1e3:.0f} GB/s")
    else:
        ctx = _ctx([a.tokens], [a.tokens])
        cache = _cache(1, a.tokens, nkv, hd, a.page)
        qkv = torch.randn(a.tokens, (nh + 2 * nkv) * hd, device="cuda").to(torch.bfloat16)
        inv = torch.rand(hd // 2, device="cuda")
        us = _time(lambda: K.rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv, hd), a.iters, a.warmup,
                   not a.no_flush)
        byt = a.tokens * hd * 2.0 * (2 * (nh + nkv) + nkv + 2 * nkv)
        print(f"rope + cache write T={a.tokens} heads={nh}/{nkv}x{hd}: {us:.1f} us  {byt / us / 1e3:.0f} GB/s")
    K.check_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())
