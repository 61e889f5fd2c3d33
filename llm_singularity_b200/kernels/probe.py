"""Run one kernel on a given size, a few times, and print its time and achieved rate.

    python -m llm_singularity_b200.kernels.probe gemm --m 8 --n 16384 --k 2048 [--gated] [--f32-out]
    python -m llm_singularity_b200.kernels.probe decode_attention --batch 8 --context 4096
    python -m llm_singularity_b200.kernels.probe prefill_attention --tokens 2048
    python -m llm_singularity_b200.kernels.probe add_rmsnorm --tokens 2048 --hidden 2048
    python -m llm_singularity_b200.kernels.probe rope --tokens 2048

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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="probe", description=__doc__.split("\n\n")[0])
    ap.add_argument("op", choices=["gemm", "decode_attention", "prefill_attention", "add_rmsnorm", "rope"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--gated", action="store_true")
    ap.add_argument("--f32-out", action="store_true")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args(argv)
    from .. import kernels as K
    torch.manual_seed(0)
    nh, nkv, hd = a.heads, a.kv_heads, a.head_dim

    if a.op == "gemm":
        x = torch.randn(a.m, a.k, device="cuda").to(torch.bfloat16)
        w = torch.randn(a.n, a.k, device="cuda").to(torch.bfloat16)
        od = torch.float32 if a.f32_out else torch.bfloat16
        us = _time(lambda: K.linear(x, w, out_dtype=od, gated=a.gated), a.iters, a.warmup, not a.no_flush)
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
