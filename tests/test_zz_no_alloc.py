"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some hosts of the kernel library cannot allocate device memory when they need attention (a pool
owns the device, or an allocation's synchronisation is not allowed in their loop), so
``lsb_decode_attention_noalloc`` keeps the split-KV scratch in a fixed device array inside the
library.  Here it is called twice in a row (the second call with other sizes, on top of what the
first left in the array) and compared with the regular entry point, which gets its scratch from
the caller.  This file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from llm_singularity_b200.kernels import build
    path = build.ensure_built(["attention_tc"])["attention_tc"]
    lib = ctypes.CDLL(path)
    lib.lsb_decode_attention_noalloc_max_floats.restype = ctypes.c_longlong
    lib.lsb_decode_attention_noalloc_error.restype = ctypes.c_char_p
    return lib


def _problem(R, nh, nkv, hd, page, kv_lens, seed):
    """Random queries and a paged cache with scattered pages; returns tensors and C arguments."""
    g = torch.Generator().manual_seed(seed)
    pages_per = -(-max(kv_lens) // page)
    n_pages = R * pages_per + 5
    table = torch.randperm(n_pages, generator=g)[:R * pages_per].view(R, pages_per).to(torch.int32).cuda()
    k = torch.randn(n_pages, nkv, page, hd, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(n_pages, nkv, page, hd, generator=g).to(torch.bfloat16).cuda()
    qkv = torch.randn(R, (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16).cuda()
    q_start = torch.arange(R + 1, dtype=torch.int32).cuda()
    kv_len = torch.tensor(kv_lens, dtype=torch.int32).cuda()
    rows = torch.arange(R, dtype=torch.int32).cuda()
    return dict(qkv=qkv, k=k, v=v, table=table, q_start=q_start, kv_len=kv_len, rows=rows,
                R=R, nh=nh, nkv=nkv, hd=hd, page=page, n_pages=n_pages)


def _args(p, out):
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    head = [P(p["qkv"].data_ptr()), I(p["qkv"].shape[1]), P(p["k"].data_ptr()), P(p["v"].data_ptr()),
            P(p["q_start"].data_ptr()), P(p["kv_len"].data_ptr()), P(p["rows"].data_ptr()),
            P(p["table"].data_ptr()), I(p["table"].shape[1]), P(out.data_ptr())]
    tail = [I(p["R"]), I(p["nh"]), I(p["nkv"]), I(p["hd"]), I(p["page"]), I(p["n_pages"]),
            F(1.0 / math.sqrt(p["hd"])), I(0)]
    return head, tail


def _both(lib, p, splits):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    want = torch.zeros(p["R"], p["nh"] * p["hd"], dtype=torch.bfloat16, device="cuda")
    got = torch.zeros_like(want)
    scratch = torch.empty(p["R"] * p["nh"] * splits * (p["hd"] + 2), dtype=torch.float32, device="cuda")
    head, tail = _args(p, want)
    rc = lib.lsb_decode_attention(*head, ctypes.c_void_p(scratch.data_ptr()), *tail,
                                  ctypes.c_int(splits), stream)
    assert rc == 0
    head, tail = _args(p, got)
    rc = lib.lsb_decode_attention_noalloc(*head, *tail, ctypes.c_int(splits), stream)
    assert rc == 0, lib.lsb_decode_attention_noalloc_error(rc).decode()
    torch.cuda.synchronize()
    return want, got


def test_no_alloc_entry_point_matches_the_regular_one_twice_in_a_row():
    lib = _lib()
    assert lib.lsb_decode_attention_noalloc_max_floats() == 1 << 20
    # first call: 5 requests, 12 splits (more than a cluster holds, so the partial results go
    # through the scratch array); second call: other sizes on top of what the first left
    p1 = _problem(5, 8, 2, 64, 16, [700, 64, 1, 333, 65], seed=1)
    want, got = _both(lib, p1, splits=12)
    assert want.abs().max() > 0.1
    assert (want.float() - got.float()).abs().max().item() <= 1e-2 * 3.0
    p2 = _problem(3, 16, 1, 128, 8, [129, 900, 40], seed=2)
    want, got = _both(lib, p2, splits=20)
    assert (want.float() - got.float()).abs().max().item() <= 1e-2 * 3.0
    assert torch.equal(want, got)           # same kernels, same order of sums: the same bits


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = _lib()
    p = _problem(2, 8, 2, 64, 16, [100, 50], seed=3)
    out = torch.zeros(2, 8 * 64, dtype=torch.bfloat16, device="cuda")
    head, tail = _args(p, out)
    tail[0] = ctypes.c_int(60000)                       # 60000 requests * 8 heads * 32 splits * 66
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.lsb_decode_attention_noalloc(*head, *tail, ctypes.c_int(32), stream)
    assert rc == -100
    assert b"exceeds" in lib.lsb_decode_attention_noalloc_error(rc)
    torch.cuda.synchronize()
    assert out.abs().max() == 0                         # nothing was launched
