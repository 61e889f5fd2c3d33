"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some hosts of the kernel library cannot allocate device memory when they need attention (a pool
owns the device, or an allocation's synchronisation is not allowed in their loop), so
``lsb_decode_attention_noalloc`` keeps the split-KV scratch in a fixed device array inside the
library.  Here it is called several times in a row (each call with other sizes, on top of what
the one before left in the array) and held to two things: a plain 64-bit attention over the same
pages, and the regular entry point, which gets its scratch from the caller.  Free device memory
is read around a call to see that none was taken.  This file sorts last on purpose: a run that
stops at the first failure has then already run every other test.
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


def _oracle(p, window=0):
    """Plain attention in 64-bit of every request's one query over its own pages."""
    R, nh, nkv, hd, page = p["R"], p["nh"], p["nkv"], p["hd"], p["page"]
    q = p["qkv"][:, :nh * hd].double().cpu().view(R, nh, hd)
    k, v, table = p["k"].double().cpu(), p["v"].double().cpu(), p["table"].cpu()
    out = torch.zeros(R, nh, hd, dtype=torch.float64)
    for r in range(R):
        n = int(p["kv_len"][r])
        idx = torch.arange(n)
        pages = table[r, idx // page].long()
        K, V = k[pages, :, idx % page], v[pages, :, idx % page]           # [n, nkv, hd]
        lo = max(0, n - window) if window else 0
        for h in range(nh):
            g = h // (nh // nkv)
            s = (K[lo:, g] @ q[r, h]) / math.sqrt(hd)
            out[r, h] = torch.softmax(s, 0) @ V[lo:, g]
    return out.view(R, nh * hd)


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


def _args(p, out, window=0):
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    head = [P(p["qkv"].data_ptr()), I(p["qkv"].shape[1]), P(p["k"].data_ptr()), P(p["v"].data_ptr()),
            P(p["q_start"].data_ptr()), P(p["kv_len"].data_ptr()), P(p["rows"].data_ptr()),
            P(p["table"].data_ptr()), I(p["table"].shape[1]), P(out.data_ptr())]
    tail = [I(p["R"]), I(p["nh"]), I(p["nkv"]), I(p["hd"]), I(p["page"]), I(p["n_pages"]),
            F(1.0 / math.sqrt(p["hd"])), I(window)]
    return head, tail


TOL = 1e-2 * 3.0          # one bfloat16 rounding of outputs of size up to 3, as the kernel tests use


def _both(lib, p, splits, window=0, watch_memory=False):
    """The regular entry point (scratch from the caller), then the one that allocates nothing;
    both against the 64-bit oracle.  Returns the two outputs."""
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    want = torch.zeros(p["R"], p["nh"] * p["hd"], dtype=torch.bfloat16, device="cuda")
    got = torch.zeros_like(want)
    scratch = torch.empty(max(1, p["R"] * p["nh"] * splits * (p["hd"] + 2)), dtype=torch.float32, device="cuda")
    head, tail = _args(p, want, window)
    rc = lib.lsb_decode_attention(*head, ctypes.c_void_p(scratch.data_ptr()), *tail,
                                  ctypes.c_int(splits), stream)
    assert rc == 0
    head, tail = _args(p, got, window)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.lsb_decode_attention_noalloc(*head, *tail, ctypes.c_int(splits), stream)
    assert rc == 0, lib.lsb_decode_attention_noalloc_error(rc).decode()
    torch.cuda.synchronize()
    if watch_memory:        # (not on a library's very first launch, which loads its kernels)
        assert torch.cuda.mem_get_info()[0] == free_before, "the call took device memory"
    ref = _oracle(p, window)
    assert ref.abs().max() > 0.1
    for name, t in (("regular", want), ("no-alloc", got)):
        worst = (t.double().cpu() - ref).abs().max().item()
        assert worst <= TOL, f"{name} entry point, {splits} splits: {worst:.3e} from the plain attention"
    return want, got


def test_no_alloc_entry_point_matches_plain_attention_and_the_regular_one():
    lib = _lib()
    assert lib.lsb_decode_attention_noalloc_max_floats() == 1 << 20
    # first call: 5 requests, 12 splits (more than a cluster holds, so the partial results go
    # through the scratch array); second call: other sizes on top of what the first left
    p1 = _problem(5, 8, 2, 64, 16, [700, 64, 1, 333, 65], seed=1)
    want, got = _both(lib, p1, splits=12)
    p2 = _problem(3, 16, 1, 128, 8, [129, 900, 40], seed=2)
    want, got = _both(lib, p2, splits=20, watch_memory=True)
    assert torch.equal(want, got)           # same kernels, same order of sums: the same bits
    # the paths that need no scratch: one split, and four splits merged inside a cluster
    for splits in (1, 4):
        want, got = _both(lib, p1, splits=splits, watch_memory=True)
        assert torch.equal(want, got)
    # a window of 100 keys, through the array again (a far key must not be seen)
    p3 = _problem(4, 8, 2, 64, 16, [500, 100, 99, 101], seed=4)
    p3["k"][p3["table"][0, 3].long(), :, 5] *= 30.0        # position 53 of request 0: outside its window
    want, got = _both(lib, p3, splits=10, window=100, watch_memory=True)
    assert torch.equal(want, got)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    """The limit is on the floats of scratch, n_requests * nh * splits * (hd + 2), and only where
    scratch is used (more than 8 splits).  hd + 2 is 66 or 130 and never divides the array's 2^20
    floats, so the nearest sizes on either side of the limit are 220 and 221 requests of 8 heads
    in 9 splits (1,045,440 and 1,050,192 floats)."""
    lib = _lib()
    cap = lib.lsb_decode_attention_noalloc_max_floats()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    fits = _problem(220, 8, 2, 64, 16, [40 + (i % 7) for i in range(220)], seed=5)
    assert 220 * 8 * 9 * 66 <= cap < 221 * 8 * 9 * 66
    _both(lib, fits, splits=9, watch_memory=True)
    p = _problem(221, 8, 2, 64, 16, [40] * 221, seed=6)
    out = torch.zeros(221, 8 * 64, dtype=torch.bfloat16, device="cuda")
    head, tail = _args(p, out)
    rc = lib.lsb_decode_attention_noalloc(*head, *tail, ctypes.c_int(9), stream)
    assert rc == -100
    assert b"exceeds" in lib.lsb_decode_attention_noalloc_error(rc)
    torch.cuda.synchronize()
    assert out.abs().max() == 0                         # nothing was launched
    # the same requests in 8 splits need no scratch and are taken
    rc = lib.lsb_decode_attention_noalloc(*head, *tail, ctypes.c_int(8), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert (out.double().cpu() - _oracle(p)).abs().max().item() <= TOL
