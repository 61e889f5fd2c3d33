"""Each CUDA kernel alone against plain tensor arithmetic, at sizes the engine's tiny models do
not use: head sizes in steps of 16 up to 256, odd widths and vocabularies, scattered pages."""
import math

import numpy as np
import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype, scale=1.0):
    # float32: accumulation-order noise only; bfloat16: one rounding of the result (2^-8 relative)
    return (2e-5 if dtype == torch.float32 else 1e-2) * scale


@pytest.fixture(scope="module")
def ops():
    from llm_singularity_b200 import kernels
    kernels.prepare(["embedding", "norm", "activation", "cache_table", "rope_cache", "attention",
                     "attention_tc", "gemm", "gemm_tc", "gemm_stream", "sampling"])
    yield kernels
    kernels.check_status()


def _rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).cuda()


# ------------------------------------------------------------------ small ones
def test_ops_refuse_cpu_tensors(ops):
    with pytest.raises(ops.KernelError, match="CUDA"):
        ops.swiglu(torch.zeros(2, 8), torch.zeros(2, 4))


@pytest.mark.parametrize("dtype", DTYPES)
def test_random_weights_are_the_same_bits_on_the_device_and_on_the_cpu(ops, dtype):
    """The random-weights stream: the kernel and the CPU statement of the same arithmetic."""
    from llm_singularity_b200.weights.random_init import normal_tensor, random_tensors, tensor_key
    key = tensor_key(12345, "model.layers.3.mlp.down_proj.weight")
    for shape, mean, scale in (((1_000_003,), 0.0, 0.02), ((257, 129), 1.0, 0.1), ((1,), 0.0, 1.0)):
        dev = normal_tensor(shape, key, mean, scale, dtype, "cuda")
        cpu = normal_tensor(shape, key, mean, scale, dtype, "cpu")
        assert dev.shape == cpu.shape
        diff = (dev.cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32)
                != cpu.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
        assert int(diff.sum()) == 0, f"{int(diff.sum())} of {diff.numel()} elements differ"
    expected = {"a.weight": ((33, 65), "matrix", "normal"), "n.weight": ((65,), "vector", "ones")}
    dev = random_tensors(expected, 9, dtype=dtype, std=0.05, norm_noise=0.1, device="cuda")
    cpu = random_tensors(expected, 9, dtype=dtype, std=0.05, norm_noise=0.1)
    assert all(torch.equal(dev[k].cpu(), cpu[k]) for k in expected)


def test_a_wait_that_runs_out_returns_and_is_reported(ops):
    """The kernels' waits on barriers are bounded.  A probe kernel of the matrix-product library
    waits, with a limit of 4,096 polls, on a barrier that nothing arrives at: it gives up and
    ends by itself, a second waiter of the block leaves on seeing that, and the status word the
    host reads afterwards says so (and is cleared by the reading)."""
    import ctypes
    lib = ops._lib("gemm_tc")
    result = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    rc = lib.lsb_gemm_tc_wait_probe(ctypes.c_int(4096), ctypes.c_void_p(result.data_ptr()),
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert result.tolist() == [1, 1]
    with pytest.raises(ops.KernelError, match="bounded wait"):
        ops.check_status()
    ops.check_status()                     # read and cleared: the library is usable again
    x = _rand(8, 64, dtype=torch.bfloat16, seed=1)
    w = _rand(32, 64, dtype=torch.bfloat16, seed=2)
    assert torch.allclose(ops.linear(x, w).float(), x.float() @ w.float().T, atol=0.5)


def test_scatter_i32(ops):
    dst = torch.full((5, 7), -1, dtype=torch.int32, device="cuda")
    idx = torch.tensor([0, 8, 34, 8], dtype=torch.int32, device="cuda")[:3]
    val = torch.tensor([4, 5, 6], dtype=torch.int32, device="cuda")
    ops.scatter_i32(dst, idx, val)
    want = torch.full((35,), -1, dtype=torch.int32)
    want[[0, 8, 34]] = torch.tensor([4, 5, 6], dtype=torch.int32)
    assert torch.equal(dst.cpu().view(-1), want)


def test_move_i32(ops):
    """dst[dst_idx[i]] = src[src_idx[i]]: sampled tokens become input tokens of the next step."""
    n = 700
    g = torch.Generator().manual_seed(0)
    src = torch.randint(0, 1 << 20, (900,), generator=g, dtype=torch.int32)
    dst = torch.full((2048,), -1, dtype=torch.int32)
    dst_idx = torch.randperm(2048, generator=g)[:n].to(torch.int32)
    src_idx = torch.randint(0, 900, (n,), generator=g, dtype=torch.int32)
    want = dst.clone()
    want[dst_idx.long()] = src[src_idx.long()]
    got = dst.cuda()
    ops.move_i32(got, dst_idx.cuda(), src.cuda(), src_idx.cuda())
    ops.check_status()
    assert torch.equal(got.cpu(), want)
    # an index outside either array is reported and nothing is written for it
    got = dst.cuda()
    ops.move_i32(got, torch.tensor([3, 2048], dtype=torch.int32, device="cuda"), src.cuda(),
                 torch.tensor([900, 1], dtype=torch.int32, device="cuda"))
    with pytest.raises(ops.KernelError, match="row index"):
        ops.check_status()
    assert torch.equal(got.cpu(), dst)
    with pytest.raises(ops.KernelError, match="differ in length"):
        ops.move_i32(got, dst_idx[:3].cuda(), src.cuda(), src_idx[:4].cuda())


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(ops, dtype):
    table = _rand(1000, 200, dtype=dtype)
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32, device="cuda")
    out = torch.empty(5, 200, dtype=torch.float32, device="cuda")
    ops.embedding(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


def test_embedding_reports_a_token_outside_the_table(ops):
    table = _rand(10, 8)
    out = torch.empty(2, 8, device="cuda")
    ops.embedding(table, torch.tensor([3, 10], dtype=torch.int32, device="cuda"), out)
    with pytest.raises(ops.KernelError, match="token id"):
        ops.check_status()
    assert torch.equal(out[1], torch.zeros(8, device="cuda")) and torch.equal(out[0], table[3])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [72, 2048, 2049, 5000])
def test_add_rmsnorm(ops, dtype, hidden):
    res = _rand(7, hidden, seed=1)
    delta = _rand(7, hidden, dtype=dtype, seed=2)
    w = 1 + 0.1 * _rand(hidden, seed=3)
    eps = 3e-6
    want_res = res.double() + delta.double()
    want = plain_llama.rms_norm(want_res, w.double(), eps)
    out = torch.empty(7, hidden, dtype=dtype, device="cuda")
    ops.add_rmsnorm(res, delta, w, eps, out)
    assert torch.allclose(res.double(), want_res, atol=1e-6)          # residual updated in 32-bit
    assert (out.double() - want).abs().max() <= _tol(dtype, want.abs().max().item())
    # without a delta the residual is left alone
    res2 = _rand(3, hidden, seed=4)
    keep = res2.clone()
    out2 = torch.empty(3, hidden, dtype=dtype, device="cuda")
    ops.add_rmsnorm(res2, None, w, eps, out2)
    assert torch.equal(res2, keep)
    want2 = plain_llama.rms_norm(keep.double(), w.double(), eps)
    assert (out2.double() - want2).abs().max() <= _tol(dtype, want2.abs().max().item())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [200, 4100])
def test_gather_add_rmsnorm_leaves_the_residual_alone(ops, dtype, hidden):
    res, delta = _rand(9, hidden, seed=1), _rand(9, hidden, dtype=dtype, seed=2)
    w = 1 + 0.1 * _rand(hidden, seed=3)
    rows = torch.tensor([8, 0, 3, 3], dtype=torch.int32, device="cuda")
    keep = res.clone()
    out = torch.empty(4, hidden, dtype=dtype, device="cuda")
    ops.gather_add_rmsnorm(res, delta, rows, w, 1e-5, out)
    want = plain_llama.rms_norm((keep.double() + delta.double())[rows.long()], w.double(), 1e-5)
    assert torch.equal(res, keep)
    assert (out.double() - want).abs().max() <= _tol(dtype, want.abs().max().item())


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(ops, dtype):
    gu = _rand(11, 200, dtype=dtype, scale=3.0)
    out = torch.empty(11, 100, dtype=dtype, device="cuda")
    ops.swiglu(gu, out)
    g, u = gu[:, 0::2].double(), gu[:, 1::2].double()       # gate and up alternate
    want = g / (1 + torch.exp(-g)) * u
    assert (out.double() - want).abs().max() <= _tol(dtype, want.abs().max().item())


@pytest.mark.parametrize("in_dtype, out_dtype", [(torch.float32, torch.float32),
                                                 (torch.bfloat16, torch.float32),
                                                 (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("M, N, K", [(1, 301, 72), (37, 301, 70), (130, 64, 2049), (64, 129, 16)])
def test_linear(ops, in_dtype, out_dtype, M, N, K):
    x, w = _rand(M, K, dtype=in_dtype, seed=1), _rand(N, K, dtype=in_dtype, seed=2)
    y = ops.linear(x, w, out_dtype=out_dtype)
    want = x.double() @ w.double().T
    assert y.dtype == out_dtype and y.shape == (M, N)
    tol = 3e-7 * K if out_dtype == torch.float32 else 1e-2 * want.abs().max().item()
    assert (y.double() - want).abs().max() <= tol


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M, N, K", [(1, 256, 64), (8, 16384, 2048), (40, 200, 72), (300, 1000, 136),
                                     (2048, 512, 256), (5, 64, 2048), (8, 19200, 200), (40, 30000, 64),
                                     (64, 16384, 2048), (17, 1616, 128), (128, 4096, 256), (100, 272, 64),
                                     (33, 16384, 2048)])
def test_gated_linear(ops, dtype, M, N, K):
    # out[m, i] = silu(x . w[2i]) * (x . w[2i + 1]); small N with large K makes the decode
    # orientation split K, so the activation has to wait for the sum of all splits; the last two
    # have more 128-row weight slabs than SMs and less than twice as many (two blocks share an SM);
    # the ones after them are batches of 17 to 128 rows, whose outputs leave the tile kernel through
    # a transposing epilogue (whole and partial slabs, whole and partial batch tiles)
    x, w = _rand(M, K, dtype=dtype, seed=1, scale=0.5), _rand(N, K, dtype=dtype, seed=2, scale=0.2)
    y = ops.linear(x, w, gated=True)
    d = x.double() @ w.double().T
    g, u = d[:, 0::2], d[:, 1::2]
    want = g / (1 + torch.exp(-g)) * u
    assert y.shape == (M, N // 2) and y.dtype == dtype
    tol = 3e-6 * K if dtype == torch.float32 else 1.5e-2 * (want.abs().max().item() + 1)
    assert (y.double() - want).abs().max() <= tol


@pytest.mark.parametrize("M, N, K", [(8, 3072, 2048), (8, 2048, 8192), (64, 2048, 2048), (3, 128, 4096)])
def test_split_k_products_are_repeatable(ops, M, N, K):
    # the decode orientation splits K over several blocks; the block arriving last sums the partial
    # tiles in split order, so the bits do not depend on arrival order, and the tile counters are
    # handed back zeroed for the next launch
    x, w = _rand(M, K, dtype=torch.bfloat16, seed=3), _rand(N, K, dtype=torch.bfloat16, seed=4)
    ops.SMALL_PRODUCTS = ops.STREAM_PRODUCTS = False     # the tile kernel, also where the others would do
    try:
        first = ops.linear(x, w, out_dtype=torch.float32)
        want = x.double() @ w.double().T
        assert (first.double() - want).abs().max() <= 3e-7 * K * 8
        for _ in range(5):
            assert torch.equal(ops.linear(x, w, out_dtype=torch.float32), first)
    finally:
        ops.SMALL_PRODUCTS = ops.STREAM_PRODUCTS = True


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M, N, K", [(1, 3072, 2048), (8, 2048, 2048), (8, 3072, 2048), (16, 2048, 2048),
                                     (9, 300, 64), (5, 4736, 128), (3, 7, 64), (13, 1000, 1024)])
def test_small_products(ops, M, N, K, out_dtype):
    # at most 16 rows times a matrix that fits the chip's shared memory: the kernel that keeps its
    # weight rows resident (the decode step's q/k/v and output projections); whole and partial
    # 16-row tiles, one and two 8-column tiles of the batch, fewer weight rows than SMs
    x, w = _rand(M, K, dtype=torch.bfloat16, seed=5), _rand(N, K, dtype=torch.bfloat16, seed=6)
    assert ops.small_gemm_ok(x, w)
    y = ops.linear(x, w, out_dtype=out_dtype)
    want = x.double() @ w.double().T
    assert y.dtype == out_dtype and y.shape == (M, N)
    tol = 3e-7 * K * 8 if out_dtype == torch.float32 else 1e-2 * want.abs().max().item()
    assert (y.double() - want).abs().max() <= tol
    for _ in range(3):
        assert torch.equal(ops.linear(x, w, out_dtype=out_dtype), y)      # a fixed summation order
    ops.SMALL_PRODUCTS = ops.STREAM_PRODUCTS = False
    try:
        other = ops.linear(x, w, out_dtype=torch.float32)                 # the tile kernel
    finally:
        ops.SMALL_PRODUCTS = ops.STREAM_PRODUCTS = True
    assert (other.double() - want).abs().max() <= 3e-7 * K * 8
    assert not ops.small_gemm_ok(_rand(17, K, dtype=torch.bfloat16, seed=1), w)
    assert not ops.small_gemm_ok(x[:, :K - 8].contiguous(), w[:, :K - 8].contiguous())


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M, N, K, act", [
    (8, 16384, 2048, "silu"), (8, 2048, 8192, None), (1, 2048, 8192, None), (16, 2048, 8192, None),
    (16, 16384, 2048, "silu"), (13, 1000, 384, None), (3, 14, 128, None), (5, 28672, 4096, "gelu_tanh"),
    (9, 40000, 256, None), (2, 302, 1152, "none"), (7, 6, 128, "silu"), (16, 5000, 128, None),
    (4, 300, 192, None), (11, 2050, 64, "silu")])
def test_streamed_products(ops, M, N, K, act, out_dtype):
    """At most 16 rows times a matrix of any size, every SM streaming its own share of the weight
    rows (the decode step's gate/up and down products): whole and partial 16-row tiles, one and
    two 8-row tiles of activations, fewer rows than SMs, more rows than one pass holds, every
    activation of a gated product; against 64-bit sums, bit for bit from call to call, and beside
    the tile kernel."""
    x = _rand(M, K, dtype=torch.bfloat16, seed=7, scale=0.5)
    w = _rand(N, K, dtype=torch.bfloat16, seed=8, scale=0.2)
    gated = act is not None
    assert ops.stream_gemm_ok(x, w, ops.ACTIVATIONS[act] if gated else 0)
    ops.SMALL_PRODUCTS = False
    try:
        y = ops.linear(x, w, out_dtype=out_dtype, gated=gated, activation=act or "silu")
        again = [ops.linear(x, w, out_dtype=out_dtype, gated=gated, activation=act or "silu") for _ in range(3)]
        ops.STREAM_PRODUCTS = False
        tile = ops.linear(x, w, out_dtype=torch.float32, gated=gated, activation=act or "silu")
    finally:
        ops.SMALL_PRODUCTS = ops.STREAM_PRODUCTS = True
    d = x.double() @ w.double().T
    if gated:
        g, u = d[:, 0::2], d[:, 1::2]
        a = {"silu": g / (1 + torch.exp(-g)), "none": g,
             "gelu_tanh": 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))}[act]
        want = a * u
    else:
        want = d
    assert y.dtype == out_dtype and y.shape == want.shape
    scale = want.abs().max().item() + 1
    tol = 3e-7 * K * 8 * scale if out_dtype == torch.float32 else 1e-2 * scale
    assert (y.double() - want).abs().max() <= tol
    assert all(torch.equal(t, y) for t in again)                       # a fixed summation order
    assert (tile.double() - want).abs().max() <= 2e-3 * scale          # (its activation is approximate)
    assert not ops.stream_gemm_ok(_rand(17, K, dtype=torch.bfloat16, seed=1), w)
    assert not ops.stream_gemm_ok(x[:, :K - 8].contiguous(), w[:, :K - 8].contiguous())


@pytest.mark.parametrize("M, K, H, N, act", [
    (8, 8192, 2048, 16384, "silu"), (8, 2048, 2048, 3072, None), (1, 2048, 2048, 3072, None),
    (16, 8192, 2048, 16384, "silu"), (13, 320, 192, 1000, None), (3, 128, 64, 28, "gelu_tanh"),
    (5, 192, 2112, 302, "none"), (9, 64, 40000 // 64 * 64, 66, None)])
def test_products_with_a_norm_folded_in(ops, M, K, H, N, act):
    """A product that adds its result to the residual stream and leaves the next norm half done
    (residual times weight, the rows' sums of squares in parts), and the product after it, which
    pays the rest by scaling its output rows: against residual add, RMS norm and product in 64-bit;
    the half-done norm finished by its own kernel; and the fallback where no kernel folds."""
    eps = 3e-5
    x = _rand(M, K, dtype=torch.bfloat16, seed=11, scale=0.5)
    w1 = _rand(H, K, dtype=torch.bfloat16, seed=12, scale=0.2)
    w2 = _rand(N, H, dtype=torch.bfloat16, seed=13, scale=0.2)
    g = (1 + 0.3 * _rand(H, seed=14)).contiguous()
    r0 = _rand(M, H, seed=15, scale=2.0)
    r0[0, 5] = 300.0                                  # one element that dominates its row's sum
    gated = act is not None
    residual = r0.clone()
    h = ops.linear(x, w1, into=(residual, g, eps))
    assert isinstance(h, ops.NormOut) and h.parts is not None and h.values.shape == (M, H)
    want_r = r0.double() + x.double() @ w1.double().T
    rs = want_r.abs().max().item()
    assert (residual.double() - want_r).abs().max() <= 3e-7 * K * 8 * (rs + 1)
    assert (h.values.double() - residual.double() * g.double()).abs().max() <= 4e-3 * (rs * 1.3 + 1)
    ss = h.parts.double().sum(0)[:M]
    assert ((ss - (residual.double() ** 2).sum(1)).abs() <= 1e-5 * ss).all()
    normed = want_r * torch.rsqrt((want_r ** 2).mean(1, keepdim=True) + eps) * g.double()
    fin = ops.finish_norm(h)
    assert (fin.double() - normed).abs().max() <= 1.2e-2 * (normed.abs().max().item() + 1)
    y = ops.linear(h, w2, gated=gated, activation=act or "silu", out_dtype=torch.float32)
    d = normed @ w2.double().T
    if gated:
        gg, u = d[:, 0::2], d[:, 1::2]
        a = {"silu": gg / (1 + torch.exp(-gg)), "none": gg,
             "gelu_tanh": 0.5 * gg * (1 + torch.tanh(math.sqrt(2 / math.pi) * (gg + 0.044715 * gg ** 3)))}[act]
        want = a * u
    else:
        want = d
    # (the inputs of the second product are rounded to bfloat16: 2^-9 relative each, summed at random)
    tol = 2.0 ** -8 * (normed.abs().double() @ w2.abs().double().T).max().item() / math.sqrt(H) * 4
    if gated:
        tol *= d.abs().max().item() + 1
    assert y.shape == want.shape and (y.double() - want).abs().max() <= tol + 1e-6
    again = ops.linear(h, w2, gated=gated, activation=act or "silu", out_dtype=torch.float32)
    assert torch.equal(again, y)
    # where no kernel folds (the streaming products off): the same meaning through separate kernels
    ops.STREAM_PRODUCTS = False
    try:
        residual2 = r0.clone()
        h2 = ops.linear(x, w1, into=(residual2, g, eps))
        assert isinstance(h2, ops.NormOut) and h2.parts is None
        y2 = ops.linear(h2, w2, gated=gated, activation=act or "silu", out_dtype=torch.float32)
    finally:
        ops.STREAM_PRODUCTS = True
    assert (residual2.double() - want_r).abs().max() <= 3e-7 * K * 8 * (rs + 1) + 1e-2 * (x.double() @ w1.double().T).abs().max().item()
    assert (h2.values.double() - normed).abs().max() <= 1.2e-2 * (normed.abs().max().item() + 1)
    assert (y2.double() - want).abs().max() <= 2 * tol + 1e-6


def test_streamed_products_warm_what_followed_them_last_time(ops):
    """A streaming product asks L2 for the first weights of the product that followed it the last
    time.  That changes no result; the follower is learnt from the calls themselves, forgotten
    when its tensor is gone, and any other kind of product ends the chain."""
    M = 8
    x = _rand(M, 2048, dtype=torch.bfloat16, seed=21, scale=0.5)
    a = _rand(4096, 2048, dtype=torch.bfloat16, seed=22, scale=0.2)      # gated: 2048 outputs
    b = _rand(2048, 2048, dtype=torch.bfloat16, seed=23, scale=0.2)
    big = _rand(300, 2048, dtype=torch.bfloat16, seed=24, scale=0.2)
    ops.SMALL_PRODUCTS = False
    try:
        def chain():
            h = ops.linear(x, a, gated=True)
            return ops.linear(h, b)
        ops.WARM_NEXT = False
        want = chain()
        ops.WARM_NEXT = True
        ops._follows.clear()
        ops._chain_ends()
        first = chain()                                   # learns: b follows a
        assert ops._follows[a.data_ptr()][0]() is b and ops._follows[a.data_ptr()][1] is False
        assert b.data_ptr() not in ops._follows
        second = chain()                                  # a warms b; and learns: a (gated) follows b
        assert ops._follows[b.data_ptr()][0]() is a and ops._follows[b.data_ptr()][1] is True
        third = chain()                                   # both warm
        assert ops._warm_after(a, True, M) is not None
        ops.linear(_rand(40, 2048, dtype=torch.bfloat16, seed=25), big)   # another kind of product
        assert ops._last_streamed is None
        assert torch.equal(first, want) and torch.equal(second, want) and torch.equal(third, want)
        gone = b.data_ptr()
        del b, chain
        import gc
        gc.collect()
        assert ops._warm_after(a, True, M) is None and a.data_ptr() not in ops._follows and gone
    finally:
        ops.SMALL_PRODUCTS = ops.WARM_NEXT = True
        ops._follows.clear()
        ops._chain_ends()


def test_linear_float32_is_true_32_bit(ops):
    # (1 + 2^-20) * 1 + 1 * (-1) = 2^-20 exactly in 32-bit; a reduced-precision matrix mode
    # (10-bit mantissa operands) rounds the first factor to 1 and returns 0
    K = 256
    x = torch.zeros(1, K, device="cuda")
    w = torch.zeros(1, K, device="cuda")
    x[0, 0], w[0, 0] = 1 + 2.0 ** -20, 1.0
    x[0, 1], w[0, 1] = 1.0, -1.0
    assert ops.linear(x, w).item() == 2.0 ** -20


# --------------------------------------------------------------- rope + cache
class _Ctx:
    pass


def _make_ctx(q_lens, kv_lens, table_rows=None):
    from llm_singularity_b200.engine.batch import ContextBuilder
    b = ContextBuilder("cuda", 4096, 64)
    R = len(q_lens)
    toks = [[0] * n for n in q_lens]
    starts = [kv - q for kv, q in zip(kv_lens, q_lens)]
    ctx, _ = b.build(toks, starts, table_rows or list(range(R)), [[] for _ in range(R)])
    ctx._keep = b
    return ctx


def _make_cache(R, max_kv, nkv, hd, page_size, dtype, seed=0, window=None, slots=None):
    from llm_singularity_b200.cache.manager import KVCacheView
    pages_per = -(-max_kv // page_size)
    slots = slots or R
    n_pages = slots * pages_per + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g)[:slots * pages_per].view(slots, pages_per)
    k = torch.zeros(n_pages, nkv, page_size, hd, dtype=dtype, device="cuda")
    v = torch.zeros_like(k)
    return KVCacheView(k, v, perm.to(torch.int32).cuda(), page_size, window, 0)


def _fill(cache, row, K, V):
    """Write dense K, V [len, nkv, hd] of one request into its pages."""
    n = K.shape[0]
    pos = torch.arange(n)
    pages = cache.block_table[row].cpu()[pos // cache.page_size].long()
    cache.k_pages[pages, :, pos % cache.page_size, :] = K.to(cache.k_pages.dtype).cuda()
    cache.v_pages[pages, :, pos % cache.page_size, :] = V.to(cache.v_pages.dtype).cuda()


def _dense(cache, row, n):
    pos = torch.arange(n)
    pages = cache.block_table[row].cpu()[pos // cache.page_size].long()
    return cache.k_pages[pages, :, pos % cache.page_size, :], cache.v_pages[pages, :, pos % cache.page_size, :]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh, nkv, hd, rot, page", [(5, 5, 80, 40, 4), (4, 1, 32, 32, 8), (6, 2, 128, 128, 16)])
def test_rope_kv_store(ops, dtype, nh, nkv, hd, rot, page):
    from llm_singularity_b200.parts.rotary import rotary_inv_freq
    q_lens, kv_lens = [3, 1, 9], [3, 30, 20]          # a fresh prompt, a decode token, a later portion
    ctx = _make_ctx(q_lens, kv_lens, table_rows=[2, 0, 1])
    cache = _make_cache(3, 32, nkv, hd, page, dtype)
    T = sum(q_lens)
    qkv = _rand(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=5)
    orig = qkv.clone()
    inv = rotary_inv_freq(rot, 10000.0).float().cuda()
    ops.rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv, rot)
    pos = ctx.positions.cpu().tolist()
    assert pos == [0, 1, 2, 29] + list(range(11, 20))
    o = orig.double().cpu()
    q0 = o[:, :nh * hd].view(T, nh, hd)
    k0 = o[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v0 = o[:, (nh + nkv) * hd:].view(T, nkv, hd)

    def rope(x):
        y = x.clone()
        y[..., :rot] = plain_llama.apply_rope(x[..., :rot], pos, inv.double().cpu())
        return y
    tol = _tol(dtype, 4.0)
    got_q = qkv[:, :nh * hd].double().cpu().view(T, nh, hd)
    assert (got_q - rope(q0)).abs().max() <= tol
    assert torch.equal(qkv[:, (nh + nkv) * hd:], orig[:, (nh + nkv) * hd:])       # values untouched
    want_k = rope(k0)
    t = 0
    for r, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        Kc, Vc = _dense(cache, [2, 0, 1][r], kl)
        sl = slice(kl - ql, kl)
        assert (Kc[sl].double().cpu() - want_k[t:t + ql]).abs().max() <= tol
        assert torch.equal(Vc[sl].cpu(), v0[t:t + ql].to(dtype))
        assert Kc[:kl - ql].abs().max() == 0 if kl > ql else True             # nothing else written
        t += ql
    # store=False rotates but leaves the pages alone
    before = cache.k_pages.clone()
    qkv2 = orig.clone()
    ops.rope_kv_store(qkv2, nh, nkv, hd, ctx, cache, inv, rot, store=False)
    assert torch.equal(cache.k_pages, before) and torch.equal(qkv2[:, :nh * hd], qkv[:, :nh * hd])


def test_rope_kv_store_reports_a_page_that_is_not_held(ops):
    ctx = _make_ctx([2], [2])
    cache = _make_cache(1, 16, 1, 16, 16, torch.float32)
    cache.block_table[0, 0] = -1
    qkv = _rand(2, 3 * 16)
    ops.rope_kv_store(qkv, 1, 1, 16, ctx, cache, None, 0)
    with pytest.raises(ops.KernelError, match="page"):
        ops.check_status()
    assert cache.k_pages.abs().max() == 0


# ------------------------------------------------------------------- attention
@pytest.mark.parametrize("nh, nkv, hd, page, window, rotary",
                         [(8, 2, 64, 16, 0, 64), (32, 8, 64, 16, 0, 64), (6, 2, 128, 32, 0, 128),
                          (16, 1, 64, 8, 0, 64), (4, 4, 64, 4, 0, 64), (8, 2, 64, 16, 40, 64),
                          (8, 2, 64, 16, 0, 32), (6, 3, 64, 8, 0, 16), (6, 2, 128, 32, 0, 32),
                          (4, 4, 128, 16, 40, 96), (18, 2, 128, 16, 0, 64)])
@pytest.mark.parametrize("q_lens, kv_lens", [([1, 1, 1, 1], [1, 16, 17, 700]), ([1, 9, 1, 130], [33, 20, 4097, 130]),
                                             ([1], [5000])])
def test_decode_kernel_rotates_and_stores_like_the_separate_kernel(ops, monkeypatch, nh, nkv, hd, page,
                                                                    window, rotary, q_lens, kv_lens):
    """rope_store_attention (single tokens rotated and stored inside the decode kernel) against
    rope_kv_store followed by paged_attention on copies of the same inputs: same outputs, same
    pages; also with store off, and with only the first `rotary` dims of a head rotated."""
    from llm_singularity_b200.parts.rotary import rotary_inv_freq
    dtype = torch.bfloat16
    R = len(q_lens)
    rows = list(reversed(range(R)))
    ctx = _make_ctx(q_lens, kv_lens, table_rows=rows)
    T = sum(q_lens)
    inv = rotary_inv_freq(rotary, 500000.0).float().cuda()
    scale = 1.0 / math.sqrt(hd)
    called = []
    call = ops._call
    monkeypatch.setattr(ops, "_call", lambda lib, name, *a: (called.append(name), call(lib, name, *a))[1])
    qkv0 = _rand(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=3)
    results = []
    for fused in (False, True):
        for store in (True, False):
            cache = _make_cache(R, max(kv_lens), nkv, hd, page, dtype, seed=1)
            for r in range(R):
                _fill(cache, rows[r], _rand(kv_lens[r], nkv, hd, dtype=dtype, seed=10 + r).cpu(),
                      _rand(kv_lens[r], nkv, hd, dtype=dtype, seed=20 + r).cpu())
            qkv = qkv0.clone()
            out = torch.empty(T, nh * hd, dtype=dtype, device="cuda")
            if fused:
                ops.rope_store_attention(qkv, nh, nkv, hd, ctx, cache, inv, rotary, store, scale, window, out)
                assert "lsb_decode_attention_rope" in called
            else:
                ops.rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv, rotary, store=store)
                ops.paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out)
                assert "lsb_decode_attention_rope" not in called
            ops.check_status()
            results.append((out.float().cpu(), cache.k_pages.float().cpu(), cache.v_pages.cpu()))
    for a, b in ((0, 2), (1, 3)):
        out_a, k_a, v_a = results[a]
        out_b, k_b, v_b = results[b]
        assert torch.equal(v_a, v_b)
        # the two kernels may contract the rotation's multiply-adds differently: one bfloat16 step
        assert (k_a - k_b).abs().max() <= 2.0 ** -7 * k_a.abs().max()
        assert (out_a - out_b).abs().max() <= _tol(dtype, 3.0)


@pytest.mark.parametrize("hd, q_lens, kv_lens", [(64, [1, 1, 150, 1, 40], [300, 17, 200, 4097, 40]),
                                                 (128, [1, 9, 1], [900, 30, 64])])
def test_decode_kernel_beside_the_prompt_kernels_gives_the_same_bits(ops, hd, q_lens, kv_lens):
    """A step with single tokens and prompt portions: the decode kernel on a second stream beside
    the rotation and the portions' attention, against all of them in a row."""
    from llm_singularity_b200 import kernels
    from llm_singularity_b200.parts.rotary import rotary_inv_freq
    nh, nkv, page, dtype = 8, 2, 16, torch.bfloat16
    R, T = len(q_lens), sum(q_lens)
    inv = rotary_inv_freq(hd, 500000.0).float().cuda()
    qkv0 = _rand(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=3)
    results = []
    try:
        for beside in (False, True, True):
            kernels.OVERLAP_ATTENTION = beside
            ctx = _make_ctx(q_lens, kv_lens)
            cache = _make_cache(R, max(kv_lens), nkv, hd, page, dtype, seed=1)
            for r in range(R):
                _fill(cache, r, _rand(kv_lens[r], nkv, hd, dtype=dtype, seed=10 + r).cpu(),
                      _rand(kv_lens[r], nkv, hd, dtype=dtype, seed=20 + r).cpu())
            qkv = qkv0.clone()
            out = torch.empty(T, nh * hd, dtype=dtype, device="cuda")
            ops.rope_store_attention(qkv, nh, nkv, hd, ctx, cache, inv, hd, True, 1.0 / math.sqrt(hd), 0, out)
            follow = out.float().sum()                   # the step's stream goes on after both
            ops.check_status()
            results.append((out.cpu(), cache.k_pages.cpu(), cache.v_pages.cpu(), follow.item()))
    finally:
        kernels.OVERLAP_ATTENTION = True
    for other in results[1:]:
        assert all(torch.equal(a, b) for a, b in zip(results[0][:3], other[:3]))
        assert results[0][3] == other[3]


def _ref_attention(q, K, V, scale, window):
    """q [n, nh, hd] are the last n positions of a sequence whose keys/values are K, V [len, nkv, hd]."""
    n, nh, hd = q.shape
    L, nkv = K.shape[0], K.shape[1]
    out = torch.zeros(n, nh, hd, dtype=torch.float64)
    for i in range(n):
        p = L - n + i
        lo = max(0, p - window + 1) if window else 0
        for h in range(nh):
            g = h // (nh // nkv)
            s = (K[lo:p + 1, g] @ q[i, h]) * scale
            out[i, h] = torch.softmax(s, 0) @ V[lo:p + 1, g]
    return out


def _run_attention(ops, dtype, nh, nkv, hd, page, q_lens, kv_lens, window=0, seed=0, qk_boost=None):
    R = len(q_lens)
    rows = list(reversed(range(R)))
    ctx = _make_ctx(q_lens, kv_lens, table_rows=rows)
    cache = _make_cache(R, max(kv_lens), nkv, hd, page, dtype, seed=seed)
    T = sum(q_lens)
    qkv = _rand(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=seed + 1)
    Ks, Vs = [], []
    for r in range(R):
        K = _rand(kv_lens[r], nkv, hd, dtype=dtype, seed=seed + 10 + r).cpu()
        V = _rand(kv_lens[r], nkv, hd, dtype=dtype, seed=seed + 20 + r).cpu()
        Ks.append(K); Vs.append(V)
    if qk_boost:
        qk_boost(qkv, Ks, ctx)
    for r in range(R):
        _fill(cache, rows[r], Ks[r], Vs[r])
    out = torch.empty(T, nh * hd, dtype=dtype, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    ops.paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out)
    t = 0
    worst = 0.0
    for r in range(R):
        q = qkv[t:t + q_lens[r], :nh * hd].double().cpu().view(q_lens[r], nh, hd)
        want = _ref_attention(q, Ks[r].double(), Vs[r].double(), scale, window)
        got = out[t:t + q_lens[r]].double().cpu().view(q_lens[r], nh, hd)
        worst = max(worst, (got - want).abs().max().item())
        t += q_lens[r]
    return worst


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh, nkv, hd, page", [(6, 3, 48, 16), (8, 1, 16, 8), (5, 5, 128, 4),
                                               (4, 2, 256, 32), (3, 1, 80, 16), (8, 2, 64, 16),
                                               (16, 1, 64, 8), (6, 2, 128, 32), (34, 2, 64, 16)])
def test_attention_mixed_batch(ops, dtype, nh, nkv, hd, page):
    # a whole prompt, a decode token on a long context, a portion in the middle, two tokens
    # (bfloat16 with head size 64/128 takes the tensor-core kernels, unless a group has > 16 heads)
    worst = _run_attention(ops, dtype, nh, nkv, hd, page, [37, 1, 12, 2, 1], [37, 300, 45, 64, 1])
    assert worst <= _tol(dtype, 3.0)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("q_lens, kv_lens", [([1], [5000]), ([1, 1, 1], [1, 64, 65]), ([200], [200]),
                                             ([130, 1], [700, 129]), ([64, 65, 63], [64, 65, 1000])])
def test_tensor_core_attention_shapes(ops, hd, q_lens, kv_lens):
    # decode with many splits, lengths on tile edges (64), prompts over several 64-row tiles,
    # a portion deep inside a long context
    worst = _run_attention(ops, torch.bfloat16, 8, 2, hd, 16, q_lens, kv_lens, seed=3)
    assert worst <= _tol(torch.bfloat16, 3.0)


@pytest.mark.parametrize("hd", [64, 128])
def test_prompt_attention_with_ragged_last_tiles_is_the_same_every_time(ops, hd):
    """Several prompt portions whose last 128-row tile is partly empty, run many times: every run
    must match the reference and the first run bit for bit.  (Rows without a query make their
    softmax warp faster than its neighbours; once it ran a whole tile ahead, its arrival was
    counted for the tile the others were still writing P for.)"""
    nh, nkv, page = 8, 2, 16
    q_lens, kv_lens = [577, 577, 577, 101], [1024, 1024, 1024, 1024]
    dtype = torch.bfloat16
    R, T = len(q_lens), sum(q_lens)
    ctx = _make_ctx(q_lens, kv_lens, table_rows=list(range(R)))
    cache = _make_cache(R, max(kv_lens), nkv, hd, page, dtype, seed=2)
    Ks = [_rand(kv_lens[r], nkv, hd, dtype=dtype, seed=30 + r).cpu() for r in range(R)]
    Vs = [_rand(kv_lens[r], nkv, hd, dtype=dtype, seed=40 + r).cpu() for r in range(R)]
    for r in range(R):
        _fill(cache, r, Ks[r], Vs[r])
    qkv = _rand(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=4)
    scale = 1.0 / math.sqrt(hd)
    first = None
    for it in range(60):
        out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device="cuda")
        ops.paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, 0, out)
        if first is None:
            first = out.clone()
            t = 0
            for r in range(R):
                q = qkv[t:t + q_lens[r], :nh * hd].double().cpu().view(q_lens[r], nh, hd)
                want = _ref_attention(q, Ks[r].double(), Vs[r].double(), scale, 0)
                got = out[t:t + q_lens[r]].double().cpu().view(q_lens[r], nh, hd)
                assert (got - want).abs().max() <= _tol(dtype, 3.0)
                t += q_lens[r]
        else:
            assert torch.equal(out, first), f"run {it} differs from the first"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kv_len", [15, 16, 17, 31, 32, 33, 64, 65])
@pytest.mark.parametrize("hd", [32, 64])
def test_attention_at_page_edges(ops, dtype, kv_len, hd):
    # lengths that end just before, on and just after a page's edge; decode and 2-token portions
    assert _run_attention(ops, dtype, 4, 2, hd, 16, [1, 2], [kv_len, kv_len]) <= _tol(dtype, 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(ops, dtype):
    # the query of the last row points at key 3 of 700 (times 6): softmax puts nearly all mass
    # there, so skipping, misplacing or mis-paging that one key changes the output by O(1)
    def boost(qkv, Ks, ctx):
        nh, hd = 4, 64
        for h in range(nh):
            qkv[-1, h * hd:(h + 1) * hd] = (Ks[0][3, h // 2] * 6).to(qkv.dtype)
    assert _run_attention(ops, dtype, 4, 2, 64, 16, [1], [700], qk_boost=boost) <= _tol(dtype, 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 17, 70])
@pytest.mark.parametrize("offset", [0, 1])
@pytest.mark.parametrize("hd, q_len", [(32, 3), (64, 3), (64, 1)])
def test_attention_window_edge(ops, dtype, window, offset, hd, q_len):
    # the stand-out key sits just outside (offset 0) or just inside (offset 1) the window of the
    # last query: taking it in or leaving it out by mistake changes the output by O(1)
    kv_len = 150

    def boost(qkv, Ks, ctx):
        j = kv_len - 1 - window + offset
        qkv[-1, :hd] = (Ks[0][j, 0] * 6).to(qkv.dtype)
    worst = _run_attention(ops, dtype, 1, 1, hd, 8, [q_len], [kv_len], window=window, qk_boost=boost)
    assert worst <= _tol(dtype, 3.0)


@pytest.mark.parametrize("q_lens, kv_lens", [([1, 200, 1, 130], [300, 330, 700, 130]), ([1, 100], [260, 100])])
def test_kernels_address_a_pool_of_more_than_two_to_the_31_elements(ops, q_lens, kv_lens):
    """300,000 pages of 8 x 16 x 64 are 2.46e9 elements per pool: offsets into it need 64 bits.  The
    requests hold the topmost pages; decode kernel, both prompt kernels and the cache write."""
    from llm_singularity_b200.cache.manager import KVCacheView
    if torch.cuda.mem_get_info()[0] < 16 << 30:
        pytest.skip("needs 10 GB of device memory")
    nh, nkv, hd, page, n_pages, dtype = 32, 8, 64, 16, 300_000, torch.bfloat16
    R, per = len(q_lens), -(-max(kv_lens) // page)
    k = torch.zeros(n_pages, nkv, page, hd, dtype=dtype, device="cuda")
    v = torch.zeros_like(k)
    assert k.numel() > 2 ** 31
    top = n_pages - 1 - torch.randperm(R * per, generator=torch.Generator().manual_seed(0))
    cache = KVCacheView(k, v, top.view(R, per).to(torch.int32).cuda(), page, None, 0)
    ctx = _make_ctx(q_lens, kv_lens)
    T = sum(q_lens)
    qkv = _rand(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=1)
    Ks = [_rand(n, nkv, hd, dtype=dtype, seed=10 + r).cpu() for r, n in enumerate(kv_lens)]
    Vs = [_rand(n, nkv, hd, dtype=dtype, seed=20 + r).cpu() for r, n in enumerate(kv_lens)]
    for r in range(R):
        _fill(cache, r, Ks[r], Vs[r])
    out = torch.empty(T, nh * hd, dtype=dtype, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    ops.paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, 0, out)
    ops.check_status()
    t = 0
    for r in range(R):
        q = qkv[t:t + q_lens[r], :nh * hd].double().cpu().view(q_lens[r], nh, hd)
        want = _ref_attention(q, Ks[r].double(), Vs[r].double(), scale, 0)
        got = out[t:t + q_lens[r]].double().cpu().view(q_lens[r], nh, hd)
        assert (got - want).abs().max().item() < _tol(dtype, 2.0)
        t += q_lens[r]
    fresh = _rand(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=3)
    before = fresh.clone()
    ops.rope_kv_store(fresh, nh, nkv, hd, ctx, cache, torch.rand(hd // 2, device="cuda"), hd)
    ops.check_status()
    t = 0
    for r in range(R):
        n, L = q_lens[r], kv_lens[r]
        kd, vd = _dense(cache, r, L)
        assert torch.equal(kd[L - n:], fresh[t:t + n, nh * hd:(nh + nkv) * hd].view(n, nkv, hd))
        assert torch.equal(vd[L - n:], before[t:t + n, (nh + nkv) * hd:].view(n, nkv, hd))
        t += n
    del k, v, cache
    torch.cuda.empty_cache()


def test_attention_refuses_sizes_it_does_not_take(ops):
    ctx = _make_ctx([1], [1])
    for hd in (24, 272):
        cache = _make_cache(1, 16, 1, hd, 16, torch.float32)
        with pytest.raises(ops.KernelError, match="head_dim"):
            ops.paged_attention(_rand(1, 3 * hd), 1, 1, hd, ctx, cache, 1.0, 0,
                                torch.empty(1, hd, device="cuda"))
    cache = _make_cache(1, 16, 2, 16, 16, torch.float32)
    with pytest.raises(ops.KernelError, match="kv heads"):
        ops.paged_attention(_rand(1, 7 * 16), 3, 2, 16, ctx, cache, 1.0, 0,
                            torch.empty(1, 48, device="cuda"))


# -------------------------------------------------------------------- sampling
def _u(i):
    from llm_singularity_b200.sampling import uniform
    return uniform(1234, i)


@pytest.mark.parametrize("vocab", [301, 5000])
def test_sampling_matches_the_plain_sampler(ops, vocab):
    g = torch.Generator().manual_seed(0)
    R = 24
    logits = (torch.randn(R, vocab, generator=g) * 3).cuda()
    combos = [(0.0, 0, 1.0, 1.0), (1.0, 0, 1.0, 1.0), (0.7, 5, 1.0, 1.0), (1.3, 0, 0.8, 1.0),
              (0.9, 40, 0.6, 1.0), (1.0, 0, 1.0, 1.7), (0.0, 0, 1.0, 50.0), (0.8, 3, 0.9, 1.3)]
    params, topk, prev, prev_start = [], [], [], [0]
    for r in range(R):
        t, k, p, pen = combos[r % len(combos)]
        params.append([t, p, pen, _u(r)])
        topk.append(k)
        mine = torch.randint(0, vocab, (6,), generator=g).tolist() + [int(logits[r].argmax())] * 2
        prev += mine
        prev_start.append(len(prev))
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(logits, torch.tensor(params, device="cuda"), torch.tensor(topk, dtype=torch.int32, device="cuda"),
               torch.tensor(prev_start, dtype=torch.int32, device="cuda"),
               torch.tensor(prev, dtype=torch.int32, device="cuda"), out)
    got = out.cpu().tolist()
    host = logits.cpu()
    for r in range(R):
        t, k, p, pen = combos[r % len(combos)]
        mine = prev[prev_start[r]:prev_start[r + 1]]
        # the plain sampler in float32 arithmetic mirrors the kernel's rounding of x / T
        row = host[r].tolist()
        want = plain_llama.sample_plain(row, t, k, p, pen, mine, params[r][3])
        if got[r] != want:
            # only acceptable when u falls within rounding of a boundary of the CDF
            lo = plain_llama.sample_plain(row, t, k, p, pen, mine, max(params[r][3] - 1e-5, 1e-9))
            hi = plain_llama.sample_plain(row, t, k, p, pen, mine, min(params[r][3] + 1e-5, 1 - 1e-9))
            assert got[r] in (lo, hi), f"row {r}: got {got[r]}, plain {want}"


def test_greedy_takes_the_first_maximum(ops):
    logits = torch.zeros(3, 70000, device="cuda")
    logits[0, [69999, 40000, 123]] = 5.0
    logits[1, 69999] = 1.0
    out = torch.empty(3, dtype=torch.int32, device="cuda")
    params = torch.tensor([[0.0, 1.0, 1.0, 0.5]] * 3, device="cuda")
    ops.sample(logits, params, torch.zeros(3, dtype=torch.int32, device="cuda"), None, None, out)
    assert out.cpu().tolist() == [123, 69999, 0]


@pytest.mark.parametrize("vocab", [128256, 20001, 16384])
def test_greedy_rows_scanned_by_several_blocks(ops, vocab):
    """A few greedy rows over a large vocabulary are scanned by several blocks each, whose partial
    maxima meet in device memory: equal maxima in different blocks' slices still give the first one,
    again and again (the arrival counter is left at zero), also beside rows that sample and rows
    with a repetition penalty (which one block scans alone)."""
    g = torch.Generator().manual_seed(3)
    R = 7
    logits = torch.randn(R, vocab, generator=g)
    per = -(-vocab // 16)
    logits[0, [per - 1, per, 5 * per + 3, vocab - 1]] = 9.0          # ties on both sides of a slice's edge
    logits[1, vocab - 1] = 9.0
    logits[2, 0] = 9.0
    logits[3] = 0.0                                                  # every value equal: index 0
    logits[5, [7 * per + 1, 12 * per]] = 9.0
    params = [[0.0, 1.0, 1.0, 0.5]] * 4 + [[1.0, 1.0, 1.0, 0.3], [0.0, 1.0, 4.0, 0.5], [0.0, 1.0, 1.0, 0.5]]
    prev_start = [0, 0, 0, 0, 0, 0, 2, 2]
    prev = [7 * per + 1, 3]                                          # row 5: its first maximum is penalised
    out = torch.full((R,), -1, dtype=torch.int32, device="cuda")
    dev = logits.cuda()
    for _ in range(3):
        out.fill_(-1)
        ops.sample(dev, torch.tensor(params, device="cuda"), torch.zeros(R, dtype=torch.int32, device="cuda"),
                   torch.tensor(prev_start, dtype=torch.int32, device="cuda"),
                   torch.tensor(prev, dtype=torch.int32, device="cuda"), out)
        got = out.cpu().tolist()
        assert got[0] == per - 1 and got[1] == vocab - 1 and got[2] == 0 and got[3] == 0
        assert got[4] == plain_llama.sample_plain(logits[4].tolist(), 1.0, 0, 1.0, 1.0, (), 0.3)
        assert got[5] == 12 * per
        assert got[6] == int(logits[6].argmax())


def test_sampling_falls_back_to_the_last_kept_token(ops):
    """When the running sum never reaches u * total (rounding at the very end of the scan; forced
    here by a draw above one), the token is the last kept one in index order, as in the reference
    (core/src/sampling.cpp:113-116), also when every later stretch of the vocabulary is empty."""
    vocab = 128256
    logits = torch.full((2, vocab), -5.0)
    for i, x in ((5, 4.0), (900, 3.0), (70000, 3.5)):
        logits[:, i] = x
    params = torch.tensor([[1.0, 1.0, 1.0, 1.5], [1.0, 1.0, 1.0, 0.999]], device="cuda")
    out = torch.empty(2, dtype=torch.int32, device="cuda")
    ops.sample(logits.cuda(), params, torch.tensor([3, 3], dtype=torch.int32, device="cuda"), None, None, out)
    row = logits[0].tolist()
    assert out.tolist() == [plain_llama.sample_plain(row, 1.0, 3, 1.0, 1.0, (), 1.5),
                            plain_llama.sample_plain(row, 1.0, 3, 1.0, 1.0, (), 0.999)] == [70000, 70000]


def test_sampling_follows_the_distribution(ops):
    # 4000 draws from softmax([2, 1, 0, -1] / 1): frequencies within 3 sigma
    R = 4000
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0] + [-30.0] * 60], device="cuda").repeat(R, 1)
    params = torch.tensor([[1.0, 1.0, 1.0, _u(i)] for i in range(R)], device="cuda")
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(logits, params, torch.zeros(R, dtype=torch.int32, device="cuda"), None, None, out)
    counts = np.bincount(out.cpu().numpy(), minlength=4)[:4] / R
    p = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0]), 0).numpy()
    assert np.all(np.abs(counts - p) < 3 * np.sqrt(p * (1 - p) / R) + 1e-3)
