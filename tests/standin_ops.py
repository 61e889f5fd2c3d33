"""Dense-tensor stand-ins for the kernel entry points, for tests without a GPU.

The product has no CPU path: ``llm_singularity_b200.kernels`` refuses to run
without its compiled CUDA libraries.  These functions mirror the signatures of
that module so that host-side logic (cache manager, block tables, step
metadata, scheduler, entry point) can be driven end to end on the CPU box where
the tests are written.  They are handed to ``Runtime(ops=...)`` explicitly by
tests and are never imported by the package.
"""
from __future__ import annotations

import torch


def prepare(names, verbose=False):
    return None


def scatter_i32(dst, idx, val):
    dst.view(-1)[idx.long()] = val


def move_i32(dst, dst_idx, src, src_idx):
    dst[dst_idx.long()] = src[src_idx.long()]


def embedding(table, ids, out):
    out.copy_(table[ids.long()].float())


def _rms(x, w, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def add_rmsnorm(residual, delta, weight, eps, out):
    if delta is not None:
        residual += delta.float()
    out.copy_(_rms(residual, weight, eps).to(out.dtype))


def gather_add_rmsnorm(residual, delta, rows, weight, eps, out):
    x = residual[rows.long()]
    if delta is not None:
        x = x + delta[rows.long()].float()
    out.copy_(_rms(x, weight, eps).to(out.dtype))


ACTIVATIONS = {"silu": 1, "gelu_tanh": 2, "none": 3}


def _act(g, name):
    if name == "silu":
        return g / (1 + torch.exp(-g))
    if name == "gelu_tanh":
        return 0.5 * g * (1 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    assert name == "none"
    return g


def linear(x, w, out_dtype=None, gated=False, activation="silu"):
    y = x.float() @ w.float().T
    if gated:
        y = _act(y[:, 0::2], activation) * y[:, 1::2]
    return y.to(out_dtype or x.dtype)


def swiglu(gate_up, out):
    g, u = gate_up[:, 0::2].float(), gate_up[:, 1::2].float()
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store=True):
    T = qkv.shape[0]
    pos = ctx.positions.long()
    q = qkv[:, :nh * hd].view(T, nh, hd)
    k = qkv[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
    if inv_freq is not None:
        half = rotary_dim // 2
        ang = pos.float()[:, None] * inv_freq[None, :]
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        for x in (q, k):
            x0, x1 = x[..., :half].float().clone(), x[..., half:rotary_dim].float().clone()
            x[..., :half] = (x0 * cos - x1 * sin).to(x.dtype)
            x[..., half:rotary_dim] = (x0 * sin + x1 * cos).to(x.dtype)
    if store:
        ps = cache.page_size
        rows = ctx.table_rows.long()[ctx.token_req.long()]
        pages = cache.block_table[rows, pos // ps].long()
        assert (pages >= 0).all(), "write into a page that is not held"
        off = pos % ps
        cache.k_pages[pages, :, off, :] = k
        cache.v_pages[pages, :, off, :] = v


def rope_store_attention(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store, scale, window, out):
    rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store)
    paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out)


def paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out):
    T = qkv.shape[0]
    q = qkv[:, :nh * hd].view(T, nh, hd).float()
    ps = cache.page_size
    group = nh // nkv
    q_start = ctx.q_start.tolist()
    for r in range(ctx.n_requests):
        row = int(ctx.table_rows[r])
        kv_len = int(ctx.kv_len[r])
        n = q_start[r + 1] - q_start[r]
        lo_all = 0
        if window:
            lo_all = max(0, (kv_len - n) - window + 1)
        idx = torch.arange(lo_all, kv_len)
        pages = cache.block_table[row, idx // ps].long()
        assert (pages >= 0).all(), "read of a page that is not held"
        K = cache.k_pages[pages, :, idx % ps, :].float()     # [len, nkv, hd]
        V = cache.v_pages[pages, :, idx % ps, :].float()
        for i in range(n):
            p = kv_len - n + i
            mask = idx <= p
            if window:
                mask &= idx > p - window
            for h in range(nh):
                s = (K[:, h // group, :] @ q[q_start[r] + i, h]) * scale
                s = s.masked_fill(~mask, float("-inf"))
                w = torch.softmax(s, 0)
                out[q_start[r] + i, h * hd:(h + 1) * hd] = (w @ V[:, h // group, :]).to(out.dtype)


def sample(logits, params, top_k, prev_start, prev_tokens, out, work=None):
    import plain_llama
    for r in range(logits.shape[0]):
        t, p, pen, u = (float(x) for x in params[r])
        prev = ()
        if prev_start is not None:
            prev = prev_tokens[int(prev_start[r]):int(prev_start[r + 1])].tolist()
        out[r] = plain_llama.sample_plain(logits[r].tolist(), t, int(top_k[r]), p, pen, prev, u)
