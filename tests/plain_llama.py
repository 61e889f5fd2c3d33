"""A plain, slow Llama decoder: whole sequences, no cache, one function per part.

This file rests on the reference's formulas only: the reference's model code
(models/llama/llama_model.cpp) has no CPU path (every step is a CUDA kernel or a
cuBLAS call), so it cannot be run where the tests are written, and llama3 rope
scaling, a configurable eps and ``head_dim`` do not exist in it at all.  Each
function cites the reference lines it restates.  It shares no code with the
engine: it has its own safetensors reader, its own config reading and uses only
dense tensor arithmetic (float64 by default).

Paths cited are relative to the reference project root.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


# --------------------------------------------------------------------------- files
def read_safetensors(path):
    """name -> float64/int64 torch tensor (core/src/safetensors.cpp:42-116: u64 LE header
    length, JSON header with dtype/shape/data_offsets, raw data after it)."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        buf = raw[base + b:base + e]
        dt = info["dtype"]
        if dt == "BF16":          # bf16 -> fp32 by a 16-bit shift (tests/debug_embed_check.py:11-20)
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            a = u.view(np.float32).astype(np.float64)
        elif dt == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif dt == "F16":
            a = np.frombuffer(buf, dtype="<f2").astype(np.float64)
        elif dt == "I32":
            a = np.frombuffer(buf, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = torch.from_numpy(a.reshape(info["shape"]).copy())
    return out


def load_model_dir(model_dir):
    """(config dict, weights dict) of a folder with config.json and model.safetensors."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


def sizes(cfg):
    """Derived sizes (models/llama/llama_model.cpp:105-107,159-183)."""
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    return nh, nkv, hd


# --------------------------------------------------------------------------- parts
def embed(table, ids):
    """h0[t,:] = E[id_t,:] (kernels/src/embedding.cu:12-26)."""
    return table[torch.as_tensor(ids, dtype=torch.long, device=table.device)]


def rms_norm(x, w, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w (kernels/src/rmsnorm.cu:42-72)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * w


def rope_inv_freq(hd, theta, scaling=None):
    """f_i = 1 / theta^(2i/hd) (kernels/src/rope.cu:15); llama3 scaling has no reference
    code: wavelengths shorter than orig/high keep f, longer than orig/low get f/factor,
    between them a linear blend in (orig/wavelength - low)/(high - low)."""
    out = []
    for i in range(hd // 2):
        f = 1.0 / (theta ** (2.0 * i / hd))
        if scaling is not None and scaling.get("rope_type", scaling.get("type")) == "llama3":
            factor = scaling["factor"]
            low, high = scaling["low_freq_factor"], scaling["high_freq_factor"]
            orig = scaling["original_max_position_embeddings"]
            wavelen = 2.0 * math.pi / f
            if wavelen < orig / high:
                pass
            elif wavelen > orig / low:
                f = f / factor
            else:
                s = (orig / wavelen - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def apply_rope(x, positions, inv_freq):
    """x [n, heads, hd]; pairs (i, i + hd/2) rotated by pos * f_i
    (kernels/src/rope.cu:13-26: x0' = x0 cos - x1 sin, x1' = x0 sin + x1 cos).
    The angle is formed in 32-bit like the engine's (pos and f_i as floats)."""
    half = x.shape[-1] // 2
    pos = torch.as_tensor(positions, dtype=torch.float32, device=x.device)
    ang = (pos[:, None] * inv_freq.to(device=x.device, dtype=torch.float32)[None, :]).to(x.dtype)   # [n, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def causal_attention(q, k, v, scale, window=None, softcap=None, slopes=None):
    """q [n, nh, hd], k/v [n, nkv, hd]; query head h reads kv head h // (nh/nkv)
    (kernels/src/attention.cu:46); scores (q.k) * scale over keys at positions <= the
    query's own (models/llama/llama_model.cpp:599-615: per-row length start+t+1), softmax,
    weighted sum of values (attention.cu:79-113,161-170).  ``window``: also key > pos - window.
    Not in the reference, for parts of other architectures: ``softcap`` replaces a scaled score s
    by softcap * tanh(s / softcap); ``slopes[h]`` times the distance to the key is subtracted."""
    n, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    out = torch.zeros_like(q)
    for h in range(nh):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale                 # [n, n]
        i = torch.arange(n, device=q.device)
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        if slopes is not None:
            s = s - float(slopes[h]) * (i[:, None] - i[None, :]).to(s.dtype)
        mask = i[None, :] <= i[:, None]
        if window is not None:
            mask &= i[None, :] > i[:, None] - window
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu_mlp(x, wg, wu, wd):
    """down( silu(gate) * up ), silu(g) = g / (1 + exp(-g))
    (models/llama/llama_model.cpp:634-649; kernels/src/activations.cu:11-21)."""
    g = x @ wg.T
    u = x @ wu.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ wd.T


def _no_rounding(t):
    return t


def bf16_rounding(t):
    """Round to bfloat16 and back: what storing an activation in bfloat16 does to it."""
    return t.to(torch.bfloat16).to(t.dtype)


def decoder_layer(x, w, i, cfg, positions, inv_freq, rnd=_no_rounding):
    """x += attn(norm(x)); x += mlp(norm(x)) (models/llama/llama_model.cpp:502-655).
    ``rnd`` is applied wherever a bfloat16 engine stores an activation (norm output,
    projections, rotated q/k, attention output, gate/up, activation, down); the residual
    stream x itself is never rounded."""
    nh, nkv, hd = sizes(cfg)
    eps = cfg.get("rms_norm_eps", 1e-5)
    p = f"model.layers.{i}."
    n = x.shape[0]
    h = rnd(rms_norm(x, w[p + "input_layernorm.weight"], eps))
    q = rnd(h @ w[p + "self_attn.q_proj.weight"].T).view(n, nh, hd)
    k = rnd(h @ w[p + "self_attn.k_proj.weight"].T).view(n, nkv, hd)
    v = rnd(h @ w[p + "self_attn.v_proj.weight"].T).view(n, nkv, hd)
    q = rnd(apply_rope(q, positions, inv_freq))
    k = rnd(apply_rope(k, positions, inv_freq))
    a = rnd(causal_attention(q, k, v, 1.0 / math.sqrt(hd), cfg.get("sliding_window")))
    x = x + rnd(a.reshape(n, nh * hd) @ w[p + "self_attn.o_proj.weight"].T)
    h = rnd(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps))
    g = rnd(h @ w[p + "mlp.gate_proj.weight"].T)
    u = rnd(h @ w[p + "mlp.up_proj.weight"].T)
    act = rnd((g / (1.0 + torch.exp(-g))) * u)           # same formula as swiglu_mlp
    return x + rnd(act @ w[p + "mlp.down_proj.weight"].T)


def forward_logits(cfg, w, token_ids, dtype=torch.float64, act_round=None, rows=None, device=None):
    """Logits [n, vocab] at every position of one whole sequence
    (models/llama/llama_model.cpp:424-425,502-666; lm_head tied to the embedding when
    absent, :257-261).  ``act_round="bfloat16"`` rounds stored activations as a bfloat16
    engine does, so that such an engine can be held to a tight tolerance.  ``rows``: only these
    positions' logits are formed (the layers still run the whole sequence).  ``device``: where
    the dense arithmetic runs (the CPU unless told otherwise; long sequences at large widths take
    hours there); the result comes back to the CPU."""
    rnd = bf16_rounding if act_round == "bfloat16" else _no_rounding
    w = {k: (v.to(device=device, dtype=dtype) if v.is_floating_point() else v.to(device=device))
         for k, v in w.items()}
    nh, nkv, hd = sizes(cfg)
    inv_freq = rope_inv_freq(hd, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"))
    positions = list(range(len(token_ids)))
    x = embed(w["model.embed_tokens.weight"], token_ids)
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg, positions, inv_freq, rnd)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long, device=x.device)]
    x = rnd(rms_norm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5)))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return (x @ head.T).cpu()


def greedy_generate(cfg, w, prompt, n_new):
    """Append the arg-max token n_new times (core/src/sampling.cpp:35-38: first maximum)."""
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward_logits(cfg, w, toks)[-1]
        t = int(torch.argmax(logits))
        out.append(t)
        toks.append(t)
    return out


# ------------------------------------------------------------------------ sampling
def sample_distribution_plain(logits, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0,
                              prev_tokens=()):
    """The distribution the reference sampler draws from (core/src/sampling.cpp:11-103):
    repetition penalty -> /T -> top-k -> top-p -> softmax.  With T == 0 it is one at the first
    maximum of the penalised logits (sampling.cpp:35-38)."""
    work = [float(x) for x in logits]
    V = len(work)
    if repetition_penalty != 1.0:
        for t in prev_tokens:
            if 0 <= t < V:
                work[t] = work[t] / repetition_penalty if work[t] > 0 else work[t] * repetition_penalty
    if temperature == 0.0:
        best = max(range(V), key=lambda i: (work[i], -i))
        return [1.0 if i == best else 0.0 for i in range(V)]
    work = [x / temperature for x in work]
    if 0 < top_k < V:
        order = sorted(range(V), key=lambda i: (-work[i], i))
        keep = set(order[:top_k])
        work = [x if i in keep else float("-inf") for i, x in enumerate(work)]
    if top_p < 1.0:
        m = max(work)
        probs = [math.exp(x - m) for x in work]
        s = sum(probs)
        probs = [p / s for p in probs]
        order = sorted(range(V), key=lambda i: (-probs[i], i))
        c = 0.0
        for n, i in enumerate(order):
            c += probs[i]
            if c > top_p:
                for j in order[n + 1:]:
                    work[j] = float("-inf")
                break
    m = max(work)
    probs = [math.exp(x - m) for x in work]
    s = sum(probs)
    return [p / s for p in probs]


def sample_plain(logits, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0,
                 prev_tokens=(), u=0.5):
    """The reference sampler (core/src/sampling.cpp:11-118) with the uniform draw ``u``
    given: the first i with u <= cumsum of the distribution above (sampling.cpp:105-117)."""
    probs = sample_distribution_plain(logits, temperature, top_k, top_p, repetition_penalty,
                                      prev_tokens)
    V = len(probs)
    if temperature == 0.0:
        return probs.index(1.0)
    c = 0.0
    for i in range(V):
        c += probs[i]
        if u <= c:
            return i
    return max(i for i in range(V) if probs[i] > 0)
