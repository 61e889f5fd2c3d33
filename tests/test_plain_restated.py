"""The plain implementation (tests/plain_llama.py, dense tensor algebra) against a second statement
of the same formulas written the way the reference's kernels walk their data: one token, one head,
one key at a time, with the running maximum and sum of its attention kernel
(kernels/src/attention.cu:79-113,161-170), rotation pair by pair (kernels/src/rope.cu:13-26), the
norm as a sum over the row (kernels/src/rmsnorm.cu:42-72).  Two statements written apart that agree
to rounding are unlikely to share a misreading.  numpy, 64-bit, tiny models, short sequences."""
import math

import numpy as np
import pytest

import plain_llama
import tiny_models


def _inv_freq(hd, theta, scaling):
    f = [1.0 / theta ** (2.0 * i / hd) for i in range(hd // 2)]
    if scaling is None:
        return f
    factor, low, high = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
    orig = scaling["original_max_position_embeddings"]
    out = []
    for fi in f:
        wavelength = 2.0 * math.pi / fi
        if wavelength < orig / high:
            out.append(fi)
        elif wavelength > orig / low:
            out.append(fi / factor)
        else:
            s = (orig / wavelength - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return out


def _norm_row(x, w, eps):
    ss = 0.0
    for v in x:
        ss += v * v
    r = 1.0 / math.sqrt(ss / len(x) + eps)
    return np.array([v * r * wi for v, wi in zip(x, w)])


def _rotate(vec, pos, inv_freq):
    hd = len(vec)
    out = vec.copy()
    for i in range(hd // 2):
        a = float(np.float32(pos) * np.float32(inv_freq[i]))      # the angle is formed in 32-bit
        c, s = math.cos(a), math.sin(a)
        out[i] = vec[i] * c - vec[i + hd // 2] * s
        out[i + hd // 2] = vec[i] * s + vec[i + hd // 2] * c
    return out


def restated_logits(cfg, w, tokens):
    w = {k: v.numpy() for k, v in w.items()}
    H, nh = cfg["hidden_size"], cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    hd = cfg.get("head_dim") or H // nh
    eps = cfg.get("rms_norm_eps", 1e-5)
    inv_freq = _inv_freq(hd, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"))
    scale = 1.0 / math.sqrt(hd)
    L = cfg["num_hidden_layers"]
    keys = [[] for _ in range(L)]           # per layer: one [nkv, hd] array per position so far
    values = [[] for _ in range(L)]
    logits = []
    for pos, tok in enumerate(tokens):      # token by token, as a decode step sees it
        x = w["model.embed_tokens.weight"][tok].copy()
        for layer in range(L):
            p = f"model.layers.{layer}."
            h = _norm_row(x, w[p + "input_layernorm.weight"], eps)
            q = (w[p + "self_attn.q_proj.weight"] @ h).reshape(nh, hd)
            k = (w[p + "self_attn.k_proj.weight"] @ h).reshape(nkv, hd)
            v = (w[p + "self_attn.v_proj.weight"] @ h).reshape(nkv, hd)
            q = np.stack([_rotate(q[i], pos, inv_freq) for i in range(nh)])
            keys[layer].append(np.stack([_rotate(k[i], pos, inv_freq) for i in range(nkv)]))
            values[layer].append(v)
            attn = np.zeros((nh, hd))
            for head in range(nh):
                g = head // (nh // nkv)
                m, total, acc = -math.inf, 0.0, np.zeros(hd)
                for j in range(pos + 1):                          # running maximum and sum
                    s = float(q[head] @ keys[layer][j][g]) * scale
                    m_new = max(m, s)
                    corr = math.exp(m - m_new) if m > -math.inf else 0.0
                    e = math.exp(s - m_new)
                    acc = acc * corr + e * values[layer][j][g]
                    total = total * corr + e
                    m = m_new
                attn[head] = acc / total if total > 0.0 else 0.0
            x = x + w[p + "self_attn.o_proj.weight"] @ attn.reshape(-1)
            h = _norm_row(x, w[p + "post_attention_layernorm.weight"], eps)
            gate, up = w[p + "mlp.gate_proj.weight"] @ h, w[p + "mlp.up_proj.weight"] @ h
            act = np.array([gi / (1.0 + math.exp(-gi)) * ui for gi, ui in zip(gate, up)])
            x = x + w[p + "mlp.down_proj.weight"] @ act
        h = _norm_row(x, w["model.norm.weight"], eps)
        head_w = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
        logits.append(head_w @ h)
    return np.stack(logits)


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
def test_two_statements_of_the_formulas_agree(model_dirs, name):
    cfg, w = plain_llama.load_model_dir(model_dirs[name])
    tokens = tiny_models.random_tokens(cfg["vocab_size"], 11, 7)
    dense = plain_llama.forward_logits(cfg, w, tokens).numpy()
    walked = restated_logits(cfg, w, tokens)
    assert walked.shape == dense.shape
    assert np.abs(walked - dense).max() <= 1e-9 * max(1.0, np.abs(dense).max())
