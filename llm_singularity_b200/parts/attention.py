"""Causal softmax attention with grouped keys/values over a paged cache.

Per layer call (reference order, models/llama/llama_model.cpp:564-622):
``q,k,v = x Wq^T, x Wk^T, x Wv^T`` (one product against the row-wise
concatenation ``[Wq; Wk; Wv]``) -> position encoding on q and k, fused with the
write of k and v into this step's cache pages -> every query row attends the
cached keys at positions ``<=`` its own (and ``> pos - window`` if a window is
set), query head ``h`` reading kv head ``h // (num_heads / num_kv_heads)``
(kernels/src/attention.cu:46) -> output projection.  Scores, softmax and the
weighted sum of values are 32-bit.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import POSITIONS, PagedKVSpec, ParamSpec, Part, register_mixer


@register_mixer("attention")
class PagedAttention(Part):
    graph_safe = True
    replayable = True
    folds_norm = True
    takes_unnormed = True
    kernels = ("gemm", "rope_cache", "attention")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads {s.num_heads} is not a multiple of num_kv_heads "
                             f"{s.num_kv_heads}")
        if s.window is not None and s.window < 1:
            raise ValueError(f"window must be at least 1, got {s.window}")
        self.position = POSITIONS.build(s.position, rt)
        if self.position.rotary_table() is None:
            self.replayable = False          # a position encoding applied with tensor operations
        if rt.dtype == torch.bfloat16 and s.head_dim in (64, 128):
            self.kernels = self.kernels + ("attention_tc", "attention_tc5")
        self.q_size = s.num_heads * s.head_dim
        self.kv_size = s.num_kv_heads * s.head_dim
        self.softcap = float(getattr(s, "logit_softcap", None) or 0.0)
        self.slopes = None
        if getattr(s, "linear_bias", False):
            # head h of n: 2^(-8 (h + 1) / n), the geometric sequence of the linear-bias scheme
            self.slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / s.num_heads) for h in range(s.num_heads)],
                                       dtype=torch.float32, device=rt.device)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        q, kv, H = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.hidden_size
        return {"q_proj": ParamSpec((q, H)), "k_proj": ParamSpec((kv, H)),
                "v_proj": ParamSpec((kv, H)), "o_proj": ParamSpec((H, q))}

    def children(self):
        return {"position": self.position}

    def load(self, tensors):
        # one product instead of three: rows of Wq, then Wk, then Wv
        self.wqkv = torch.cat([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]], dim=0)
        self.wqkv = self.wqkv.contiguous()
        self.wo = tensors["o_proj"].contiguous()

    def cache_spec(self):
        return PagedKVSpec(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def _modifiers(self) -> dict:
        """Keyword arguments for the attention operations: only what the spec asks for."""
        mods = {}
        if self.softcap:
            mods["softcap"] = self.softcap
        if self.slopes is not None:
            mods["slopes"] = self.slopes
        return mods

    def forward(self, x, ctx, cache, writes_cache: bool = True, into=None):
        s, ops = self.spec, self.rt.ops
        qkv = ops.linear(x, self.wqkv)
        table = self.position.rotary_table()
        out = self.rt.empty(x.shape[0], self.q_size)
        if table is None:
            self.position.apply(qkv[:, :self.q_size], qkv[:, self.q_size:self.q_size + self.kv_size], ctx)
            ops.rope_kv_store(qkv, s.num_heads, s.num_kv_heads, s.head_dim, ctx, cache, None, 0,
                              store=writes_cache)
            ops.paged_attention(qkv, s.num_heads, s.num_kv_heads, s.head_dim, ctx, cache,
                                s.scale, s.window or 0, out, **self._modifiers())
        else:
            inv_freq, rotary_dim = table
            ops.rope_store_attention(qkv, s.num_heads, s.num_kv_heads, s.head_dim, ctx, cache,
                                     inv_freq, rotary_dim, writes_cache, s.scale, s.window or 0, out,
                                     **self._modifiers())
        if into is not None:
            return ops.linear(out, self.wo, into=into)
        return ops.linear(out, self.wo)
