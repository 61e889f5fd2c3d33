"""A toy norm defined here and registered without a change to the framework's files: it centres a
row, divides by its standard deviation and applies a weight and a bias, so it cannot be folded
into the products around it the way the stock norm is in steps of a few rows.  It is the norm of one
block (both places) and of the head, beside a block with the stock norm: in a decode step the first
block's products stay whole, its feed-forward folds the second block's first norm into its last
product, and the second block folds its own.  A plain whole-sequence computation in float64 is the
reference.  The toy is not a model of anybody's."""
import json
import math
import os
from dataclasses import dataclass, field

import pytest
import torch

import plain_llama
import tiny_models

pytestmark = pytest.mark.gpu


def _register():
    from llm_singularity_b200 import register_architecture
    from llm_singularity_b200.config.specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMLPSpec,
                                                   HeadSpec, LayerCall, ModelSpec, PartSpec, RMSNormSpec,
                                                   RotarySpec)
    from llm_singularity_b200.parts import ParamSpec, Part, register_norm

    @dataclass(frozen=True)
    class CentredNormSpec(PartSpec):
        size: int = 0
        eps: float = 1e-5
        kind: str = field(init=False, default="toy_centred")

    @register_norm("toy_centred")
    class CentredNorm(Part):
        """(x - mean) / sqrt(var + eps) * weight + bias over a row, in 32-bit; ``add_norm`` adds the
        delta to the residual stream first, as every norm does."""
        graph_safe = True            # the same work whatever the host-side values are
        replayable = False           # not launched through the framework's kernels: nothing to record
        foldable = False             # a product cannot take the centring upon itself

        @classmethod
        def params(cls, spec):
            return {"weight": ParamSpec((spec.size,), role="vector", init="ones"),
                    "bias": ParamSpec((spec.size,), role="vector")}

        def load(self, tensors):
            self.weight, self.bias = tensors["weight"], tensors["bias"]

        def _norm(self, x):
            mu = x.mean(dim=-1, keepdim=True)
            var = (x - mu).square().mean(dim=-1, keepdim=True)
            return ((x - mu) * torch.rsqrt(var + self.spec.eps) * self.weight + self.bias).to(self.rt.dtype)

        def add_norm(self, residual, delta):
            if delta is not None:
                residual += delta.float()
            return self._norm(residual)

        def gather_add_norm(self, residual, delta, rows):
            x = residual[rows.long()]
            if delta is not None:
                x = x + delta[rows.long()].float()
            return self._norm(x)

    class ToyConfig:
        architecture = "ToyCentredNormForCausalLM"

        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_model_spec(self):
            d = self.d
            toy = CentredNormSpec(size=d["width"], eps=d["toy_eps"])
            rms = RMSNormSpec(size=d["width"], eps=d["eps"])
            rot = RotarySpec(head_dim=d["head"], rotary_dim=d["head"], theta=d["theta"])
            att = AttentionSpec(hidden_size=d["width"], num_heads=d["heads"], num_kv_heads=d["kv"],
                                head_dim=d["head"], scale=1 / math.sqrt(d["head"]), position=rot)
            mlp = GatedMLPSpec(hidden_size=d["width"], intermediate_size=d["inner"])
            names = [("emb", ("embedding", "weight")), ("out_norm.w", ("head.norm", "weight")),
                     ("out_norm.b", ("head.norm", "bias"))]
            for i in (0, 1):
                names += [(f"b{i}.{k}", (f"blocks.{i}.mixer", k)) for k in ("q_proj", "k_proj", "v_proj", "o_proj")]
                names += [(f"b{i}.{k}", (f"blocks.{i}.ffn", k)) for k in ("gate_proj", "up_proj", "down_proj")]
                names += [(f"b{i}.n1.w", (f"blocks.{i}.mixer_norm", "weight")),
                          (f"b{i}.n2.w", (f"blocks.{i}.ffn_norm", "weight"))]
            names += [("b0.n1.b", ("blocks.0.mixer_norm", "bias")), ("b0.n2.b", ("blocks.0.ffn_norm", "bias"))]
            return ModelSpec(architecture=self.architecture,
                             embedding=EmbeddingSpec(vocab_size=d["vocab"], hidden_size=d["width"]),
                             blocks=(BlockSpec(mixer=att, ffn=mlp, mixer_norm=toy, ffn_norm=toy),
                                     BlockSpec(mixer=att, ffn=mlp, mixer_norm=rms, ffn_norm=rms)),
                             order=(LayerCall(0, 0), LayerCall(1, 1)),
                             head=HeadSpec(vocab_size=d["vocab"], hidden_size=d["width"], tied=True, norm=toy),
                             tensor_names=tuple(names))

    register_architecture(ToyConfig.architecture, ToyConfig)
    return ToyConfig


def _plain(cfg, w, toks):
    n, nh, nkv, hd = len(toks), cfg["heads"], cfg["kv"], cfg["head"]
    inv = plain_llama.rope_inv_freq(hd, cfg["theta"])

    def centred(x, name):
        mu = x.mean(dim=-1, keepdim=True)
        var = (x - mu).square().mean(dim=-1, keepdim=True)
        return (x - mu) / torch.sqrt(var + cfg["toy_eps"]) * w[name + ".w"] + w[name + ".b"]

    def rms(x, name):
        return plain_llama.rms_norm(x, w[name + ".w"], cfg["eps"])

    x = w["emb"][torch.tensor(toks)]
    for i, norm in ((0, centred), (1, rms)):
        h = norm(x, f"b{i}.n1")
        q = plain_llama.apply_rope((h @ w[f"b{i}.q_proj"].T).view(n, nh, hd), range(n), inv)
        k = plain_llama.apply_rope((h @ w[f"b{i}.k_proj"].T).view(n, nkv, hd), range(n), inv)
        v = (h @ w[f"b{i}.v_proj"].T).view(n, nkv, hd)
        a = plain_llama.causal_attention(q, k, v, 1 / math.sqrt(hd))
        x = x + a.reshape(n, -1) @ w[f"b{i}.o_proj"].T
        h = norm(x, f"b{i}.n2")
        x = x + plain_llama.swiglu_mlp(h, w[f"b{i}.gate_proj"], w[f"b{i}.up_proj"], w[f"b{i}.down_proj"])
    return centred(x, "out_norm") @ w["emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_norm_registers_builds_and_steps_beside_the_stock_one(tmp_path, dtype):
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    from llm_singularity_b200.engine.runner import expected_tensors_of
    from llm_singularity_b200.weights import random_tensors, write_safetensors
    ToyConfig = _register()
    cfg = dict(architectures=["ToyCentredNormForCausalLM"], width=192, heads=4, kv=2, head=64, inner=208,
               vocab=157, eps=1e-5, toy_eps=3e-4, theta=10000.0)
    d = str(tmp_path)
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    expected = expected_tensors_of(ToyConfig(cfg).to_model_spec())
    assert {"b0.n1.b", "b0.n2.b", "out_norm.b"} <= set(expected) and "b1.n1.b" not in expected
    tensors = random_tensors(expected, seed=23, dtype=torch.bfloat16, std=0.08, norm_noise=0.1)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    w = {k: v.double() for k, v in tensors.items()}
    assert w["b0.n1.b"].abs().max() > 0.05                 # the bias matters

    runner = ModelRunner(d, dtype=dtype, page_size=16, num_pages=24, max_requests=2)
    seqs = {"a": tiny_models.random_tokens(157, 180, 3), "b": tiny_models.random_tokens(157, 60, 4)}
    # a portion on the tensor-core kernels, small portions, then single tokens through the graph
    # (rows few enough for the stock norm to be folded into the products around it)
    plan = [[("a", 140)], [("a", 9), ("b", 30)], [("a", 1), ("b", 2)]] + [[("a", 1), ("b", 1)]] * 28
    got, pos = {"a": [], "b": []}, {"a": 0, "b": 0}
    runner.open("a"); runner.open("b")
    for step in plan:
        entries = [StepEntry(r, seqs[r][pos[r]:pos[r] + n], list(range(n))) for r, n in step]
        out = runner.step(entries)
        k = 0
        for r, n in step:
            got[r].append(out[k:k + n].clone()); k += n; pos[r] += n      # graph logits are overwritten
    runner.check_kernels()
    assert pos == {"a": 178, "b": 60}
    assert runner.graph_replays >= 20 or not runner.cuda_graphs
    for r in "ab":
        want = _plain(cfg, w, seqs[r][:pos[r]])
        have = torch.cat(got[r]).double().cpu()
        bound = 2e-4 if dtype == "float32" else 4e-2 * want.abs().max().item()
        assert (have - want).abs().max().item() <= bound, (r, (have - want).abs().max().item(), bound)
    runner.close("a"); runner.close("b")
    runner.cache.check_invariants()
