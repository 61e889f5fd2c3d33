"""A toy mixer with per-request state of its own, defined here, is registered, built into a
model beside attention layers, and stepped in portions, without a change to the framework's
files.  The model's run order names one block twice, each call with a cache of its own."""
import json
import math
import os
from dataclasses import dataclass, field

import pytest
import torch

import plain_llama
import tiny_models

pytestmark = pytest.mark.gpu

H, NH, HD, INTER, VOCAB, DECAY = 48, 3, 16, 40, 97, 0.75


def _register():
    from llm_singularity_b200 import register_architecture
    from llm_singularity_b200.config.specs import (AttentionSpec, BlockSpec, EmbeddingSpec,
                                                   GatedMLPSpec, HeadSpec, LayerCall, ModelSpec,
                                                   PartSpec, RMSNormSpec, RotarySpec)
    from llm_singularity_b200.parts import ParamSpec, Part, StateSpec, register_mixer

    @dataclass(frozen=True)
    class DecaySpec(PartSpec):
        hidden_size: int = 0
        decay: float = 0.5
        kind: str = field(init=False, default="toy_decay")

    @register_mixer("toy_decay")
    class DecayMixer(Part):
        """s_t = decay * s_{t-1} + x_t W_in^T ;  out_t = s_t W_out^T   (state: one vector per request)"""

        @classmethod
        def params(cls, spec):
            return {"w_in": ParamSpec((spec.hidden_size, spec.hidden_size)),
                    "w_out": ParamSpec((spec.hidden_size, spec.hidden_size))}

        def load(self, tensors):
            self.w_in, self.w_out = tensors["w_in"], tensors["w_out"]

        def cache_spec(self):
            return StateSpec((self.spec.hidden_size,), torch.float32)

        def forward(self, x, ctx, cache, writes_cache=True):
            u = self.rt.ops.linear(x, self.w_in).float()
            states = torch.empty_like(u)
            for r in range(ctx.n_requests):
                a, b = int(ctx.h_q_start[r]), int(ctx.h_q_start[r + 1])
                s = cache.state[int(ctx.h_table_rows[r])]
                for t in range(a, b):
                    s.mul_(self.spec.decay).add_(u[t])
                    states[t] = s
            return self.rt.ops.linear(states.to(x.dtype), self.w_out)

    class ToyConfig:
        architecture = "ToyDecayForCausalLM"

        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_model_spec(self):
            d = self.d
            norm = RMSNormSpec(size=d["width"], eps=d["eps"])
            mlp = GatedMLPSpec(hidden_size=d["width"], intermediate_size=d["inner"])
            toy = BlockSpec(mixer=DecaySpec(hidden_size=d["width"], decay=d["decay"]), ffn=mlp,
                            mixer_norm=norm, ffn_norm=norm)
            att = BlockSpec(mixer=AttentionSpec(hidden_size=d["width"], num_heads=d["heads"],
                                                num_kv_heads=d["heads"], head_dim=d["head"],
                                                scale=1 / math.sqrt(d["head"]),
                                                position=RotarySpec(head_dim=d["head"], rotary_dim=d["head"],
                                                                    theta=d["theta"])),
                            ffn=mlp, mixer_norm=norm, ffn_norm=norm)
            names = [("emb", ("embedding", "weight")), ("out_norm", ("head.norm", "weight")),
                     ("out", ("head", "weight"))]
            for i, kinds in enumerate((("w_in", "w_out"), ("q_proj", "k_proj", "v_proj", "o_proj"))):
                names += [(f"b{i}.{k}", (f"blocks.{i}.mixer", k)) for k in kinds]
                names += [(f"b{i}.{k}", (f"blocks.{i}.ffn", k)) for k in ("gate_proj", "up_proj", "down_proj")]
                names += [(f"b{i}.n1", (f"blocks.{i}.mixer_norm", "weight")),
                          (f"b{i}.n2", (f"blocks.{i}.ffn_norm", "weight"))]
            return ModelSpec(
                architecture=self.architecture,
                embedding=EmbeddingSpec(vocab_size=d["vocab"], hidden_size=d["width"]),
                blocks=(toy, att),
                # block 0 runs twice, each call with its own state
                order=(LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2)),
                head=HeadSpec(vocab_size=d["vocab"], hidden_size=d["width"], tied=False, norm=norm),
                tensor_names=tuple(names))

    register_architecture(ToyConfig.architecture, ToyConfig)
    return ToyConfig


def _plain(cfg, w, toks):
    """The same model written out whole-sequence in float64."""
    x = w["emb"][torch.tensor(toks)]
    n = len(toks)

    def mlp(x, i):
        h = plain_llama.rms_norm(x, w[f"b{i}.n2"], cfg["eps"])
        return x + plain_llama.swiglu_mlp(h, w[f"b{i}.gate_proj"], w[f"b{i}.up_proj"], w[f"b{i}.down_proj"])

    def toy(x):
        h = plain_llama.rms_norm(x, w["b0.n1"], cfg["eps"])
        u = h @ w["b0.w_in"].T
        s, out = torch.zeros(cfg["width"], dtype=torch.float64), []
        for t in range(n):
            s = cfg["decay"] * s + u[t]
            out.append(s)
        return mlp(x + torch.stack(out) @ w["b0.w_out"].T, 0)

    def att(x):
        h = plain_llama.rms_norm(x, w["b1.n1"], cfg["eps"])
        q, k, v = ((h @ w[f"b1.{p}"].T).view(n, cfg["heads"], cfg["head"]) for p in ("q_proj", "k_proj", "v_proj"))
        inv = plain_llama.rope_inv_freq(cfg["head"], cfg["theta"])
        q, k = plain_llama.apply_rope(q, range(n), inv), plain_llama.apply_rope(k, range(n), inv)
        a = plain_llama.causal_attention(q, k, v, 1 / math.sqrt(cfg["head"]))
        return mlp(x + a.reshape(n, -1) @ w["b1.o_proj"].T, 1)

    x = toy(att(toy(x)))
    return plain_llama.rms_norm(x, w["out_norm"], cfg["eps"]) @ w["out"].T


def test_toy_state_mixer_registers_builds_and_steps(tmp_path):
    run_toy_model(tmp_path)


def run_toy_model(tmp_path, **runner_options):
    """Register, build and step the toy model; ``runner_options`` go to the ModelRunner (the
    host-side test runs the same on the CPU with stand-in kernels)."""
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    from llm_singularity_b200.engine.runner import expected_tensors_of
    from llm_singularity_b200.parts import StateSpec
    from llm_singularity_b200.weights import random_tensors, write_safetensors
    ToyConfig = _register()
    cfg = dict(architectures=["ToyDecayForCausalLM"], width=H, heads=NH, head=HD, inner=INTER,
               vocab=VOCAB, decay=DECAY, eps=1e-5, theta=10000.0)
    d = str(tmp_path)
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    expected = expected_tensors_of(ToyConfig(cfg).to_model_spec())
    tensors = random_tensors(expected, seed=3, dtype=torch.float32, std=0.15, norm_noise=0.1)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    w = {k: v.double() for k, v in tensors.items()}

    runner = ModelRunner(d, dtype="float32", page_size=16, num_pages=8, max_requests=2, **runner_options)
    specs = runner.model.cache_specs()
    assert isinstance(specs[0], StateSpec) and isinstance(specs[2], StateSpec) and len(specs) == 3
    a, b, c = (tiny_models.random_tokens(VOCAB, n, s) for n, s in ((23, 1), (40, 2), (9, 3)))
    got = {"a": [], "b": [], "c": []}
    runner.open("a"); runner.open("b")
    plan = [[("a", 5), ("b", 17)], [("a", 1), ("b", 2)], [("b", 21)], [("a", 17)]]
    pos = {"a": 0, "b": 0, "c": 0}
    seqs = {"a": a, "b": b, "c": c}
    for step in plan:
        entries = [StepEntry(r, seqs[r][pos[r]:pos[r] + n], list(range(n))) for r, n in step]
        out = runner.step(entries)
        k = 0
        for r, n in step:
            got[r].append(out[k:k + n]); k += n; pos[r] += n
    runner.close("a")
    runner.open("c")                      # takes a's slot: its state must start from zero
    got["c"].append(runner.step([StepEntry("c", c, list(range(9)))]))
    runner.check_kernels()
    for r in "abc":
        want = _plain(cfg, w, seqs[r])
        diff = (torch.cat(got[r]).double().cpu() - want).abs().max().item()
        assert diff <= 1e-4, (r, diff)
