"""Two more toy parts defined here and registered without a change to the framework's files: a
feed-forward that routes every token to one of several small experts, and a position encoding
that is not rotary (a learned vector per position, added to queries and keys).  They sit in
different layers of one model beside the stock attention and gated feed-forward, and the model is
stepped in portions and single tokens; a plain whole-sequence computation in float64 is the
reference.  Neither toy is a model of anybody's."""
import json
import math
import os
from dataclasses import dataclass, field

import pytest
import torch

import plain_llama
import tiny_models

pytestmark = pytest.mark.gpu

W, NH, NKV, HD, INNER, VOCAB, EXPERTS, EINNER, MAXPOS = 40, 3, 1, 16, 56, 83, 3, 24, 64


def _register():
    from llm_singularity_b200 import register_architecture
    from llm_singularity_b200.config.specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMLPSpec,
                                                   HeadSpec, LayerCall, ModelSpec, PartSpec, RMSNormSpec,
                                                   RotarySpec)
    from llm_singularity_b200.parts import ParamSpec, Part, register_feed_forward, register_position

    @dataclass(frozen=True)
    class RoutedSpec(PartSpec):
        hidden_size: int = 0
        inner: int = 0
        experts: int = 0
        kind: str = field(init=False, default="toy_routed")

    @register_feed_forward("toy_routed")
    class RoutedFeedForward(Part):
        """Each token goes to the expert with the largest router logit (32-bit); the expert is
        relu(x W1^T) W2^T, weighted by the softmax probability of that logit."""

        @classmethod
        def params(cls, spec):
            p = {"router": ParamSpec((spec.experts, spec.hidden_size))}
            for e in range(spec.experts):
                p[f"e{e}_in"] = ParamSpec((spec.inner, spec.hidden_size))
                p[f"e{e}_out"] = ParamSpec((spec.hidden_size, spec.inner))
            return p

        def load(self, tensors):
            self.t = tensors

        def forward(self, x, ctx):
            ops = self.rt.ops
            logits = ops.linear(x, self.t["router"], out_dtype=torch.float32)
            prob, choice = torch.softmax(logits, dim=-1).max(dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.spec.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    h = torch.relu(ops.linear(x[rows].contiguous(), self.t[f"e{e}_in"]))
                    y = ops.linear(h, self.t[f"e{e}_out"]).float() * prob[rows, None]
                    out[rows] = y.to(x.dtype)
            return out

    @dataclass(frozen=True)
    class LearnedPositionSpec(PartSpec):
        head_dim: int = 0
        max_positions: int = 0
        kind: str = field(init=False, default="toy_learned")

    @register_position("toy_learned")
    class LearnedPosition(Part):
        """q[t, h] += table[pos_t], k[t, h] += table[pos_t]: nothing rotary, so the mixer calls
        ``apply`` and then only stores keys and values."""

        @classmethod
        def params(cls, spec):
            return {"table": ParamSpec((spec.max_positions, spec.head_dim))}

        def load(self, tensors):
            self.table = tensors["table"]

        def rotary_table(self):
            return None

        def apply(self, q, k, ctx):
            add = self.table[ctx.positions.long()]                       # [T, head_dim]
            hd = self.spec.head_dim
            for x in (q, k):
                v = x.view(x.shape[0], -1, hd) if x.is_contiguous() else None
                if v is not None:
                    v += add[:, None, :]
                else:                                                     # a column slice of qkv
                    x += add.repeat(1, x.shape[1] // hd)

    class ToyConfig:
        architecture = "ToyRoutedForCausalLM"

        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_model_spec(self):
            d = self.d
            norm = RMSNormSpec(size=d["width"], eps=d["eps"])

            def attention(position):
                return AttentionSpec(hidden_size=d["width"], num_heads=d["heads"], num_kv_heads=d["kv"],
                                     head_dim=d["head"], scale=1 / math.sqrt(d["head"]), position=position)
            b0 = BlockSpec(mixer=attention(LearnedPositionSpec(head_dim=d["head"], max_positions=d["maxpos"])),
                           ffn=RoutedSpec(hidden_size=d["width"], inner=d["einner"], experts=d["experts"]),
                           mixer_norm=norm, ffn_norm=norm)
            b1 = BlockSpec(mixer=attention(RotarySpec(head_dim=d["head"], rotary_dim=d["head"], theta=d["theta"])),
                           ffn=GatedMLPSpec(hidden_size=d["width"], intermediate_size=d["inner"]),
                           mixer_norm=norm, ffn_norm=norm)
            names = [("emb", ("embedding", "weight")), ("out_norm", ("head.norm", "weight"))]
            for i in (0, 1):
                names += [(f"b{i}.{k}", (f"blocks.{i}.mixer", k)) for k in ("q_proj", "k_proj", "v_proj", "o_proj")]
                names += [(f"b{i}.n1", (f"blocks.{i}.mixer_norm", "weight")),
                          (f"b{i}.n2", (f"blocks.{i}.ffn_norm", "weight"))]
            names += [("b0.pos", ("blocks.0.mixer.position", "table")), ("b0.router", ("blocks.0.ffn", "router"))]
            for e in range(d["experts"]):
                names += [(f"b0.e{e}_in", ("blocks.0.ffn", f"e{e}_in")), (f"b0.e{e}_out", ("blocks.0.ffn", f"e{e}_out"))]
            names += [(f"b1.{k}", ("blocks.1.ffn", k)) for k in ("gate_proj", "up_proj", "down_proj")]
            return ModelSpec(
                architecture=self.architecture,
                embedding=EmbeddingSpec(vocab_size=d["vocab"], hidden_size=d["width"]),
                blocks=(b0, b1), order=(LayerCall(0, 0), LayerCall(1, 1)),
                head=HeadSpec(vocab_size=d["vocab"], hidden_size=d["width"], tied=True, norm=norm),
                tensor_names=tuple(names))

    register_architecture(ToyConfig.architecture, ToyConfig)
    return ToyConfig


def _plain(cfg, w, toks):
    n, nh, nkv, hd = len(toks), cfg["heads"], cfg["kv"], cfg["head"]
    x = w["emb"][torch.tensor(toks)]

    def attend(x, i, positional):
        h = plain_llama.rms_norm(x, w[f"b{i}.n1"], cfg["eps"])
        q = (h @ w[f"b{i}.q_proj"].T).view(n, nh, hd)
        k = (h @ w[f"b{i}.k_proj"].T).view(n, nkv, hd)
        v = (h @ w[f"b{i}.v_proj"].T).view(n, nkv, hd)
        q, k = positional(q, k)
        a = plain_llama.causal_attention(q, k, v, 1 / math.sqrt(hd))
        return x + a.reshape(n, -1) @ w[f"b{i}.o_proj"].T

    def learned(q, k):
        add = w["b0.pos"][:n][:, None, :]
        return q + add, k + add

    def rotary(q, k):
        inv = plain_llama.rope_inv_freq(hd, cfg["theta"])
        return plain_llama.apply_rope(q, range(n), inv), plain_llama.apply_rope(k, range(n), inv)

    x = attend(x, 0, learned)
    h = plain_llama.rms_norm(x, w["b0.n2"], cfg["eps"])
    prob, choice = torch.softmax(h @ w["b0.router"].T, dim=-1).max(dim=-1)
    y = torch.stack([torch.relu(h[t] @ w[f"b0.e{int(choice[t])}_in"].T) @ w[f"b0.e{int(choice[t])}_out"].T * prob[t]
                     for t in range(n)])
    x = x + y
    x = attend(x, 1, rotary)
    h = plain_llama.rms_norm(x, w["b1.n2"], cfg["eps"])
    x = x + plain_llama.swiglu_mlp(h, w["b1.gate_proj"], w["b1.up_proj"], w["b1.down_proj"])
    return plain_llama.rms_norm(x, w["out_norm"], cfg["eps"]) @ w["emb"].T, choice


def test_toy_routed_feed_forward_and_learned_positions_register_build_and_step(tmp_path):
    run_routed_model(tmp_path)


def run_routed_model(tmp_path, **runner_options):
    """``runner_options`` go to the ModelRunner (tests/test_toy_parts_host.py runs the same models
    on the CPU with stand-in kernels)."""
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    from llm_singularity_b200.engine.runner import expected_tensors_of
    from llm_singularity_b200.weights import random_tensors, write_safetensors
    ToyConfig = _register()
    cfg = dict(architectures=["ToyRoutedForCausalLM"], width=W, heads=NH, kv=NKV, head=HD, inner=INNER,
               vocab=VOCAB, experts=EXPERTS, einner=EINNER, maxpos=MAXPOS, eps=1e-6, theta=10000.0)
    d = str(tmp_path)
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    expected = expected_tensors_of(ToyConfig(cfg).to_model_spec())
    assert "b0.pos" in expected and "b0.router" in expected and f"b0.e{EXPERTS - 1}_out" in expected
    tensors = random_tensors(expected, seed=11, dtype=torch.float32, std=0.2, norm_noise=0.1)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    w = {k: v.double() for k, v in tensors.items()}

    runner = ModelRunner(d, dtype="float32", page_size=8, num_pages=12, max_requests=2, **runner_options)
    seqs = {"a": tiny_models.random_tokens(VOCAB, 37, 5), "b": tiny_models.random_tokens(VOCAB, 50, 6)}
    got = {"a": [], "b": []}
    pos = {"a": 0, "b": 0}
    runner.open("a"); runner.open("b")
    plan = [[("a", 9), ("b", 2)], [("a", 1), ("b", 30)], [("a", 1), ("b", 1)], [("a", 26), ("b", 1)], [("b", 16)]]
    for step in plan:
        entries = [StepEntry(r, seqs[r][pos[r]:pos[r] + n], list(range(n))) for r, n in step]
        out = runner.step(entries)
        k = 0
        for r, n in step:
            got[r].append(out[k:k + n]); k += n; pos[r] += n
    runner.check_kernels()
    assert pos == {"a": 37, "b": 50}
    used = set()
    for r in "ab":
        want, choice = _plain(cfg, w, seqs[r])
        used |= set(choice.tolist())
        diff = (torch.cat(got[r]).double().cpu() - want).abs().max().item()
        assert diff <= 2e-4, (r, diff)
    assert len(used) >= 2                     # the router really sends tokens to different experts
    runner.close("a"); runner.close("b")
    runner.cache.check_invariants()


# ------------------------------------------------------------------ a windowed layer beside a full one
def _register_window():
    from llm_singularity_b200 import register_architecture
    from llm_singularity_b200.config.specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMLPSpec,
                                                   HeadSpec, LayerCall, ModelSpec, RMSNormSpec, RotarySpec)

    class WindowConfig:
        architecture = "ToyWindowForCausalLM"

        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_model_spec(self):
            d = self.d
            norm = RMSNormSpec(size=d["width"], eps=d["eps"])
            rot = RotarySpec(head_dim=d["head"], rotary_dim=d["head"], theta=d["theta"])
            mlp = GatedMLPSpec(hidden_size=d["width"], intermediate_size=d["inner"])

            def block(window):
                return BlockSpec(mixer=AttentionSpec(hidden_size=d["width"], num_heads=d["heads"], num_kv_heads=d["kv"],
                                                     head_dim=d["head"], scale=1 / math.sqrt(d["head"]),
                                                     window=window, position=rot),
                                 ffn=mlp, mixer_norm=norm, ffn_norm=norm)
            names = [("emb", ("embedding", "weight")), ("out_norm", ("head.norm", "weight"))]
            for i in (0, 1):
                names += [(f"b{i}.{k}", (f"blocks.{i}.mixer", k)) for k in ("q_proj", "k_proj", "v_proj", "o_proj")]
                names += [(f"b{i}.{k}", (f"blocks.{i}.ffn", k)) for k in ("gate_proj", "up_proj", "down_proj")]
                names += [(f"b{i}.n1", (f"blocks.{i}.mixer_norm", "weight")), (f"b{i}.n2", (f"blocks.{i}.ffn_norm", "weight"))]
            return ModelSpec(architecture=self.architecture,
                             embedding=EmbeddingSpec(vocab_size=d["vocab"], hidden_size=d["width"]),
                             blocks=(block(d["window"]), block(None)), order=(LayerCall(0, 0), LayerCall(1, 1)),
                             head=HeadSpec(vocab_size=d["vocab"], hidden_size=d["width"], tied=True, norm=norm),
                             tensor_names=tuple(names))

    register_architecture(WindowConfig.architecture, WindowConfig)
    return WindowConfig


def _plain_window(cfg, w, toks):
    n, nh, nkv, hd = len(toks), cfg["heads"], cfg["kv"], cfg["head"]
    x = w["emb"][torch.tensor(toks)]
    inv = plain_llama.rope_inv_freq(hd, cfg["theta"])
    for i, window in ((0, cfg["window"]), (1, None)):
        h = plain_llama.rms_norm(x, w[f"b{i}.n1"], cfg["eps"])
        q = plain_llama.apply_rope((h @ w[f"b{i}.q_proj"].T).view(n, nh, hd), range(n), inv)
        k = plain_llama.apply_rope((h @ w[f"b{i}.k_proj"].T).view(n, nkv, hd), range(n), inv)
        v = (h @ w[f"b{i}.v_proj"].T).view(n, nkv, hd)
        a = plain_llama.causal_attention(q, k, v, 1 / math.sqrt(hd), window)
        x = x + a.reshape(n, -1) @ w[f"b{i}.o_proj"].T
        h = plain_llama.rms_norm(x, w[f"b{i}.n2"], cfg["eps"])
        x = x + plain_llama.swiglu_mlp(h, w[f"b{i}.gate_proj"], w[f"b{i}.up_proj"], w[f"b{i}.down_proj"])
    return plain_llama.rms_norm(x, w["out_norm"], cfg["eps"]) @ w["emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_windowed_layer_beside_a_full_one_keeps_pages_of_its_own(tmp_path, dtype):
    run_windowed_model(tmp_path, dtype)


def run_windowed_model(tmp_path, dtype, graphs=True, **runner_options):
    """Two attention layers, one seeing the last 40 keys only, one seeing all: two cache groups.
    Heads of 64, so bfloat16 runs the tensor-core kernels with their window arguments.  The
    windowed group gives pages back as the window passes them; logits match the plain model in
    portions of 150 tokens (the tcgen05 kernel), small portions and single tokens."""
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    from llm_singularity_b200.engine.runner import expected_tensors_of
    from llm_singularity_b200.weights import random_tensors, write_safetensors
    WindowConfig = _register_window()
    cfg = dict(architectures=["ToyWindowForCausalLM"], width=128, heads=4, kv=2, head=64, inner=160, vocab=211,
               window=40, eps=1e-5, theta=10000.0)
    d = str(tmp_path)
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    tensors = random_tensors(expected_tensors_of(WindowConfig(cfg).to_model_spec()), seed=17,
                             dtype=torch.bfloat16, std=0.08, norm_noise=0.1)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    w = {k: v.double() for k, v in tensors.items()}

    runner = ModelRunner(d, dtype=dtype, page_size=16, num_pages=40, max_requests=2, **runner_options)
    cache = runner.cache
    assert sorted(g.window or 0 for g in cache.groups) == [0, 40]
    windowed = next(g for g in cache.groups if g.window)
    full = next(g for g in cache.groups if not g.window)
    seqs = {"a": tiny_models.random_tokens(211, 230, 1), "b": tiny_models.random_tokens(211, 200, 2)}
    # the run of single tokens at the end goes through the captured decode graph (two block tables
    # to patch inside it, pages leaving the windowed one as it goes)
    plan = [[("a", 150)], [("a", 30), ("b", 150)], [("a", 1), ("b", 7)], [("a", 1), ("b", 1)], [("a", 28), ("b", 22)]] \
        + [[("a", 1), ("b", 1)]] * 20
    got, pos = {"a": [], "b": []}, {"a": 0, "b": 0}
    runner.open("a"); runner.open("b")
    for step in plan:
        entries = [StepEntry(r, seqs[r][pos[r]:pos[r] + n], list(range(n))) for r, n in step]
        out = runner.step(entries)
        k = 0
        for r, n in step:
            got[r].append(out[k:k + n].clone()); k += n; pos[r] += n      # graph logits are overwritten
    runner.check_kernels()
    assert pos == {"a": 230, "b": 200} and (runner.graph_replays >= 15 or not graphs)
    # 430 tokens are held: 28 pages in the full group, only the windows' pages in the other
    assert full.pool.num_used == -(-230 // 16) + -(-200 // 16)
    assert windowed.pool.num_used <= 2 * (-(-40 // 16) + 1)
    cache.check_invariants()
    tol = 2e-4 if dtype == "float32" else None
    for r in "ab":
        want = _plain_window(cfg, w, seqs[r])
        have = torch.cat(got[r]).double().cpu()
        bound = tol if tol is not None else 4e-2 * want.abs().max().item()
        assert (have - want).abs().max().item() <= bound, r
    runner.close("a"); runner.close("b")
    assert windowed.pool.num_used == 0 and full.pool.num_used == 0


# ------------------------------------------------------------------ a layer that reads another layer's cache
def _register_shared():
    from llm_singularity_b200 import register_architecture
    from llm_singularity_b200.config.specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMLPSpec,
                                                   HeadSpec, LayerCall, ModelSpec, RMSNormSpec, RotarySpec)

    class SharedConfig:
        architecture = "ToySharedCacheForCausalLM"

        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_model_spec(self):
            d = self.d
            norm = RMSNormSpec(size=d["width"], eps=d["eps"])
            rot = RotarySpec(head_dim=d["head"], rotary_dim=d["head"], theta=d["theta"])
            blk = BlockSpec(mixer=AttentionSpec(hidden_size=d["width"], num_heads=d["heads"], num_kv_heads=d["kv"],
                                                head_dim=d["head"], scale=1 / math.sqrt(d["head"]), position=rot),
                            ffn=GatedMLPSpec(hidden_size=d["width"], intermediate_size=d["inner"]),
                            mixer_norm=norm, ffn_norm=norm)
            names = [("emb", ("embedding", "weight")), ("out_norm", ("head.norm", "weight"))]
            for i in (0, 1):
                names += [(f"b{i}.{k}", (f"blocks.{i}.mixer", k)) for k in ("q_proj", "k_proj", "v_proj", "o_proj")]
                names += [(f"b{i}.{k}", (f"blocks.{i}.ffn", k)) for k in ("gate_proj", "up_proj", "down_proj")]
                names += [(f"b{i}.n1", (f"blocks.{i}.mixer_norm", "weight")), (f"b{i}.n2", (f"blocks.{i}.ffn_norm", "weight"))]
            # the second layer writes no keys or values: it attends over what the first one cached;
            # the third call runs the first block again, on a cache of its own
            return ModelSpec(architecture=self.architecture,
                             embedding=EmbeddingSpec(vocab_size=d["vocab"], hidden_size=d["width"]),
                             blocks=(blk, blk),
                             order=(LayerCall(0, 0), LayerCall(1, 0, writes_cache=False), LayerCall(0, 1)),
                             head=HeadSpec(vocab_size=d["vocab"], hidden_size=d["width"], tied=True, norm=norm),
                             tensor_names=tuple(names))

    register_architecture(SharedConfig.architecture, SharedConfig)
    return SharedConfig


def _plain_shared(cfg, w, toks):
    n, nh, nkv, hd = len(toks), cfg["heads"], cfg["kv"], cfg["head"]
    x = w["emb"][torch.tensor(toks)]
    inv = plain_llama.rope_inv_freq(hd, cfg["theta"])
    kept = None
    for i, own_cache in ((0, True), (1, False), (0, True)):
        h = plain_llama.rms_norm(x, w[f"b{i}.n1"], cfg["eps"])
        q = plain_llama.apply_rope((h @ w[f"b{i}.q_proj"].T).view(n, nh, hd), range(n), inv)
        if own_cache:
            k = plain_llama.apply_rope((h @ w[f"b{i}.k_proj"].T).view(n, nkv, hd), range(n), inv)
            v = (h @ w[f"b{i}.v_proj"].T).view(n, nkv, hd)
            if kept is None:
                kept = (k, v)
        else:
            k, v = kept                                     # the first layer's keys and values
        a = plain_llama.causal_attention(q, k, v, 1 / math.sqrt(hd))
        x = x + a.reshape(n, -1) @ w[f"b{i}.o_proj"].T
        h = plain_llama.rms_norm(x, w[f"b{i}.n2"], cfg["eps"])
        x = x + plain_llama.swiglu_mlp(h, w[f"b{i}.gate_proj"], w[f"b{i}.up_proj"], w[f"b{i}.down_proj"])
    return plain_llama.rms_norm(x, w["out_norm"], cfg["eps"]) @ w["emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_reads_another_layers_cache(tmp_path, dtype):
    run_shared_cache_model(tmp_path, dtype)


def run_shared_cache_model(tmp_path, dtype, graphs=True, **runner_options):
    """The run order lets the second layer attend over the keys and values the first one cached
    (it stores none of its own) and names the first block a second time with a cache of its own."""
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    from llm_singularity_b200.engine.runner import expected_tensors_of
    from llm_singularity_b200.weights import random_tensors, write_safetensors
    SharedConfig = _register_shared()
    cfg = dict(architectures=["ToySharedCacheForCausalLM"], width=128, heads=4, kv=2, head=64, inner=96, vocab=157,
               eps=1e-5, theta=10000.0)
    d = str(tmp_path)
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    tensors = random_tensors(expected_tensors_of(SharedConfig(cfg).to_model_spec()), seed=23,
                             dtype=torch.bfloat16, std=0.08, norm_noise=0.1)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    w = {k: v.double() for k, v in tensors.items()}
    runner = ModelRunner(d, dtype=dtype, page_size=16, num_pages=24, max_requests=2, **runner_options)
    assert len(runner.model.cache_specs()) == 2             # two caches for three layer calls
    seqs = {"a": tiny_models.random_tokens(157, 170, 3), "b": tiny_models.random_tokens(157, 60, 4)}
    plan = [[("a", 140)], [("a", 1), ("b", 33)], [("a", 1), ("b", 1)], [("a", 16), ("b", 14)]] + [[("a", 1), ("b", 1)]] * 12
    got, pos = {"a": [], "b": []}, {"a": 0, "b": 0}
    runner.open("a"); runner.open("b")
    for step in plan:
        entries = [StepEntry(r, seqs[r][pos[r]:pos[r] + n], list(range(n))) for r, n in step]
        out = runner.step(entries)
        k = 0
        for r, n in step:
            got[r].append(out[k:k + n].clone()); k += n; pos[r] += n
    runner.check_kernels()
    assert pos == {"a": 170, "b": 60} and (runner.graph_replays >= 8 or not graphs)
    for r in "ab":
        want = _plain_shared(cfg, w, seqs[r])
        have = torch.cat(got[r]).double().cpu()
        bound = 2e-4 if dtype == "float32" else 4e-2 * want.abs().max().item()
        assert (have - want).abs().max().item() <= bound, r
    runner.cache.check_invariants()
