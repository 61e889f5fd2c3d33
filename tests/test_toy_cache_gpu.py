"""A cache kind of the test's own and the activations of the stock gated feed-forward, with no
change to the framework's files.

The toy cache keeps one short latent vector per token in pages of its own shape ([pages,
page_size, latent], 32-bit, keys and values in one), handed out through the block table like
key/value pages: it is a ``CacheSpec`` subclass defined here, which the cache manager allocates,
groups, views and frees without knowing it.  The toy mixer that uses it attends over the latents
(one head, the latent is key and value at once).  Its two blocks run the stock gated feed-forward
with the tanh form of gelu and with no activation at all (gate * up), through the same kernels
as silu.  The model is stepped in portions and single tokens, two requests at a time, with pages
used again; a plain whole-sequence computation in float64 is the reference.  The toy is nobody's
model."""
import json
import math
import os
from dataclasses import dataclass, field

import pytest
import torch

import plain_llama
import tiny_models

W, LATENT, INNER, VOCAB = 40, 24, 56, 91


def _register():
    from llm_singularity_b200 import register_architecture
    from llm_singularity_b200.config.specs import (BlockSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec,
                                                   LayerCall, ModelSpec, PartSpec, RMSNormSpec)
    from llm_singularity_b200.parts import CacheSpec, ParamSpec, Part, register_mixer

    @dataclass
    class LatentView:
        pages: torch.Tensor            # [num_pages, page_size, latent] float32
        block_table: torch.Tensor      # int32 [slots, max_pages]
        page_size: int

    @dataclass(frozen=True)
    class LatentPagesSpec(CacheSpec):
        """One latent vector per token, in pages addressed through the group's block table."""
        latent: int = 0
        window = None
        paged = True

        def allocate(self, rt, page_size, num_pages, slots):
            return torch.zeros(num_pages, page_size, self.latent, dtype=torch.float32, device=rt.device)

        def view(self, storage, group):
            return LatentView(storage, group.dev_table, group.page_size)

        def bytes_per_page(self, page_size, element_size):
            return page_size * self.latent * 4

    @dataclass(frozen=True)
    class LatentMixerSpec(PartSpec):
        hidden_size: int = 0
        latent: int = 0
        kind: str = field(init=False, default="toy_latent")

    @register_mixer("toy_latent")
    class LatentMixer(Part):
        """c_t = x_t Wc^T is cached; out_t = (sum_s softmax_s(q_t . c_s / sqrt(L)) c_s) Wo^T over
        s <= t, with q_t = x_t Wq^T."""

        @classmethod
        def params(cls, spec):
            return {"w_c": ParamSpec((spec.latent, spec.hidden_size)),
                    "w_q": ParamSpec((spec.latent, spec.hidden_size)),
                    "w_o": ParamSpec((spec.hidden_size, spec.latent))}

        def load(self, tensors):
            self.t = tensors

        def cache_spec(self):
            return LatentPagesSpec(latent=self.spec.latent)

        def forward(self, x, ctx, cache, writes_cache=True):
            ops, L = self.rt.ops, self.spec.latent
            c = ops.linear(x, self.t["w_c"], out_dtype=torch.float32)
            q = ops.linear(x, self.t["w_q"], out_dtype=torch.float32)
            ps = cache.page_size
            pos = ctx.positions.long()
            rows = ctx.table_rows.long()[ctx.token_req.long()]
            if writes_cache:
                pages = cache.block_table[rows, pos // ps].long()
                assert bool((pages >= 0).all()), "write into a page that is not held"
                cache.pages[pages, pos % ps] = c
            mixed = torch.empty_like(c)
            for r in range(ctx.n_requests):
                a, b = int(ctx.h_q_start[r]), int(ctx.h_q_start[r + 1])
                n = int(ctx.h_kv_len[r])
                idx = torch.arange(n, device=x.device)
                held = cache.block_table[int(ctx.h_table_rows[r]), idx // ps].long()
                lat = cache.pages[held, idx % ps]                                  # [n, L]
                s = (q[a:b] @ lat.T) / math.sqrt(L)
                mask = idx[None, :] <= pos[a:b, None]
                p = torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1)
                mixed[a:b] = p @ lat
            return ops.linear(mixed.to(x.dtype), self.t["w_o"])

    class ToyConfig:
        architecture = "ToyLatentForCausalLM"

        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_model_spec(self):
            d = self.d
            norm = RMSNormSpec(size=d["width"], eps=d["eps"])
            mixer = LatentMixerSpec(hidden_size=d["width"], latent=d["latent"])
            blocks = tuple(BlockSpec(mixer=mixer, mixer_norm=norm, ffn_norm=norm,
                                     ffn=GatedMLPSpec(hidden_size=d["width"], intermediate_size=d["inner"],
                                                      activation=act))
                           for act in d["activations"])
            names = [("emb", ("embedding", "weight")), ("out_norm", ("head.norm", "weight")),
                     ("out", ("head", "weight"))]
            for i in range(len(blocks)):
                names += [(f"b{i}.{k}", (f"blocks.{i}.mixer", k)) for k in ("w_c", "w_q", "w_o")]
                names += [(f"b{i}.{k}", (f"blocks.{i}.ffn", k)) for k in ("gate_proj", "up_proj", "down_proj")]
                names += [(f"b{i}.n1", (f"blocks.{i}.mixer_norm", "weight")),
                          (f"b{i}.n2", (f"blocks.{i}.ffn_norm", "weight"))]
            return ModelSpec(
                architecture=self.architecture,
                embedding=EmbeddingSpec(vocab_size=d["vocab"], hidden_size=d["width"]),
                blocks=blocks, order=tuple(LayerCall(i, i) for i in range(len(blocks))),
                head=HeadSpec(vocab_size=d["vocab"], hidden_size=d["width"], tied=False, norm=norm),
                tensor_names=tuple(names))

    register_architecture(ToyConfig.architecture, ToyConfig)
    return ToyConfig, LatentPagesSpec


def _act(g, name):
    if name == "gelu_tanh":
        return 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
    return g if name == "none" else g / (1 + torch.exp(-g))


def _plain(cfg, w, toks, rnd):
    """The same model whole-sequence in float64; ``rnd`` rounds where a bfloat16 engine stores."""
    n = len(toks)
    x = w["emb"][torch.tensor(toks)]
    mask = torch.tril(torch.ones(n, n, dtype=torch.bool))
    for i, act in enumerate(cfg["activations"]):
        h = rnd(plain_llama.rms_norm(x, w[f"b{i}.n1"], cfg["eps"]))
        c, q = h @ w[f"b{i}.w_c"].T, h @ w[f"b{i}.w_q"].T          # kept in 32-bit by the mixer
        p = torch.softmax(((q @ c.T) / math.sqrt(cfg["latent"])).masked_fill(~mask, float("-inf")), dim=-1)
        x = x + rnd(rnd(p @ c) @ w[f"b{i}.w_o"].T)
        h = rnd(plain_llama.rms_norm(x, w[f"b{i}.n2"], cfg["eps"]))
        g, u = h @ w[f"b{i}.gate_proj"].T, h @ w[f"b{i}.up_proj"].T
        x = x + rnd(rnd(_act(g, act) * u) @ w[f"b{i}.down_proj"].T)
    return rnd(plain_llama.rms_norm(x, w["out_norm"], cfg["eps"])) @ w["out"].T


def run_latent_model(tmp_path, dtype, **runner_options):
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    from llm_singularity_b200.engine.runner import expected_tensors_of
    from llm_singularity_b200.weights import random_tensors, write_safetensors
    ToyConfig, LatentPagesSpec = _register()
    cfg = dict(architectures=["ToyLatentForCausalLM"], width=W, latent=LATENT, inner=INNER, vocab=VOCAB,
               eps=1e-5, activations=["gelu_tanh", "none"])
    d = str(tmp_path)
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = random_tensors(expected_tensors_of(ToyConfig(cfg).to_model_spec()), seed=29, dtype=store,
                             std=0.3, norm_noise=0.1)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    w = {k: v.double() for k, v in tensors.items()}

    runner = ModelRunner(d, dtype=dtype, page_size=8, num_pages=9, max_requests=2, **runner_options)
    specs = runner.model.cache_specs()
    assert all(isinstance(s, LatentPagesSpec) for s in specs) and len(runner.cache.groups) == 1
    assert runner.cache.bytes_per_page(0) == 2 * 8 * LATENT * 4
    seqs = {r: tiny_models.random_tokens(VOCAB, n, s) for r, n, s in (("a", 30, 1), ("b", 41, 2), ("c", 25, 3))}
    got = {r: [] for r in seqs}
    pos = {r: 0 for r in seqs}
    plan = [[("a", 7), ("b", 20)], [("a", 1), ("b", 2)], [("a", 22), ("b", 1)], [("b", 10), ("c", 9)],
            [("c", 1), ("b", 8)], [("c", 15)]]     # c starts on pages that a gave back, beside b
    runner.open("a"); runner.open("b")
    pages_seen = {}
    for step in plan:
        for r, _ in step:
            if not runner.cache.has(r):
                runner.open(r)
        out = runner.step([StepEntry(r, seqs[r][pos[r]:pos[r] + n], list(range(n))) for r, n in step])
        k = 0
        for r, n in step:
            got[r].append(out[k:k + n]); k += n; pos[r] += n
            for page in runner.cache.pages_of(r):
                pages_seen.setdefault(page, set()).add(r)
            if pos[r] == len(seqs[r]):
                runner.close(r)
    runner.check_kernels()
    assert any(len(who) > 1 for who in pages_seen.values())          # a page was used again
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == 9
    rnd = plain_llama.bf16_rounding if dtype == "bfloat16" else (lambda t: t)
    for r in seqs:
        want = _plain(cfg, w, seqs[r], rnd)
        tol = 1e-4 if dtype == "float32" else 4e-2 * float(want.abs().max())
        diff = (torch.cat(got[r]).double().cpu() - want).abs().max().item()
        assert diff <= tol, (r, diff, tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_cache_kind_and_activations_of_the_tests_own(tmp_path, dtype):
    run_latent_model(tmp_path, dtype)


def test_a_cache_kind_of_the_tests_own_on_the_host(tmp_path):
    import standin_ops
    run_latent_model(tmp_path, "float32", device="cpu", ops=standin_ops)
