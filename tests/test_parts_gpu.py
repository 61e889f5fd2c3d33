"""Each part of a layer alone (norm, rotary attention with its cache, feed-forward, block,
embedding and head), built from its spec outside any model, against the plain functions."""
import math

import pytest
import torch

import plain_llama
from test_kernels_gpu import _make_ctx, _rand

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _rt(dtype):
    from llm_singularity_b200.parts import Runtime
    return Runtime("cuda", dtype)


def _tol(dtype, scale):
    return (3e-5 if dtype == torch.float32 else 2e-2) * scale


def _w(*shape, dtype, seed, std=0.05):
    return _rand(*shape, dtype=dtype, seed=seed, scale=std)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from llm_singularity_b200.config.specs import RMSNormSpec
    from llm_singularity_b200.parts import NORMS
    norm = NORMS.build(RMSNormSpec(size=200, eps=2e-6), _rt(dtype))
    assert type(norm).params(norm.spec)["weight"].role == "vector"
    w = 1 + 0.1 * _rand(200, seed=1)
    norm.load({"weight": w})
    res, delta = _rand(5, 200, seed=2), _rand(5, 200, dtype=dtype, seed=3)
    want = plain_llama.rms_norm(res.double() + delta.double(), w.double(), 2e-6)
    out = norm.add_norm(res, delta)
    assert out.dtype == dtype and (out.double() - want).abs().max() <= _tol(dtype, 4)
    rows = torch.tensor([4, 1], dtype=torch.int32, device="cuda")
    out2 = norm.gather_add_norm(res, None, rows)          # res already holds res + delta
    assert (out2.double() - want[[4, 1]]).abs().max() <= _tol(dtype, 4)


def _attention_setup(dtype, window=None, scaling=None, nh=6, nkv=2, hd=48, H=72, page=8, rotary=None, **more):
    from llm_singularity_b200.cache import CacheManager
    from llm_singularity_b200.config.specs import AttentionSpec, Llama3RopeScaling, RotarySpec
    from llm_singularity_b200.parts import MIXERS
    rt = _rt(dtype)
    sc = Llama3RopeScaling(8.0, 1.0, 4.0, 32) if scaling else None
    spec = AttentionSpec(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                         scale=1 / math.sqrt(hd), window=window,
                         position=RotarySpec(head_dim=hd, rotary_dim=rotary or hd, theta=20000.0, scaling=sc),
                         **more)
    att = MIXERS.build(spec, rt)
    ws = {"q_proj": _w(nh * hd, H, dtype=dtype, seed=1, std=0.3), "k_proj": _w(nkv * hd, H, dtype=dtype, seed=2, std=0.3),
          "v_proj": _w(nkv * hd, H, dtype=dtype, seed=3), "o_proj": _w(H, nh * hd, dtype=dtype, seed=4)}
    att.load(ws)
    cache = CacheManager([att.cache_spec()], page, 24, 3, 16, rt=rt)
    return rt, att, ws, cache, sc


def _plain_attention(x, ws, nh, nkv, hd, theta, sc, window, softcap=None, slopes=None, rotary=None):
    n = x.shape[0]
    d = {k: v.double().cpu() for k, v in ws.items()}
    q = (x @ d["q_proj"].T).view(n, nh, hd)
    k = (x @ d["k_proj"].T).view(n, nkv, hd)
    v = (x @ d["v_proj"].T).view(n, nkv, hd)
    scd = None if sc is None else dict(rope_type="llama3", factor=sc.factor, low_freq_factor=sc.low_freq_factor,
                                       high_freq_factor=sc.high_freq_factor,
                                       original_max_position_embeddings=sc.original_max_position_embeddings)
    rot = rotary or hd
    inv = plain_llama.rope_inv_freq(rot, theta, scd)
    q, k = (torch.cat([plain_llama.apply_rope(t[..., :rot], range(n), inv), t[..., rot:]], dim=-1) for t in (q, k))
    a = plain_llama.causal_attention(q, k, v, 1 / math.sqrt(hd), window, softcap, slopes)
    return a.reshape(n, nh * hd) @ d["o_proj"].T


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window, scaling, hd, rotary", [(None, False, 48, None), (None, True, 48, None),
                                                         (11, False, 48, None), (None, False, 48, 20),
                                                         (None, True, 64, 32), (11, False, 128, 48)])
def test_attention_part_in_portions_and_decode(dtype, window, scaling, hd, rotary):
    """One sequence of 45 tokens fed as 20 + 2 + 1 + ... through the part's own cache equals plain
    attention over the whole sequence; with a window, pages the window has passed are given back.
    Also with heads of which only the first `rotary` dims rotate (in bfloat16 the 64- and 128-wide
    ones take the decode kernel's own rotation for their single tokens)."""
    from llm_singularity_b200.engine.batch import ContextBuilder
    rt, att, ws, cache, sc = _attention_setup(dtype, window, scaling, hd=hd, rotary=rotary)
    x = _rand(45, 72, dtype=dtype, seed=9)
    want = _plain_attention(x.double().cpu(), ws, 6, 2, hd, 20000.0, sc, window, rotary=rotary)
    builder = ContextBuilder("cuda", 64, 3)
    cache.open("s")
    outs, pos = [], 0
    for n in [20, 2, 1, 1, 13, 1, 7]:
        assert cache.reserve("s", pos + n)
        ups = dict(cache.take_updates(0))
        if ups:
            idx = torch.tensor(list(ups.keys()), dtype=torch.int32, device="cuda")
            val = torch.tensor(list(ups.values()), dtype=torch.int32, device="cuda")
            rt.ops.scatter_i32(cache.groups[0].dev_table, idx, val)
        ctx, _ = builder.build([[0] * n], [pos], [cache.slot("s")], [[]])
        outs.append(att.forward(x[pos:pos + n].contiguous(), ctx, cache.view(0, ctx)))
        pos += n
        cache.commit("s", pos)
    got = torch.cat(outs).double().cpu()
    rt.ops.check_status()
    assert (got - want).abs().max() <= _tol(dtype, want.abs().max().item() + 1)
    if window:
        assert cache.groups[0].pool.num_used <= -(-window // 8) + 1      # only the window's pages
    cache.close("s")
    cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd, softcap, bias", [(48, 5.0, False), (64, None, True), (64, 3.0, True)])
def test_attention_part_with_score_modifiers(dtype, hd, softcap, bias):
    """A soft cap on the scores and a linear position bias per head (neither is Llama's: what another
    architecture's attention would set in its spec), in portions and decode tokens through the cache,
    against plain attention with the same modifiers.  Head size 64 in bfloat16 would run the tensor-core
    kernels; a spec with a modifier goes to the generic kernel, and it must show in the result: the
    queries are large enough that the cap moves the scores by far more than the tolerance."""
    from llm_singularity_b200.engine.batch import ContextBuilder
    nh, nkv, H = 4, 2, 64
    rt, att, ws, cache, sc = _attention_setup(dtype, None, None, nh=nh, nkv=nkv, hd=hd, H=H,
                                              logit_softcap=softcap, linear_bias=bias)
    x = _rand(40, H, dtype=dtype, seed=11) * (3 if softcap else 1)    # (large scores only where the cap bounds them)
    slopes = [2.0 ** (-8.0 * (h + 1) / nh) for h in range(nh)] if bias else None
    want = _plain_attention(x.double().cpu(), ws, nh, nkv, hd, 20000.0, sc, None, softcap, slopes)
    plain = _plain_attention(x.double().cpu(), ws, nh, nkv, hd, 20000.0, sc, None)
    builder = ContextBuilder("cuda", 64, 3)
    cache.open("s")
    outs, pos = [], 0
    for n in [17, 1, 1, 9, 1, 11]:
        assert cache.reserve("s", pos + n)
        ups = dict(cache.take_updates(0))
        if ups:
            idx = torch.tensor(list(ups.keys()), dtype=torch.int32, device="cuda")
            val = torch.tensor(list(ups.values()), dtype=torch.int32, device="cuda")
            rt.ops.scatter_i32(cache.groups[0].dev_table, idx, val)
        ctx, _ = builder.build([[0] * n], [pos], [cache.slot("s")], [[]])
        outs.append(att.forward(x[pos:pos + n].contiguous(), ctx, cache.view(0, ctx)))
        pos += n
        cache.commit("s", pos)
    got = torch.cat(outs).double().cpu()
    rt.ops.check_status()
    tol = _tol(dtype, want.abs().max().item() + 1)
    assert (got - want).abs().max() <= tol
    assert (plain - want).abs().max() > 0.1 * want.abs().max()   # the modifiers matter at these sizes
    cache.close("s")


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_mlp_part(dtype):
    from llm_singularity_b200.config.specs import GatedMLPSpec
    from llm_singularity_b200.parts import FEED_FORWARDS
    mlp = FEED_FORWARDS.build(GatedMLPSpec(hidden_size=72, intermediate_size=100), _rt(dtype))
    ws = {"gate_proj": _w(100, 72, dtype=dtype, seed=1, std=0.2), "up_proj": _w(100, 72, dtype=dtype, seed=2, std=0.2),
          "down_proj": _w(72, 100, dtype=dtype, seed=3, std=0.2)}
    mlp.load(ws)
    x = _rand(9, 72, dtype=dtype, seed=4)
    want = plain_llama.swiglu_mlp(x.double().cpu(), *(ws[k].double().cpu() for k in ("gate_proj", "up_proj", "down_proj")))
    got = mlp.forward(x, None).double().cpu()
    assert (got - want).abs().max() <= _tol(dtype, want.abs().max().item() + 1)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from llm_singularity_b200.config.specs import EmbeddingSpec, HeadSpec, RMSNormSpec
    from llm_singularity_b200.parts.embedding import Embedding, LMHead
    rt = _rt(dtype)
    emb = Embedding(EmbeddingSpec(vocab_size=301, hidden_size=72), rt)
    table = _w(301, 72, dtype=dtype, seed=1, std=1.0)
    emb.load({"weight": table})
    ids = torch.tensor([300, 0, 17], dtype=torch.int32, device="cuda")
    h = emb.forward(ids)
    assert h.dtype == torch.float32 and torch.equal(h, table[ids.long()].float())
    for tied in (True, False):
        head = LMHead(HeadSpec(vocab_size=301, hidden_size=72, tied=tied,
                               norm=RMSNormSpec(size=72, eps=1e-5)), rt)
        nw = 1 + 0.1 * _rand(72, seed=2)
        head.norm.load({"weight": nw})
        w = table if tied else _w(301, 72, dtype=dtype, seed=3, std=1.0)
        if tied:
            assert type(head).params(head.spec) == {}
            head.tie(emb)
        else:
            head.load({"weight": w})
        pending = _rand(3, 72, dtype=dtype, seed=4)
        rows = torch.tensor([2, 0], dtype=torch.int32, device="cuda")
        logits = head.forward(h, pending, rows)
        x = (h.double() + pending.double())[[2, 0]].cpu()
        want = plain_llama.rms_norm(x, nw.double().cpu(), 1e-5) @ w.double().cpu().T
        assert logits.dtype == torch.float32 and logits.shape == (2, 301)
        assert (logits.double().cpu() - want).abs().max() <= _tol(dtype, want.abs().max().item())


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part_carries_the_pending_delta(dtype):
    """A pre-norm block: the feed-forward output comes back un-added and the next norm adds it."""
    from llm_singularity_b200.cache import CacheManager
    from llm_singularity_b200.config.specs import (AttentionSpec, BlockSpec, GatedMLPSpec,
                                                   NoPositionSpec, RMSNormSpec)
    from llm_singularity_b200.engine.batch import ContextBuilder
    from llm_singularity_b200.parts import BLOCKS
    rt = _rt(dtype)
    H, nh, hd = 64, 2, 32
    norm = RMSNormSpec(size=H, eps=1e-5)
    spec = BlockSpec(mixer=AttentionSpec(hidden_size=H, num_heads=nh, num_kv_heads=nh, head_dim=hd,
                                         scale=0.2, position=NoPositionSpec()),
                     ffn=GatedMLPSpec(hidden_size=H, intermediate_size=48), mixer_norm=norm, ffn_norm=norm)
    blk = BLOCKS.build(spec, rt)
    ws = {"q_proj": _w(H, H, dtype=dtype, seed=1, std=0.2), "k_proj": _w(H, H, dtype=dtype, seed=2, std=0.2),
          "v_proj": _w(H, H, dtype=dtype, seed=3), "o_proj": _w(H, H, dtype=dtype, seed=4),
          "gate_proj": _w(48, H, dtype=dtype, seed=5), "up_proj": _w(48, H, dtype=dtype, seed=6),
          "down_proj": _w(H, 48, dtype=dtype, seed=7)}
    n1, n2 = 1 + 0.1 * _rand(H, seed=8), 1 + 0.1 * _rand(H, seed=9)
    blk.mixer_norm.load({"weight": n1}); blk.ffn_norm.load({"weight": n2})
    blk.mixer.load({k: ws[k] for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
    blk.ffn.load({k: ws[k] for k in ("gate_proj", "up_proj", "down_proj")})
    cache = CacheManager([blk.mixer.cache_spec()], 16, 4, 1, 4, rt=rt)
    cache.open("s"); cache.reserve("s", 10)
    ups = dict(cache.take_updates(0))
    rt.ops.scatter_i32(cache.groups[0].dev_table, torch.tensor(list(ups), dtype=torch.int32, device="cuda"),
                       torch.tensor(list(ups.values()), dtype=torch.int32, device="cuda"))
    ctx, _ = ContextBuilder("cuda", 16, 1).build([[0] * 10], [0], [0], [[]])
    x0, pend = _rand(10, H, seed=10), _rand(10, H, dtype=dtype, seed=11)
    res = x0.clone()
    out = blk.forward(res, pend, ctx, cache.view(0, ctx))
    d = {k: v.double().cpu() for k, v in ws.items()}
    x = x0.double().cpu() + pend.double().cpu()
    h = plain_llama.rms_norm(x, n1.double().cpu(), 1e-5)
    q, k, v = ((h @ d[n].T).view(10, nh, hd) for n in ("q_proj", "k_proj", "v_proj"))
    x = x + plain_llama.causal_attention(q, k, v, 0.2).reshape(10, H) @ d["o_proj"].T
    h = plain_llama.rms_norm(x, n2.double().cpu(), 1e-5)
    want = plain_llama.swiglu_mlp(h, d["gate_proj"], d["up_proj"], d["down_proj"])
    assert (res.double().cpu() - x).abs().max() <= _tol(dtype, 4)          # residual after attention
    assert (out.double().cpu() - want).abs().max() <= _tol(dtype, want.abs().max().item() + 1)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_replayed_layers_give_the_same_bits_as_layers_run_one_by_one(tmp_path, dtype):
    """From the second layer on a step records a layer's launches and repeats them for the layers
    after it with their own weights and pages.  A step of decode tokens beside prompt portions
    (two streams), a prompt alone and a decode step (captured graph), each against the same step
    with the repetition switched off: identical logits, identical cache pages."""
    from llm_singularity_b200 import kernels
    from llm_singularity_b200.engine import ModelRunner, StepEntry
    import tiny_models
    import json, os
    from llm_singularity_b200.config.llama import LlamaConfig
    from llm_singularity_b200.weights import write_random_model
    name = "tiny_b" if dtype == "float32" else "tiny_d"      # generic kernels / heads of 64, five layers each
    cfg = dict(tiny_models.CONFIGS[name], num_hidden_layers=5)
    model_dir = str(tmp_path / "five_layers")
    write_random_model(model_dir, LlamaConfig.from_dict(cfg), seed=77, std=0.08, norm_noise=0.1)
    json.dump(cfg, open(os.path.join(model_dir, "config.json"), "w"))
    vocab = cfg["vocab_size"]
    ps = tiny_models.PAGE_SIZE[name]
    toks = {r: tiny_models.random_tokens(vocab, n, 70 + i) for i, (r, n) in enumerate((("a", 150), ("b", 40), ("c", 9)))}
    results = []
    launches = []
    try:
        for on in (False, True):
            kernels.LAYER_REPLAY = on
            runner = ModelRunner(model_dir, dtype=dtype, page_size=ps, num_pages=64, max_requests=4)
            for r in toks:
                runner.open(r)
            n0 = kernels.launch_count()
            outs = [runner.step([StepEntry("b", toks["b"][:30], [29]), StepEntry("c", toks["c"][:8], [7])]).clone()]
            outs.append(runner.step([StepEntry("b", toks["b"][30:31], [0]), StepEntry("c", toks["c"][8:], [0]),
                                     StepEntry("a", toks["a"][:140], [0, 139])]).clone())
            for k in range(31, 35):                                              # decode steps: eager, captured, replayed
                outs.append(runner.step([StepEntry("b", [toks["b"][k]], [0]), StepEntry("a", [toks["a"][109 + k]], [0])]).clone())
            launches.append(kernels.launch_count() - n0)
            runner.check_kernels()
            pages = [t.clone() for cid in range(len(runner.model.cache_specs())) for t in runner.cache._store[cid]]
            results.append((outs, pages))
    finally:
        kernels.LAYER_REPLAY = True
    for a, b in zip(results[0][0], results[1][0]):
        assert torch.equal(a, b)
    for a, b in zip(results[0][1], results[1][1]):
        assert torch.equal(a, b)
    assert launches[0] == launches[1]                 # the same kernels were launched, as many times
