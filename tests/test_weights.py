"""Safetensors container, checked loading and random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

import plain_llama
import tiny_models
from llm_singularity_b200.config.llama import LlamaConfig
from llm_singularity_b200.engine.runner import expected_tensors_of
from llm_singularity_b200.weights import (SafetensorsError, SafetensorsFile, WeightError,
                                         load_checkpoint, write_random_model, write_safetensors)


def _expected(name):
    spec = LlamaConfig.from_dict(tiny_models.CONFIGS[name]).to_model_spec()
    return {n: (shape, role) for n, (shape, role, _) in expected_tensors_of(spec).items()}, spec


def test_round_trip_keeps_dtype_and_values(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7),
         "c": torch.arange(6, dtype=torch.int32).view(2, 3)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    f = SafetensorsFile(p)
    assert sorted(f.names()) == ["a", "b", "c"]
    for n, v in t.items():
        got = f.tensor(n)
        assert got.dtype == v.dtype and torch.equal(got, v)
    # an independent reader (the plain implementation's) sees the same numbers
    plain = plain_llama.read_safetensors(p)
    assert torch.equal(plain["a"], t["a"].double()) and torch.equal(plain["b"], t["b"].double())


def test_container_errors(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too small"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "F8_E4M3", "shape": [1], "data_offsets": [0, 1]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0")
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="needs 8"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFile(str(tmp_path / "absent.safetensors"))


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    cfg = LlamaConfig.from_dict(tiny_models.CONFIGS["tiny_b"])
    d = str(tmp_path / "m")
    write_random_model(d, cfg, seed=5, norm_noise=0.1)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    expected, spec = _expected("tiny_b")
    w = load_checkpoint(d, expected, spec.ignorable)
    assert set(w) == set(expected)
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    q = w["model.layers.1.self_attn.q_proj.weight"].float()
    assert q.shape == (128, 128) and abs(q.std().item() - 0.02) < 0.002
    n = w["model.norm.weight"].float()
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.15
    # same seed, same tensors; another seed, others; a tensor does not depend on its neighbours
    d2, d3 = str(tmp_path / "m2"), str(tmp_path / "m3")
    write_random_model(d2, cfg, seed=5, norm_noise=0.1)
    write_random_model(d3, cfg, seed=6, norm_noise=0.1)
    w2, w3 = load_checkpoint(d2, expected), load_checkpoint(d3, expected)
    assert all(torch.equal(w[k], w2[k]) for k in w)
    assert not torch.equal(w["lm_head.weight"], w3["lm_head.weight"])
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["LlamaForCausalLM"]


def test_random_stream_is_counter_based():
    """Element i of a tensor is a function of (seed, name, i) alone: a piece made on its own is
    the same piece, another name or seed gives another stream, and the values are standard normal.
    The first values are written down here, so that a change of the arithmetic (which would make
    models of earlier seeds unrepeatable) is seen."""
    from llm_singularity_b200.weights.random_init import _normal_cpu, normal_tensor, tensor_key
    key = tensor_key(7, "model.embed_tokens.weight")
    head = _normal_cpu(key, 0, 6)
    pinned = [-0.210832417011261, 0.22373543679714203, -1.0792911052703857, 0.40433570742607117,
              0.9879299402236938, 0.8777292370796204]
    assert head.tolist() == pinned
    assert torch.equal(_normal_cpu(key, 3, 3), head[3:])
    big = normal_tensor((1 << 20) + 5, key, 0.0, 1.0, torch.float32)        # crosses a chunk's edge
    assert torch.equal(big[:6], head) and torch.equal(big[(1 << 20) - 2:], _normal_cpu(key, (1 << 20) - 2, 7))
    assert not torch.equal(_normal_cpu(tensor_key(7, "lm_head.weight"), 0, 6), head)
    assert not torch.equal(_normal_cpu(tensor_key(8, "model.embed_tokens.weight"), 0, 6), head)
    x = big.double()
    assert torch.isfinite(x).all()
    assert abs(x.mean()) < 4e-3 and abs(x.var() - 1) < 6e-3
    assert abs((x ** 3).mean()) < 1.5e-2 and abs((x ** 4).mean() - 3) < 5e-2
    assert (x.abs() > 3).double().mean() == pytest.approx(0.0027, abs=4e-4)   # the tails are there
    # mean and scale, and one rounding to the stored dtype
    w = normal_tensor((4, 5), key, 1.0, 0.1, torch.bfloat16)
    assert torch.equal(w.view(-1)[:6], (1.0 + torch.tensor(0.1) * head).to(torch.bfloat16))


def test_32_bit_tensors_stay_32_bit(tmp_path):
    cfg = LlamaConfig.from_dict(tiny_models.CONFIGS["tiny_a"])
    d = str(tmp_path / "m")
    write_random_model(d, cfg, seed=1, dtype=torch.float32)
    expected, spec = _expected("tiny_a")
    w = load_checkpoint(d, expected, spec.ignorable)
    assert all(t.dtype == torch.float32 for t in w.values())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = LlamaConfig.from_dict(tiny_models.CONFIGS["tiny_a"])
    d = str(tmp_path / "m")
    write_random_model(d, cfg, seed=1)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    del t["model.layers.0.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    t["model.layers.1.self_attn.q_proj.weight"] = torch.zeros(3, 64)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    expected, spec = _expected("tiny_a")
    with pytest.raises(WeightError) as ei:
        load_checkpoint(d, expected, spec.ignorable)
    e = ei.value
    assert e.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.7.mlp.up_proj.weight"]
    assert [(n, tuple(g), tuple(w)) for n, g, w in e.wrong_shape] == \
        [("model.layers.1.self_attn.q_proj.weight", (3, 64), (64, 64))]
    msg = str(e)
    for word in ("missing", "unexpected", "wrong shape", "model.norm.weight", "[3, 64]"):
        assert word in msg


def test_tied_checkpoint_may_carry_lm_head_but_untied_must(tmp_path):
    cfg = LlamaConfig.from_dict(tiny_models.CONFIGS["tiny_a"])          # tied
    d = str(tmp_path / "m")
    write_random_model(d, cfg, seed=1)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    expected, spec = _expected("tiny_a")
    assert "lm_head.weight" not in load_checkpoint(d, expected, spec.ignorable)
    untied = dict(tiny_models.CONFIGS["tiny_a"], tie_word_embeddings=False)
    spec_u = LlamaConfig.from_dict(untied).to_model_spec()
    exp_u = {n: (s, r) for n, (s, r, _) in expected_tensors_of(spec_u).items()}
    del t["lm_head.weight"]
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_checkpoint(d, exp_u, spec_u.ignorable)


def test_no_safetensors_file(tmp_path):
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_checkpoint(str(tmp_path), {})
