"""Configuration and registry (no GPU)."""
import json
import math

import pytest

import tiny_models
from llm_singularity_b200 import load_config, known_architectures, register_architecture
from llm_singularity_b200.config.llama import ConfigError, LlamaConfig
from llm_singularity_b200.registry import UnknownArchitecture


def test_every_key_is_read_from_config_json():
    d = tiny_models.CONFIGS["tiny_b"]
    c = LlamaConfig.from_dict(d)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads,
            c.head_dim, c.intermediate_size, c.vocab_size) == (3, 128, 4, 1, 32, 320, 512)
    assert c.rope_theta == 500000.0 and c.rms_norm_eps == 1e-6 and not c.tie_word_embeddings
    rs = c.rope_scaling
    assert (rs.factor, rs.low_freq_factor, rs.high_freq_factor,
            rs.original_max_position_embeddings) == (32.0, 1.0, 4.0, 64)
    assert c.eos_token_ids == (510, 511)


def test_defaults_follow_the_reference():
    c = LlamaConfig.from_dict(dict(num_hidden_layers=1, hidden_size=64, num_attention_heads=4,
                                   intermediate_size=8, vocab_size=10))
    assert c.num_key_value_heads == 4            # llama_model.cpp:162-163
    assert c.head_dim == 16                      # hidden / heads, llama_model.cpp:105-107
    assert c.rope_theta == 10000.0               # llama_model.cpp:183
    assert c.rms_norm_eps == 1e-5                # llama_model.cpp:507
    assert c.max_position_embeddings == 2048     # llama_model.cpp:166
    assert c.rope_scaling is None and c.eos_token_ids == ()


def test_head_dim_may_differ_from_hidden_over_heads():
    c = LlamaConfig.from_dict(tiny_models.CONFIGS["tiny_c"])
    assert c.head_dim == 48 and c.hidden_size // c.num_attention_heads == 12
    spec = c.to_model_spec()
    assert spec.blocks[0].mixer.head_dim == 48
    assert math.isclose(spec.blocks[0].mixer.scale, 1 / math.sqrt(48))


@pytest.mark.parametrize("patch, word", [
    ({"num_attention_heads": 5, "num_key_value_heads": 2}, "multiple"),
    ({"head_dim": 15}, "multiple of 16"),
    ({"head_dim": 24}, "multiple of 16"),
    ({"head_dim": 272}, "at most 256"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "lacks"),
    ({"hidden_act": "gelu"}, "gelu"),
    ({"attention_bias": True}, "attention_bias"),
    ({"vocab_size": None}, "vocab_size"),
    ({"hidden_size": -4}, "positive"),
    ({"rms_norm_eps": 0.0}, "eps"),
])
def test_bad_values_are_refused(patch, word):
    d = dict(tiny_models.CONFIGS["tiny_a"])
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict(d)


def test_registry_picks_the_class_by_architecture(tmp_path):
    assert "LlamaForCausalLM" in known_architectures()
    (tmp_path / "config.json").write_text(json.dumps(tiny_models.CONFIGS["tiny_a"]))
    assert isinstance(load_config(str(tmp_path)), LlamaConfig)
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["NopeForCausalLM"]}))
    with pytest.raises(UnknownArchitecture, match="LlamaForCausalLM"):
        load_config(str(tmp_path))
    with pytest.raises(FileNotFoundError):
        load_config(str(tmp_path / "absent"))


def test_spec_has_one_block_per_layer_and_reference_tensor_names():
    c = LlamaConfig.from_dict(tiny_models.CONFIGS["tiny_b"])
    spec = c.to_model_spec()
    assert len(spec.blocks) == 3 and [lc.block for lc in spec.order] == [0, 1, 2]
    names = dict(spec.tensor_names)
    assert names["model.layers.2.self_attn.k_proj.weight"] == ("blocks.2.mixer", "k_proj")
    assert "lm_head.weight" in names
    tied = LlamaConfig.from_dict(tiny_models.CONFIGS["tiny_a"]).to_model_spec()
    assert "lm_head.weight" not in dict(tied.tensor_names) and tied.head.tied
    assert tied.stop_token_ids == (255,)


def test_config_round_trips_through_to_dict():
    for d in tiny_models.CONFIGS.values():
        c = LlamaConfig.from_dict(d)
        assert LlamaConfig.from_dict(c.to_dict()) == c
