"""LlamaConfig: the Llama decoder's configuration, read from config.json keys.

The reference reads ``num_hidden_layers, hidden_size, num_attention_heads,
num_key_value_heads, intermediate_size, vocab_size, max_position_embeddings,
eos_token_id, rope_theta`` (models/llama/llama_model.cpp:159-183), derives the
head size (llama_model.cpp:105-107), fixes the norm eps at 1e-5
(llama_model.cpp:507,630,659) and infers tied embeddings from a missing
``lm_head.weight`` (llama_model.cpp:257-261).  Here every one of those is a typed
field taken from config.json (``head_dim``, ``rms_norm_eps``,
``tie_word_embeddings``, ``rope_scaling``), with the reference's value as the
default where the key is absent.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec,
                    LayerCall, Llama3RopeScaling, ModelSpec, RMSNormSpec, RotarySpec)


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value the engine cannot run."""


def _require(d: Mapping[str, Any], key: str, typ):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        if v <= 0:
            raise ConfigError(f"config.json: '{key}' must be positive, got {v}")
    return v


@dataclass(frozen=True)
class LlamaConfig:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    rope_scaling: Optional[Llama3RopeScaling]
    rms_norm_eps: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    eos_token_ids: Tuple[int, ...]

    architecture = "LlamaForCausalLM"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        nh = _require(d, "num_attention_heads", int)
        hidden = _require(d, "hidden_size", int)
        nkv = d.get("num_key_value_heads")
        if nkv is None:
            nkv = nh                                   # llama_model.cpp:162-163
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % nh:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not divisible by "
                    f"num_attention_heads {nh} and no 'head_dim' is given")
            head_dim = hidden // nh                    # llama_model.cpp:105-107
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (silu only)")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(f"config.json: '{key}' = true is not supported")

        eos = d.get("eos_token_id")                    # int or list: llama_model.cpp:170-181
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)

        cfg = cls(
            num_hidden_layers=_require(d, "num_hidden_layers", int),
            hidden_size=hidden,
            num_attention_heads=nh,
            num_key_value_heads=int(nkv),
            head_dim=int(head_dim),
            intermediate_size=_require(d, "intermediate_size", int),
            vocab_size=_require(d, "vocab_size", int),
            rope_theta=float(d.get("rope_theta", 10000.0)),   # llama_model.cpp:183
            rope_scaling=cls._parse_rope_scaling(d.get("rope_scaling")),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_position_embeddings=int(d.get("max_position_embeddings", 2048)),
            eos_token_ids=eos_ids,
        )
        cfg.validate()
        return cfg

    @staticmethod
    def _parse_rope_scaling(rs) -> Optional[Llama3RopeScaling]:
        if rs is None:
            return None
        if not isinstance(rs, Mapping):
            raise ConfigError(f"config.json: rope_scaling must be an object or null, got {rs!r}")
        rope_type = rs.get("rope_type", rs.get("type"))
        if rope_type in (None, "default"):
            return None
        if rope_type != "llama3":
            raise ConfigError(
                f"config.json: rope_scaling type '{rope_type}' is not supported "
                f"(known: 'llama3', 'default')")
        try:
            return Llama3RopeScaling(
                factor=float(rs["factor"]),
                low_freq_factor=float(rs["low_freq_factor"]),
                high_freq_factor=float(rs["high_freq_factor"]),
                original_max_position_embeddings=int(rs["original_max_position_embeddings"]))
        except KeyError as e:
            raise ConfigError(f"config.json: rope_scaling (llama3) lacks key {e}") from None

    def validate(self) -> None:
        if self.num_key_value_heads <= 0 or self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} must be a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim <= 0 or self.head_dim % 16 or self.head_dim > 256:
            # what the attention kernels take (csrc/attention.cu); refused here, when the
            # configuration is read, not at the first step
            raise ConfigError(f"head_dim {self.head_dim} must be a multiple of 16, at most 256")
        if self.rms_norm_eps <= 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.rope_theta <= 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        rs = self.rope_scaling
        if rs is not None:
            if rs.factor <= 0 or rs.high_freq_factor <= rs.low_freq_factor:
                raise ConfigError(
                    "rope_scaling (llama3) needs factor > 0 and high_freq_factor > low_freq_factor")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "hidden_act": "silu",
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
        }
        if self.rope_scaling is not None:
            rs = self.rope_scaling
            d["rope_scaling"] = {
                "rope_type": "llama3", "factor": rs.factor,
                "low_freq_factor": rs.low_freq_factor, "high_freq_factor": rs.high_freq_factor,
                "original_max_position_embeddings": rs.original_max_position_embeddings}
        if len(self.eos_token_ids) == 1:
            d["eos_token_id"] = self.eos_token_ids[0]
        elif self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # -------------------------------------------------------------- translation
    def to_model_spec(self) -> ModelSpec:
        """Every layer: RMSNorm -> GQA attention with rotary keys -> RMSNorm -> SwiGLU.

        Order inside a block and the tensor names are the reference's
        (llama_model.cpp:209-245, 502-655).
        """
        H, L = self.hidden_size, self.num_hidden_layers
        rotary = RotarySpec(head_dim=self.head_dim, rotary_dim=self.head_dim,
                            theta=self.rope_theta, scaling=self.rope_scaling)
        attention = AttentionSpec(
            hidden_size=H, num_heads=self.num_attention_heads,
            num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
            scale=1.0 / math.sqrt(self.head_dim),        # kernels/src/attention.cu:184
            window=None, position=rotary)
        mlp = GatedMLPSpec(hidden_size=H, intermediate_size=self.intermediate_size,
                           activation="silu")
        norm = RMSNormSpec(size=H, eps=self.rms_norm_eps)
        block = BlockSpec(mixer=attention, ffn=mlp, mixer_norm=norm, ffn_norm=norm)

        names = [("model.embed_tokens.weight", ("embedding", "weight")),
                 ("model.norm.weight", ("head.norm", "weight"))]
        if not self.tie_word_embeddings:
            names.append(("lm_head.weight", ("head", "weight")))
        for i in range(L):
            p = f"model.layers.{i}."
            names += [
                (p + "input_layernorm.weight", (f"blocks.{i}.mixer_norm", "weight")),
                (p + "post_attention_layernorm.weight", (f"blocks.{i}.ffn_norm", "weight")),
                (p + "self_attn.q_proj.weight", (f"blocks.{i}.mixer", "q_proj")),
                (p + "self_attn.k_proj.weight", (f"blocks.{i}.mixer", "k_proj")),
                (p + "self_attn.v_proj.weight", (f"blocks.{i}.mixer", "v_proj")),
                (p + "self_attn.o_proj.weight", (f"blocks.{i}.mixer", "o_proj")),
                (p + "mlp.gate_proj.weight", (f"blocks.{i}.ffn", "gate_proj")),
                (p + "mlp.up_proj.weight", (f"blocks.{i}.ffn", "up_proj")),
                (p + "mlp.down_proj.weight", (f"blocks.{i}.ffn", "down_proj")),
            ]
        return ModelSpec(
            architecture=self.architecture,
            embedding=EmbeddingSpec(vocab_size=self.vocab_size, hidden_size=H),
            blocks=tuple(block for _ in range(L)),
            order=tuple(LayerCall(block=i, cache=i) for i in range(L)),
            head=HeadSpec(vocab_size=self.vocab_size, hidden_size=H,
                          tied=self.tie_word_embeddings, norm=norm),
            tensor_names=tuple(names),
            # a tied checkpoint may still carry a copy of the table under lm_head
            ignorable=("lm_head.weight",) if self.tie_word_embeddings else (),
            stop_token_ids=self.eos_token_ids,
            max_position_embeddings=self.max_position_embeddings,
        )
