"""Typed descriptions of a model, one dataclass per kind of part.

An architecture's configuration (read from its own config.json keys) is
translated once into a :class:`ModelSpec`: a list of blocks, each naming its
mixer, feed-forward, norms and position encoding with every size and constant
as a field, plus the order in which the blocks run.  The parts are built from
these specs and never see the architecture's configuration, so no part knows
which model it is in, and two layers of one model may use different parts.

The reference has a single generic ``ModelConfig`` (models/include/models/
model_interface.h:11-23) and hard-wires one layer shape; the spec layer is
what replaces the ``-DMODEL=llama`` compile-time switch (CMakeLists.txt:12,27).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """Base of all part descriptions; ``kind`` selects the implementing class."""

    kind: str = field(init=False, default="")


# --------------------------------------------------------------------------- norms
@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    size: int = 0
    eps: float = 1e-5
    kind: str = field(init=False, default="rmsnorm")


# ---------------------------------------------------------------- position encodings
@dataclass(frozen=True)
class Llama3RopeScaling:
    """Frequency-dependent stretching of the rotary wavelengths ("llama3")."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotary position encoding with split-half pairing (i, i + rotary_dim/2)."""

    head_dim: int = 0
    rotary_dim: int = 0           # leading dims of each head that rotate
    theta: float = 10000.0
    scaling: Optional[Llama3RopeScaling] = None
    kind: str = field(init=False, default="rotary")


@dataclass(frozen=True)
class NoPositionSpec(PartSpec):
    kind: str = field(init=False, default="none")


# --------------------------------------------------------------------------- mixers
@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Causal softmax attention with grouped keys/values over a paged cache."""

    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0            # multiplies q.k before the softmax
    window: Optional[int] = None  # keys further back than this many are not seen
    position: PartSpec = field(default_factory=NoPositionSpec)
    # score modifiers (this architecture has neither): cap * tanh(s / cap) on the scaled scores, and
    # a linear position bias -slope[h] * distance with the usual geometric slopes over the heads
    logit_softcap: Optional[float] = None
    linear_bias: bool = False
    kind: str = field(init=False, default="attention")


# -------------------------------------------------------------------- feed-forwards
@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """down( act(gate(x)) * up(x) ), dense, no bias."""

    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    kind: str = field(init=False, default="gated_mlp")


# --------------------------------------------------------------------------- blocks
@dataclass(frozen=True)
class BlockSpec(PartSpec):
    """x += mixer(norm1(x)); x += ffn(norm2(x))   (the "pre_norm" arrangement)."""

    mixer: PartSpec = None
    ffn: PartSpec = None
    mixer_norm: PartSpec = None
    ffn_norm: PartSpec = None
    kind: str = field(init=False, default="pre_norm")


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``block`` indexes ``ModelSpec.blocks``; a block may be named more than once.
    ``cache`` is the id of the cache (pages or state) the mixer uses in this
    call, ``writes_cache`` says whether the call appends this step's tokens to
    it or only reads what an earlier call of the same step wrote (a layer that
    reads another layer's keys and values).
    """

    block: int
    cache: int
    writes_cache: bool = True


# ---------------------------------------------------------------------------- model
@dataclass(frozen=True)
class EmbeddingSpec(PartSpec):
    vocab_size: int = 0
    hidden_size: int = 0
    kind: str = field(init=False, default="embedding")


@dataclass(frozen=True)
class HeadSpec(PartSpec):
    """Final norm followed by the projection to the vocabulary."""

    vocab_size: int = 0
    hidden_size: int = 0
    tied: bool = False            # reuse the embedding table as the projection
    norm: PartSpec = None
    kind: str = field(init=False, default="lm_head")


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    embedding: EmbeddingSpec
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[LayerCall, ...]
    head: HeadSpec
    # checkpoint tensor name -> (owner path, local parameter name); owner paths are
    # "embedding", "head", "head.norm", "blocks.<i>.mixer", "blocks.<i>.ffn",
    # "blocks.<i>.mixer_norm", "blocks.<i>.ffn_norm".
    tensor_names: Tuple[Tuple[str, Tuple[str, str]], ...]
    # names that may be present in a checkpoint and are skipped without complaint
    ignorable: Tuple[str, ...] = ()
    stop_token_ids: Tuple[int, ...] = ()
    max_position_embeddings: int = 0

    @property
    def num_caches(self) -> int:
        return 1 + max((c.cache for c in self.order), default=-1)
