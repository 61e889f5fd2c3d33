"""Interfaces of the parts a model is put together from, and their registries.

A part is built from its spec (``config.specs``) and a :class:`Runtime`; it
declares its parameters (name, shape, role), receives them once through
``load``, and exposes ``forward``.  Parts are looked up by ``spec.kind`` in one
registry per family, so a test or another architecture can add a mixer,
feed-forward, norm, position encoding or block arrangement without editing this
package: decorate the class with ``@register_mixer("kind")`` (and so on) and
name that kind in a spec.

Interfaces
----------
Norm            ``add_norm(residual, delta) -> normed``: ``residual += delta`` in
                place (fp32), returns ``norm(residual)`` in the compute dtype;
                ``delta`` may be ``None``.  ``gather_add_norm(residual, delta,
                rows)`` does the same for selected rows without touching
                ``residual``.
PositionEncoding ``rotary_table() -> (inv_freq, rotary_dim) | None`` for encodings
                that rotate q and k (fused with the cache write), and
                ``apply(q, k, ctx)`` for anything else.
Mixer           ``cache_spec() -> PagedKVSpec | StateSpec | None`` and
                ``forward(x, ctx, cache, writes_cache) -> delta``.
FeedForward     ``forward(x, ctx) -> delta``.
Block           ``forward(residual, pending, ctx, cache, writes_cache) -> pending``
                where ``pending`` is a delta not yet added to the residual stream.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch


# ------------------------------------------------------------------- parameters
@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part needs.

    role: ``matrix`` and ``table`` are matrix-product operands and live in the
    compute dtype; ``vector`` (norm weights and the like) is kept in 32-bit;
    ``int_table`` is kept as int32.
    init: ``normal`` -> N(0, std); ``ones`` -> 1 + N(0, noise).
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


# ------------------------------------------------------------------ cache needs
@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every past token (or of the last ``window`` tokens)."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size (one tensor of ``shape`` per request)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ---------------------------------------------------------------------- runtime
class Runtime:
    """What every part shares: device, compute dtype and the kernel library.

    ``ops`` is the module of kernel entry points (``llm_singularity_b200.kernels``
    in the product; the tests may hand in a stand-in to exercise host logic
    where no GPU exists).
    """

    def __init__(self, device, dtype: torch.dtype, ops=None, page_size: int = 16):
        self.device = torch.device(device)
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self._ops = ops
        self.page_size = page_size

    @property
    def ops(self):
        if self._ops is None:
            from .. import kernels
            self._ops = kernels
        return self._ops

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


class Part:
    """Base class: parameters in, ``forward`` out.

    ``graph_safe``: the part's ``forward`` launches the same kernels with the same arguments
    whatever the step's host-side values are (it reads lengths, positions and rows only on the
    device), so a decode step through it can be captured once in a CUDA graph and replayed.
    """

    graph_safe = False

    def __init__(self, spec, rt: Runtime):
        self.spec = spec
        self.rt = rt

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        return {}

    def children(self) -> Dict[str, "Part"]:
        """Sub-parts whose parameters are loaded under ``<name>.``."""
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive this part's own parameters (on device, dtype by role)."""
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no parameters, got {sorted(tensors)}")


# ------------------------------------------------------------------- registries
class _Registry:
    def __init__(self, family: str):
        self.family = family
        self._classes: Dict[str, Any] = {}

    def register(self, kind: str) -> Callable:
        def deco(cls):
            self._classes[kind] = cls
            return cls
        return deco

    def get(self, kind: str):
        try:
            return self._classes[kind]
        except KeyError:
            raise KeyError(f"no {self.family} of kind '{kind}' is registered "
                           f"(known: {', '.join(sorted(self._classes))})") from None

    def build(self, spec, rt: Runtime):
        return self.get(spec.kind)(spec, rt)


NORMS = _Registry("norm")
POSITIONS = _Registry("position encoding")
MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
BLOCKS = _Registry("block arrangement")

register_norm = NORMS.register
register_position = POSITIONS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_block = BLOCKS.register
