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
Mixer           ``cache_spec() -> CacheSpec | None`` (``PagedKVSpec``, ``StateSpec`` or a
                kind of the mixer's own) and
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
class CacheSpec:
    """What a mixer keeps between steps, as the cache manager sees it.

    A mixer returns one of these from ``cache_spec()`` (or ``None``).  The manager knows no
    cache kind by name: it asks the spec.  ``paged`` says whether the kind lives in pages that
    grow with the sequence (it then gets page ids through the block table of its group; kinds
    with the same ``window`` share a group, and a page id addresses one slot in the storage of
    every cache of the group) or in one row per request slot.  Another kind (pages of another
    shape, a compressed cache, a second state) is a subclass; nothing in the manager changes.

    ``allocate(rt, page_size, num_pages, slots)`` -> device storage, any object (``num_pages``
    is the group's pool size for paged kinds, ``None`` otherwise);
    ``view(storage, group)`` -> what the mixer's ``forward`` gets as ``cache`` (``group`` has
    ``dev_table`` int32 [slots, max_pages], ``window``, ``index`` and ``page_size`` for paged
    kinds; it is ``None`` otherwise);
    ``reset(storage, slot)`` is called when a request takes a slot;
    ``bytes_per_page(page_size, element_size)`` -> bytes one page id stands for in this cache.
    ``shareable``: full pages of this kind mean the same for every request with the same
    tokens before them, so a prefix tree may hand them to other requests.
    """

    paged = False
    shareable = False
    window: Optional[int] = None

    def allocate(self, rt, page_size: int, num_pages: Optional[int], slots: int):
        raise NotImplementedError

    def view(self, storage, group):
        raise NotImplementedError

    def reset(self, storage, slot: int) -> None:
        pass

    def bytes_per_page(self, page_size: int, element_size: int) -> int:
        return 0


@dataclass
class KVCacheView:
    """What an attention call sees of its cache."""

    k_pages: torch.Tensor          # [num_pages, kv_heads, page_size, head_dim]
    v_pages: torch.Tensor
    block_table: torch.Tensor      # int32 [slots, max_pages]; rows picked by ctx.table_rows
    page_size: int
    window: Optional[int]
    group: int


@dataclass
class StateView:
    """What a mixer with fixed-size state sees: ``state[ctx.table_rows[r]]`` is request r's."""

    state: torch.Tensor            # [slots, *shape]


@dataclass(frozen=True)
class PagedKVSpec(CacheSpec):
    """Keys and values of every past token (or of the last ``window`` tokens)."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    paged = True
    shareable = True

    def allocate(self, rt, page_size, num_pages, slots):
        shape = (num_pages, self.num_kv_heads, page_size, self.head_dim)
        return (torch.zeros(shape, dtype=rt.dtype, device=rt.device),
                torch.zeros(shape, dtype=rt.dtype, device=rt.device))

    def view(self, storage, group):
        return KVCacheView(storage[0], storage[1], group.dev_table, group.page_size, group.window,
                           group.index)

    def bytes_per_page(self, page_size, element_size):
        return 2 * self.num_kv_heads * page_size * self.head_dim * element_size


@dataclass(frozen=True)
class StateSpec(CacheSpec):
    """Per-request state of fixed size (one tensor of ``shape`` per request), zero when a
    request begins."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32

    def allocate(self, rt, page_size, num_pages, slots):
        return torch.zeros((slots,) + tuple(self.shape), dtype=self.dtype, device=rt.device)

    def view(self, storage, group):
        return StateView(storage)

    def reset(self, storage, slot):
        storage[slot].zero_()


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
    # ``replayable``: everything ``forward`` does on the device goes through the kernel entry points
    # (no tensor-library operations, no values read back), with the same launches for another part
    # of the same spec and the same step, so that a layer's launches can be recorded once and
    # repeated for the layers after it (``kernels.LayerRecording``).
    replayable = False
    # Folding a norm into the products on either side of it (a step of a few rows, where a norm's
    # own kernel costs more than the bytes it moves; ``ops.folds_norm`` says when).  A mixer or
    # feed-forward with ``folds_norm`` takes ``into=(residual, weight, eps)`` in ``forward``: its last
    # product adds its result to the residual stream and hands back what follows the norm with
    # that weight, an ``ops.NormOut``, as ``ops.linear`` does with the same argument.  One with
    # ``takes_unnormed`` accepts an ``ops.NormOut`` for ``x`` and passes it to its first product
    # (any other gets the finished rows).  A norm with ``foldable`` has ``fold() -> (weight, eps)``.
    # A block with ``folds_next`` takes ``next_norm`` in ``forward`` (the norm its output will meet
    # first) and tells through ``first_norm()`` which norm of its own the block before may fold.
    folds_norm = False
    takes_unnormed = False
    foldable = False
    folds_next = False

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
