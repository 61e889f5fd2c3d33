"""Parts a model is assembled from: norms, position encodings, mixers,
feed-forwards and block arrangements, each chosen by the ``kind`` of its spec."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, CacheSpec, KVCacheView,
                   PagedKVSpec, ParamSpec, Part, Runtime, StateSpec, StateView, register_block, register_feed_forward,
                   register_mixer, register_norm, register_position)
from . import attention, block, embedding, mlp, norm, rotary  # noqa: F401  (registration)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "CacheSpec", "KVCacheView",
           "PagedKVSpec", "ParamSpec", "Part", "Runtime", "StateSpec", "StateView", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_position"]
