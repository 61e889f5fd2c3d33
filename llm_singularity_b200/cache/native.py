"""Loading the host runtime (``csrc/host_memory.cpp``: pools, block tables, slots, prefix tree;
``csrc/host_scheduler.cpp``: the scheduler; ``csrc/host_step.cpp``: a step's metadata packed into
one buffer) and declaring its C interface.

The library is host code only; it is compiled at first use like the CUDA libraries and needs no
GPU to run, so the cache manager and the scheduler can be exercised anywhere.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int32, c_longlong, c_void_p
from typing import Optional

import numpy as np

from ..kernels import build as _build

ERR = -1000                      # what a failed call returns; the message is in lsbm_last_error
_IP = POINTER(c_int)

_SIGNATURES = {
    "lsbm_create": (c_void_p, [c_int, c_int, c_int, c_int, _IP, _IP]),
    "lsbm_destroy": (None, [c_void_p]),
    "lsbm_last_error": (c_char_p, [c_void_p]),
    "lsbm_pool_allocate": (c_int, [c_void_p, c_int]),
    "lsbm_pool_retain": (c_int, [c_void_p, c_int, c_int]),
    "lsbm_pool_release": (c_int, [c_void_p, c_int, c_int]),
    "lsbm_pool_refcount": (c_int, [c_void_p, c_int, c_int]),
    "lsbm_pool_num_free": (c_int, [c_void_p, c_int]),
    "lsbm_pool_num_pages": (c_int, [c_void_p, c_int]),
    "lsbm_pool_check": (c_int, [c_void_p, c_int]),
    "lsbm_open": (c_int, [c_void_p]),
    "lsbm_close": (c_int, [c_void_p, c_int]),
    "lsbm_length": (c_longlong, [c_void_p, c_int]),
    "lsbm_num_pages": (c_int, [c_void_p, c_int]),
    "lsbm_first_live": (c_int, [c_void_p, c_int, c_int]),
    "lsbm_free_pages": (c_int, [c_void_p]),
    "lsbm_reserve": (c_int, [c_void_p, c_int, c_longlong]),
    "lsbm_commit": (c_int, [c_void_p, c_int, c_longlong]),
    "lsbm_adopt": (c_int, [c_void_p, c_int, _IP, c_int, c_longlong]),
    "lsbm_pages_of": (c_int, [c_void_p, c_int, c_int, _IP, c_int]),
    "lsbm_table": (POINTER(c_int32), [c_void_p, c_int]),
    "lsbm_num_updates": (c_int, [c_void_p, c_int]),
    "lsbm_take_updates": (c_int, [c_void_p, c_int, _IP, c_int]),
    "lsbm_take_updates_last": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int]),
    "lsbm_check": (c_int, [c_void_p]),
    "lsbh_pack_step": (c_longlong, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_longlong, c_void_p, c_void_p]),
    "lsbp_enable": (c_int, [c_void_p]),
    "lsbp_match": (c_int, [c_void_p, _IP, c_longlong, _IP, c_int]),
    "lsbp_adopt": (c_longlong, [c_void_p, c_int, _IP, c_int]),
    "lsbp_release": (c_int, [c_void_p, _IP, c_int]),
    "lsbp_insert": (c_int, [c_void_p, _IP, c_longlong, c_int]),
    "lsbp_share": (c_int, [c_void_p, _IP, c_longlong, c_int, _IP, c_int, _IP, c_int]),
    "lsbp_evictable": (c_int, [c_void_p]),
    "lsbp_num_nodes": (c_int, [c_void_p]),
    "lsbp_hits": (c_longlong, [c_void_p]),
    "lsbp_evict": (c_int, [c_void_p, c_int]),
    "lsbp_node_users": (c_int, [c_void_p, c_int]),
    "lsbp_node_pages": (c_int, [c_void_p, c_int, _IP]),
    "lsbp_idle_on": (c_int, [c_void_p, _IP, c_int]),
    "lsbs_create": (c_void_p, [c_void_p, c_int, c_int, c_int, c_int, _IP, c_int, c_longlong]),
    "lsbs_destroy": (None, [c_void_p]),
    "lsbs_set_stop_ids": (None, [c_void_p, _IP, c_int]),
    "lsbs_last_error": (c_char_p, [c_void_p]),
    "lsbs_add": (c_int, [c_void_p, _IP, c_longlong, c_int, c_int, c_int]),
    "lsbs_forget": (c_int, [c_void_p, c_int]),
    "lsbs_has_work": (c_int, [c_void_p]),
    "lsbs_plans_in_flight": (c_int, [c_void_p]),
    "lsbs_plan": (c_int, [c_void_p, c_int]),
    "lsbs_update": (c_int, [c_void_p, _IP, _IP, c_int]),
    "lsbs_num_events": (c_int, [c_void_p]),
    "lsbs_events": (c_int, [c_void_p, POINTER(c_longlong), c_int]),
    "lsbs_request_error": (c_char_p, [c_void_p, c_int]),
    "lsbs_request_slot": (c_int, [c_void_p, c_int]),
    "lsbs_request_state": (c_int, [c_void_p, c_int, POINTER(c_longlong)]),
    "lsbs_request_tokens": (c_int, [c_void_p, c_int, _IP, c_longlong]),
    "lsbs_stats": (c_int, [c_void_p, POINTER(c_longlong)]),
}

_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    """The loaded library; compiled first if its current build is absent."""
    global _lib
    if _lib is None:
        path = _build.ensure_built(["host_runtime"])["host_runtime"]
        try:
            loaded = ctypes.CDLL(path)
        except OSError as e:
            raise RuntimeError(f"cannot load the host runtime from {path}: {e}") from None
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(loaded, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = loaded
    return _lib


def ints(values) -> ctypes.Array:
    """A C int array holding ``values`` (any sequence of Python ints)."""
    return (c_int * len(values))(*values)


def token_array(tokens):
    """(keep-alive array, C pointer) for a sequence of token ids."""
    a = np.ascontiguousarray(tokens, dtype=np.int32)
    return a, a.ctypes.data_as(_IP)
