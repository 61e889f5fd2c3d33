"""Kernel entry points: checked Python wrappers over the compiled sm_100a libraries.

Every function here launches hand-written CUDA on the current stream of its
tensors' device.  There is no CPU path and no fallback: a tensor that is not on
a CUDA device, or a library that cannot be compiled or loaded, raises.  Shapes,
dtypes, contiguity and size limits are checked here, before the launch, so that
a size a kernel does not take is refused with a message and never computed
wrongly.
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Dict, Iterable, Optional

import torch

from . import build as _build

_libs: Dict[str, ctypes.CDLL] = {}

_F32, _BF16 = 0, 1
_STATUS_TEXT = {
    1: "a block-table entry outside the page pool was met (page not held by the request)",
    2: "a token id outside the vocabulary was met",
    3: "a row index outside its tensor was met",
    4: "a bounded wait inside a kernel ran out",
}


class KernelError(RuntimeError):
    pass


# ------------------------------------------------------------------ loading
def prepare(names: Iterable[str], verbose: bool = False) -> None:
    """Compile (if needed) and load the named libraries; raises if that is impossible."""
    names = [n for n in dict.fromkeys(names) if n not in _libs]
    if not names:
        return
    paths = _build.ensure_built(names, verbose=verbose)
    for n in names:
        try:
            _libs[n] = ctypes.CDLL(paths[n])
        except OSError as e:
            raise KernelError(f"cannot load kernel library '{n}' from {paths[n]}: {e}") from None
        _libs[n].lsb_error_string.restype = ctypes.c_char_p


def loaded_libraries() -> Dict[str, str]:
    return {n: lib._name for n, lib in _libs.items()}


def _lib(name: str) -> ctypes.CDLL:
    if name not in _libs:
        prepare([name])
    return _libs[name]


def check_status() -> None:
    """Read (and clear) every loaded library's status word; raises if a kernel recorded a fault.
    Synchronises the device."""
    for n, lib in _libs.items():
        code = ctypes.c_int(0)
        rc = lib.lsb_take_status(ctypes.byref(code))
        if rc != 0:
            raise KernelError(f"{n}: reading the status word failed: "
                              f"{lib.lsb_error_string(rc).decode()}")
        if code.value != 0:
            raise KernelError(f"{n}: {_STATUS_TEXT.get(code.value, f'status {code.value}')}")


_launches = 0
_scratch: Dict[tuple, torch.Tensor] = {}      # scratch buffers by use and size, kept for reuse


def launch_count() -> int:
    """How many kernel launches this process has made through this module."""
    return _launches


def _call(libname: str, fn: str, *args) -> None:
    global _launches
    lib = _lib(libname)
    _launches += 1
    cfn = getattr(lib, fn)
    rc = cfn(*args)
    if rc != 0:
        raise KernelError(f"{fn} failed: {lib.lsb_error_string(rc).decode()} (code {rc})")
    if _recording is not None:
        _recording.ops.append([cfn, list(args), fn, lib, ()])


# ------------------------------------------------------ a layer's launches, recorded
# The layers of a model are the same sequence of launches with other weights.  What the host does
# per launch (checks, choosing a kernel, sizing grids, allocating the output) is the same work for
# every layer of a step, and in steps that hold prompt portions (launched kernel by kernel, unlike
# decode steps, which replay a captured graph) it is most of the host's time.  So the model records
# the launches of one layer call and repeats them for the calls after it that have the same shape,
# with the pointers of that layer's own tensors (weights, cache pages, the delta coming in and
# going out) exchanged for the next layer's; every other buffer is the recorded layer's, reused in
# stream order.
LAYER_REPLAY = True
_recording: Optional["LayerRecording"] = None


class LayerRecording:
    """The launches of one layer call: C entry points with their packed arguments and, between
    them, stream operations (the second stream of steps that hold decode tokens and portions)."""

    def __init__(self):
        self.ops = []          # [cfunction, args, name, lib, slots] or a callable (a stream operation)
        self.keep = []         # tensors whose memory the recorded launches use
        self._before = None

    def __enter__(self):
        global _recording
        self._before, _recording = _recording, self
        return self

    def __exit__(self, *exc):
        global _recording
        _recording = self._before
        return False

    def bind(self, roles: Dict[int, object]) -> None:
        """``roles``: device address -> name, for every tensor that is the recorded layer's own.
        Arguments that hold such an address become slots that :meth:`replay` fills."""
        for op in self.ops:
            if not callable(op):
                op[4] = tuple((i, roles[a.value]) for i, a in enumerate(op[1])
                              if isinstance(a, ctypes.c_void_p) and a.value in roles)

    def replay(self, addresses: Dict[object, int]) -> None:
        """Launch everything again with the slots pointing at ``addresses[name]``."""
        global _launches
        for op in self.ops:
            if callable(op):
                op()
                continue
            cfn, args, name, lib, slots = op
            for i, role in slots:
                args[i] = ctypes.c_void_p(addresses[role])
            _launches += 1
            rc = cfn(*args)
            if rc != 0:
                raise KernelError(f"{name} failed: {lib.lsb_error_string(rc).decode()} (code {rc})")


def _stream_op(fn) -> None:
    """Do a stream or event operation now and, when a layer is being recorded, again at every replay."""
    fn()
    if _recording is not None:
        _recording.ops.append(fn)


# ------------------------------------------------------------------- helpers
def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _req(t: torch.Tensor, name: str, dtype=None, dim: Optional[int] = None, contiguous=True):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name} must have {dim} dims, got shape {tuple(t.shape)}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


def _p(t: Optional[torch.Tensor]):
    if _recording is not None and t is not None:
        _recording.keep.append(t)
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = torch._C._cuda_getCurrentRawStream      # (device index) -> cudaStream_t as int


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(_raw_stream(t.device.index))


_i = ctypes.c_int
_ll = ctypes.c_longlong
_f = ctypes.c_float


# ---------------------------------------------------------------------- ops
def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor) -> None:
    """dst.flat[idx[i]] = val[i]."""
    _req(dst, "dst", torch.int32)
    _req(idx, "idx", torch.int32, 1)
    _req(val, "val", torch.int32, 1)
    if idx.numel() != val.numel():
        raise KernelError("scatter_i32: idx and val differ in length")
    _call("cache_table", "lsb_scatter_i32", _p(dst), _p(idx), _p(val), _i(idx.numel()),
          _ll(dst.numel()), _stream(dst))


def move_i32(dst: torch.Tensor, dst_idx: torch.Tensor, src: torch.Tensor, src_idx: torch.Tensor) -> None:
    """dst[dst_idx[i]] = src[src_idx[i]]."""
    for name, t in (("dst", dst), ("dst_idx", dst_idx), ("src", src), ("src_idx", src_idx)):
        _req(t, name, torch.int32, 1)
    if dst_idx.numel() != src_idx.numel():
        raise KernelError("move_i32: dst_idx and src_idx differ in length")
    _call("cache_table", "lsb_move_i32", _p(dst), _p(dst_idx), _p(src), _p(src_idx), _i(dst_idx.numel()),
          _ll(dst.numel()), _ll(src.numel()), _stream(dst))


def scatter_i32_counted(dst: torch.Tensor, packed: torch.Tensor, cap: int) -> None:
    """dst.flat[idx[i]] = val[i] for i < n, with packed = [n, idx[cap], val[cap]] on the device."""
    _req(dst, "dst", torch.int32)
    _req(packed, "packed", torch.int32, 1)
    if packed.numel() != 1 + 2 * cap:
        raise KernelError("scatter_i32_counted: packed must hold 1 + 2 * cap ints")
    _call("cache_table", "lsb_scatter_i32_counted", _p(dst), _p(packed), _i(cap), _ll(dst.numel()),
          _stream(dst))


def random_normal(out: torch.Tensor, key: int, mean: float, scale: float) -> None:
    """out.flat[i] = mean + scale * normal(key, i): the counter-based stream of the random-weights
    mode (``weights/random_init.py`` states the same arithmetic for the CPU)."""
    _req(out, "out")
    _call("random_init", "lsb_random_normal", _p(out), _i(_dt(out)), _ll(out.numel()),
          ctypes.c_ulonglong(key & ((1 << 64) - 1)), _f(mean), _f(scale), _stream(out))


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] = float(table[ids[t], :])."""
    _req(table, "table", dim=2)
    _req(ids, "ids", torch.int32, 1)
    _req(out, "out", torch.float32, 2)
    if out.shape != (ids.shape[0], table.shape[1]):
        raise KernelError(f"embedding: out is {tuple(out.shape)}, expected "
                          f"{(ids.shape[0], table.shape[1])}")
    _call("embedding", "lsb_embedding", _p(table), _i(_dt(table)), _p(ids), _p(out),
          _i(ids.shape[0]), _i(table.shape[1]), _i(table.shape[0]), _stream(out))


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: torch.Tensor) -> None:
    """residual += delta (in place, 32-bit); out = rmsnorm(residual) * weight."""
    _req(residual, "residual", torch.float32, 2)
    _req(weight, "weight", torch.float32, 1)
    _req(out, "out", dim=2)
    T, H = residual.shape
    if out.shape != (T, H) or weight.shape[0] != H:
        raise KernelError("add_rmsnorm: shapes of residual, weight and out disagree")
    if delta is not None:
        _req(delta, "delta", out.dtype, 2)
        if delta.shape != (T, H):
            raise KernelError("add_rmsnorm: delta has another shape than residual")
    _call("norm", "lsb_add_rmsnorm", _p(residual), _p(delta), _p(weight), _p(out), _i(_dt(out)),
          _i(T), _i(H), _f(eps), _stream(out))


def gather_add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor,
                       weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[i] = rmsnorm(residual[rows[i]] + delta[rows[i]]) * weight; residual unchanged."""
    _req(residual, "residual", torch.float32, 2)
    _req(rows, "rows", torch.int32, 1)
    _req(weight, "weight", torch.float32, 1)
    _req(out, "out", dim=2)
    T, H = residual.shape
    if out.shape != (rows.shape[0], H) or weight.shape[0] != H:
        raise KernelError("gather_add_rmsnorm: shapes disagree")
    if delta is not None:
        _req(delta, "delta", out.dtype, 2)
        if delta.shape != (T, H):
            raise KernelError("gather_add_rmsnorm: delta has another shape than residual")
    _call("norm", "lsb_gather_add_rmsnorm", _p(residual), _p(delta), _p(rows), _p(weight), _p(out),
          _i(_dt(out)), _i(rows.shape[0]), _i(T), _i(H), _f(eps), _stream(out))


ACTIVATIONS = {"silu": 1, "gelu_tanh": 2, "none": 3}     # act(gate) * up of a gated product


def _activation_id(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation '{name}' is not implemented "
                          f"(known: {', '.join(sorted(ACTIVATIONS))})") from None


class NormOut:
    """Rows as they leave an RMS norm that a product folded in.  ``values`` [M, H] is the residual
    row times the norm's weight, rounded to the compute dtype; ``parts`` [P, 16] holds each row's
    sum of squares in P parts (row m in column m), and the factor ``rsqrt(sum / H + eps)`` per row
    is still owed: the next product scales its output rows by it (``linear`` takes a NormOut for
    ``x``), which is the same as normalising first.  ``parts`` None: nothing is owed, ``values``
    are the normalised rows (where no kernel could fold the norm).  ``finish_norm`` gives the
    normalised rows in either case."""
    __slots__ = ("values", "parts", "eps")

    def __init__(self, values: torch.Tensor, parts: Optional[torch.Tensor] = None, eps: float = 0.0):
        self.values, self.parts, self.eps = values, parts, float(eps)

    shape = property(lambda self: self.values.shape)
    dtype = property(lambda self: self.values.dtype)
    device = property(lambda self: self.values.device)


FOLD_NORMS = True               # decode steps fold each norm into the products on either side of it

# Warming.  A streaming product (csrc/gemm_stream.cu) can ask L2, while it ends, for the first
# weights of the streaming product after it, so that HBM works through the gap between the two
# kernels (csrc/stream_warm.cuh).  Which product comes next is not something a part knows; it is
# learnt here: the matrix that followed a matrix the last time is expected to follow it again,
# which holds from a model's second step on (and a decode step runs once before it is captured in
# a graph).  A wrong guess costs a few prefetched bytes; nothing depends on it.  Any other product
# in between (more than 16 rows, the output head) ends the chain.
WARM_NEXT = True
_follows: Dict[int, tuple] = {}         # address of a matrix -> (weak reference to its follower, gated)
_warm_structs: Dict[tuple, object] = {}  # (address, rows, gated) -> (weak reference, filled-in StreamWarm)
_last_streamed: Optional[int] = None


def _warm_after(w: torch.Tensor, gated: bool, M: int):
    """Note that ``w`` is being streamed now; the StreamWarm for what followed it last time, or None."""
    global _last_streamed
    if not WARM_NEXT:
        return None
    here = w.data_ptr()
    if _last_streamed is not None and _last_streamed != here:
        _follows[_last_streamed] = (weakref.ref(w), gated)
    _last_streamed = here
    nxt = _follows.get(here)
    if nxt is None:
        return None
    t = nxt[0]()
    if t is None:
        del _follows[here]
        return None
    key = (t.data_ptr(), M, nxt[1])
    made = _warm_structs.get(key)
    if made is None or made[0]() is not t:
        lib = _lib("gemm_stream")
        buf = ctypes.create_string_buffer(lib.lsb_stream_warm_bytes())
        rc = lib.lsb_gemm_stream_warm(_p(t), _i(M), _i(t.shape[0]), _i(t.shape[1]),
                                      _i(ACTIVATIONS["silu"] if nxt[1] else 0), _i(0), buf)
        made = _warm_structs[key] = (weakref.ref(t), buf if rc == 0 else None)
    return made[1]


def _chain_ends() -> None:
    global _last_streamed
    _last_streamed = None


def folds_norm(rows: int, dtype: torch.dtype) -> bool:
    """Does a step of this many rows fold its norms into the neighbouring products?  (The products
    of at most 16 bfloat16 rows, which one kernel streams: there a norm's own kernel costs more
    than the bytes it moves.)"""
    return FOLD_NORMS and STREAM_PRODUCTS and dtype == torch.bfloat16 and 0 < rows <= 16


def finish_norm(x: NormOut) -> torch.Tensor:
    """The normalised rows a NormOut stands for."""
    if x.parts is None:
        return x.values
    M, H = x.values.shape
    out = torch.empty_like(x.values)
    _call("norm", "lsb_finish_norm", _p(x.values), _p(x.parts), _i(x.parts.shape[0]), _p(out), _i(_dt(out)),
          _i(M), _i(H), _f(x.eps), _stream(out))
    return out


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           gated: bool = False, activation: str = "silu", into=None):
    """x [M, K] times w [N, K] transposed -> [M, N]; 32-bit accumulation.

    ``x`` may be a ``NormOut`` (the norm before this product, possibly half done: see there).
    ``into = (residual, norm_weight, eps)``: the product is added to ``residual`` ([M, N] 32-bit, in
    place) and what comes back is a ``NormOut``: what follows the RMS norm with that weight.

    float32 operands run on the CUDA cores in true 32-bit.  bfloat16 operands run on the
    tensor cores (tcgen05, accumulators in TMEM) when K is a multiple of 8, else on the CUDA
    cores as well.

    ``gated``: the rows of ``w`` alternate gate_i, up_i and the result is [M, N / 2] with
    ``out[m, i] = act(d[m, 2i]) * d[m, 2i + 1]`` (applied in the product's epilogue on the
    tensor-core path, by the activation kernel otherwise); ``activation`` names act: "silu",
    "gelu_tanh" or "none".
    """
    act = _activation_id(activation) if gated else 0
    owed = None
    if isinstance(x, NormOut):
        owed, x = (x if x.parts is not None else None), x.values
    _req(x, "x", dim=2)
    _req(w, "w", x.dtype, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    if gated and N % 2:
        raise KernelError("linear: a gated product needs an even number of weight rows")
    out_dtype = out_dtype or x.dtype
    if out_dtype not in (x.dtype, torch.float32):
        raise KernelError(f"linear: output must be {x.dtype} or float32")
    if into is not None:
        residual, norm_w, eps = into
        if gated or out_dtype != x.dtype:
            raise KernelError("linear: a product into the residual is plain and in the compute dtype")
        _req(residual, "residual", torch.float32, 2)
        _req(norm_w, "norm weight", torch.float32, 1)
        if residual.shape != (M, N) or norm_w.shape[0] != N:
            raise KernelError("linear: residual and norm weight do not fit the product")
    if (owed is not None or into is not None) and x.dtype == torch.bfloat16 and STREAM_PRODUCTS \
            and M <= 16 and stream_gemm_ok(x, w, act):
        lib = _lib("gemm_stream")
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
        parts = None
        if into is not None:
            parts = torch.empty((lib.lsb_gemm_stream_blocks(_i(M), _i(N), _i(K), _i(act)), 16),
                                dtype=torch.float32, device=x.device)
        _call("gemm_stream", "lsb_gemm_stream_folded", _p(x), _p(w), _p(out),
              _i(1 if out_dtype == torch.float32 else 0), _i(M), _i(N), _i(K), _i(act),
              _p(owed.parts if owed is not None else None), _i(owed.parts.shape[0] if owed is not None else 0),
              _i(K), _f(owed.eps if owed is not None else 0.0),
              _p(into[0] if into is not None else None), _p(into[1] if into is not None else None), _p(parts),
              _warm_after(w, gated, M), _stream(out))
        return NormOut(out, parts, into[2]) if into is not None else out
    if owed is not None:
        x = finish_norm(owed)
    if into is not None:
        delta = linear(x, w, out_dtype)
        out = torch.empty_like(delta)
        add_rmsnorm(into[0], delta, into[1], into[2], out)
        return NormOut(out)
    if x.dtype == torch.bfloat16 and SMALL_PRODUCTS and not gated and M <= 16 and small_gemm_ok(x, w):
        # a few rows times a matrix that fits the chip's shared memory (decode: q/k/v, output
        # projection): weights resident before the previous kernel has ended, no cluster
        _chain_ends()
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        _call("gemm_small", "lsb_gemm_small", _p(x), _p(w), _p(out), _i(1 if out_dtype == torch.float32 else 0),
              _i(M), _i(N), _i(K), _stream(out))
        return out
    if x.dtype == torch.bfloat16 and STREAM_PRODUCTS and M <= 16 and stream_gemm_ok(x, w, act):
        # a few rows times a matrix of any size (decode: gate/up, down): every SM streams its own
        # share of the weight rows, the first chunks before the previous kernel has ended
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
        _call("gemm_stream", "lsb_gemm_stream_folded", _p(x), _p(w), _p(out),
              _i(1 if out_dtype == torch.float32 else 0), _i(M), _i(N), _i(K), _i(act), _p(None), _i(0), _i(K),
              _f(0.0), _p(None), _p(None), _p(None), _warm_after(w, gated, M), _stream(out))
        return out
    _chain_ends()
    if x.dtype == torch.bfloat16 and tensor_core_gemm_ok(x, w):
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
        _call("gemm_tc", "lsb_gemm_tc", _p(x), _p(w), _p(out), _i(1 if out_dtype == torch.float32 else 0),
              _i(M), _i(N), _i(K), _i(act), _stream(out))
        return out
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _call("gemm", "lsb_gemm_nt", _p(x), _p(w), _p(out), _i(_dt(x)), _i(_dt(out)), _i(M), _i(N), _i(K),
          _ll(K), _ll(K), _ll(N), _stream(out))
    if gated:
        half = torch.empty((M, N // 2), dtype=out_dtype, device=x.device)
        gated_activation(out, half, activation)
        return half
    return out


SMALL_PRODUCTS = True           # products of at most 16 rows with a small matrix: csrc/gemm_small.cu
STREAM_PRODUCTS = True          # products of at most 16 rows with any matrix: csrc/gemm_stream.cu
STREAM_MAX_ROWS = 65536         # weight rows beyond which the tile kernel's persistent form is used


def stream_gemm_ok(x: torch.Tensor, w: torch.Tensor, act: int = 0) -> bool:
    """Does the streaming kernel take x [M, K] times w [N, K] transposed?  (bfloat16, M <= 16, K a
    multiple of 64; the output head, far more rows than the SMs can share out in a few passes,
    stays with the persistent tile kernel.)"""
    M, K = x.shape
    N = w.shape[0]
    if M > 16 or K % 64 or N > STREAM_MAX_ROWS:
        return False
    return bool(_lib("gemm_stream").lsb_gemm_stream_supported(_p(x), _p(w), _i(M), _i(N), _i(K), _i(act)))



def small_gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Does the small-product kernel take x [M, K] times w [N, K] transposed?  (bfloat16, M <= 16,
    K a multiple of 64, N / SMs rows of w and the rows of x within one block's shared memory.)"""
    M, K = x.shape
    N = w.shape[0]
    per_sm = -(-N // num_sms(x.device))
    if M > 16 or K % 64 or per_sm > 32 or (per_sm + 16) * K * 2 > 180 * 1024:
        return False                                  # cheap refusals first; the library has the last word
    return bool(_lib("gemm_small").lsb_gemm_small_supported(_p(x), _p(w), _i(M), _i(N), _i(K)))


def tensor_core_gemm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """TMA needs 16-byte aligned bases and row strides: K a multiple of 8 for bfloat16."""
    return (x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gated_activation(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[t, i] = act(gate_up[t, 2i]) * gate_up[t, 2i + 1] (gate and up alternate)."""
    _req(gate_up, "gate_up", dim=2)
    _req(out, "out", gate_up.dtype, 2)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError(f"gated_activation: gate_up is {tuple(gate_up.shape)}, out is {tuple(out.shape)}")
    _call("activation", "lsb_gated_act", _p(gate_up), _p(out), _i(_dt(out)), _i(T), _i(I),
          _i(_activation_id(activation)), _stream(out))


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, 2i]) * gate_up[t, 2i + 1]."""
    gated_activation(gate_up, out, "silu")


def _check_cache(cache, nkv: int, hd: int, dtype) -> None:
    for name in ("k_pages", "v_pages"):
        t = _req(getattr(cache, name), name, dtype, 4)
        if t.shape[1:] != (nkv, cache.page_size, hd):
            raise KernelError(f"{name} is {tuple(t.shape)}, expected [pages, {nkv}, "
                              f"{cache.page_size}, {hd}]")
    _req(cache.block_table, "block_table", torch.int32, 2)


def rope_kv_store(qkv: torch.Tensor, nh: int, nkv: int, hd: int, ctx, cache,
                  inv_freq: Optional[torch.Tensor], rotary_dim: int, store: bool = True,
                  skip_single: bool = False) -> None:
    """Rotate queries and keys of the fused projection in place and write keys and values
    of this step's tokens into their cache pages.  ``skip_single`` leaves the tokens of requests
    that bring one token alone (their attention kernel does the same work itself)."""
    _req(qkv, "qkv", dim=2)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise KernelError(f"qkv is {tuple(qkv.shape)}, expected [T, {(nh + 2 * nkv) * hd}]")
    if hd % 2 or rotary_dim % 2 or rotary_dim > hd:
        raise KernelError(f"rope: head_dim {hd} and rotary_dim {rotary_dim} must be even, "
                          f"rotary_dim <= head_dim")
    if rotary_dim:
        _req(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rotary_dim // 2:
            raise KernelError("inv_freq must have rotary_dim / 2 entries")
    _check_cache(cache, nkv, hd, qkv.dtype)
    if ctx.n_tokens != T:
        raise KernelError(f"qkv has {T} rows, the step has {ctx.n_tokens} tokens")
    _call("rope_cache", "lsb_rope_kv_store", _p(qkv), _i(_dt(qkv)), _i(T), _i(nh), _i(nkv), _i(hd),
          _p(ctx.positions), _p(ctx.token_req), _p(ctx.table_rows), _p(cache.block_table),
          _i(cache.block_table.shape[1]), _p(inv_freq if rotary_dim else None), _i(rotary_dim),
          _p(cache.k_pages), _p(cache.v_pages), _i(cache.page_size), _i(cache.k_pages.shape[0]),
          _i(1 if store else 0), _p(ctx.q_start if skip_single else None), _stream(qkv))


_sm_counts: Dict[int, int] = {}


def num_sms(device=None) -> int:
    """Streaming multiprocessors of ``device`` (the current one by default), asked once."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


USE_TCGEN05_ATTENTION = True    # prompt portions of 128 tokens and more
FUSE_DECODE_ROPE = True         # single tokens: rotation and cache write inside the decode kernel
_TC_HEAD_DIMS = (64, 128)


_decode_occupancy: Dict[tuple, int] = {}


def decode_splits(n_decode: int, nkv: int, device=None, hd: int = 64, group: int = 4) -> int:
    """How many ways each request's keys are split among thread blocks in the decode kernel: as many
    as fill four fifths of the blocks the SMs hold at once (four an SM at head size 64, two at 128,
    where a block has twice the registers and shared memory), never a second round of blocks.
    Measured inside decode steps at context 4096: head size 64, 8 requests: 7 splits (6: 1 % slower,
    9: 10 %); 32 requests: 2 (1: 14 % slower, 3: 10 %); head size 128, 8 requests: 4 or 5 splits 27 -
    28 us a layer, 7 splits (a second round for four blocks) 42 us; 32 requests: 1 split 84 us, 2
    splits 108 us.  A function of the batch alone, so that a captured launch stays valid as
    sequences grow."""
    key = (hd, group)
    if key not in _decode_occupancy:
        fits = 4
        if hd in _TC_HEAD_DIMS:
            fits = int(_lib("attention_tc").lsb_decode_blocks_per_sm(_i(hd), _i(group)))
        _decode_occupancy[key] = max(1, fits)
    room = _decode_occupancy[key] * num_sms(device)
    return max(1, min(32, int(0.8 * room / max(1, n_decode * nkv) + 0.5)))


_cluster_caps: Dict[int, int] = {}


def _decode_cluster_cap(hd: int) -> int:
    """The largest thread-block cluster the decode kernel can be launched with here (8 or 16)."""
    if hd not in _cluster_caps:
        _cluster_caps[hd] = int(_lib("attention_tc").lsb_decode_max_cluster(_i(hd)))
    return _cluster_caps[hd]


def tensor_core_attention_ok(dtype, hd: int, nh: int, nkv: int) -> bool:
    return dtype == torch.bfloat16 and hd in _TC_HEAD_DIMS and nh // nkv <= 16


OVERLAP_ATTENTION = True        # decode kernel beside the prompt kernels in steps that hold both
_side: Dict[torch.device, tuple] = {}


def _fork_join(ctx, device):
    """(the step's stream, a second stream, two events), looked up once per step."""
    got = getattr(ctx, "_fork_join", None)
    if got is None:
        if device not in _side:
            _side[device] = (torch.cuda.Stream(device), torch.cuda.Event(), torch.cuda.Event())
        got = ctx._fork_join = (torch.cuda.current_stream(device),) + _side[device]
    return got


def _batch_shape(ctx):
    """(single-token requests, first and one past the last request with more tokens) of a step;
    worked out once per step and kept on the context."""
    shape = getattr(ctx, "_batch_shape", None)
    if shape is None:
        many = ctx.h_q_len != 1
        idx = many.nonzero()[0]
        shape = (int(len(many) - len(idx)),) + ((int(idx[0]), int(idx[-1]) + 1) if len(idx) else (0, 0))
        ctx._batch_shape = shape
    return shape


def rope_store_attention(qkv: torch.Tensor, nh: int, nkv: int, hd: int, ctx, cache,
                         inv_freq: Optional[torch.Tensor], rotary_dim: int, store: bool,
                         scale: float, window: int, out: torch.Tensor, softcap: float = 0.0,
                         slopes: Optional[torch.Tensor] = None) -> None:
    """``rope_kv_store`` followed by ``paged_attention``, as one operation.  Where the decode
    kernel can do the rotation and the cache write of single tokens itself (tensor-core path,
    the rotated part of the head a multiple of 16 wide, no score modifier), the separate kernel
    runs only for the tokens of prompt portions, or not at all."""
    if softcap or slopes is not None:
        rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store)
        paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out, softcap=softcap, slopes=slopes)
        return
    fuse = (FUSE_DECODE_ROPE and 0 < rotary_dim <= hd and rotary_dim % 16 == 0 and inv_freq is not None
            and tensor_core_attention_ok(qkv.dtype, hd, nh, nkv))
    n_decode = _batch_shape(ctx)[0] if fuse else 0
    if not n_decode:
        rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store)
        paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out)
        return
    if n_decode < ctx.n_requests:
        if OVERLAP_ATTENTION and not getattr(ctx, "fixed_launch", False):
            # Single tokens and prompt portions are different requests with different pages: the
            # decode kernel (memory-bound) runs on a second stream beside the rotation and the
            # attention of the portions (compute-bound), and the step's stream waits for both.
            main, side, fork, join = _fork_join(ctx, qkv.device)
            _stream_op(lambda: fork.record(main))             # qkv is whole here
            _stream_op(lambda: side.wait_event(fork))
            paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out,
                            decode_rope=(inv_freq, store, rotary_dim), only="single", stream=side.cuda_stream)
            _stream_op(lambda: join.record(side))
            rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store, skip_single=True)
            paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out, only="portions")
            _stream_op(lambda: main.wait_event(join))
            return
        rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store, skip_single=True)
    else:
        _req(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rotary_dim // 2 or qkv.shape[1] != (nh + 2 * nkv) * hd:
            raise KernelError("rope: inv_freq or qkv do not fit the head size")
    paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out,
                    decode_rope=(inv_freq, store, rotary_dim))


def paged_attention(qkv: torch.Tensor, nh: int, nkv: int, hd: int, ctx, cache, scale: float,
                    window: int, out: torch.Tensor, decode_rope=None, only: Optional[str] = None,
                    stream: Optional[int] = None, softcap: float = 0.0,
                    slopes: Optional[torch.Tensor] = None) -> None:
    """Causal attention of this step's query rows over their requests' cached keys and values.

    Score modifiers: ``softcap`` > 0 replaces a scaled score s by ``softcap * tanh(s / softcap)``;
    ``slopes`` (float32 [heads]) subtracts ``slopes[h] * (query position - key position)``.  A
    call with either runs the generic kernel, whatever the dtype and head size.

    bfloat16 with head size 64 or 128 runs on the tensor cores: single decode tokens in the
    split-KV kernel, prompt portions in the tiled kernel.  Everything else (32-bit, other head
    sizes) runs the generic kernel.  ``decode_rope = (inv_freq, store, rotary_dim)`` says that
    single tokens come unrotated and not yet in the cache (see ``rope_store_attention``).  ``only``: "single"
    or "portions" launches just that kernel; ``stream``: a raw stream to launch on instead of the
    current one."""
    _req(qkv, "qkv", dim=2)
    _req(out, "out", qkv.dtype, 2)
    T = qkv.shape[0]
    if qkv.shape[1] < nh * hd or out.shape != (T, nh * hd):
        raise KernelError(f"attention: qkv {tuple(qkv.shape)} / out {tuple(out.shape)} do not fit "
                          f"{nh} heads of {hd}")
    if hd % 16 or not 16 <= hd <= 256:
        raise KernelError(f"attention: head_dim must be a multiple of 16 in [16, 256], got {hd}")
    if nkv <= 0 or nh % nkv:
        raise KernelError(f"attention: {nh} heads cannot share {nkv} kv heads")
    if ctx.n_requests > 65535 or nh > 65535:
        raise KernelError("attention: at most 65535 requests and heads per step")
    _check_cache(cache, nkv, hd, qkv.dtype)
    common = (_p(qkv), _i(qkv.shape[1]), _p(cache.k_pages), _p(cache.v_pages), _p(ctx.q_start),
              _p(ctx.kv_len), _p(ctx.table_rows), _p(cache.block_table),
              _i(cache.block_table.shape[1]), _p(out))
    tail = (_i(nh), _i(nkv), _i(hd), _i(cache.page_size), _i(cache.k_pages.shape[0]), _f(scale),
            _i(window))
    modified = bool(softcap) or slopes is not None
    if slopes is not None:
        _req(slopes, "slopes", torch.float32, 1)
        if slopes.shape[0] != nh:
            raise KernelError(f"attention: {slopes.shape[0]} slopes for {nh} heads")
    if softcap < 0:
        raise KernelError("attention: the soft cap must be positive (0: none)")
    if modified or not tensor_core_attention_ok(qkv.dtype, hd, nh, nkv):
        if decode_rope is not None:
            raise KernelError("attention: only the tensor-core decode kernel rotates by itself")
        _call("attention", "lsb_paged_attention_generic", *common, _i(_dt(qkv)),
              _i(ctx.n_requests), _i(ctx.max_q_len), *tail, _f(softcap), _p(slopes), _stream(out))
        return
    R = ctx.n_requests
    n_decode, first, last = _batch_shape(ctx)
    on = _stream(out) if stream is None else ctypes.c_void_p(stream)
    if n_decode and only != "portions":
        splits = decode_splits(n_decode, nkv, qkv.device, hd, nh // nkv)
        if not getattr(ctx, "fixed_launch", False):
            splits = min(splits, -(-ctx.max_kv_len // 128))
        cluster_cap = _decode_cluster_cap(hd)
        if cluster_cap >= 16 and splits > 8 and n_decode * nkv <= 16:
            splits = 16                 # a few requests: one 16-block cluster each, no merge kernel
                                        # (with more clusters than that the merge kernel was faster)
        elif splits > 12:
            splits = 12                 # finer splits than this only lengthen the merge
        scratch = None
        if splits > cluster_cap:        # splits of a cluster merge through distributed shared memory
            key = (qkv.device, R, nh, hd, splits)
            scratch = _scratch.get(key)
            if scratch is None:
                scratch = torch.empty(R * nh * splits * (hd + 2), dtype=torch.float32,
                                      device=qkv.device)
                _scratch[key] = scratch
        if decode_rope is None:
            _call("attention_tc", "lsb_decode_attention", *common, _p(scratch), _i(R), *tail,
                  _i(splits), on)
        else:
            _call("attention_tc", "lsb_decode_attention_rope", *common, _p(scratch), _i(R), *tail,
                  _i(splits), _p(decode_rope[0]), _i(decode_rope[2]), _i(1 if decode_rope[1] else 0), on)
    if n_decode < R and only != "single":
        # prompt portions: tcgen05 kernel for long ones (128-row tiles), mma.sync kernel otherwise
        # The grid has a slab of blocks per request, and blocks that find a single token leave at
        # once, but thousands of them still cost tens of microseconds: the kernels get only the
        # requests from the first to the last prompt portion (the scheduler puts single tokens
        # first), by way of offset pointers into the per-request arrays.
        off = 4 * first
        per_request = (ctypes.c_void_p(ctx.q_start.data_ptr() + off),
                       ctypes.c_void_p(ctx.kv_len.data_ptr() + off),
                       ctypes.c_void_p(ctx.table_rows.data_ptr() + off))
        skip = _i(1 if n_decode > first + (R - last) else 0)      # single tokens among them
        if (USE_TCGEN05_ATTENTION and ctx.max_q_len >= 128
                and cache.page_size in (8, 16, 32, 64) and qkv.shape[1] % 8 == 0):
            _call("attention_tc5", "lsb_prefill_attention_tc5", _p(qkv), _i(qkv.shape[1]), _i(T),
                  _p(cache.k_pages), _p(cache.v_pages), *per_request, _p(cache.block_table),
                  _i(cache.block_table.shape[1]), _p(out), _i(last - first), _i(ctx.max_q_len), *tail,
                  skip, on)
        else:
            _call("attention_tc", "lsb_prefill_attention", _p(qkv), _i(qkv.shape[1]), _p(cache.k_pages),
                  _p(cache.v_pages), *per_request, _p(cache.block_table), _i(cache.block_table.shape[1]),
                  _p(out), _i(last - first), _i(ctx.max_q_len), *tail, skip, on)


def sample(logits: torch.Tensor, params: torch.Tensor, top_k: torch.Tensor,
           prev_start: Optional[torch.Tensor], prev_tokens: Optional[torch.Tensor],
           out: torch.Tensor, work: Optional[torch.Tensor] = None) -> None:
    """One token per row of ``logits``.  ``params[r] = (temperature, top_p, repetition_penalty,
    u)``; ``top_k[r]`` (0 = off); ``prev_tokens[prev_start[r]:prev_start[r+1]]`` are the tokens the
    repetition penalty applies to; ``work`` is scratch shaped like ``logits`` (needed only when
    a penalty is in use)."""
    _req(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    _req(params, "params", torch.float32, 2)
    _req(top_k, "top_k", torch.int32, 1)
    _req(out, "out", torch.int32, 1)
    if params.shape != (R, 4) or top_k.shape[0] != R or out.shape[0] != R:
        raise KernelError("sample: per-row arrays do not match the logits")
    if prev_start is not None:
        _req(prev_start, "prev_start", torch.int32, 1)
        _req(prev_tokens, "prev_tokens", torch.int32, 1)
        if work is None:
            work = torch.empty_like(logits)
        _req(work, "work", torch.float32, 2)
        if work.shape != logits.shape:
            raise KernelError("sample: work must be shaped like logits")
    _call("sampling", "lsb_sample", _p(logits), _p(work), _i(R), _i(V), _p(params), _p(top_k),
          _p(prev_start), _p(prev_tokens), _p(out), _stream(out))
