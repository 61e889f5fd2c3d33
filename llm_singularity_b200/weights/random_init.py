"""Random-weights mode: make a model folder from a configuration and a seed.

The reference has no such mode (it needs a downloaded checkpoint,
app/main.cpp:149-160).  Matrices and the embedding table are N(0, std); norm
weights are ``1 + N(0, norm_noise)``.

The values come from a counter-based stream: element ``i`` of the tensor called
``name`` is a function of ``(seed, name, i)`` and of nothing else, so a tensor's
values do not depend on which other tensors exist, in which order or in how many
pieces they are made, or where.  On a CUDA device a kernel of the package makes
them (``csrc/random_init.cu``); on the CPU the same arithmetic is stated below with
tensor operations.  The two agree bit for bit, so a model made on the GPU by
``--random-weights --seed S`` can be rebuilt anywhere from ``S``.

``normal(key, i)``: ``z = splitmix64(key + (i + 1) * golden)``; ``a`` its top 24
bits, ``b`` the next 24; ``u = (a + 1) / 2^24`` lies in (0, 1]; the value is
``sqrt(-2 ln u) * cos(2 pi b / 2^24)`` (Box-Muller).  Logarithm and cosine are short
polynomials evaluated in 32-bit, every product and sum rounded on its own (no
fused multiply-add), division and square root correctly rounded: arithmetic
that IEEE 754 pins down, which library functions are not.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Mapping, Tuple

import numpy as np
import torch

from .safetensors_io import write_safetensors

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
_CHUNK = 1 << 20                  # elements made at a time on the CPU


def _splitmix64_int(x: int) -> int:
    z = x & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of one tensor's stream."""
    return _splitmix64_int(int(seed) * _GOLDEN + zlib.crc32(name.encode("utf-8")))


def _f32(x) -> torch.Tensor:
    return torch.tensor(x, dtype=torch.float32)


def _normal_cpu(key: int, start: int, count: int) -> torch.Tensor:
    """normal(key, i) for i in [start, start + count), float32, on the CPU."""
    with np.errstate(over="ignore"):
        i = np.arange(start + 1, start + count + 1, dtype=np.uint64)
        z = np.uint64(key) + i * np.uint64(_GOLDEN)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    a = (z >> np.uint64(40)).astype(np.int64)
    b = ((z >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.int64)
    # ln u: t = a + 1 = m * 2^e with m in (sqrt(1/2), sqrt(2)]
    t = torch.from_numpy(a + 1).to(torch.float32)                  # exact: at most 2^24
    mant, exp = torch.frexp(t)                                     # t = mant * 2^exp, mant in [0.5, 1)
    m, e = mant * 2.0, exp - 1
    big = m > _f32(1.41421356)
    m = torch.where(big, m * 0.5, m)
    e = torch.where(big, e + 1, e)
    s = (m + (-1.0)) / (m + 1.0)
    s2 = s * s
    one = np.float32(1.0)
    p = torch.full_like(s, float(one / np.float32(9.0)))
    for d in (7.0, 5.0, 3.0, 1.0):
        p = p * s2 + float(one / np.float32(d))
    lnm = (s * 2.0) * p
    lnu = (e - 24).to(torch.float32) * _f32(0.69314718) + lnm
    # (the tensor library's 32-bit square root is not correctly rounded on every CPU; numpy's is)
    r = torch.from_numpy(np.sqrt((lnu * (-2.0)).numpy()))
    # cos(2 pi b / 2^24): quadrant q, then the sine of an angle in [0, pi/2]
    q, f = b >> 22, b & 0x3FFFFF
    g = np.where(q & 1, f, 0x400000 - f)
    x = torch.from_numpy(g).to(torch.float32) * _f32(3.7450703e-07)
    x2 = x * x
    c = torch.full_like(x, float(one / np.float32(6227020800.0)))
    for d, sign in ((39916800.0, -1.0), (362880.0, 1.0), (5040.0, -1.0), (120.0, 1.0), (6.0, -1.0)):
        c = c * x2 + float(np.float32(sign) / np.float32(d))
    c = c * x2 + 1.0
    v = x * c
    v = torch.where(torch.from_numpy((q == 1) | (q == 2)), -v, v)
    return r * v


def normal_tensor(shape, key: int, mean: float, scale: float, dtype: torch.dtype,
                  device="cpu") -> torch.Tensor:
    """``mean + scale * normal(key, i)`` in ``dtype`` (rounded to nearest even from 32-bit), element
    ``i`` counted in row-major order."""
    device = torch.device(device)
    shape = (int(shape),) if isinstance(shape, int) else tuple(shape)
    n = 1
    for d in shape:
        n *= int(d)
    if device.type == "cuda":
        from .. import kernels
        out = torch.empty(tuple(shape), dtype=dtype, device=device)
        kernels.random_normal(out, key, mean, scale)
        return out
    out = torch.empty(n, dtype=dtype)
    mean32, scale32 = _f32(mean), _f32(scale)
    for start in range(0, n, _CHUNK):
        count = min(_CHUNK, n - start)
        out[start:start + count] = (mean32 + scale32 * _normal_cpu(key, start, count)).to(dtype)
    return out.reshape(tuple(shape))


def random_tensors(expected: Mapping[str, Tuple[Tuple[int, ...], str, str]], seed: int,
                   dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                   norm_noise: float = 0.0, device="cpu") -> Dict[str, torch.Tensor]:
    """``expected``: name -> (shape, role, init).  Matrices/tables in ``dtype``, vectors in
    ``dtype`` too (a checkpoint stores one dtype), integer tables as int32 zeros.  The same
    values whatever ``device`` is."""
    out: Dict[str, torch.Tensor] = {}
    for name, (shape, role, init) in expected.items():
        if role == "int_table":
            out[name] = torch.zeros(shape, dtype=torch.int32, device=device)
            continue
        key = tensor_key(seed, name)
        if init == "ones":
            out[name] = normal_tensor(shape, key, 1.0, norm_noise, dtype, device)
        else:
            out[name] = normal_tensor(shape, key, 0.0, std, dtype, device)
    return out


def write_random_model(model_dir: str, config, seed: int, dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02, norm_noise: float = 0.0, device="cpu") -> None:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` into ``model_dir``.
    ``device``: where the values are made (the file is the same either way)."""
    from ..engine.runner import expected_tensors_of
    os.makedirs(model_dir, exist_ok=True)
    expected = expected_tensors_of(config.to_model_spec())
    tensors = random_tensors(expected, seed, dtype=dtype, std=std, norm_noise=norm_noise, device=device)
    tensors = {n: t.cpu() for n, t in tensors.items()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
