"""Random-weights mode: make a model folder from a configuration and a seed.

The reference has no such mode (it needs a downloaded checkpoint,
app/main.cpp:149-160).  Matrices and the embedding table are N(0, std); norm
weights are ``1 + N(0, norm_noise)``.  Every tensor has its own generator seeded
from ``(seed, tensor name)``, so a tensor's values do not depend on which other
tensors exist or in which order they are made.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Mapping, Tuple

import torch

from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B97F4A7C15 + zlib.crc32(name.encode("utf-8"))) % (1 << 63)


def random_tensors(expected: Mapping[str, Tuple[Tuple[int, ...], str, str]], seed: int,
                   dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                   norm_noise: float = 0.0, device="cpu") -> Dict[str, torch.Tensor]:
    """``expected``: name -> (shape, role, init).  Matrices/tables in ``dtype``, vectors in
    ``dtype`` too (a checkpoint stores one dtype), integer tables as int32 zeros."""
    out: Dict[str, torch.Tensor] = {}
    device = torch.device(device)
    for name, (shape, role, init) in expected.items():
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(seed, name))
        if role == "int_table":
            out[name] = torch.zeros(shape, dtype=torch.int32, device=device)
            continue
        t = torch.randn(shape, generator=g, dtype=torch.float32, device=device)
        if init == "ones":
            t = 1.0 + norm_noise * t
        else:
            t = std * t
        out[name] = t.to(dtype)
    return out


def write_random_model(model_dir: str, config, seed: int, dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02, norm_noise: float = 0.0) -> None:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` into ``model_dir``."""
    from ..engine.runner import expected_tensors_of
    os.makedirs(model_dir, exist_ok=True)
    expected = expected_tensors_of(config.to_model_spec())
    tensors = random_tensors(expected, seed, dtype=dtype, std=std, norm_noise=norm_noise)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
