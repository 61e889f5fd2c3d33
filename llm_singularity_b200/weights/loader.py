"""Loading a checkpoint by tensor name, with one error that tells everything.

Files: every ``model*.safetensors`` in the folder, sorted (the reference's regex,
models/llama/llama_model.cpp:189-197).  The reference routes twelve names to
member pointers and is silent about what is missing, mis-shaped or unknown
(llama_model.cpp:209-255); here the model declares every tensor it expects with
its shape, and a single :class:`WeightError` lists all missing tensors, all
unexpected ones and all wrong shapes.  Tensors keep their stored dtype on the way
in (bfloat16 stays bfloat16, 32-bit stays 32-bit, integers become int32); the
model then places each by role.
"""
from __future__ import annotations

import glob
import os
from typing import Dict, Iterable, Mapping, Tuple

import torch

from .safetensors_io import SafetensorsFile


class WeightError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is {got}")
        super().__init__("\n".join(lines))


def checkpoint_files(model_dir: str):
    files = sorted(glob.glob(os.path.join(model_dir, "model*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no model*.safetensors file in {model_dir}")
    return files


_FLOAT = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INT = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


def load_checkpoint(model_dir: str, expected: Mapping[str, Tuple[Tuple[int, ...], str]],
                    ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Read the tensors named in ``expected`` (name -> (shape, role)).

    Returns CPU tensors: floating tensors in bfloat16 or float32 as stored (float16
    and float64 are widened/narrowed to float32), integer tables as int32.
    """
    ignorable = set(ignorable)
    found: Dict[str, torch.Tensor] = {}
    unexpected, wrong_shape, wrong_dtype = [], [], []
    for path in checkpoint_files(model_dir):
        f = SafetensorsFile(path)
        for name in f.names():
            if name not in expected:
                if name not in ignorable:
                    unexpected.append(name)
                continue
            dtype, shape = f.info(name)
            want_shape, role = expected[name]
            if tuple(shape) != tuple(want_shape):
                wrong_shape.append((name, shape, want_shape))
                continue
            if role == "int_table":
                if dtype not in _INT:
                    wrong_dtype.append((name, f"{dtype}, expected an integer table"))
                    continue
                found[name] = f.tensor(name).to(torch.int32)
            else:
                if dtype not in _FLOAT:
                    wrong_dtype.append((name, f"{dtype}, expected a floating type"))
                    continue
                t = f.tensor(name)
                found[name] = t if dtype in (torch.float32, torch.bfloat16) else t.to(torch.float32)
    missing = [n for n in expected if n not in found
               and not any(n == w[0] for w in wrong_shape)
               and not any(n == w[0] for w in wrong_dtype)]
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype)
    return found
