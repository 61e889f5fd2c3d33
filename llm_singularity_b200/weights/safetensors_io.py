"""A reader and a writer for the safetensors container, with no dependency.

Layout (as the reference reads it, core/src/safetensors.cpp:42-116): an
unsigned 64-bit little-endian header length, a JSON header mapping each tensor
name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative
to the end of the header; the ``__metadata__`` entry is skipped), then the raw
little-endian data.  The file is memory-mapped and tensors are views into the
map, so opening a large checkpoint copies nothing.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from typing import Dict, Iterable, Mapping, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "F64": torch.float64, "I64": torch.int64, "I32": torch.int32,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """Read-only view of one ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e.strerror}") from None
        size = self._f.seek(0, 2)
        if size < 8:                                           # safetensors.cpp:60-64
            raise SafetensorsError(f"{path}: file too small ({size} bytes) to hold a header")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if 8 + hlen > size:                                    # safetensors.cpp:79-85
            raise SafetensorsError(f"{path}: header length {hlen} exceeds file size {size}")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self._data_start = 8 + hlen
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            dt = info.get("dtype")
            if dt not in _DTYPES:                              # safetensors.cpp:27-32
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            offs = info.get("data_offsets")
            if not isinstance(offs, list) or len(offs) != 2:   # safetensors.cpp:107-110
                raise SafetensorsError(f"{path}: tensor '{name}' needs two data_offsets")
            shape = tuple(int(s) for s in info.get("shape", []))
            begin, end = int(offs[0]), int(offs[1])
            n = 1
            for s in shape:
                n *= s
            want = n * torch.empty((), dtype=_DTYPES[dt]).element_size()
            if end - begin != want or self._data_start + end > size or begin < 0:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' spans {end - begin} bytes, "
                    f"shape {list(shape)} of {dt} needs {want}")
            self._entries[name] = (_DTYPES[dt], shape, begin, end)

    def names(self):
        return list(self._entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        if name not in self._entries:                          # safetensors.cpp:143-145
            raise SafetensorsError(f"{self.path}: no tensor named '{name}'")
        dt, shape, _, _ = self._entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that aliases the mapped file (do not write to it)."""
        dt, shape = self.info(name)
        _, _, begin, end = self._entries[name]
        n = 1
        for s in shape:
            n *= s
        if n == 0:
            return torch.empty(shape, dtype=dt)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # the map is read-only by design
            flat = torch.frombuffer(self._map, dtype=dt, count=n,
                                    offset=self._data_start + begin)
        return flat.view(shape)

    def close(self):
        # tensors handed out keep the map alive through the buffer protocol
        try:
            self._map.close()
        except BufferError:
            pass
        self._f.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] | None = None) -> None:
    """Write CPU tensors to ``path`` in name order, data aligned to 8 bytes."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    ordered = sorted(tensors.items())
    for name, t in ordered:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((-len(blob)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in ordered:
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))


def read_all(paths: Iterable[str]) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for p in paths:
        f = SafetensorsFile(p)
        for n in f.names():
            out[n] = f.tensor(n)
    return out
