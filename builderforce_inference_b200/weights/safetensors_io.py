"""Reading and writing safetensors files: an 8-byte little-endian header length, a JSON header
(name -> dtype, shape, byte offsets) and the raw tensors.  Tensors are handed out as views of
a private memory map, so nothing is copied on the host before the one copy to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors file."""


_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


def _no_duplicates(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise SafetensorsError(f"duplicate tensor name '{k}' in header")
        out[k] = v
    return out


class SafetensorsFile:
    """One open file: ``names()``, ``info(name)``, ``tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a header ({size} bytes)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"), object_pairs_hook=_no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
        self._base = 8 + n
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dt, shape = info["dtype"], tuple(int(s) for s in info["shape"])
                b, e = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as err:
                raise SafetensorsError(f"{path}: malformed entry for '{name}'") from err
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            tdt = _DTYPES[dt]
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty((), dtype=tdt).element_size()
            if e - b != want:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' spans {e - b} bytes but {dt}{list(shape)} needs {want}")
            if b < 0 or self._base + e > size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' ends at byte {self._base + e} but the file has {size} "
                    f"(truncated?)")
            self._entries[name] = (tdt, shape, b, e)
        self._mm = None

    def names(self) -> List[str]:
        return list(self._entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self._entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A host view of the tensor (shares the private mapping; copy or move it before close)."""
        dt, shape, b, e = self._entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        if self._mm is None:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY)
        numel = 1
        for s in shape:
            numel *= s
        t = torch.frombuffer(self._mm, dtype=dt, count=numel, offset=self._base + b)
        return t.reshape(shape)

    def close(self) -> None:
        # Views handed out keep the mapping alive; dropping our references is enough.
        self._mm = None
        self._f.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Write ``(name, tensor)`` pairs in the given order."""
    items = [(n, t.detach().to("cpu").contiguous()) for n, t in tensors]
    header = {}
    off = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} (tensor '{name}')")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
