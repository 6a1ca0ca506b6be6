"""Weights by tensor name.

The model says which tensors it wants (name -> shape); the folder says which it has.  Every
disagreement (missing, unexpected, wrong shape, unusable dtype) is collected and raised as ONE
``WeightsError`` that lists them all, before anything is copied to the device
(the reference stops at the first: crates/bfi-models/src/qwen3.rs:101-148, 379-425).

Storage rule: in a bfloat16 run a 16-bit tensor is kept as bfloat16 and a tensor stored in
32-bit stays 32-bit (the kernels take either); integer tables become int32; in a float32 run
every floating tensor is widened to float32, which is exact.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Mapping, Optional, Sequence, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors_io import SafetensorsError, SafetensorsFile

SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"


class WeightsError(ValueError):
    """The tensors of a model folder do not fit the model."""

    def __init__(self, folder: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 bad_dtype: Sequence[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.bad_dtype = list(bad_dtype)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, dt in self.bad_dtype:
            lines.append(f"  unusable dtype: {name} is stored as {dt}")
        super().__init__("\n".join(lines))


def _open_folder(folder: str) -> Dict[str, SafetensorsFile]:
    """tensor name -> the open file that holds it."""
    index = os.path.join(folder, INDEX_FILE)
    single = os.path.join(folder, SINGLE_FILE)
    where: Dict[str, SafetensorsFile] = {}
    if os.path.isfile(single):
        f = SafetensorsFile(single)
        for n in f.names():
            where[n] = f
        return where
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as fh:
            weight_map = json.load(fh).get("weight_map", {})
        files: Dict[str, SafetensorsFile] = {}
        for fname in sorted(set(weight_map.values())):
            files[fname] = SafetensorsFile(os.path.join(folder, fname))
        for f in files.values():
            for n in f.names():
                if n in where:
                    raise SafetensorsError(f"{folder}: tensor '{n}' appears in two shards")
                where[n] = f
        return where
    raise FileNotFoundError(f"{folder}: neither {SINGLE_FILE} nor {INDEX_FILE} found")


def stored_dtype_for(run_dtype: torch.dtype, file_dtype: torch.dtype) -> Optional[torch.dtype]:
    """The dtype a tensor is kept in on the device, or None if it cannot be used."""
    if file_dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return torch.int32
    if not file_dtype.is_floating_point:
        return None
    if run_dtype == torch.float32:
        return torch.float32
    if file_dtype in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_names(folder: str, have: Mapping[str, Tuple[torch.dtype, Tuple[int, ...]]],
                expected: Mapping[str, ParamSpec], ignored: Iterable[str],
                run_dtype: torch.dtype) -> None:
    ignored = set(ignored)
    missing = [n for n, s in expected.items() if n not in have and not s.optional]
    unexpected = [n for n in have if n not in expected and n not in ignored]
    wrong, bad = [], []
    for n, s in expected.items():
        if n in have:
            dt, shape = have[n]
            if tuple(shape) != tuple(s.shape):
                wrong.append((n, tuple(shape), tuple(s.shape)))
            if stored_dtype_for(run_dtype, dt) is None:
                bad.append((n, str(dt)))
    if missing or unexpected or wrong or bad:
        raise WeightsError(folder, missing, unexpected, wrong, bad)


def load_folder(folder: str, expected: Mapping[str, ParamSpec], ignored: Iterable[str],
                run_dtype: torch.dtype, device: torch.device) -> Dict[str, torch.Tensor]:
    """Check the folder against ``expected`` and bring every expected tensor to ``device``."""
    where = _open_folder(folder)
    have = {n: f.info(n) for n, f in where.items()}
    check_names(folder, have, expected, ignored, run_dtype)
    out: Dict[str, torch.Tensor] = {}
    for n in expected:
        if n not in where:
            continue
        host = where[n].tensor(n)
        keep = stored_dtype_for(run_dtype, host.dtype)
        both = (torch.float32, torch.bfloat16)
        if torch.device(device).type == "cuda" and host.dtype != keep and host.dtype in both and keep in both:
            # widened (or narrowed) on the device by the library's own conversion kernel
            from ..kernels import ops
            out[n] = ops.convert(host.to(device=device), keep)
        else:
            out[n] = host.to(device=device, dtype=keep).contiguous()
    for f in set(where.values()):
        f.close()
    return out
