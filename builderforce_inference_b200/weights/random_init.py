"""Random weights from a configuration and a seed.

Matrices and tables are N(0, 0.02); norm weights are 1 + N(0, 0.1).  Every value is a closed
formula of (seed, tensor name, element index), so a tensor's values do not depend on which other
tensors exist, on the order they are made in, or on the machine that makes them: the model folder
written on the CPU and the model filled straight into device memory hold the same bits, and any
other implementation can rebuild them (the reference builds its toy models from a closed formula
for the same reason: crates/bfi-models/src/lib.rs:52-79).

The formula, for element ``i`` (row-major) of the tensor called ``name``:

    key = the first 8 bytes (little endian) of sha256("<seed>:<name>")
    x_j = mix64(key + (2 i + j + 1) * 0x9E3779B97F4A7C15)        j = 0, 1, modulo 2^64
    s   = the sum of the eight 16-bit fields of x_0 and x_1
    c   = 2 s - 8 * 65535
    v   = offset + float32(c) * scale                             rounded to float32 after each step

``mix64`` is the splitmix64 finalizer.  ``s`` is a sum of eight uniform integers (Irwin-Hall: close
to normal, no value beyond 4.9 standard deviations) with standard deviation 65536 * sqrt(2/3);
``scale`` is ``std / (131072 * sqrt(2/3))`` rounded to float32.  A bfloat16 tensor is ``v`` rounded
to nearest even.  On the CPU the formula runs in numpy; on the GPU in ``csrc/utility.cu``.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from concurrent.futures import ThreadPoolExecutor
from ctypes import c_float, c_int, c_long, c_ulonglong, c_void_p
from typing import Any, Dict, Iterator, Mapping, Tuple

import numpy as np
import torch

from ..parts.base import ParamSpec
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1
_GOLDEN = 0x9E3779B97F4A7C15
_UNIT_STD = 131072.0 * math.sqrt(2.0 / 3.0)       # standard deviation of c
_CHUNK = 1 << 16                                   # elements per numpy pass (stays in cache)


def tensor_key(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()[:8], "little")


def fill_constants(role: str) -> Tuple[float, float]:
    """``(scale, offset)`` of a tensor's role, both exactly representable in float32."""
    std, offset = (NORM_STD, 1.0) if role == "norm" else (MATRIX_STD, 0.0)
    return float(np.float32(std / _UNIT_STD)), offset


def _mix64(z: np.ndarray) -> np.ndarray:
    z ^= z >> np.uint64(30)
    z *= np.uint64(0xBF58476D1CE4E5B9)
    z ^= z >> np.uint64(27)
    z *= np.uint64(0x94D049BB133111EB)
    z ^= z >> np.uint64(31)
    return z


def _fields16(x: np.ndarray) -> np.ndarray:
    m = np.uint64(0xFFFF)
    return ((x & m) + ((x >> np.uint64(16)) & m) + ((x >> np.uint64(32)) & m) + (x >> np.uint64(48))).astype(np.int64)


def _fill_range(out: np.ndarray, first: int, key: int, scale: float, offset: float) -> None:
    n = out.shape[0]
    with np.errstate(over="ignore"):
        i = np.arange(first, first + n, dtype=np.uint64)
        base = np.uint64(key) + (np.uint64(2) * i + np.uint64(1)) * np.uint64(_GOLDEN)
        s = _fields16(_mix64(base.copy())) + _fields16(_mix64(base + np.uint64(_GOLDEN)))
    c = (2 * s - 8 * 65535).astype(np.float32)
    np.multiply(c, np.float32(scale), out=out)
    if offset != 0.0:
        np.add(out, np.float32(offset), out=out)


def random_values_cpu(n: int, key: int, scale: float, offset: float) -> np.ndarray:
    """``n`` float32 values of the formula above."""
    out = np.empty(n, dtype=np.float32)
    pieces = [(a, min(a + _CHUNK, n)) for a in range(0, n, _CHUNK)]

    def work(piece):
        a, b = piece
        _fill_range(out[a:b], a, key, scale, offset)

    if len(pieces) > 8:
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as pool:
            list(pool.map(work, pieces))
    else:
        for piece in pieces:
            work(piece)
    return out


def random_tensor(name: str, spec: ParamSpec, seed: int, dtype: torch.dtype,
                  device: torch.device) -> torch.Tensor:
    device = torch.device(device)
    key = tensor_key(seed, name)
    scale, offset = fill_constants(spec.role)
    n = 1
    for d in spec.shape:
        n *= d
    if device.type != "cuda":
        values = torch.from_numpy(random_values_cpu(n, key, scale, offset)).reshape(spec.shape)
        return values.to(dtype)
    from ..kernels.library import library
    from ..kernels.ops import _stream, dtype_code
    out = torch.empty(spec.shape, dtype=dtype, device=device)
    with torch.cuda.device(device):
        library("core").call("bfi_fill_random", c_void_p(out.data_ptr()), c_int(dtype_code(dtype)), c_long(n),
                             c_ulonglong(key), c_float(scale), c_float(offset), _stream())
    return out


def random_tensors(expected: Mapping[str, ParamSpec], seed: int, dtype: torch.dtype,
                   device: torch.device) -> Iterator[Tuple[str, torch.Tensor]]:
    for name, spec in expected.items():
        if spec.optional:
            continue
        yield name, random_tensor(name, spec, seed, dtype, device)


def write_model_folder(config: Dict[str, Any], seed: int, folder: str,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a config.json dictionary)
    with random weights from ``seed``; returns the folder."""
    from ..registry import describe_model  # late: the registry imports the architectures

    spec = describe_model(config)
    expected = expected_tensors(spec)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(expected, seed, dtype, torch.device("cpu")))
    return folder


def expected_tensors(spec) -> Dict[str, ParamSpec]:
    """Every checkpoint tensor a ``ModelSpec`` wants: name -> ParamSpec."""
    from ..engine.decoder import expected_tensors as _expected
    return _expected(spec)
