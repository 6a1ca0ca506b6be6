"""Random weights from a configuration and a seed.

Matrices and tables are N(0, 0.02); norm weights are 1 + N(0, 0.1).  Each tensor has its own
generator, seeded from the seed and the tensor's name, so a tensor's values do not depend on
which other tensors exist or on the order they are made in.  The same function fills a model
folder (config.json, model.safetensors) and, for benchmarks, device memory directly.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Iterator, Mapping, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec: ParamSpec, seed: int, dtype: torch.dtype,
                  device: torch.device) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    t = torch.empty(spec.shape, dtype=torch.float32, device=device)
    t.normal_(0.0, 1.0, generator=g)
    if spec.role == "norm":
        t.mul_(NORM_STD).add_(1.0)
    else:
        t.mul_(MATRIX_STD)
    return t.to(dtype)


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
