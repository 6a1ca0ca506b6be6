"""Rotate-half (NEOX) rotary position encoding: dim ``i`` pairs with ``i + rot_dim/2`` and the
pair turns by ``pos * theta^(-2i/rot_dim)`` (crates/bfi-core/src/cpu.rs:650-670; qwen3 uses the
whole head, no frequency scaling: crates/bfi-models/src/qwen3.rs:150-163).

The angles are evaluated in float64 on the host, once, and the table of (cos, sin) is rounded to
float32: it is at least as exact as evaluating ``pos / theta^(2i/d)`` in float32 per token, which
is what the reference does.  The attention kernels read the table in the same pass as the q/k
norms and the cache write.
"""
from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, PositionEncoding


def rotary_table(theta: float, rot_dim: int, positions: int, device) -> torch.Tensor:
    """float32 ``[positions, rot_dim/2, 2]`` of (cos, sin)."""
    half = rot_dim // 2
    i = torch.arange(half, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / rot_dim)
    ang = torch.arange(positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
    table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32)
    return table.contiguous().to(device)


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, theta: float, rot_dim: int):
        if rot_dim % 2 != 0 or rot_dim <= 0:
            raise ValueError(f"rotary width must be even and positive, got {rot_dim}")
        self.theta = float(theta)
        self.rot_dim = int(rot_dim)
        self.table = None

    def prepare(self, runtime, max_positions: int) -> None:
        key = ("rotary", self.theta, self.rot_dim, max_positions)
        table = runtime.shared.get(key)
        if table is None:
            table = rotary_table(self.theta, self.rot_dim, max_positions, runtime.device)
            runtime.shared[key] = table
        self.table = table

    def fused_rotary(self):
        return self.table, self.rot_dim


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    graph_safe = True

    def fused_rotary(self):
        return None, 0
