"""Gated dense feed-forward: ``down(silu(gate(h)) * up(h))``, no bias
(crates/bfi-models/src/qwen3.rs:244-250; SiLU*mul crates/bfi-core/src/cpu.rs:169-180).

The gate and up matrices are stored interleaved row by row (gate_j, up_j, gate_j+1, ...), so
one matrix product yields both and its epilogue applies SiLU*mul while the pair is still in
registers; the down product adds into the residual stream.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels.linear import EPI_ACCUMULATE, EPI_SWIGLU, linear
from .base import FEED_FORWARDS, FeedForward, ParamSpec


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, width: int, inner: int, activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"gated_mlp supports the silu activation, got {activation!r}")
        self.width, self.inner = int(width), int(inner)
        self.w_gate_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"gate_proj": ParamSpec((self.inner, self.width)),
                "up_proj": ParamSpec((self.inner, self.width)),
                "down_proj": ParamSpec((self.width, self.inner))}

    def load(self, tensors, runtime) -> None:
        g, u = tensors["gate_proj"], tensors["up_proj"]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.stack([g, u], dim=1).reshape(2 * self.inner, self.width).contiguous()
        self.w_down = tensors["down_proj"]

    def forward(self, ctx, h, residual) -> None:
        act = ctx.rows("mlp.act", self.inner)
        linear(h, self.w_gate_up, act, EPI_SWIGLU)
        linear(act, self.w_down, residual, EPI_ACCUMULATE)
