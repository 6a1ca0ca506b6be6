"""RMS norm: ``y = x * rsqrt(mean(x^2) + eps) * w`` over the last dim, the weight as stored
(crates/bfi-core/src/cpu.rs:92-122).  The statistics are float32; the input is the float32
residual stream and the output is in the activation dtype."""
from __future__ import annotations

from typing import Dict

from ..kernels import ops
from .base import NORMS, Norm, ParamSpec


@NORMS.register("rms")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float):
        self.width = int(width)
        self.eps = float(eps)
        self.weight = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.width,), "norm")}

    def load(self, tensors, runtime) -> None:
        self.weight = tensors["weight"]

    def forward(self, ctx, x, rows=None, tag: str = "norm.out"):
        n = x.shape[0] if rows is None else rows.numel()
        out = ctx.rows(tag, self.width, n_rows=n)
        ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out
