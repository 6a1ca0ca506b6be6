"""``out = a @ w.T`` with a choice of epilogue: the one place that decides which matrix-product
kernel runs for a shape and a pair of storage types.

* float32 anywhere in the product: the CUDA-core kernels (float32 multiply-add; this is the
  whole of the 32-bit path, no tensor-core mode is involved);
* bfloat16 x bfloat16: few rows stream the weights once through the tensor-core skinny kernel,
  many rows run the tcgen05 kernel; shapes those kernels refuse go to the CUDA-core kernels.
"""
from __future__ import annotations

import torch

from . import ops
from .ops import EPI_ACCUMULATE, EPI_STORE, EPI_SWIGLU  # noqa: F401  (re-exported)

_fast = None


def _fast_ops():
    global _fast
    if _fast is None:
        from . import fast_ops
        _fast = fast_ops
    return _fast


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if _fast_ops().linear_bf16(a, w, out, epilogue):
            return
    ops.gemm_simt(a, w, out, epilogue)
