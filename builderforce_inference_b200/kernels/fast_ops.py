"""Faces of the bfloat16 kernels of the ``fast`` library.  Each returns False when it does not
take the shape (the caller then uses the general kernel); it never computes a wrong result.
"""
from __future__ import annotations

import torch


def linear_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> bool:
    return False
