"""Choice of the attention kernel for a step.  Returns False when no specialised kernel takes
the step; the caller then runs the general paged kernel."""
from __future__ import annotations


def attend(ctx, qkv, out, kv, n_heads: int, scale: float) -> bool:
    return False
