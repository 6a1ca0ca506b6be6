"""Choice of the attention kernel for a step.  Returns False when no specialised kernel takes
the step; the caller then runs the general paged kernel."""
from __future__ import annotations

import torch


def attend(ctx, qkv, out, kv, n_heads: int, scale: float) -> bool:
    if qkv.dtype != torch.bfloat16:
        return False
    from . import fast_ops
    if ctx.max_seq_tokens == 1 and ctx.n_tokens == ctx.n_seqs:
        return fast_ops.attention_decode_bf16(ctx, qkv, out, kv, n_heads, scale)
    if ctx.max_seq_tokens >= fast_ops.TCGEN05_ATTENTION_MIN_TOKENS and \
            fast_ops.attention_prefill_tcgen05_bf16(ctx, qkv, out, kv, n_heads, scale):
        return True
    return fast_ops.attention_prefill_bf16(ctx, qkv, out, kv, n_heads, scale)
