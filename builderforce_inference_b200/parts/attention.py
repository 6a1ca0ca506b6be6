"""Grouped-query attention over the paged cache, as a mixer.

Order of operations (crates/bfi-models/src/qwen3.rs:220-242): q, k, v projections without bias;
per-head RMS norm of q and k when ``qk_norm``; position encoding of q and k; k and v appended to
the sequence's cache; causal attention of every new token over the cached keys (all of them, or
the last ``window``); output projection added to the residual stream.

The three projections are one matrix product over the concatenated weights.  Keys and values
are always read from the cache, so a step may bring whole prompts, a continuation of a cached
prefix, or single tokens, and a run may read another run's cache (``run.writes_cache`` false:
this layer then has no k and v projections of its own).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..kernels import ops
from ..kernels.linear import EPI_ACCUMULATE, EPI_STORE, linear
from .base import MIXERS, POSITION_ENCODINGS, KVNeed, Mixer, ParamSpec, PartSpec


@MIXERS.register("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: Optional[PartSpec] = None, qk_norm: bool = False, eps: float = 1e-6,
                 window: Optional[int] = None, scale: Optional[float] = None, own_kv: bool = True):
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"GQA: {n_heads} query heads do not divide into {n_kv_heads} kv heads")
        if head_dim % 16 != 0 or head_dim > 512:
            raise ValueError(f"attention kernels take head sizes in steps of 16 up to 512, got {head_dim}")
        if window is not None and window < 1:
            raise ValueError(f"window must be positive, got {window}")
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = width, n_heads, n_kv_heads, head_dim
        self.qk_norm, self.eps, self.window = bool(qk_norm), float(eps), window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.own_kv = bool(own_kv)
        self.position = POSITION_ENCODINGS.build(position) if position is not None \
            else POSITION_ENCODINGS.build(PartSpec("none"))
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    def children(self):
        return {"position": self.position}

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, h = self.head_dim, self.width
        specs = {"q_proj": ParamSpec((self.n_heads * d, h)), "o_proj": ParamSpec((h, self.n_heads * d))}
        if self.own_kv:
            specs["k_proj"] = ParamSpec((self.n_kv_heads * d, h))
            specs["v_proj"] = ParamSpec((self.n_kv_heads * d, h))
        if self.qk_norm:
            specs["q_norm"] = ParamSpec((d,), "norm")
            if self.own_kv:
                specs["k_norm"] = ParamSpec((d,), "norm")
        return specs

    def cache_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window)

    def prepare(self, runtime, max_positions: int) -> None:
        self.position.prepare(runtime, max_positions)

    def load(self, tensors, runtime) -> None:
        mats = [tensors["q_proj"]]
        if self.own_kv:
            mats += [tensors["k_proj"], tensors["v_proj"]]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.w_o = tensors["o_proj"]
        self.q_norm = tensors.get("q_norm")
        self.k_norm = tensors.get("k_norm")
        if self.q_norm is not None and self.k_norm is not None and self.q_norm.dtype != self.k_norm.dtype:
            self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    def forward(self, ctx, h, residual, run) -> None:
        kv = run.kv
        if kv is None:
            raise RuntimeError("attention needs a key/value cache for its run")
        n_kv_in = self.n_kv_heads if self.own_kv else 0
        if run.writes_cache != self.own_kv:
            raise RuntimeError("an attention layer writes the cache exactly when it has k and v projections")
        d = self.head_dim
        qkv = ctx.rows("attn.qkv", (self.n_heads + 2 * n_kv_in) * d)
        linear(h, self.w_qkv, qkv, EPI_STORE)

        fused = self.position.fused_rotary()
        write = ops.FLAG_WRITE_CACHE if run.writes_cache else 0
        if fused is not None:
            table, rot = fused
            ops.qk_norm_rope_cache(qkv, self.n_heads, n_kv_in, d, self.q_norm, self.k_norm, self.eps,
                                   table, rot, ctx.token_pos, ctx.token_slot, kv, write, ctx.status)
        else:
            # a position encoding with code of its own: norms first, then its transform, then the cache
            ops.qk_norm_rope_cache(qkv, self.n_heads, n_kv_in, d, self.q_norm, self.k_norm, self.eps,
                                   None, 0, ctx.token_pos, ctx.token_slot, kv, ops.FLAG_K_IN_PLACE, ctx.status)
            q_view = qkv[:, :self.n_heads * d].view(-1, self.n_heads, d)
            k_view = qkv[:, self.n_heads * d:(self.n_heads + n_kv_in) * d].view(-1, n_kv_in, d)
            self.position.apply(ctx, q_view, k_view)
            if write:
                ops.qk_norm_rope_cache(qkv, self.n_heads, n_kv_in, d, None, None, self.eps, None, 0,
                                       ctx.token_pos, ctx.token_slot, kv, write, ctx.status)

        out = ctx.rows("attn.out", self.n_heads * d)
        self.attend(ctx, qkv, out, kv)
        linear(out, self.w_o, residual, EPI_ACCUMULATE)

    def attend(self, ctx, qkv, out, kv) -> None:
        from ..kernels import attention as fast_attention
        if fast_attention.attend(ctx, qkv, out, kv, self.n_heads, self.scale):
            return
        ops.attention_paged(qkv, qkv.stride(0), out, kv, ctx.cu_seqlens, ctx.seq_slot, ctx.seq_start,
                            ctx.n_seqs, ctx.max_seq_tokens, self.n_heads, self.scale)
