"""Plain Qwen3 dense decoder: whole sequences, no cache, one function per part.

Every function restates one formula of the reference (Rust; paths are relative
to the reference project).  Shapes follow the reference: activations are
``[tokens, heads, head_dim]`` or ``[tokens, width]``, matrices are
``[out, in]`` row-major.  The working dtype is float32 as in the reference
(``crates/bfi-models/src/state.rs:52-59``: every activation and the cache are
f32); ``dtype=torch.float64`` gives a tighter oracle for the 32-bit tests.

This file shares no code with the product package.  It rests on the reference's formulas alone:
the reference is a Rust workspace that cannot be built or imported here (no Rust toolchain, no
network) and ships no numeric golden for this architecture, so there is nothing to compare it
with but the cited lines themselves.
"""
from __future__ import annotations

import json
import math
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

# --------------------------------------------------------------------------
# configuration and weights, read independently of the product's loader
# --------------------------------------------------------------------------


@dataclass
class PlainConfig:
    """Hyper-parameters, named as in ``Qwen3Config``
    (crates/bfi-models/src/qwen3.rs:26-38) with the config.json key each is read from."""

    n_layer: int          # num_hidden_layers
    n_embd: int           # hidden_size
    n_ff: int             # intermediate_size
    n_vocab: int          # vocab_size
    n_ctx: int            # max_position_embeddings
    n_head: int           # num_attention_heads
    n_head_kv: int        # num_key_value_heads (default: n_head, qwen3.rs:334-337)
    head_dim: int         # head_dim (default n_embd / n_head, qwen3.rs:343-348)
    rms_eps: float        # rms_norm_eps (default 1e-6, qwen3.rs:349-351)
    rope_freq_base: float  # rope_theta (default 1e6, qwen3.rs:352)
    tied: bool            # tie_word_embeddings (reference: absence of output.weight, qwen3.rs:144)
    windows: List[Optional[int]]  # per layer; None = all keys (the reference has no window)

    @staticmethod
    def from_dict(d: dict) -> "PlainConfig":
        n_layer = int(d["num_hidden_layers"])
        n_head = int(d["num_attention_heads"])
        n_embd = int(d["hidden_size"])
        windows: List[Optional[int]] = [None] * n_layer
        if d.get("use_sliding_window") and d.get("sliding_window"):
            w = int(d["sliding_window"])
            kinds = d.get("layer_types")
            first = int(d.get("max_window_layers", n_layer))
            for i in range(n_layer):
                sliding = (kinds[i] == "sliding_attention") if kinds else (i >= first)
                windows[i] = w if sliding else None
        return PlainConfig(
            n_layer=n_layer,
            n_embd=n_embd,
            n_ff=int(d["intermediate_size"]),
            n_vocab=int(d["vocab_size"]),
            n_ctx=int(d["max_position_embeddings"]),
            n_head=n_head,
            n_head_kv=int(d.get("num_key_value_heads", n_head)),
            head_dim=int(d.get("head_dim", n_embd // n_head)),
            rms_eps=float(d.get("rms_norm_eps", 1e-6)),
            rope_freq_base=float(d.get("rope_theta", 1_000_000.0)),
            tied=bool(d.get("tie_word_embeddings", False)),
            windows=windows,
        )


_ST_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of one safetensors file, in their stored dtype."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    base = 8 + n
    out: Dict[str, torch.Tensor] = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt, _ = _ST_DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        buf = bytearray(raw[base + b:base + e])
        t = torch.frombuffer(buf, dtype=dt) if e > b else torch.empty(0, dtype=dt)
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_folder(folder: str, dtype: torch.dtype = torch.float32):
    """(config, weights widened to ``dtype``) of a model folder."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = PlainConfig.from_dict(json.load(f))
    w = {k: v.to(dtype) for k, v in read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    return cfg, w


# --------------------------------------------------------------------------
# the parts
# --------------------------------------------------------------------------


def embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """``x[t,:] = E[id_t,:]``; ids outside ``[0, V)`` are an error
    (crates/bfi-core/src/cpu.rs:402-438, range check :795-801)."""
    n_vocab = table.shape[0]
    for i in ids:
        if not 0 <= int(i) < n_vocab:
            raise ValueError(f"get_rows: id {i} out of range for n_vocab {n_vocab}")
    return table[torch.tensor(list(ids), dtype=torch.long)].clone()


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``y_j = x_j * (mean(x^2) + eps)^(-1/2) * w_j`` over the last dim; the weight
    multiplies as stored (no ``1 + w``) and eps sits inside the square root
    (crates/bfi-core/src/cpu.rs:92-122)."""
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    scale = 1.0 / torch.sqrt(mean_sq + eps)
    return x * scale * weight


def linear(w: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``y[t,o] = sum_e W[o,e] * x[t,e]``, no bias
    (crates/bfi-core/src/cpu.rs:78-90, 498-514)."""
    return x @ w.t()


def rope_neox(x: torch.Tensor, pos: Sequence[int], freq_base: float) -> torch.Tensor:
    """Rotate-half (NEOX) rotary encoding over the whole head: for ``i < d/2``,
    ``theta = pos / base^(2i/d)`` and ``(x_i, x_{i+d/2})`` turns by ``theta``
    (crates/bfi-core/src/cpu.rs:650-670; called with n_rot = head_dim, freq_scale 1,
    attn_factor 1 from crates/bfi-models/src/qwen3.rs:150-163).  The reference evaluates
    the angle in f32; here it is evaluated in float64 and rounded once."""
    t, _, d = x.shape
    half = d // 2
    i = torch.arange(half, dtype=torch.float64)
    p = torch.tensor(list(pos), dtype=torch.float64)
    theta = p[:, None] / torch.pow(torch.tensor(freq_base, dtype=torch.float64), 2.0 * i / d)[None, :]
    cos = torch.cos(theta).to(x.dtype)[:, None, :]
    sin = torch.sin(theta).to(x.dtype)[:, None, :]
    x0 = x[..., :half]
    x1 = x[..., half:2 * half]
    out = x.clone()
    out[..., :half] = x0 * cos - x1 * sin
    out[..., half:2 * half] = x0 * sin + x1 * cos
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              window: Optional[int] = None) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    ``q [T,hq,d]``, ``k,v [T,hkv,d]``; query head ``h`` reads kv head ``h // (hq/hkv)``;
    score ``q.k / sqrt(d)`` for keys ``s <= t``; max-subtracted softmax; weighted sum of V
    (crates/bfi-core/src/cpu.rs:328-392: scale :345, head map :344-349, mask :356-359,
    softmax :366-379, PV :381-388).  ``window`` (not in the reference) keeps only the last
    ``window`` keys, ``t - window < s <= t``."""
    tq, hq, d = q.shape
    tk, hkv, _ = k.shape
    assert tq == tk and hq % hkv == 0
    reps = hq // hkv
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    s_idx = torch.arange(tk)
    for h in range(hq):
        kh = k[:, h // reps, :]
        vh = v[:, h // reps, :]
        scores = (q[:, h, :] @ kh.t()) * scale            # [tq, tk]
        t_idx = torch.arange(tq)[:, None]
        masked = s_idx[None, :] > t_idx
        if window is not None:
            masked = masked | (s_idx[None, :] <= t_idx - window)
        scores = scores.masked_fill(masked, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ vh
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """``x * sigmoid(x)`` (crates/bfi-core/src/cpu.rs:708-720)."""
    return x * torch.sigmoid(x)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` (crates/bfi-core/src/cpu.rs:169-180)."""
    return silu(gate) * up


def attention_half(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, cfg: PlainConfig,
                   pos: Sequence[int], window: Optional[int]) -> torch.Tensor:
    """Pre-norm attention half of a block, with the residual add
    (crates/bfi-models/src/qwen3.rs:217-242)."""
    t = x.shape[0]
    h = rms_norm(x, w[p + "input_layernorm.weight"], cfg.rms_eps)
    q = linear(w[p + "self_attn.q_proj.weight"], h).reshape(t, cfg.n_head, cfg.head_dim)
    k = linear(w[p + "self_attn.k_proj.weight"], h).reshape(t, cfg.n_head_kv, cfg.head_dim)
    v = linear(w[p + "self_attn.v_proj.weight"], h).reshape(t, cfg.n_head_kv, cfg.head_dim)
    q = rms_norm(q, w[p + "self_attn.q_norm.weight"], cfg.rms_eps)
    k = rms_norm(k, w[p + "self_attn.k_norm.weight"], cfg.rms_eps)
    q = rope_neox(q, pos, cfg.rope_freq_base)
    k = rope_neox(k, pos, cfg.rope_freq_base)
    a = attention(q, k, v, window).reshape(t, cfg.n_head * cfg.head_dim)
    return x + linear(w[p + "self_attn.o_proj.weight"], a)


def mlp_half(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, cfg: PlainConfig) -> torch.Tensor:
    """Pre-norm SwiGLU half of a block, with the residual add
    (crates/bfi-models/src/qwen3.rs:244-250)."""
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.rms_eps)
    g = linear(w[p + "mlp.gate_proj.weight"], h)
    u = linear(w[p + "mlp.up_proj.weight"], h)
    return x + linear(w[p + "mlp.down_proj.weight"], swiglu(g, u))


def hidden(w: Dict[str, torch.Tensor], cfg: PlainConfig, tokens: Sequence[int]) -> torch.Tensor:
    """Every block over one whole sequence starting at position 0
    (crates/bfi-models/src/qwen3.rs:190-255)."""
    if len(tokens) == 0:
        raise ValueError("forward: empty token list")
    if len(tokens) > cfg.n_ctx:
        raise ValueError(f"forward: KV overflow n=0 + t={len(tokens)} > n_ctx={cfg.n_ctx}")
    pos = list(range(len(tokens)))
    x = embedding(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg.n_layer):
        p = f"model.layers.{i}."
        x = attention_half(x, w, p, cfg, pos, cfg.windows[i])
        x = mlp_half(x, w, p, cfg)
    return x


def head(w: Dict[str, torch.Tensor], cfg: PlainConfig, x: torch.Tensor) -> torch.Tensor:
    """Output norm and lm_head over every given row; the head is the embedding table
    when tied (crates/bfi-models/src/qwen3.rs:184-186, 258-266)."""
    h = rms_norm(x, w["model.norm.weight"], cfg.rms_eps)
    table = w["model.embed_tokens.weight"] if cfg.tied else w["lm_head.weight"]
    return linear(table, h)


def forward_each(w: Dict[str, torch.Tensor], cfg: PlainConfig, tokens: Sequence[int]) -> torch.Tensor:
    """Logits ``[T, V]`` at every position (crates/bfi-models/src/qwen3.rs:306-314)."""
    return head(w, cfg, hidden(w, cfg, tokens))


# --------------------------------------------------------------------------
# sampling and generation
# --------------------------------------------------------------------------


@dataclass
class PlainSampleParams:
    """crates/bfi-runtime/src/sample.rs:10-50 (the options that are in scope)."""

    max_tokens: int = 256
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    presence_penalty: float = 0.0
    seed: int = 0


def argmax_first(vals: Sequence[float]) -> int:
    """First maximum wins (strict ``>`` scan, crates/bfi-runtime/src/sample.rs:429-439)."""
    best_i, best_v = 0, float("-inf")
    for i, v in enumerate(vals):
        if v > best_v:
            best_v, best_i = v, i
    return best_i


def target(logits: Sequence[float], prev: Sequence[int], p: PlainSampleParams):
    """The distribution a token is drawn from: either ``("token", id)`` or
    ``("weights", [(id, weight), ...])`` (crates/bfi-runtime/src/sample.rs:326-427)."""
    f32 = torch.float32
    vals = torch.tensor(list(logits), dtype=f32).clone()
    ids = list(range(len(vals)))
    seen = set(int(t) for t in prev)
    if abs(p.repeat_penalty - 1.0) > 1.1920929e-07 and seen:       # :345-357
        for i in seen:
            if 0 <= i < len(vals):
                vals[i] = vals[i] / p.repeat_penalty if vals[i] > 0 else vals[i] * p.repeat_penalty
    if p.presence_penalty != 0.0 and seen:                         # :359-367
        for i in seen:
            if 0 <= i < len(vals):
                vals[i] = vals[i] - p.presence_penalty
    if p.temperature <= 0.0:                                       # :369-371
        return ("token", argmax_first(vals.tolist()))
    vals = vals / p.temperature                                    # :373-375
    vals = torch.exp(vals - vals.max())                            # :377-390
    s = vals.sum()
    if s > 0:
        vals = vals / s
    pairs = list(zip(ids, vals.tolist()))
    if p.top_k > 0 and p.top_k < len(pairs):                       # :392-395
        pairs.sort(key=lambda kv: -kv[1])
        pairs = pairs[:p.top_k]
    if p.top_p < 1.0:                                              # :397-409
        pairs.sort(key=lambda kv: -kv[1])
        cum, cut = 0.0, len(pairs)
        for i, (_, pr) in enumerate(pairs):
            cum += pr
            if cum >= p.top_p:
                cut = i + 1
                break
        pairs = pairs[:max(cut, 1)]
    if p.min_p > 0.0:                                              # :411-424
        max_p = max(pr for _, pr in pairs)
        pairs = [(i, pr) for i, pr in pairs if pr >= p.min_p * max_p]
        if not pairs:
            return ("token", argmax_first(list(logits)))
    return ("weights", pairs)


def draw(pairs, u: float) -> int:
    """Inverse CDF over ``(id, weight)`` in list order at ``u`` in ``[0,1)``
    (crates/bfi-runtime/src/sample.rs:312-323)."""
    total = sum(pr for _, pr in pairs)
    r = u * max(total, 0.0)
    cum = 0.0
    for i, pr in pairs:
        cum += pr
        if r <= cum:
            return i
    return pairs[-1][0] if pairs else 0


def xorshift_unit(state: int) -> float:
    """One step of the reference generator and its map to ``[0,1)``:
    ``x ^= x<<13; x ^= x>>7; x ^= x<<17; u = (x >> 40) / 2^24``, zero state replaced by a
    constant (crates/bfi-runtime/src/sample.rs:442-460)."""
    mask = (1 << 64) - 1
    x = state & mask
    if x == 0:
        x = 0x9E3779B97F4A7C15
    x ^= (x << 13) & mask
    x ^= x >> 7
    x ^= (x << 17) & mask
    return float(x >> 40) / float(1 << 24)


def greedy_generate(w, cfg: PlainConfig, prompt: Sequence[int], max_tokens: int,
                    stop_ids: Sequence[int] = ()) -> List[int]:
    """Greedy decoding by recomputing the whole sequence for every token; a stop token
    ends the sequence and is not appended (crates/bfi-runtime/src/engine/mod.rs:410-462)."""
    ids = list(prompt)
    out: List[int] = []
    while len(out) < max_tokens and len(ids) < cfg.n_ctx:
        logits = forward_each(w, cfg, ids)[-1]
        nxt = argmax_first(logits.tolist())
        if nxt in stop_ids:
            break
        out.append(nxt)
        ids.append(nxt)
    return out
