"""Typed Python faces of the exported kernels: they check devices, dtypes, shapes and strides of
torch tensors, then pass raw pointers and the current CUDA stream to the library.

Nothing here computes anything, and nothing falls back to another implementation.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from .library import KernelError, library

EPI_STORE = 0
EPI_ACCUMULATE = 1
EPI_SWIGLU = 2

FLAG_WRITE_CACHE = 1
FLAG_K_IN_PLACE = 2

STATUS_BAD_TOKEN = 1
STATUS_NO_PAGE = 2
STATUS_BAD_POSITION = 4


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return 0
    if dt == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 storage, not {dt}")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current CUDA stream of the current device, as a handle for the launchers."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must live on the GPU; there is no CPU path")


def _rows_2d(t: torch.Tensor, what: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what} must be 2-D with unit stride along the last dim, got shape "
                          f"{tuple(t.shape)} strides {t.stride()}")


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{what} must be a contiguous int32 tensor")


def convert(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A contiguous copy of ``src`` (float32 or bfloat16, on the GPU) in ``dtype``; rounding to
    bfloat16 is to nearest even."""
    _need_cuda(src)
    src = src.contiguous()
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    with torch.cuda.device(src.device):
        library("core").call("bfi_convert", _ptr(src), c_int(dtype_code(src.dtype)), _ptr(out),
                             c_int(dtype_code(dtype)), c_long(src.numel()), _stream())
    return out


def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor,
               status: Optional[torch.Tensor] = None) -> None:
    _need_cuda(table, ids, out, status)
    _rows_2d(table, "embedding table")
    _rows_2d(out, "embedding output")
    _i32(ids, "token ids")
    if out.dtype != torch.float32 or not out.is_contiguous() or out.shape != (ids.numel(), table.shape[1]):
        raise KernelError("embedding output must be contiguous float32 [tokens, width]")
    if not table.is_contiguous():
        raise KernelError("embedding table must be contiguous")
    library("core").call("bfi_embed_rows", _ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), _ptr(out),
                         c_int(ids.numel()), c_int(table.shape[1]), c_int(table.shape[0]), _ptr(status), _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """``out[r] = norm(x[rows[r]]) * w`` (``rows`` None: every row in order)."""
    _need_cuda(x, w, out, rows)
    _rows_2d(x, "norm input")
    _rows_2d(out, "norm output")
    _i32(rows, "row indices")
    width = x.shape[1]
    n_rows = rows.numel() if rows is not None else x.shape[0]
    if w.dim() != 1 or w.shape[0] != width or not w.is_contiguous():
        raise KernelError(f"norm weight must be [{width}], got {tuple(w.shape)}")
    if out.shape != (n_rows, width):
        raise KernelError(f"norm output must be [{n_rows}, {width}], got {tuple(out.shape)}")
    library("core").call("bfi_rmsnorm", _ptr(x), c_int(dtype_code(x.dtype)), c_long(x.stride(0)), _ptr(rows),
                         _ptr(w), c_int(dtype_code(w.dtype)), _ptr(out), c_int(dtype_code(out.dtype)),
                         c_long(out.stride(0)), c_int(n_rows), c_int(width), c_float(eps), _stream())


def silu_mul(gu: torch.Tensor, out: torch.Tensor, interleaved: bool) -> None:
    _need_cuda(gu, out)
    _rows_2d(gu, "gate/up input")
    _rows_2d(out, "gated output")
    if gu.dtype != out.dtype or gu.shape[0] != out.shape[0] or gu.shape[1] != 2 * out.shape[1]:
        raise KernelError("silu_mul: input must be [rows, 2*width] and output [rows, width] of one dtype")
    library("core").call("bfi_silu_mul", _ptr(gu), c_long(gu.stride(0)), _ptr(out), c_long(out.stride(0)),
                         c_int(dtype_code(gu.dtype)), c_int(gu.shape[0]), c_int(out.shape[1]),
                         c_int(1 if interleaved else 0), _stream())


def residual_add(x: torch.Tensor, y: torch.Tensor) -> None:
    _need_cuda(x, y)
    if x.dtype != torch.float32 or not x.is_contiguous() or not y.is_contiguous() or x.shape != y.shape:
        raise KernelError("residual_add: x must be contiguous float32 and y contiguous of the same shape")
    library("core").call("bfi_residual_add", _ptr(x), _ptr(y), c_int(dtype_code(y.dtype)), c_long(x.numel()),
                         _stream())


def qk_norm_rope_cache(qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                       q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                       rope_table: Optional[torch.Tensor], rot_dim: int,
                       token_pos: torch.Tensor, token_slot: torch.Tensor, kv, flags: int,
                       status: Optional[torch.Tensor] = None) -> None:
    """``kv`` is a ``KVView`` or None; ``rope_table`` is float32 ``[positions, rot_dim/2, 2]``."""
    _need_cuda(qkv, q_norm_w, k_norm_w, rope_table, token_pos, token_slot, status)
    _rows_2d(qkv, "qkv")
    _i32(token_pos, "token positions")
    _i32(token_slot, "token slots")
    n_tokens = qkv.shape[0]
    if token_pos.numel() < n_tokens or token_slot.numel() < n_tokens:
        raise KernelError("qk_norm_rope_cache: position/slot arrays shorter than the tokens")
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError(f"qkv row must hold ({n_q}+2*{n_kv})*{head_dim} values, got {qkv.shape[1]}")
    norm_dt = 0
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            if w.shape != (head_dim,) or not w.is_contiguous():
                raise KernelError(f"q/k norm weight must be [{head_dim}]")
            norm_dt = dtype_code(w.dtype)
    if q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype:
        raise KernelError("q and k norm weights must share a dtype")
    positions = 0
    if rope_table is not None:
        if rope_table.dtype != torch.float32 or not rope_table.is_contiguous() or rope_table.dim() != 3 \
                or rope_table.shape[1] != rot_dim // 2 or rope_table.shape[2] != 2:
            raise KernelError("rotation table must be contiguous float32 [positions, rot_dim/2, 2]")
        positions = rope_table.shape[0]
    k_pages = v_pages = table = None
    stride = 0
    if kv is not None and (flags & FLAG_WRITE_CACHE):
        if kv.k.dtype != qkv.dtype or kv.n_kv_heads != n_kv or kv.head_dim != head_dim:
            raise KernelError("cache pages do not fit the heads being written")
        k_pages, v_pages, table = kv.k, kv.v, kv.block_table
        stride = table.stride(0)
    library("core").call(
        "bfi_qk_norm_rope_cache", _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_long(qkv.stride(0)), c_int(n_tokens),
        c_int(n_q), c_int(n_kv), c_int(head_dim), _ptr(q_norm_w), _ptr(k_norm_w), c_int(norm_dt), c_float(eps),
        _ptr(rope_table), c_int(rot_dim), c_int(positions), _ptr(token_pos), _ptr(token_slot), _ptr(k_pages),
        _ptr(v_pages), _ptr(table), c_int(stride), c_int(flags), _ptr(status), _stream())


def attention_paged(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv, cu_seqlens: torch.Tensor,
                    seq_slot: torch.Tensor, seq_start: torch.Tensor, n_seqs: int, max_tokens: int,
                    n_q: int, scale: float) -> None:
    """``q`` is the first query element of the step (a view into the qkv buffer); token ``t``, head
    ``h`` lies at ``q + t*q_stride + h*head_dim``.  ``out`` is ``[tokens, n_q*head_dim]``."""
    _need_cuda(q, out, cu_seqlens, seq_slot, seq_start)
    _rows_2d(out, "attention output")
    _i32(cu_seqlens, "cu_seqlens")
    _i32(seq_slot, "sequence slots")
    _i32(seq_start, "sequence starts")
    if q.dtype != out.dtype or kv.k.dtype != q.dtype:
        raise KernelError("attention: q, output and cache must share a dtype")
    library("core").call(
        "bfi_attention_paged", _ptr(q), c_int(dtype_code(q.dtype)), c_long(q_stride), _ptr(out),
        c_long(out.stride(0)), _ptr(kv.k), _ptr(kv.v), _ptr(kv.block_table), c_int(kv.block_table.stride(0)),
        _ptr(cu_seqlens), _ptr(seq_slot), _ptr(seq_start), c_int(n_seqs), c_int(max_tokens), c_int(n_q),
        c_int(kv.n_kv_heads), c_int(kv.head_dim), c_int(kv.window or 0), c_float(scale), _stream())


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """``out = a @ w.T`` on the CUDA cores in float32 arithmetic (any dtypes, any sizes)."""
    _need_cuda(a, w, out)
    _rows_2d(a, "A")
    _rows_2d(w, "W")
    _rows_2d(out, "C")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"matrix product: A is {tuple(a.shape)} but W is {tuple(w.shape)}")
    cols = n // 2 if epilogue == EPI_SWIGLU else n
    if out.shape != (m, cols):
        raise KernelError(f"matrix product: output must be [{m}, {cols}], got {tuple(out.shape)}")
    library("core").call("bfi_gemm_simt", _ptr(a), c_int(dtype_code(a.dtype)), c_long(a.stride(0)), _ptr(w),
                         c_int(dtype_code(w.dtype)), c_long(w.stride(0)), _ptr(out), c_int(dtype_code(out.dtype)),
                         c_long(out.stride(0)), c_int(m), c_int(n), c_int(k), c_int(epilogue), _stream())


def argmax_rows(logits: torch.Tensor, out: torch.Tensor, scratch: Optional[torch.Tensor] = None) -> None:
    """``scratch`` (int32 or float32, at least ``2 * rows * ceil(vocab / 8192)`` values) lets many
    blocks search each row of a large vocabulary."""
    _need_cuda(logits, out, scratch)
    _rows_2d(logits, "logits")
    _i32(out, "argmax output")
    if logits.dtype != torch.float32 or out.numel() < logits.shape[0]:
        raise KernelError("argmax: logits must be float32 and the output hold one id per row")
    n_scratch = 0
    if scratch is not None:
        if scratch.element_size() != 4 or not scratch.is_contiguous():
            raise KernelError("argmax: scratch must be a contiguous tensor of 4-byte values")
        n_scratch = scratch.numel()
    library("core").call("bfi_argmax_rows", _ptr(logits), c_long(logits.stride(0)), c_int(logits.shape[0]),
                         c_int(logits.shape[1]), _ptr(out), _ptr(scratch), c_long(n_scratch), _stream())


def sample_sorted_rows(logits: torch.Tensor, temperature: torch.Tensor, u: torch.Tensor, out: torch.Tensor,
                       probs: torch.Tensor, top_k: int = 0, top_p: float = 1.0, repeat_penalty: float = 1.0,
                       presence_penalty: float = 0.0, min_p: float = 0.0, seen: Optional[torch.Tensor] = None,
                       seen_cu: Optional[torch.Tensor] = None, work: Optional[torch.Tensor] = None) -> None:
    """Top-k / top-p sampling in the reference's order (probability descending, index ascending)
    without a sort; ``probs`` is float32 scratch ``[rows, vocab]``."""
    _need_cuda(logits, temperature, u, out, probs, seen, seen_cu, work)
    _rows_2d(logits, "logits")
    _i32(out, "sample output")
    _i32(seen, "seen ids")
    _i32(seen_cu, "seen offsets")
    rows, vocab = logits.shape
    for t, what in ((temperature, "temperature"), (u, "uniform draws")):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() < rows:
            raise KernelError(f"{what} must be contiguous float32 with one value per row")
    if logits.dtype != torch.float32 or out.numel() < rows:
        raise KernelError("sample: logits must be float32 and the output hold one id per row")
    for buf, what in ((probs, "probability"), (work, "work")):
        if buf is not None and (buf.dtype != torch.float32 or not buf.is_contiguous() or buf.numel() < rows * vocab):
            raise KernelError(f"sample: {what} buffer must be contiguous float32 [rows, vocab]")
    library("core").call("bfi_sample_sorted_rows", _ptr(logits), c_long(logits.stride(0)), _ptr(work), _ptr(probs),
                         c_int(rows), c_int(vocab), _ptr(seen), _ptr(seen_cu), _ptr(temperature), _ptr(u),
                         c_float(repeat_penalty), c_float(presence_penalty), c_int(int(top_k)), c_float(top_p),
                         c_float(min_p), _ptr(out), _stream())


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, u: torch.Tensor, out: torch.Tensor,
                repeat_penalty: float = 1.0, presence_penalty: float = 0.0, min_p: float = 0.0,
                seen: Optional[torch.Tensor] = None, seen_cu: Optional[torch.Tensor] = None,
                work: Optional[torch.Tensor] = None) -> None:
    _need_cuda(logits, temperature, u, out, seen, seen_cu, work)
    _rows_2d(logits, "logits")
    _i32(out, "sample output")
    _i32(seen, "seen ids")
    _i32(seen_cu, "seen offsets")
    rows, vocab = logits.shape
    for t, what in ((temperature, "temperature"), (u, "uniform draws")):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() < rows:
            raise KernelError(f"{what} must be contiguous float32 with one value per row")
    if logits.dtype != torch.float32 or out.numel() < rows:
        raise KernelError("sample: logits must be float32 and the output hold one id per row")
    if work is not None and (work.dtype != torch.float32 or not work.is_contiguous() or work.numel() < rows * vocab):
        raise KernelError("sample: work buffer must be contiguous float32 [rows, vocab]")
    library("core").call("bfi_sample_rows", _ptr(logits), c_long(logits.stride(0)), _ptr(work), c_int(rows),
                         c_int(vocab), _ptr(seen), _ptr(seen_cu), _ptr(temperature), _ptr(u),
                         c_float(repeat_penalty), c_float(presence_penalty), c_float(min_p), _ptr(out), _stream())
