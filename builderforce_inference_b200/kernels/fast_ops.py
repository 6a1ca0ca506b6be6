"""Faces of the bfloat16 kernels of the ``fast`` library.  Each returns False when it does not
take the shape (the caller then uses the general kernel); it never computes a wrong result.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_long

import torch

from .library import KernelError, library
from .ops import _ptr, _rows_2d, _stream, dtype_code

SKINNY_MAX_ROWS = 64

_sm_count = {}


def sm_count(device=None) -> int:
    """Multiprocessors of ``device`` (the current one by default), asked of the driver once."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    n = _sm_count.get(index)
    if n is None:
        with torch.cuda.device(index):
            n = int(library("fast").lib.bfi_device_sm_count())
        _sm_count[index] = n
    return n


class _SplitScratch:
    """Scratch of the weight streamer when it splits K between blocks: float32 partial sums and one
    counter per tile.  The counters start at zero and every launch leaves them at zero.  Buffers
    only ever grow, and outgrown ones are kept alive, because captured graphs hold their addresses.
    One stream at a time may use them."""

    def __init__(self):
        self.floats = {}
        self.counters = {}
        self.retired = []

    def get(self, device, n_floats: int, n_counters: int):
        f = self.floats.get(device)
        if f is None or f.numel() < n_floats:
            if f is not None:
                self.retired.append(f)
            f = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
            self.floats[device] = f
        c = self.counters.get(device)
        if c is None or c.numel() < n_counters:
            if c is not None:
                self.retired.append(c)
            c = torch.zeros(max(n_counters, 1 << 14), dtype=torch.int32, device=device)
            self.counters[device] = c
        return f, c


_split_scratch = _SplitScratch()
_plan_cache = {}


_tc_status = {}


def tc_status(device) -> torch.Tensor:
    """The word in which the tcgen05 kernels record a bounded wait that ran out (bit 8), followed
    by the prompt attention's two counters (tickets drawn, blocks finished; zero between launches)."""
    t = _tc_status.get(device)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=device)
        _tc_status[device] = t
    return t


def _check_product(a, w, out, epilogue):
    m, k = a.shape
    n = w.shape[0]
    _rows_2d(a, "A")
    _rows_2d(w, "W")
    _rows_2d(out, "C")
    cols = n // 2 if epilogue == 2 else n
    if w.shape[1] != k or out.shape != (m, cols):
        raise KernelError(f"matrix product: A {tuple(a.shape)}, W {tuple(w.shape)}, output {tuple(out.shape)}")
    return m, n, k


def _scratch_for(func: str, m: int, n: int, k: int, device):
    key = (func, m, n, k)
    need = _plan_cache.get(key)
    if need is None:
        sizes = (c_long * 2)()
        getattr(library("fast").lib, func)(c_int(m), c_int(n), c_int(k), sizes)
        need = (int(sizes[0]), int(sizes[1]))
        _plan_cache[key] = need
    if need[0] == 0:
        return None, None
    return _split_scratch.get(device, need[0], need[1])


def _skinny_scratch_need(m: int, n: int, k: int):
    key = ("bfi_skinny_gemm_scratch", m, n, k)
    if key not in _plan_cache:
        sizes = (c_long * 2)()
        library("fast").lib.bfi_skinny_gemm_scratch(c_int(m), c_int(n), c_int(k), sizes)
        _plan_cache[key] = (int(sizes[0]), int(sizes[1]))
    return _plan_cache[key]


def skinny_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> bool:
    """The weight streamer (mma.sync), up to 64 rows."""
    m, n, k = _check_product(a, w, out, epilogue)
    if m > SKINNY_MAX_ROWS:
        return False
    scratch, counters = _scratch_for("bfi_skinny_gemm_scratch", m, n, k, a.device)
    return library("fast").call_optional(
        "bfi_skinny_gemm_bf16", _ptr(a), c_long(a.stride(0)), _ptr(w), c_long(w.stride(0)), _ptr(out),
        c_int(dtype_code(out.dtype)), c_long(out.stride(0)), c_int(m), c_int(n), c_int(k), c_int(epilogue),
        _ptr(scratch), c_long(scratch.numel() if scratch is not None else 0), _ptr(counters),
        c_int(counters.numel() if counters is not None else 0), _stream())


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> bool:
    """The tcgen05 / TMA kernel, any number of rows."""
    m, n, k = _check_product(a, w, out, epilogue)
    return library("fast").call_optional(
        "bfi_gemm_tcgen05_bf16", _ptr(a), c_long(a.stride(0)), _ptr(w), c_long(w.stride(0)), _ptr(out),
        c_int(dtype_code(out.dtype)), c_long(out.stride(0)), c_int(m), c_int(n), c_int(k), c_int(epilogue),
        _ptr(tc_status(a.device)), _stream())


def gemm_tcgen05_wait_probe(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, spin_limit: int,
                            hold_producer: bool) -> bool:
    """The tcgen05 product with every bounded wait cut to ``spin_limit`` polls and, if asked, a
    producer that issues no copy: the consumers' waits then run out by construction, the launch
    records the time-out in ``tc_status`` and returns.  For the tests of that path."""
    m, n, k = _check_product(a, w, out, epilogue)
    return library("fast").call_optional(
        "bfi_gemm_tcgen05_bf16_wait_probe", _ptr(a), c_long(a.stride(0)), _ptr(w), c_long(w.stride(0)), _ptr(out),
        c_int(dtype_code(out.dtype)), c_long(out.stride(0)), c_int(m), c_int(n), c_int(k), c_int(epilogue),
        _ptr(tc_status(a.device)), c_int(int(spin_limit)), c_int(1 if hold_producer else 0), _stream())


_stream_sinks = {}


def weight_stream(w: torch.Tensor, stages: int = 6, ksplit: int = 1) -> bool:
    """Reads ``w`` once through the few-row products' TMA rings and does nothing with it: the time
    of this launch is the floor under a product of that shape (see ``csrc/weight_stream.cu``)."""
    if w.dtype != torch.bfloat16 or w.dim() != 2 or w.stride(1) != 1:
        raise KernelError("weight_stream wants a bfloat16 matrix with unit column stride")
    sink = _stream_sinks.get(w.device)
    if sink is None:
        sink = _stream_sinks[w.device] = torch.zeros(1, dtype=torch.int64, device=w.device)
    return library("fast").call_optional("bfi_weight_stream_bf16", _ptr(w), c_long(w.stride(0)), c_int(w.shape[0]),
                                         c_int(w.shape[1]), c_int(stages), c_int(ksplit), _ptr(tc_status(w.device)),
                                         _ptr(sink), _stream())


def linear_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> bool:
    """bfloat16 x bfloat16 -> ``out`` (float32 or bfloat16): the tcgen05 kernel, whose blocks start
    streaming W into their shared memory while the kernel before them still runs; the register-fed
    weight streamer for the shapes TMA cannot address; False if neither takes the shape."""
    if gemm_tcgen05(a, w, out, epilogue):
        return True
    if a.shape[0] <= SKINNY_MAX_ROWS:
        return skinny_gemm(a, w, out, epilogue)
    return False


DECODE_PAGES_PER_BLOCK = 24     # a block's range should not be much longer than this many pages


def decode_splits(n_seqs: int, n_kv: int, group: int, max_pages: int, n_sm: int) -> int:
    """Into how many page ranges every (sequence, kv head) is cut: enough blocks to fill the GPU
    once (two to three blocks are resident on an SM), and enough that no block walks a very long
    range alone (with many sequences one range each fills the GPU, but 64 pages in a row make a
    long tail); never more than a sequence can have pages.  Depends only on sizes that are fixed
    when a step is captured."""
    blocks = n_seqs * n_kv * ((group + 15) // 16)
    fill = (n_sm * 5 // 2 + blocks - 1) // blocks
    length = (max_pages + DECODE_PAGES_PER_BLOCK - 1) // DECODE_PAGES_PER_BLOCK
    return max(1, min(max(fill, length), max_pages, 32))


def attention_decode_bf16(ctx, qkv: torch.Tensor, out: torch.Tensor, kv, n_heads: int, scale: float,
                          probe=None) -> bool:
    """One new token per sequence over its cached pages, which arrive by TMA: the cache must be
    contiguous.  A wait for a page that ran out shows in ``tc_status``.  ``probe``: (polls, hold
    the producer), for ``attention_decode_wait_probe``."""
    d = kv.head_dim
    if d not in (64, 128) or qkv.dtype != torch.bfloat16 or kv.k.dtype != torch.bfloat16:
        return False
    if not kv.k.is_contiguous() or not kv.v.is_contiguous():
        return False
    max_pages = kv.block_table.shape[1]
    bucket = getattr(ctx, "pages_bucket", 0)
    if bucket:
        max_pages = min(max_pages, bucket)           # what the step's sequences hold now, rounded up
    if kv.window:
        max_pages = min(max_pages, (kv.window + 62) // 64 + 1)
    group = n_heads // kv.n_kv_heads
    max_splits = decode_splits(ctx.n_seqs, kv.n_kv_heads, group, max_pages, sm_count(qkv.device))
    part_o = part_ml = None
    if max_splits > 1:
        part_o = ctx.workspace.vector("attn.part_o", ctx.n_seqs * n_heads * max_splits * d, torch.float32)
        part_ml = ctx.workspace.vector("attn.part_ml", ctx.n_seqs * n_heads * max_splits * 2, torch.float32)
    args = [_ptr(qkv), c_long(qkv.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(kv.k), _ptr(kv.v),
            c_long(kv.k.shape[0]), _ptr(kv.block_table), c_int(kv.block_table.stride(0)), _ptr(ctx.seq_slot),
            _ptr(ctx.seq_start), c_int(ctx.n_seqs), c_int(n_heads), c_int(kv.n_kv_heads), c_int(d), c_int(kv.window or 0),
            c_float(scale), c_int(max_splits), _ptr(part_o), _ptr(part_ml), _ptr(tc_status(qkv.device))]
    if probe is None:
        return library("fast").call_optional("bfi_attention_decode_bf16", *args, _stream())
    return library("fast").call_optional("bfi_attention_decode_bf16_wait_probe", *args, c_int(int(probe[0])),
                                         c_int(1 if probe[1] else 0), _stream())


def attention_decode_wait_probe(ctx, qkv: torch.Tensor, out: torch.Tensor, kv, n_heads: int, scale: float,
                                spin_limit: int, hold_producer: bool) -> bool:
    """The decode attention with its bounded waits cut to ``spin_limit`` polls and, if asked, a
    thread that asks for no page: see ``gemm_tcgen05_wait_probe``."""
    return attention_decode_bf16(ctx, qkv, out, kv, n_heads, scale, probe=(spin_limit, hold_producer))


def attention_prefill_bf16(ctx, qkv: torch.Tensor, out: torch.Tensor, kv, n_heads: int, scale: float) -> bool:
    """Tensor-core attention for steps that bring more than one token per sequence."""
    d = kv.head_dim
    if d not in (64, 128) or qkv.dtype != torch.bfloat16 or kv.k.dtype != torch.bfloat16:
        return False
    return library("fast").call_optional(
        "bfi_attention_prefill_bf16", _ptr(qkv), c_long(qkv.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(kv.k),
        _ptr(kv.v), _ptr(kv.block_table), c_int(kv.block_table.stride(0)), _ptr(ctx.cu_seqlens), _ptr(ctx.seq_slot),
        _ptr(ctx.seq_start), c_int(ctx.n_seqs), c_int(ctx.max_seq_tokens), c_int(n_heads), c_int(kv.n_kv_heads),
        c_int(d), c_int(kv.window or 0), c_float(scale), _stream())


TCGEN05_ATTENTION_MIN_TOKENS = 128     # shorter steps: the mma.sync kernel with 64-token tiles


def attention_prefill_tcgen05_bf16(ctx, qkv: torch.Tensor, out: torch.Tensor, kv, n_heads: int, scale: float) -> bool:
    """tcgen05 / TMA attention for steps with long runs of new tokens: one block per SM draws
    items of 128 tokens of one head, scores and output in tensor memory.  A wait that ran out
    shows in ``tc_status``."""
    d = kv.head_dim
    if d not in (64, 128) or qkv.dtype != torch.bfloat16 or kv.k.dtype != torch.bfloat16:
        return False
    if not kv.k.is_contiguous() or not kv.v.is_contiguous():
        return False
    return library("fast").call_optional(
        "bfi_attention_prefill_tcgen05_bf16", _ptr(qkv), c_long(qkv.stride(0)), _ptr(out), c_long(out.stride(0)),
        _ptr(kv.k), _ptr(kv.v), c_long(kv.k.shape[0]), _ptr(kv.block_table), c_int(kv.block_table.stride(0)),
        _ptr(ctx.cu_seqlens), _ptr(ctx.seq_slot), _ptr(ctx.seq_start), c_int(ctx.n_seqs), c_long(qkv.shape[0]),
        c_int(ctx.max_seq_tokens), c_int(n_heads), c_int(kv.n_kv_heads), c_int(d), c_int(kv.window or 0), c_float(scale),
        _ptr(tc_status(qkv.device)), _stream())


def attention_prefill_tcgen05_wait_probe(ctx, qkv: torch.Tensor, out: torch.Tensor, kv, n_heads: int, scale: float,
                                         spin_limit: int, hold_producer: bool) -> bool:
    """The tcgen05 prompt attention with its bounded waits cut to ``spin_limit`` polls and, if asked,
    a producer warp that draws no item: see ``gemm_tcgen05_wait_probe``."""
    return library("fast").call_optional(
        "bfi_attention_prefill_tcgen05_bf16_wait_probe", _ptr(qkv), c_long(qkv.stride(0)), _ptr(out),
        c_long(out.stride(0)), _ptr(kv.k), _ptr(kv.v), c_long(kv.k.shape[0]), _ptr(kv.block_table),
        c_int(kv.block_table.stride(0)), _ptr(ctx.cu_seqlens), _ptr(ctx.seq_slot), _ptr(ctx.seq_start), c_int(ctx.n_seqs),
        c_long(qkv.shape[0]), c_int(ctx.max_seq_tokens), c_int(n_heads), c_int(kv.n_kv_heads), c_int(kv.head_dim),
        c_int(kv.window or 0), c_float(scale), _ptr(tc_status(qkv.device)), c_int(int(spin_limit)),
        c_int(1 if hold_producer else 0), _stream())
