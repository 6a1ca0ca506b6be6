"""The engine: a decoder, its cache, and ONE step function.

``Engine.step`` takes a batch of sequences, each with the next tokens it brings (a whole prompt,
a further piece of one, or a single token), runs exactly those tokens as one packed batch from
the cache that earlier steps left, and returns float32 logits at the wanted places.  It is what
generation, trace replay, the benchmark and the tests all drive; there is no second forward pass.

The reference's counterpart is ``Model::forward`` / ``forward_each`` for one sequence
(crates/bfi-models/src/arch.rs:29-59; qwen3.rs:190-314) looped over by the runtime
(crates/bfi-runtime/src/engine/mod.rs:297-337); here the batch reaches the kernels.

Steps in which every sequence brings one token are captured in CUDA graphs, one per padded batch
size, when every part of the model is graph-safe.  Padding rows carry slot -1, which every kernel
skips, so padding changes no result.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.cache import SequenceCache
from ..cache.pages import PAGE_TOKENS, CacheError
from ..cache.plan import plan_cache
from ..config.base import read_json, stop_ids_of_folder
from ..kernels import ops
from ..kernels.library import total_calls
from ..parts.base import ModelSpec
from ..registry import describe_model
from ..weights.loader import load_folder
from ..weights.random_init import random_tensors
from .context import StepContext, Workspace
from .decoder import Decoder, Runtime, expected_tensors

PINNED_RING = 4          # pinned staging buffers per size of a step's index arrays


def pack_meta(dst: np.ndarray, tok, pos, slot_of, cu, n_tok: int, n_seq: int, seq_slots, seq_starts, pages: int,
              want_rows=()) -> int:
    """Write a step's index arrays into ``dst`` (int32) in the layout the kernels read:
    token_ids[T] token_pos[T] token_slot[T] cu_seqlens[B+1] seq_slot[B] seq_start[B] total_pages[1]
    want_rows[W], with T = n_tok and B = n_seq; rows and sequences past the real ones are padding
    (ids and positions 0, slots -1, cu_seqlens repeating the last offset).  Returns the count written."""
    k, b, last = len(tok), len(seq_slots), cu[-1]
    o = 0
    dst[o:o + k] = tok
    dst[o + k:o + n_tok] = 0
    o += n_tok
    dst[o:o + k] = pos
    dst[o + k:o + n_tok] = 0
    o += n_tok
    dst[o:o + k] = slot_of
    dst[o + k:o + n_tok] = -1
    o += n_tok
    dst[o:o + len(cu)] = cu
    dst[o + len(cu):o + n_seq + 1] = last
    o += n_seq + 1
    dst[o:o + b] = seq_slots
    dst[o + b:o + n_seq] = -1
    o += n_seq
    dst[o:o + b] = seq_starts
    dst[o + b:o + n_seq] = 0
    o += n_seq
    dst[o] = pages
    o += 1
    dst[o:o + len(want_rows)] = want_rows
    return o + len(want_rows)



class PinnedRings:
    """Page-locked staging buffers for the steps' index arrays: ``PINNED_RING`` buffers in rotation
    per capacity, capacities being powers of two (at least ``MIN_CAPACITY`` values).  However many
    distinct lengths are asked for, at most ``PINNED_RING * log2(largest / MIN_CAPACITY)`` buffers
    ever exist.  An entry is ``[buffer, event]``; ``take`` waits for the event of the entry it hands
    out, so a buffer is never rewritten while a copy still reads it."""

    MIN_CAPACITY = 64

    def __init__(self, make=None):
        self._rings: Dict[int, dict] = {}
        self._make = make or (lambda cap: torch.empty(cap, dtype=torch.int32, pin_memory=True))

    @classmethod
    def capacity_for(cls, n: int) -> int:
        cap = cls.MIN_CAPACITY
        while cap < n:
            cap *= 2
        return cap

    def take(self, n: int) -> list:
        ring = self._rings.setdefault(self.capacity_for(n), {"next": 0, "slots": []})
        if len(ring["slots"]) < PINNED_RING:
            ring["slots"].append([self._make(self.capacity_for(n)), None])
            return ring["slots"][-1]
        entry = ring["slots"][ring["next"]]
        ring["next"] = (ring["next"] + 1) % PINNED_RING
        if entry[1] is not None:
            entry[1].synchronize()
        return entry

    def n_buffers(self) -> int:
        return sum(len(r["slots"]) for r in self._rings.values())


DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class StepError(RuntimeError):
    """A step was refused before any launch, or a device-side check recorded a fault."""


@dataclass
class SequenceStep:
    """What one sequence brings to a step: its next tokens, and the places among them whose
    logits are wanted (indices into ``tokens``; may be empty)."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"run dtype must be bfloat16 or float32, got {name}")
        return name
    if name not in DTYPES:
        raise ValueError(f"run dtype must be one of {sorted(DTYPES)}, got {name!r}")
    return DTYPES[name]


def _require_gpu(device: torch.device) -> None:
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("this engine runs on an NVIDIA GPU only (sm_100a kernels); no CUDA device is available")


PAGE_BUCKETS_STEP = 4     # page-count buckets of single-token steps: 1, 4, 16, 64, ... pages per sequence


def pages_bucket(most_pages: int, limit: int) -> int:
    """The smallest bucket (a power of ``PAGE_BUCKETS_STEP``) that holds ``most_pages``, capped by
    the bucket that holds ``limit`` (the most pages a sequence can have)."""
    b = 1
    while b < most_pages and b < limit:
        b *= PAGE_BUCKETS_STEP
    return b


class _DecodeGraphs:
    """The captured single-token steps of one padded batch size: per page-count bucket (kernels
    cut their work by the most pages a sequence of the step holds) the step's stages, all over
    the same index arrays and logits.  A stage whose parts are all graph-safe is a CUDA graph; a
    stage with a part that is not (it reads the host's lists of slots and lengths, or launches
    shapes that depend on them) runs as it is written, between the graphs.  Every bucket is
    captured when the batch size is first seen, so no capture falls into the middle of a
    generation."""

    def __init__(self, engine: "Engine", batch: int):
        self.batch = batch
        dev = engine.device
        self.meta = torch.zeros(engine._meta_len(batch, batch, 0), dtype=torch.int32, device=dev)
        self.logits = torch.empty((batch, engine.spec.vocab_size), dtype=torch.float32, device=dev)
        self.rows = torch.arange(batch, dtype=torch.int32, device=dev)
        # every row starts as padding (slot -1), so the runs below touch no sequence's cache
        engine._fill_meta(self.meta, [], [], [], [0], batch, batch)
        self.stages = engine.decoder.stages()
        self.graphs: Dict[int, list] = {}           # bucket -> [CUDAGraph or None per stage]
        self.n_kernels: Dict[int, int] = {}
        limit = engine.cache.n_blocks
        buckets, b = [], 1
        while True:
            buckets.append(b)
            if b >= limit:
                break
            b *= PAGE_BUCKETS_STEP
        # eager runs first (no sequence: the host lists are empty): they load kernels, size the
        # workspace and set launch attributes
        for b in buckets:
            ctx = self.context(engine, b, ([], [], []))
            for _, ops in self.stages:
                self.run_ops(engine, ctx, ops)
        torch.cuda.synchronize(dev)
        self.stamp = engine._stamp()
        for b in buckets:
            ctx = self.context(engine, b, None)
            ctx.capturing = True
            graphs, count = [], 0
            for safe, ops in self.stages:
                if not safe:
                    graphs.append(None)
                    continue
                graph = torch.cuda.CUDAGraph()
                before = total_calls()
                with torch.cuda.graph(graph):
                    self.run_ops(engine, ctx, ops)
                count += total_calls() - before
                graphs.append(graph)
            self.graphs[b] = graphs
            self.n_kernels[b] = count                   # launches the replays of one step stand for

    def context(self, engine: "Engine", bucket: int, host) -> StepContext:
        ctx = engine._context_from_meta(self.meta, self.batch, self.batch, 1, host)
        ctx.pages_bucket = bucket
        return ctx

    def run_ops(self, engine: "Engine", ctx: StepContext, ops) -> None:
        x = ctx.rows("residual", engine.spec.width, torch.float32)
        for op in ops:
            if op[0] == "embed":
                engine.decoder.embed(ctx)
            elif op[0] == "runs":
                engine.decoder.run_layers(ctx, x, engine.cache, op[1], op[2])
            else:
                engine.decoder.logits(ctx, x, self.rows, self.logits)

    def replay(self, engine: "Engine", bucket: int, host) -> None:
        ctx = None
        for (safe, ops), graph in zip(self.stages, self.graphs[bucket]):
            if graph is not None:
                graph.replay()
            else:
                if ctx is None:
                    ctx = self.context(engine, bucket, host)
                self.run_ops(engine, ctx, ops)


class Engine:
    """A loaded model with its cache.  Build with ``Engine.load`` or ``Engine.from_random``."""

    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device, max_tokens: int, max_seq_len: Optional[int] = None,
                 use_graphs: bool = True, prefill_chunk_tokens: int = 8192,
                 config: Optional[Dict[str, Any]] = None, cache_bytes: Optional[int] = None,
                 cache_slots: int = 64):
        """``max_tokens`` sizes the cache in tokens (summed over live sequences, each rounded up to
        a page).  ``cache_bytes``, when given, sizes it from a byte budget instead: the tokens that
        fit beside the fixed-size state of ``cache_slots`` sequences (``cache.plan.plan_cache``)."""
        _require_gpu(device)
        self.spec = spec
        self.config = config
        self.dtype = dtype
        self.device = device
        self.runtime = Runtime(device, dtype)
        self.decoder = Decoder(spec, self.runtime)
        self.stop_ids = tuple(spec.stop_ids)      # a loaded folder may add its generation_config.json's
        self.cache_plan = None
        if cache_bytes is not None:
            self.cache_plan = plan_cache(self.decoder.run_needs(), self.decoder.run_cache_of(), int(cache_bytes),
                                         2 if dtype == torch.bfloat16 else 4, cache_slots)
            max_tokens = self.cache_plan.max_tokens
        limit = spec.max_positions if spec.max_positions > 0 else max_tokens
        self.max_seq_len = min(limit, max_seq_len) if max_seq_len else limit
        self.max_seq_len = max(1, min(self.max_seq_len,
                                      ((max_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS) * PAGE_TOKENS))
        self.decoder.load(tensors, self.max_seq_len)
        self.cache = SequenceCache(self.decoder.run_needs(), self.decoder.run_cache_of(), max_tokens,
                                   self.max_seq_len, dtype, device, initial_slots=max(1, int(cache_slots)))
        self.workspace = Workspace(device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.prefill_chunk_tokens = max(PAGE_TOKENS, int(prefill_chunk_tokens))
        # single-token steps are replayed from CUDA graphs, stage by stage: the stages whose parts are
        # all graph-safe (for a model of such parts only, the whole step is one graph)
        self.use_graphs = bool(use_graphs) and any(safe and any(op[0] == "runs" for op in ops)
                                                   for safe, ops in self.decoder.stages())
        self._graphs: Dict[int, _DecodeGraphs] = {}
        self._pinned = PinnedRings()
        self.last_h2d_bytes = 0        # bytes of index arrays the last step copied to the device
        self.graph_kernel_launches = 0  # kernels launched through graph replays so far

    # ---- construction ----------------------------------------------------------------
    @classmethod
    def load(cls, folder: str, dtype="bfloat16", max_tokens: int = 16384, max_seq_len: Optional[int] = None,
             device="cuda:0", **kw) -> "Engine":
        """Load ``folder`` (config.json + model.safetensors); the model class comes from config.json."""
        dt = parse_dtype(dtype)
        dev = torch.device(device)
        _require_gpu(dev)
        config = read_json(os.path.join(folder, "config.json"))
        spec = describe_model(config)
        tensors = load_folder(folder, expected_tensors(spec), spec.ignored_names, dt, dev)
        eng = cls(spec, tensors, dt, dev, max_tokens, max_seq_len, config=config, **kw)
        eng.stop_ids = stop_ids_of_folder(folder, spec.stop_ids)
        return eng

    @classmethod
    def from_random(cls, config: Dict[str, Any], seed: int, dtype="bfloat16", max_tokens: int = 16384,
                    max_seq_len: Optional[int] = None, device="cuda:0", **kw) -> "Engine":
        """Random weights made directly in device memory (same distributions as a written folder)."""
        dt = parse_dtype(dtype)
        dev = torch.device(device)
        _require_gpu(dev)
        spec = describe_model(config)
        tensors = dict(random_tensors(expected_tensors(spec), seed, dt, dev))
        return cls(spec, tensors, dt, dev, max_tokens, max_seq_len, config=config, **kw)

    # ---- slots -----------------------------------------------------------------------
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def rewind(self, slot: int, length: int) -> None:
        """Keep only the first ``length`` tokens of the sequence in ``slot``; the next step goes on
        from there (crates/bfi-models/src/session.rs:50-62).  Refused by name for models with
        windowed layers or per-sequence state of fixed size."""
        try:
            self.cache.rewind(slot, length)
        except CacheError as e:
            raise StepError(str(e)) from e

    # ---- the step function -----------------------------------------------------------
    def step(self, seqs: Sequence[SequenceStep], check: bool = True) -> torch.Tensor:
        """Run the given tokens of the given sequences as one batch; returns float32 logits
        ``[wanted, vocab]`` on the device, in the order of ``seqs`` and of each ``want``.
        The tensor is valid until the next call of ``step``."""
        if not seqs:
            raise StepError("a step needs at least one sequence")
        vocab = self.spec.vocab_size
        slots, counts = [], []
        for s in seqs:
            n = len(s.tokens)
            if n == 0:
                raise StepError(f"slot {s.slot}: empty token list")
            if n > 16:
                try:
                    arr = np.asarray(s.tokens, dtype=np.int64)
                except (OverflowError, ValueError, TypeError) as e:
                    raise StepError(f"slot {s.slot}: token ids must be integers below the vocabulary {vocab}: {e}") from e
                bad = np.nonzero((arr < 0) | (arr >= vocab))[0]
                if bad.size:
                    raise StepError(f"slot {s.slot}: token id {int(arr[bad[0]])} out of range for vocabulary {vocab}")
            else:
                for t in s.tokens:
                    if not 0 <= int(t) < vocab:
                        raise StepError(f"slot {s.slot}: token id {t} out of range for vocabulary {vocab}")
            for w in s.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"slot {s.slot}: wanted place {w} is not among its {n} tokens")
            slots.append(int(s.slot))
            counts.append(n)
        try:
            self.cache.begin_step(slots, counts)
        except CacheError as e:
            raise StepError(str(e)) from e
        starts = [self.cache.length(s) for s in slots]

        if all(c == 1 for c in counts):
            out = self._decode_step([int(s.tokens[0]) for s in seqs], [i for i, s in enumerate(seqs) if len(s.want) > 0],
                                    slots, starts)
        else:
            out = self._prefill_step(seqs, slots, starts, counts)
        self.cache.end_step(slots, counts)
        if check:
            self.check_status()
        return out

    def step_sampled(self, slots: Sequence[int], token_ids: torch.Tensor, check: bool = True) -> torch.Tensor:
        """One token for each of ``slots``, the ids taken from ``token_ids`` (int32 on the device,
        for instance where the sampler left them) without a trip through the host; logits for every
        sequence.  The ids must be valid: nothing but the embedding's own check sees them."""
        slots = [int(s) for s in slots]
        if not slots:
            raise StepError("a step needs at least one sequence")
        if token_ids.dtype != torch.int32 or not token_ids.is_cuda or token_ids.numel() != len(slots) \
                or not token_ids.is_contiguous():
            raise StepError(f"step_sampled wants {len(slots)} contiguous int32 ids on the device")
        counts = [1] * len(slots)
        try:
            self.cache.begin_step(slots, counts)
        except CacheError as e:
            raise StepError(str(e)) from e
        starts = [self.cache.length(s) for s in slots]
        out = self._decode_step([0] * len(slots), list(range(len(slots))), slots, starts, token_ids)
        self.cache.end_step(slots, counts)
        if check:
            self.check_status()
        return out

    def check_status(self) -> None:
        bits = int(self.status.item())
        if self.dtype == torch.bfloat16:
            from ..kernels import fast_ops
            tc = fast_ops.tc_status(self.device)
            tc_bits = int(tc[0].item())
            if tc_bits:
                tc.zero_()
                raise StepError("device-side check failed: a bounded wait in the tensor-core matrix product ran out "
                                f"(status {tc_bits}); its results are not to be trusted")
        if bits:
            self.status.zero_()
            what = []
            if bits & ops.STATUS_BAD_TOKEN:
                what.append("a token id outside the vocabulary reached the embedding")
            if bits & ops.STATUS_NO_PAGE:
                what.append("a token had no cache page to be written to")
            if bits & ops.STATUS_BAD_POSITION:
                what.append("a position outside the rotation table")
            raise StepError("device-side check failed: " + "; ".join(what))

    # ---- single-token steps ----------------------------------------------------------
    def _decode_step(self, tokens, want_rows, slots, starts, device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``device_tokens`` (int32 on the device, one per sequence) replace ``tokens`` after the
        step's index arrays have been copied: the ids then never pass through the host."""
        b = len(slots)
        # the most pages a sequence of this step holds, rounded up to a bucket: kernels cut their
        # work by it, so a step over short sequences does not launch for the longest possible one
        bucket = pages_bucket(max((st + PAGE_TOKENS) // PAGE_TOKENS for st in starts), self.cache.n_blocks)
        if self.use_graphs:
            padded = 1
            while padded < b:
                padded *= 2
            if padded > 16:
                padded = ((b + 15) // 16) * 16
            g = self._graphs.get(padded)
            if g is None or g.stamp != self._stamp():
                g = _DecodeGraphs(self, padded)
                self._graphs[padded] = g
            self._fill_meta(g.meta, tokens, starts, slots, list(range(b + 1)), padded, padded)
            if device_tokens is not None:
                g.meta[:b].copy_(device_tokens, non_blocking=True)
            g.replay(self, bucket, (slots, starts, [1] * b))
            self.graph_kernel_launches += g.n_kernels[bucket]
            logits = g.logits
        else:
            meta = self._meta_buffer(b, b, 0)
            self._fill_meta(meta, tokens, starts, slots, list(range(b + 1)), b, b)
            if device_tokens is not None:
                meta[:b].copy_(device_tokens, non_blocking=True)
            ctx = self._context_from_meta(meta, b, b, 1, (slots, starts, [1] * b))
            ctx.pages_bucket = bucket
            logits = self.workspace.rows("logits", b, self.spec.vocab_size, torch.float32)
            rows = torch.arange(b, dtype=torch.int32, device=self.device)
            self._forward(ctx, rows, logits)
        if len(want_rows) == b:
            return logits[:b]
        if not want_rows:
            return logits[:0]
        idx = torch.tensor(want_rows, dtype=torch.long, device=self.device)
        return logits.index_select(0, idx)

    # ---- steps with longer pieces ----------------------------------------------------
    def _prefill_step(self, seqs, slots, starts, counts) -> torch.Tensor:
        n_want = sum(len(s.want) for s in seqs)
        out = self.workspace.rows("logits.prefill", max(n_want, 1), self.spec.vocab_size, torch.float32)[:n_want]
        # cut into micro-batches of at most prefill_chunk_tokens tokens; a long sequence is cut too
        budget = self.prefill_chunk_tokens
        pieces: List[List[Tuple[int, int, int]]] = [[]]      # (sequence index, first token, count)
        used = 0
        for i, n in enumerate(counts):
            off = 0
            while off < n:
                if used == budget:
                    pieces.append([])
                    used = 0
                take = min(n - off, budget - used)
                pieces[-1].append((i, off, take))
                used += take
                off += take
        # where each wanted place lands in `out`
        want_base = []
        acc = 0
        for s in seqs:
            want_base.append(acc)
            acc += len(s.want)
        for piece in pieces:
            tok_parts, pos_parts, slot_parts = [], [], []
            cu, p_slots, p_starts, p_counts = [0], [], [], []
            rows, dest = [], []
            for (i, off, take) in piece:
                s = seqs[i]
                base = cu[-1]
                tok_parts.append(np.asarray(s.tokens[off:off + take], dtype=np.int32))
                pos_parts.append(np.arange(starts[i] + off, starts[i] + off + take, dtype=np.int32))
                slot_parts.append(np.full(take, slots[i], dtype=np.int32))
                cu.append(base + take)
                p_slots.append(slots[i])
                p_starts.append(starts[i] + off)
                p_counts.append(take)
                for j, w in enumerate(s.want):
                    if off <= w < off + take:
                        rows.append(base + (w - off))
                        dest.append(want_base[i] + j)
            tok, pos, slot_of = np.concatenate(tok_parts), np.concatenate(pos_parts), np.concatenate(slot_parts)
            n_tok, n_seq = cu[-1], len(piece)
            meta = self._meta_buffer(n_tok, n_seq, len(rows))
            self._fill_meta(meta, tok, pos, slot_of, cu, n_tok, n_seq, p_slots, p_starts, rows)
            ctx = self._context_from_meta(meta, n_tok, n_seq, max(p_counts), (p_slots, p_starts, p_counts))
            x = self.decoder.embed(ctx)
            self.decoder.run_layers(ctx, x, self.cache)
            if rows:
                row_idx = self._meta_slices(meta, n_tok, n_seq, len(rows))[7]
                contiguous = dest == list(range(dest[0], dest[0] + len(dest)))
                if contiguous:
                    self.decoder.logits(ctx, x, row_idx, out[dest[0]:dest[0] + len(dest)])
                else:
                    tmp = self.workspace.rows("logits.tmp", len(rows), self.spec.vocab_size, torch.float32)
                    self.decoder.logits(ctx, x, row_idx, tmp)
                    out.index_copy_(0, torch.tensor(dest, dtype=torch.long, device=self.device), tmp)
        return out

    # ---- one forward over a prepared context -----------------------------------------
    def _forward(self, ctx: StepContext, rows: torch.Tensor, logits: torch.Tensor) -> None:
        x = self.decoder.embed(ctx)
        self.decoder.run_layers(ctx, x, self.cache)
        self.decoder.logits(ctx, x, rows, logits[:rows.numel()])

    # ---- the packed index arrays of a step -------------------------------------------
    # layout of `meta` (int32): token_ids[T] token_pos[T] token_slot[T] cu_seqlens[B+1] seq_slot[B]
    #                           seq_start[B] total_pages[1] want_rows[W]
    @staticmethod
    def _meta_len(n_tok: int, n_seq: int, n_want: int) -> int:
        return 3 * n_tok + (n_seq + 1) + 2 * n_seq + 1 + n_want

    def _meta_buffer(self, n_tok: int, n_seq: int, n_want: int) -> torch.Tensor:
        n = self._meta_len(n_tok, n_seq, n_want)
        return self.workspace.vector("meta", n, torch.int32)

    @staticmethod
    def _meta_slices(meta, n_tok, n_seq, n_want):
        o = 0
        out = []
        for n in (n_tok, n_tok, n_tok, n_seq + 1, n_seq, n_seq, 1, n_want):
            out.append(meta[o:o + n])
            o += n
        return out

    def _fill_meta(self, meta, tok, pos, slot_of, cu, n_tok, n_seq, seq_slots=None, seq_starts=None,
                   want_rows=()) -> None:
        """Pack the step's index arrays on the host and copy them to ``meta`` in one transfer.
        In a single-token step ``pos`` doubles as the sequences' starts and ``slot_of`` as their slots."""
        if seq_slots is None:
            seq_slots, seq_starts = slot_of, pos
        # pages the sequences hold after this step, summed: kernels size their work split by it
        pages = sum((int(st) + (int(cu[i + 1]) - int(cu[i])) + PAGE_TOKENS - 1) // PAGE_TOKENS
                    for i, st in enumerate(seq_starts))
        n = self._meta_len(n_tok, n_seq, len(want_rows))
        # a ring of pinned staging buffers per capacity (the next power of two at or above the
        # length, so the number of rings is bounded whatever lengths the steps have): a buffer is
        # rewritten only after the copy that last read it has completed (its event), which with
        # four in rotation was steps ago, so the host packs the next step while the GPU still
        # runs this one
        entry = self._pinned.take(n)
        pinned = entry[0]
        pack_meta(pinned.numpy(), tok, pos, slot_of, cu, n_tok, n_seq, seq_slots, seq_starts, pages, want_rows)
        meta[:n].copy_(pinned[:n], non_blocking=True)
        if entry[1] is None:
            entry[1] = torch.cuda.Event()
        entry[1].record(torch.cuda.current_stream(self.device))
        self.last_h2d_bytes = 4 * n

    def _context_from_meta(self, meta, n_tok, n_seq, max_seq_tokens, host) -> StepContext:
        ids, pos, slot_of, cu, seq_slot, seq_start, pages, _ = self._meta_slices(meta, n_tok, n_seq, 0)
        ctx = StepContext(
            n_tokens=n_tok, n_seqs=n_seq, max_seq_tokens=max_seq_tokens, act_dtype=self.dtype,
            workspace=self.workspace, token_ids=ids, token_pos=pos, token_slot=slot_of, cu_seqlens=cu,
            seq_slot=seq_slot, seq_start=seq_start, total_pages=pages, status=self.status)
        if host is not None:
            ctx.host_seq_slot, ctx.host_seq_start, ctx.host_seq_tokens = host
        return ctx

    def _stamp(self) -> Tuple[int, int]:
        return (self.workspace.generation, self.cache.generation)

    # ---- accounting ------------------------------------------------------------------
    def kernel_launches(self) -> int:
        """Kernels of this package launched so far, directly or through graph replays."""
        return total_calls() + self.graph_kernel_launches

    def decode_step_bytes(self) -> int:
        """Bytes a single-token step has to read: every weight once and the live sequences' cache."""
        return self.decoder.n_weight_bytes + self.cache.live_kv_bytes()
