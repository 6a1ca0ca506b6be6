"""What a part sees of a step: the tokens' positions and slots, the sequences' boundaries, and a
workspace for its buffers.

All index arrays are int32 on the device and are the only source of lengths, positions and
slots that graph-safe parts may use; the host copies are for parts that are not graph-safe and
for checks before a launch.  Rows past ``n_tokens`` / ``n_seqs`` (padding of a captured step)
carry slot -1, which every kernel skips.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


class Workspace:
    """Reusable device buffers, one per (tag, columns, dtype), grown on demand and never shrunk.
    ``generation`` changes whenever a buffer is replaced, so captured graphs know they are stale."""

    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: Dict[Tuple[str, int, torch.dtype], torch.Tensor] = {}
        self.generation = 0

    def rows(self, tag: str, n_rows: int, n_cols: int, dtype: torch.dtype) -> torch.Tensor:
        key = (tag, n_cols, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.shape[0] < n_rows:
            cap = max(n_rows, 1)
            if buf is not None:
                cap = max(cap, buf.shape[0] * 2)
            buf = torch.empty((cap, n_cols), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        return buf[:n_rows]

    def vector(self, tag: str, n: int, dtype: torch.dtype) -> torch.Tensor:
        return self.rows(tag, n, 1, dtype).view(-1)[:n]

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class StepContext:
    """One (micro-)batch of a step."""

    n_tokens: int                 # rows of the packed token dimension (including padding rows)
    n_seqs: int                   # sequences (including padding sequences)
    max_seq_tokens: int           # most tokens any sequence brings in this step
    act_dtype: torch.dtype
    workspace: Workspace
    # device arrays (int32)
    token_ids: torch.Tensor       # [n_tokens]
    token_pos: torch.Tensor       # [n_tokens] absolute position of each token in its sequence
    token_slot: torch.Tensor      # [n_tokens] slot of the token's sequence, -1 for padding
    cu_seqlens: torch.Tensor      # [n_seqs + 1] first row of each sequence in the packed tokens
    seq_slot: torch.Tensor        # [n_seqs] slot, -1 for padding
    seq_start: torch.Tensor       # [n_seqs] tokens the sequence held before this step
    total_pages: torch.Tensor     # [1] cache pages (64 positions) the sequences hold after this step, summed
    status: torch.Tensor          # [1] int32, bits set by device-side checks
    # host copies (None while a captured graph is replayed)
    host_seq_slot: Optional[List[int]] = None
    host_seq_start: Optional[List[int]] = None
    host_seq_tokens: Optional[List[int]] = None
    capturing: bool = False
    # single-token steps: a power of two at or above the most cache pages any sequence of the step
    # holds (0: unknown).  Kernels may size their work split by it; no result depends on it.
    pages_bucket: int = 0
    extras: dict = field(default_factory=dict)

    def rows(self, tag: str, n_cols: int, dtype: Optional[torch.dtype] = None,
             n_rows: Optional[int] = None) -> torch.Tensor:
        return self.workspace.rows(tag, self.n_tokens if n_rows is None else n_rows, n_cols,
                                   dtype or self.act_dtype)


def build_context(seqs, act_dtype: torch.dtype, workspace: Workspace, device,
                  status: Optional[torch.Tensor] = None) -> StepContext:
    """A context for ``seqs = [(slot, start, tokens), ...]``: each sequence brings ``tokens`` at
    positions ``start, start+1, ...``.  Plain and unhurried; the engine packs its own arrays in one
    transfer, this is for driving a part alone."""
    ids: List[int] = []
    pos: List[int] = []
    slot_of: List[int] = []
    cu = [0]
    for slot, start, tokens in seqs:
        ids += [int(t) for t in tokens]
        pos += list(range(start, start + len(tokens)))
        slot_of += [slot] * len(tokens)
        cu.append(len(ids))

    def i32(xs):
        return torch.tensor(xs, dtype=torch.int32, device=device)

    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=device)
    return StepContext(
        n_tokens=len(ids), n_seqs=len(seqs), max_seq_tokens=max(len(t) for _, _, t in seqs),
        act_dtype=act_dtype, workspace=workspace, token_ids=i32(ids), token_pos=i32(pos),
        token_slot=i32(slot_of), cu_seqlens=i32(cu), seq_slot=i32([s for s, _, _ in seqs]),
        seq_start=i32([st for _, st, _ in seqs]),
        total_pages=i32([sum((st + len(t) + 63) // 64 for _, st, t in seqs)]), status=status,
        host_seq_slot=[s for s, _, _ in seqs], host_seq_start=[st for _, st, _ in seqs],
        host_seq_tokens=[len(t) for _, _, t in seqs])
