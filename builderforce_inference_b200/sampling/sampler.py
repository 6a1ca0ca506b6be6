"""Choosing next tokens on the device.

Everything runs in this package's kernels: greedy (``argmax_rows``), temperature with penalties
and min-p, drawn in vocabulary order (``sample_rows``), and top-k / top-p, whose kept set and draw
follow the reference's order after its stable sort (probability descending, index ascending,
crates/bfi-runtime/src/sample.rs:392-409) and are found without sorting (``sample_sorted_rows``).

The uniform number of a draw depends on (seed, request index, step), so a run is reproducible
and every step and request draws its own number.  The reference restarts its generator from the
seed at every call (sample.rs:304-309), which hands every step the same number; the generator's
update and its map to [0, 1) are kept (sample.rs:442-460).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..kernels import ops
from .params import SampleParams

_MASK = (1 << 64) - 1


def uniform_draw(seed: int, request: int, step: int) -> float:
    """A number in [0, 1) for one draw: a 64-bit mix of the three counters, then one step of the
    reference's xorshift (13, 7, 17) and its ``(x >> 40) / 2^24``."""
    x = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & _MASK
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _MASK
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _MASK
    x ^= x >> 31
    if x == 0:
        x = 0x9E3779B97F4A7C15
    x ^= (x << 13) & _MASK
    x ^= x >> 7
    x ^= (x << 17) & _MASK
    return float(x >> 40) / float(1 << 24)


class Sampler:
    """Holds the small device buffers sampling needs."""

    def __init__(self, device: torch.device, vocab_size: int):
        self.device = device
        self.vocab = vocab_size
        self._out = torch.empty(0, dtype=torch.int32, device=device)
        self._work: Optional[torch.Tensor] = None
        self._probs: Optional[torch.Tensor] = None
        self._scratch = torch.empty(0, dtype=torch.int32, device=device)

    def _out_rows(self, n: int) -> torch.Tensor:
        if self._out.numel() < n:
            self._out = torch.empty(max(n, 2 * self._out.numel()), dtype=torch.int32, device=self.device)
        return self._out[:n]

    def sample(self, logits: torch.Tensor, params: SampleParams, requests: Sequence[int], steps: Sequence[int],
               histories: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """``logits`` float32 ``[rows, vocab]`` on the device; returns int32 ids ``[rows]`` on the
        device.  ``histories[i]`` (prompt + generated so far) is needed only with penalties."""
        rows = logits.shape[0]
        out = self._out_rows(rows)
        if rows == 0:
            return out
        if params.greedy and not params.has_penalties:
            need = 2 * rows * ((self.vocab + 8191) // 8192)
            if self._scratch.numel() < need:
                self._scratch = torch.empty(2 * need, dtype=torch.int32, device=self.device)
            ops.argmax_rows(logits, out, self._scratch)
            return out
        u = [uniform_draw(params.seed, r, s) for r, s in zip(requests, steps)]
        seen = seen_cu = work = None
        if params.has_penalties:
            if histories is None:
                raise ValueError("penalties need the token history of every row")
            flat: List[int] = []
            cu = [0]
            for h in histories:
                uniq = sorted({int(t) for t in h if 0 <= int(t) < self.vocab})
                flat.extend(uniq)
                cu.append(len(flat))
            if flat:
                seen = torch.tensor(flat, dtype=torch.int32, device=self.device)
                seen_cu = torch.tensor(cu, dtype=torch.int32, device=self.device)
                if self._work is None or self._work.numel() < rows * self.vocab:
                    self._work = torch.empty(rows * self.vocab, dtype=torch.float32, device=self.device)
                work = self._work
        temp = torch.full((rows,), float(params.temperature), dtype=torch.float32, device=self.device)
        ut = torch.tensor(u, dtype=torch.float32, device=self.device)
        if params.needs_sort:
            if self._probs is None or self._probs.numel() < rows * self.vocab:
                self._probs = torch.empty(rows * self.vocab, dtype=torch.float32, device=self.device)
            ops.sample_sorted_rows(logits, temp, ut, out, self._probs, params.top_k, params.top_p, params.repeat_penalty,
                                   params.presence_penalty, params.min_p, seen, seen_cu, work)
            return out
        ops.sample_rows(logits, temp, ut, out, params.repeat_penalty, params.presence_penalty, params.min_p,
                        seen, seen_cu, work)
        return out
