"""The sequence cache: a slot per live sequence, pages of keys and values per group of layers,
and per-sequence state of fixed size beside them.

The model's runs say what they need (``KVNeed`` with or without a window, ``StateNeed``, or
nothing).  Runs with the same need form a group; each group has storage, a page pool and a
page table of its own, so layers that keep every key and layers that keep a window of them do
not share pages.  A page holds ``PAGE_TOKENS`` positions as ``[kv_head][row][head_dim]``, so
one head's rows of a page are contiguous.

Storage of a key/value group: ``[runs, 2, pages, kv_heads, PAGE_TOKENS, head_dim]`` in the run
dtype.  The page table ``[slots, blocks]`` (int32, -1 where no page is held) is mirrored on the
device; kernels find position ``p`` of slot ``s`` at page ``table[s, p // PAGE_TOKENS]``, row
``p % PAGE_TOKENS``.

Sizing follows the reference's arithmetic (crates/bfi-models/src/kv_plan.rs:49-51): bytes per
token = runs * 2 * kv_heads * head_dim * element size.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from ..parts.base import KVNeed, StateNeed
from .pages import PAGE_TOKENS, CacheError, FreeList, PageTable

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class KVView:
    """What an attention kernel needs to reach one run's keys and values."""

    k: torch.Tensor            # [pages, kv_heads, PAGE_TOKENS, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor  # [slots, blocks] int32 on the device
    n_kv_heads: int
    head_dim: int
    window: Optional[int]
    page_tokens: int = PAGE_TOKENS


@dataclass
class RunCache:
    """The cache of one run of the schedule, as handed to its mixer.  A mixer that declared
    several needs finds one entry per need, in the order it declared them, in ``entries``
    (a ``KVView`` for a ``KVNeed``, a ``[slots, *shape]`` tensor for a ``StateNeed``); ``kv`` and
    ``state`` are the first entry of each sort."""

    kv: Optional[KVView] = None
    state: Optional[torch.Tensor] = None   # [slots, *shape]
    writes_cache: bool = True
    entries: tuple = ()


def needs_of(need) -> tuple:
    """What a mixer's ``cache_need()`` returned, as a tuple of needs: it may name none, one, or
    several (keys and values beside a fixed-size state, for instance)."""
    if need is None:
        return ()
    if isinstance(need, (KVNeed, StateNeed)):
        return (need,)
    return tuple(need)


class _KVGroup:
    def __init__(self, need: KVNeed, keys: List[Any], n_pages: int, n_slots: int, n_blocks: int,
                 dtype: torch.dtype, device: torch.device):
        self.need = need
        self.keys = keys                       # (run, index among the run's needs) per place
        self.runs = [r for r, _ in keys]
        self.table = PageTable(n_pages, need.window)
        self.n_blocks = n_blocks
        self.device = device
        self.storage = torch.empty(
            (len(keys), 2, n_pages, need.n_kv_heads, PAGE_TOKENS, need.head_dim),
            dtype=dtype, device=device)
        self._alloc_tables(n_slots)

    def _alloc_tables(self, n_slots: int) -> None:
        # The host mirror is pageable on purpose: a copy from pageable memory is staged before
        # the call returns, so a row may be edited again while earlier work is still queued.
        self.block_host = torch.full((n_slots, self.n_blocks), -1, dtype=torch.int32)
        self.block_dev = torch.full((n_slots, self.n_blocks), -1, dtype=torch.int32, device=self.device)

    def grow_slots(self, n_slots: int) -> None:
        old_host = self.block_host
        self._alloc_tables(n_slots)
        self.block_host[:old_host.shape[0]] = old_host
        self.block_dev.copy_(self.block_host)

    def sync_row(self, slot: int) -> None:
        row = self.table.rows.get(slot, [])
        host = self.block_host[slot]
        host.fill_(-1)
        if row:
            if len(row) > self.n_blocks:
                raise CacheError(f"slot {slot} needs {len(row)} page blocks, table has {self.n_blocks}")
            host[:len(row)] = torch.tensor(row, dtype=torch.int32)
        self.block_dev[slot].copy_(host)

    def view(self, key) -> KVView:
        i = self.keys.index(key)
        return KVView(k=self.storage[i, 0], v=self.storage[i, 1], block_table=self.block_dev,
                      n_kv_heads=self.need.n_kv_heads, head_dim=self.need.head_dim,
                      window=self.need.window)

    def bytes_per_token(self) -> int:
        return len(self.runs) * 2 * self.need.n_kv_heads * self.need.head_dim * self.storage.element_size()


class _StateGroup:
    def __init__(self, need: StateNeed, keys: List[Any], n_slots: int, device: torch.device):
        self.need = need
        self.keys = keys
        self.runs = [r for r, _ in keys]
        self.device = device
        self.dtype = _TORCH_DTYPES[need.dtype]
        self.storage = {k: torch.zeros((n_slots,) + tuple(need.shape), dtype=self.dtype, device=device)
                        for k in keys}

    def grow_slots(self, n_slots: int) -> None:
        for r, old in list(self.storage.items()):
            new = torch.zeros((n_slots,) + tuple(self.need.shape), dtype=self.dtype, device=self.device)
            new[:old.shape[0]] = old
            self.storage[r] = new

    def reset(self, slot: int) -> None:
        for t in self.storage.values():
            t[slot].zero_()

    def bytes_per_slot(self) -> int:
        n = 1
        for s in self.need.shape:
            n *= s
        return len(self.runs) * n * torch.empty((), dtype=self.dtype).element_size()


class SequenceCache:
    """Slots, pages and fixed-size state for the live sequences of one model.

    ``needs[i]`` is what run ``i`` of the schedule keeps (None for nothing); ``cache_of[i]``
    names the run whose cache run ``i`` reads instead of keeping its own.
    ``max_tokens`` is the most tokens all live sequences hold together, each sequence's count
    rounded up to a whole page; ``max_seq_len`` the most one sequence may hold.
    """

    def __init__(self, needs: Sequence[Union[KVNeed, StateNeed, None]],
                 cache_of: Sequence[Optional[int]], max_tokens: int, max_seq_len: int,
                 dtype: torch.dtype, device: torch.device, initial_slots: int = 64):
        if max_tokens < 1 or max_seq_len < 1:
            raise CacheError("max_tokens and max_seq_len must be positive")
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_seq_len = max_seq_len
        self.n_pages = (max_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.n_blocks = (max_seq_len + PAGE_TOKENS - 1) // PAGE_TOKENS
        n_slots = max(1, min(initial_slots, self.n_pages))
        self.slots = FreeList(n_slots, "slot")
        self.lengths: Dict[int, int] = {}
        self.generation = 0          # bumped when device tensors are replaced (graphs must be re-captured)

        self.cache_of = list(cache_of)
        self.kv_groups: List[_KVGroup] = []
        self.state_groups: List[_StateGroup] = []
        self._owner: Dict[int, List[Any]] = {}     # run -> [(need index, group, key in the group)]
        by_need: Dict[Any, List[Any]] = {}
        for run, need in enumerate(needs):
            if self.cache_of[run] is not None:
                src = self.cache_of[run]
                if not 0 <= src < run or self.cache_of[src] is not None:
                    raise CacheError(f"run {run} reads the cache of run {src}, which keeps none of its own")
                continue
            self._owner[run] = []
            for j, one in enumerate(needs_of(need)):
                # a run that names the same need twice gets two places in that need's group
                by_need.setdefault(one, []).append((run, j))
        for need, keys in by_need.items():
            if isinstance(need, KVNeed):
                g = _KVGroup(need, keys, self.n_pages, n_slots, self.n_blocks, dtype, self.device)
                self.kv_groups.append(g)
            elif isinstance(need, StateNeed):
                g = _StateGroup(need, keys, n_slots, self.device)
                self.state_groups.append(g)
            else:
                raise CacheError(f"unknown cache need {need!r}")
            for key in keys:
                self._owner[key[0]].append((key[1], g, key))
        for own in self._owner.values():
            own.sort(key=lambda e: e[0])           # the order in which the mixer declared its needs

    # ---- what a run sees -------------------------------------------------------------
    def run_cache(self, run: int) -> RunCache:
        src = self.cache_of[run]
        owner_run = run if src is None else src
        entries = tuple(g.view(key) if isinstance(g, _KVGroup) else g.storage[key]
                        for _, g, key in self._owner.get(owner_run, ()))
        kv = next((e for e in entries if isinstance(e, KVView)), None)
        state = next((e for e in entries if not isinstance(e, KVView)), None)
        return RunCache(kv=kv, state=state, writes_cache=src is None, entries=entries)

    # ---- slots -----------------------------------------------------------------------
    def acquire(self) -> int:
        if self.slots.n_free == 0 and self.slots.capacity < self.n_pages:
            self._grow_slots(min(self.n_pages, self.slots.capacity * 2))
        slot = self.slots.take()
        self.lengths[slot] = 0
        for g in self.kv_groups:
            g.table.open(slot)
        for g in self.state_groups:
            g.reset(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} is not held (released twice?)")
        for g in self.kv_groups:
            g.table.close(slot)
            g.sync_row(slot)
        del self.lengths[slot]
        self.slots.give_back(slot)

    def _grow_slots(self, n: int) -> None:
        self.slots.grow(n)
        for g in self.kv_groups:
            g.grow_slots(n)
        for g in self.state_groups:
            g.grow_slots(n)
        self.generation += 1

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    @property
    def n_slots(self) -> int:
        return self.slots.capacity

    # ---- a step ----------------------------------------------------------------------
    def begin_step(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """Make room for ``counts[i]`` more tokens of ``slots[i]``; nothing changes on failure."""
        if len(set(slots)) != len(slots):
            raise CacheError("a slot appears twice in one step")
        for s, c in zip(slots, counts):
            if s not in self.lengths:
                raise CacheError(f"slot {s} is not held")
            if c < 1:
                raise CacheError(f"slot {s}: a step must bring at least one token")
            if self.lengths[s] + c > self.max_seq_len:
                raise CacheError(
                    f"context_exceeded: slot {s} holds {self.lengths[s]} tokens, {c} more would pass "
                    f"the limit of {self.max_seq_len}")
        for g in self.kv_groups:
            need = sum(g.table.pages_needed(s, self.lengths[s], self.lengths[s] + c)
                       for s, c in zip(slots, counts))
            if need > g.table.pool.n_free:
                raise CacheError(
                    f"cache full: the step needs {need} more pages of {PAGE_TOKENS} tokens, "
                    f"{g.table.pool.n_free} of {g.table.pool.capacity} are free")
        for g in self.kv_groups:
            for s, c in zip(slots, counts):
                if g.table.ensure(s, self.lengths[s], self.lengths[s] + c):
                    g.sync_row(s)

    def end_step(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """The step ran: lengths advance, and windowed groups let go of pages behind the window."""
        for s, c in zip(slots, counts):
            self.lengths[s] += c
        for g in self.kv_groups:
            if g.need.window is None:
                continue
            for s in slots:
                if g.table.trim(s, self.lengths[s]):
                    g.sync_row(s)

    def rewind(self, slot: int, length: int) -> None:
        """Keep only the first ``length`` tokens of ``slot``: its fill mark moves back and the pages
        past it return to the pool (crates/bfi-models/src/session.rs:50-62).  Only a cache that
        keeps every key can do that: a windowed group has already let go of pages the shorter
        sequence would read, and a fixed-size state cannot be wound back at all, so a model with
        either refuses by name and changes nothing."""
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} is not held")
        if not 0 <= length <= self.lengths[slot]:
            raise CacheError(f"rewind: slot {slot} holds {self.lengths[slot]} tokens, cannot keep {length}")
        if length == self.lengths[slot]:
            return
        if self.state_groups:
            raise CacheError("rewind unsupported: the model keeps per-sequence state of fixed size, "
                             "which cannot be wound back; release the slot and start again")
        windowed = [g.need.window for g in self.kv_groups if g.need.window is not None]
        if windowed:
            raise CacheError(f"rewind unsupported: layers with a window of {windowed[0]} keys have given "
                             "back pages the shorter sequence would read; release the slot and start again")
        for g in self.kv_groups:
            if g.table.shrink(slot, length):
                g.sync_row(slot)
        self.lengths[slot] = length

    # ---- accounting and checks -------------------------------------------------------
    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.kv_groups)

    def state_bytes_per_slot(self) -> int:
        return sum(g.bytes_per_slot() for g in self.state_groups)

    def live_kv_bytes(self) -> int:
        """Bytes of keys and values the live sequences hold (what a decode step has to read)."""
        total = 0
        for g in self.kv_groups:
            for s, n in self.lengths.items():
                kept = n - g.table.first_kept_position(n) if g.need.window is not None else n
                total += kept * g.bytes_per_token()
        return total

    def check(self) -> None:
        self.slots.check()
        for g in self.kv_groups:
            g.table.check()
            if set(g.table.rows) != set(self.lengths):
                raise CacheError("page rows and held slots differ")

    def poison(self, value: float = float("nan")) -> None:
        """Fill every page with ``value`` (tests: rows past a sequence's length must never matter)."""
        for g in self.kv_groups:
            g.storage.fill_(value)
