"""Host-side bookkeeping of the cache: which slots and which pages are held, and by whom.

Pure Python, no device: the tests drive these classes on a machine without a GPU.  A slot is
one live sequence; a page holds the keys and values of ``PAGE_TOKENS`` consecutive positions
of one sequence for one group of layers.  Both are handed out from free lists and given back
when a sequence ends, to be used again without being cleared: rows at or past a sequence's
length are never read.
"""
from __future__ import annotations

from typing import Dict, List, Optional

PAGE_TOKENS = 64


class CacheError(RuntimeError):
    """A slot or page was misused, or the cache is too small for what was asked."""


class FreeList:
    """Ids ``0..n-1``, each either free or held.  Lowest free id first, so reuse is
    deterministic."""

    def __init__(self, n: int, what: str):
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))
        self._held: set = set()
        self.capacity = n

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what} (all {self.capacity} are held)")
        i = self._free.pop()
        self._held.add(i)
        return i

    def give_back(self, i: int) -> None:
        if i not in self._held:
            raise CacheError(f"{self.what} {i} is not held (freed twice, or never taken)")
        self._held.remove(i)
        self._free.append(i)
        # keep "lowest id first"
        if len(self._free) > 1 and self._free[-2] < i:
            self._free.sort(reverse=True)

    def grow(self, n: int) -> None:
        if n <= self.capacity:
            return
        self._free = sorted(self._free + list(range(self.capacity, n)), reverse=True)
        self.capacity = n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return len(self._held)

    def is_held(self, i: int) -> bool:
        return i in self._held

    def check(self) -> None:
        """No id lost, none both free and held, none twice in the free list."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError(f"a {self.what} is twice in the free list")
        if free & self._held:
            raise CacheError(f"a {self.what} is both free and held")
        if len(free) + len(self._held) != self.capacity:
            raise CacheError(f"a {self.what} was lost")


class PageTable:
    """For one group of layers: per slot, which page holds positions ``64*i .. 64*i+63``.

    ``window`` is None when every earlier position is kept.  Otherwise only pages that still
    hold a position inside the window of the sequence's next token are kept; ``trim`` gives the
    others back.
    """

    def __init__(self, n_pages: int, window: Optional[int] = None):
        self.pool = FreeList(n_pages, "page")
        self.window = window
        self.rows: Dict[int, List[int]] = {}      # slot -> page id per position block (-1: none)

    def open(self, slot: int) -> None:
        if slot in self.rows:
            raise CacheError(f"slot {slot} already has a page row")
        self.rows[slot] = []

    def first_kept_position(self, length: int) -> int:
        """The oldest position the next token (at ``length``) may still read."""
        if self.window is None:
            return 0
        return max(0, length - self.window + 1)

    def pages_needed(self, slot: int, start: int, end: int) -> int:
        """How many new pages ``ensure(slot, start, end)`` would take."""
        row = self.rows[slot]
        hi = (end + PAGE_TOKENS - 1) // PAGE_TOKENS
        return sum(1 for b in range(start // PAGE_TOKENS, hi) if b >= len(row) or row[b] < 0)

    def ensure(self, slot: int, start: int, end: int) -> bool:
        """Make pages present for positions ``[start, end)`` (and whatever of the window before
        ``start`` is already present stays).  Returns True if the row changed."""
        row = self.rows[slot]
        changed = False
        hi = (end + PAGE_TOKENS - 1) // PAGE_TOKENS
        while len(row) < hi:
            row.append(-1)
        for b in range(start // PAGE_TOKENS, hi):
            if row[b] < 0:
                row[b] = self.pool.take()
                changed = True
        return changed

    def trim(self, slot: int, length: int) -> bool:
        """Give back pages that lie wholly before the window of the token at ``length``."""
        if self.window is None:
            return False
        row = self.rows[slot]
        first_block = self.first_kept_position(length) // PAGE_TOKENS
        changed = False
        for b in range(min(first_block, len(row))):
            if row[b] >= 0:
                self.pool.give_back(row[b])
                row[b] = -1
                changed = True
        return changed

    def shrink(self, slot: int, length: int) -> bool:
        """Give back pages that hold no position below ``length`` (the sequence is cut back to its
        first ``length`` tokens).  Returns True if the row changed."""
        row = self.rows[slot]
        keep = (length + PAGE_TOKENS - 1) // PAGE_TOKENS
        changed = False
        for b in range(keep, len(row)):
            if row[b] >= 0:
                self.pool.give_back(row[b])
                changed = True
        if len(row) > keep:
            del row[keep:]
            changed = True
        return changed

    def close(self, slot: int) -> None:
        row = self.rows.pop(slot, None)
        if row is None:
            raise CacheError(f"slot {slot} has no page row (freed twice?)")
        for p in row:
            if p >= 0:
                self.pool.give_back(p)

    def held_pages(self) -> int:
        return sum(1 for row in self.rows.values() for p in row if p >= 0)

    def check(self) -> None:
        self.pool.check()
        seen = set()
        for slot, row in self.rows.items():
            for p in row:
                if p < 0:
                    continue
                if p in seen:
                    raise CacheError(f"page {p} is held twice")
                if not self.pool.is_held(p):
                    raise CacheError(f"page {p} of slot {slot} is on the free list")
                seen.add(p)
        if len(seen) != self.pool.n_held:
            raise CacheError("a page is held by no slot (lost)")
