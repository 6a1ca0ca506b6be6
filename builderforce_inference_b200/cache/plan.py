"""Sizing the cache from a byte budget.  Pure arithmetic, no device.

The reference's arithmetic (crates/bfi-models/src/kv_plan.rs:1-74): keys and values of one
token cost ``layers * 2 * kv_heads * head_dim * element bytes``; the served context is the
budget divided by that, capped by the trained context and by the largest single buffer, and
rounded down to a multiple of 256 (left as it is below 256).

Here the cache is paged and grouped: every group of runs with the same need has a pool of
``max_tokens / 64`` pages of its own, so a token of capacity costs the sum over the groups, and
the fixed-size state of every slot is taken off the budget first.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

from ..parts.base import KVNeed, StateNeed
from .pages import PAGE_TOKENS, CacheError

CONTEXT_STEP = 256          # kv_plan.rs:26
_ELEMENT_BYTES = {"float32": 4, "bfloat16": 2, "int32": 4}


def element_bytes(dtype) -> int:
    name = str(dtype).replace("torch.", "")
    if name not in _ELEMENT_BYTES:
        raise CacheError(f"no element size known for dtype {dtype}")
    return _ELEMENT_BYTES[name]


def round_context(n: int) -> int:
    """Down to a multiple of 256; a count below 256 stays (at least 1) (kv_plan.rs:67-73)."""
    return n // CONTEXT_STEP * CONTEXT_STEP if n >= CONTEXT_STEP else max(n, 1)


def served_context(n_layers: int, n_kv_heads: int, head_dim: int, elem_bytes: int, budget_bytes: int,
                   trained_context: int, max_buffer_bytes: Optional[int] = None) -> int:
    """The context one sequence can be served with under ``budget_bytes`` for all layers' keys and
    values, when one layer's keys (or values) must also fit ``max_buffer_bytes``
    (kv_plan.rs:59-65)."""
    per_token = max(1, n_layers * 2 * n_kv_heads * head_dim * elem_bytes)
    cap = budget_bytes // per_token
    if max_buffer_bytes is not None:
        cap = min(cap, max_buffer_bytes // max(1, n_kv_heads * head_dim * elem_bytes))
    return round_context(min(cap, trained_context))


def _own_needs(needs, cache_of):
    from .cache import needs_of
    for run, need in enumerate(needs):
        if cache_of[run] is None:
            yield from needs_of(need)


def kv_bytes_per_token(needs: Sequence, cache_of: Sequence[Optional[int]], elem_bytes: int) -> int:
    """Bytes of keys and values one token of cache capacity costs, over all runs that keep a
    cache of their own."""
    return sum(2 * n.n_kv_heads * n.head_dim * elem_bytes for n in _own_needs(needs, cache_of)
               if isinstance(n, KVNeed))


def state_bytes_per_slot(needs: Sequence, cache_of: Sequence[Optional[int]]) -> int:
    total = 0
    for n in _own_needs(needs, cache_of):
        if isinstance(n, StateNeed):
            count = 1
            for d in n.shape:
                count *= d
            total += count * element_bytes(n.dtype)
    return total


@dataclass(frozen=True)
class CachePlan:
    max_tokens: int             # tokens all live sequences may hold together (a multiple of 64)
    bytes_per_token: int
    state_bytes_per_slot: int
    n_slots: int
    kv_bytes: int               # what the pages take
    state_bytes: int            # what the slots' fixed-size state takes


def plan_cache(needs: Sequence, cache_of: Sequence[Optional[int]], budget_bytes: int, elem_bytes: int,
               n_slots: int = 64) -> CachePlan:
    """How many tokens a cache of ``budget_bytes`` holds for a model whose runs need ``needs``,
    with room for ``n_slots`` live sequences' fixed-size state.  The count is rounded like the
    reference's served context (down to a multiple of 256, which is also whole pages); a budget
    that does not hold one page is refused."""
    per_token = kv_bytes_per_token(needs, cache_of, elem_bytes)
    per_slot = state_bytes_per_slot(needs, cache_of)
    left = int(budget_bytes) - n_slots * per_slot
    if per_token == 0:
        if left < 0:
            raise CacheError(f"a cache budget of {budget_bytes} bytes does not hold the fixed-size state of "
                             f"{n_slots} sequences ({n_slots * per_slot} bytes)")
        # nothing is kept per token: the count only bounds the sequences' lengths
        return CachePlan(PAGE_TOKENS * n_slots, 0, per_slot, n_slots, 0, n_slots * per_slot)
    tokens = left // per_token if left > 0 else 0
    tokens = round_context(tokens) if tokens >= CONTEXT_STEP else tokens // PAGE_TOKENS * PAGE_TOKENS
    if tokens < PAGE_TOKENS:
        raise CacheError(f"a cache budget of {budget_bytes} bytes holds no page of {PAGE_TOKENS} tokens "
                         f"({per_token} bytes per token, {n_slots * per_slot} bytes of fixed-size state)")
    return CachePlan(tokens, per_token, per_slot, n_slots, tokens * per_token, n_slots * per_slot)
