"""The cache's bookkeeping on the CPU: no slot or page lost, held twice or freed twice; reuse;
windows; limits; fixed-size state beside the pages."""
import random

import pytest
import torch

from builderforce_inference_b200.cache import PAGE_TOKENS, CacheError, FreeList, SequenceCache
from builderforce_inference_b200.parts.base import KVNeed, StateNeed

CPU = torch.device("cpu")


def make(needs=None, cache_of=None, max_tokens=64 * 8, max_seq_len=256, slots=4):
    needs = needs if needs is not None else [KVNeed(2, 16), KVNeed(2, 16)]
    cache_of = cache_of if cache_of is not None else [None] * len(needs)
    return SequenceCache(needs, cache_of, max_tokens, max_seq_len, torch.float32, CPU, initial_slots=slots)


def test_free_list_lowest_first_and_double_free():
    f = FreeList(3, "slot")
    assert [f.take(), f.take(), f.take()] == [0, 1, 2]
    with pytest.raises(CacheError, match="no free slot"):
        f.take()
    f.give_back(1)
    f.give_back(0)
    with pytest.raises(CacheError, match="not held"):
        f.give_back(1)
    assert f.take() == 0 and f.take() == 1
    f.check()


def test_slots_are_given_back_and_used_again():
    c = make()
    a, b = c.acquire(), c.acquire()
    c.begin_step([a, b], [70, 3]); c.end_step([a, b], [70, 3])
    assert c.length(a) == 70 and c.length(b) == 3
    g = c.kv_groups[0]
    assert g.table.held_pages() == 3
    c.release(a)
    with pytest.raises(CacheError):
        c.release(a)                       # freed twice
    with pytest.raises(CacheError):
        c.begin_step([a], [1])             # not held
    a2 = c.acquire()
    assert a2 == a and c.length(a2) == 0   # same slot again, empty
    assert g.table.held_pages() == 1
    c.begin_step([a2], [1]); c.end_step([a2], [1])
    assert g.table.held_pages() == 2
    assert g.block_host[a2, 0] >= 0 and g.block_host[a2, 1] == -1
    c.check()


def test_pages_grow_with_length_and_block_table_mirrors_them():
    c = make()
    s = c.acquire()
    g = c.kv_groups[0]
    c.begin_step([s], [64]); c.end_step([s], [64])
    assert g.table.held_pages() == 1
    c.begin_step([s], [1])                 # position 64 needs the second page
    assert g.table.held_pages() == 2
    c.end_step([s], [1])
    row = g.table.rows[s]
    assert g.block_dev[s, :2].tolist() == row and g.block_dev[s, 2].item() == -1
    c.check()


def test_limits_are_refused_before_anything_changes():
    c = make(max_tokens=64 * 3, max_seq_len=128)
    a, b = c.acquire(), c.acquire()
    with pytest.raises(CacheError, match="context_exceeded"):
        c.begin_step([a], [129])
    with pytest.raises(CacheError, match="twice"):
        c.begin_step([a, a], [1, 1])
    with pytest.raises(CacheError, match="at least one"):
        c.begin_step([a], [0])
    c.begin_step([a], [128]); c.end_step([a], [128])      # two pages
    with pytest.raises(CacheError, match="cache full"):
        c.begin_step([b], [65])                            # needs two, one is free
    assert c.kv_groups[0].table.held_pages() == 2 and c.length(b) == 0
    c.begin_step([b], [64]); c.end_step([b], [64])
    with pytest.raises(CacheError, match="context_exceeded"):
        c.begin_step([a], [1])
    c.check()


def test_slot_table_grows_up_to_the_page_count():
    c = make(max_tokens=64 * 6, slots=2)
    got = [c.acquire() for _ in range(6)]
    assert got == list(range(6)) and c.n_slots >= 6 and c.generation > 0
    with pytest.raises(CacheError, match="no free slot"):
        c.acquire()
    for s in got:
        c.release(s)
    c.check()


def test_window_group_lets_go_of_pages_behind_the_window():
    c = make(needs=[KVNeed(1, 16), KVNeed(1, 16, window=40)], max_tokens=64 * 16, max_seq_len=1024)
    full, win = c.kv_groups
    assert full.need.window is None and win.need.window == 40
    s = c.acquire()
    c.begin_step([s], [200])
    assert win.table.held_pages() == 4         # the whole prompt is present during its step
    c.end_step([s], [200])
    # next token is at 200; it reads keys 161..200: blocks 2 and 3
    assert full.table.held_pages() == 4 and win.table.held_pages() == 2
    assert win.block_host[s, :4].tolist()[:2] == [-1, -1]
    for _ in range(60):
        c.begin_step([s], [1]); c.end_step([s], [1])
    # length 260: next token at 260 reads 221..260 -> blocks 3 and 4
    assert win.table.held_pages() == 2 and full.table.held_pages() == 5
    assert c.live_kv_bytes() == 260 * full.bytes_per_token() + 39 * win.bytes_per_token()
    c.release(s)
    assert win.table.held_pages() == 0 and full.table.held_pages() == 0
    c.check()


def test_groups_and_shared_caches():
    needs = [KVNeed(2, 16), KVNeed(2, 16), KVNeed(2, 16, window=8), StateNeed((3, 5)), None, KVNeed(2, 16)]
    cache_of = [None, None, None, None, None, 1]
    c = make(needs=needs, cache_of=cache_of)
    assert [g.runs for g in c.kv_groups] == [[0, 1], [2]]
    assert [g.runs for g in c.state_groups] == [[3]]
    r1, r5 = c.run_cache(1), c.run_cache(5)
    assert r5.kv.k.data_ptr() == r1.kv.k.data_ptr() and r1.writes_cache and not r5.writes_cache
    assert c.run_cache(4).kv is None and c.run_cache(4).state is None
    assert c.run_cache(3).state.shape[1:] == (3, 5)
    with pytest.raises(CacheError):
        make(needs=[KVNeed(2, 16), KVNeed(2, 16)], cache_of=[None, 1])
    assert c.bytes_per_token() == (2 + 1) * 2 * 2 * 16 * 4          # kv_plan.rs:49-51 per group
    assert c.state_bytes_per_slot() == 3 * 5 * 4


def test_fixed_state_is_per_slot_and_reset_on_acquire():
    c = make(needs=[StateNeed((4,)), KVNeed(1, 16)], slots=2)
    a = c.acquire()
    st = c.run_cache(0).state
    st[a] += 3.0
    b = c.acquire()
    assert st[b].abs().sum() == 0 and st[a].sum() == 12.0
    c.release(a)
    a2 = c.acquire()
    assert a2 == a and c.run_cache(0).state[a2].abs().sum() == 0
    # growing the slot table keeps live state
    c.run_cache(0).state[b] += 1.0
    more = [c.acquire() for _ in range(3)]
    assert c.run_cache(0).state[b].sum() == 4.0
    for s in more + [a2, b]:
        c.release(s)
    c.check()


def test_random_traffic_never_loses_or_duplicates_anything():
    rng = random.Random(0)
    c = make(needs=[KVNeed(1, 16), KVNeed(1, 16, window=70)], max_tokens=64 * 24, max_seq_len=512, slots=2)
    live = {}
    for it in range(600):
        r = rng.random()
        if r < 0.25 and len(live) < 8:
            try:
                s = c.acquire()
                live[s] = 0
            except CacheError:
                pass
        elif r < 0.45 and live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        elif r < 0.5 and live:
            # wind a sequence back: the windowed group refuses and nothing may change
            s = rng.choice(list(live))
            if live[s] > 0:
                with pytest.raises(CacheError, match="rewind unsupported"):
                    c.rewind(s, live[s] // 2)
        elif live:
            batch = rng.sample(list(live), rng.randint(1, len(live)))
            counts = [rng.choice([1, 1, 1, 5, 64, 100]) for _ in batch]
            try:
                c.begin_step(batch, counts)
            except CacheError as e:
                assert "context_exceeded" in str(e) or "cache full" in str(e)
                continue
            c.end_step(batch, counts)
            for s, n in zip(batch, counts):
                live[s] += n
        c.check()
        assert {s: c.length(s) for s in live} == live
        for g in c.kv_groups:
            for s, n in live.items():
                row = g.table.rows[s]
                first = g.table.first_kept_position(n) // PAGE_TOKENS
                for blk in range((n + PAGE_TOKENS - 1) // PAGE_TOKENS):
                    assert (row[blk] >= 0) == (blk >= first), (g.need, s, n, blk, row)
                assert g.block_host[s, :len(row)].tolist() == row
    for s in list(live):
        c.release(s)
    for g in c.kv_groups:
        assert g.table.held_pages() == 0 and g.table.pool.n_free == g.table.pool.capacity
    assert c.slots.n_held == 0


def test_rewind_gives_pages_back_and_refuses_what_cannot_be_wound_back():
    c = make(max_tokens=64 * 8, max_seq_len=512)
    a, b = c.acquire(), c.acquire()
    c.begin_step([a, b], [200, 70]); c.end_step([a, b], [200, 70])
    g = c.kv_groups[0]
    assert g.table.held_pages() == 4 + 2
    kept = list(g.table.rows[a][:2])
    c.rewind(a, 100)                                   # session.rs:53-62: the fill mark moves back
    assert c.length(a) == 100 and g.table.rows[a] == kept and g.table.held_pages() == 2 + 2
    assert g.block_host[a, :4].tolist() == kept + [-1, -1]
    c.rewind(a, 100)                                   # nothing to do
    with pytest.raises(CacheError, match="cannot keep"):
        c.rewind(a, 101)
    with pytest.raises(CacheError, match="not held"):
        c.rewind(7, 0)
    c.begin_step([a], [130]); c.end_step([a], [130])   # grows again over the freed pages
    assert c.length(a) == 230 and g.table.held_pages() == 4 + 2
    c.rewind(b, 0)
    assert c.length(b) == 0 and g.table.rows[b] == []
    c.check()
    w = make(needs=[KVNeed(1, 16), KVNeed(1, 16, window=40)], max_seq_len=512)
    s = w.acquire()
    w.begin_step([s], [100]); w.end_step([s], [100])
    with pytest.raises(CacheError, match="rewind unsupported.*window of 40"):
        w.rewind(s, 50)
    assert w.length(s) == 100
    st = make(needs=[KVNeed(1, 16), StateNeed((4,))])
    s = st.acquire()
    st.begin_step([s], [10]); st.end_step([s], [10])
    with pytest.raises(CacheError, match="rewind unsupported.*fixed size"):
        st.rewind(s, 5)
    st.rewind(s, 10)
    st.check()


def test_a_run_may_declare_several_needs():
    """Keys and values AND a fixed-size state for one mixer; the same need twice gives two places."""
    both = (KVNeed(2, 16), StateNeed((3,)))
    needs = [both, KVNeed(2, 16), (StateNeed((3,)), StateNeed((3,)), StateNeed((5,), "int32")), both]
    c = make(needs=needs, cache_of=[None, None, None, 0])
    assert [g.keys for g in c.kv_groups] == [[(0, 0), (1, 0)]]
    assert [g.keys for g in c.state_groups] == [[(0, 1), (2, 0), (2, 1)], [(2, 2)]]
    r0, r2, r3 = c.run_cache(0), c.run_cache(2), c.run_cache(3)
    assert isinstance(r0.entries[0], type(r0.kv)) and r0.entries[1] is r0.state and r0.state.shape[1:] == (3,)
    assert r0.kv is not None and r0.kv.k.data_ptr() != c.run_cache(1).kv.k.data_ptr()
    assert len(r2.entries) == 3 and r2.kv is None and r2.entries[0].data_ptr() != r2.entries[1].data_ptr()
    assert r2.entries[2].dtype == torch.int32 and r2.entries[2].shape[1:] == (5,)
    assert r3.kv.k.data_ptr() == r0.kv.k.data_ptr() and r3.state.data_ptr() == r0.state.data_ptr()
    assert not r3.writes_cache
    a = c.acquire()
    r2.entries[1][a] += 2.0
    c.release(a)
    assert c.acquire() == a and c.run_cache(2).entries[1][a].abs().sum() == 0
    assert c.bytes_per_token() == 2 * 2 * 2 * 16 * 4
    assert c.state_bytes_per_slot() == (3 + 3 + 3) * 4 + 5 * 4


def test_cache_sized_from_a_byte_budget():
    from builderforce_inference_b200.cache import plan_cache, served_context
    # the reference's own predictions (kv_plan.rs:166-176): 36 / 28 layers, 8 kv heads of 128
    gib2, binding = 2 << 30, 128 << 20
    assert served_context(36, 8, 128, 2, gib2, 65536, binding) == 14336
    assert served_context(36, 8, 128, 4, gib2, 65536, binding) == 7168
    assert served_context(28, 8, 128, 2, gib2, 32768, binding) == 18688
    assert served_context(28, 8, 128, 4, gib2, 32768, binding) == 9216
    assert served_context(28, 8, 128, 2, 1 << 62, 4096, None) == 4096           # kv_plan.rs:180-181
    assert served_context(36, 8, 128, 2, 1 << 62, 65536, 1 << 20) == 512        # kv_plan.rs:183
    needs = [KVNeed(8, 128)] * 36
    p = plan_cache(needs, [None] * 36, gib2, 2)
    assert p.bytes_per_token == 147456 and p.max_tokens == 14336 and p.kv_bytes <= gib2
    # fixed-size state comes off the budget first; a run that reads another's cache costs nothing
    needs = [(KVNeed(2, 16), StateNeed((100,))), KVNeed(2, 16, window=8), KVNeed(2, 16)]
    p = plan_cache(needs, [None, None, 0], 1_000_000, 4, n_slots=10)
    assert p.state_bytes_per_slot == 400 and p.bytes_per_token == 2 * (2 * 2 * 16 * 4)
    assert p.max_tokens == (1_000_000 - 4000) // 512 // 256 * 256 == 1792
    assert p.kv_bytes + p.state_bytes <= 1_000_000
    assert plan_cache(needs, [None, None, 0], 4000 + 512 * 200, 4, n_slots=10).max_tokens == 192
    with pytest.raises(CacheError, match="holds no page"):
        plan_cache(needs, [None, None, 0], 4000 + 512 * 63, 4, n_slots=10)
    # the plan is what a cache of that size really allocates
    c = SequenceCache(needs, [None, None, 0], p.max_tokens, 256, torch.float32, CPU, initial_slots=10)
    assert sum(g.storage.numel() * 4 for g in c.kv_groups) == p.kv_bytes
    assert c.bytes_per_token() == p.bytes_per_token and c.state_bytes_per_slot() == p.state_bytes_per_slot


def test_random_traffic_with_rewinds():
    rng = random.Random(3)
    c = make(needs=[KVNeed(1, 16), KVNeed(2, 16)], max_tokens=64 * 20, max_seq_len=400, slots=2)
    live = {}
    for it in range(800):
        r = rng.random()
        if r < 0.2 and len(live) < 6:
            try:
                live[c.acquire()] = 0
            except CacheError:
                pass
        elif r < 0.35 and live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        elif r < 0.55 and live:
            s = rng.choice(list(live))
            keep = rng.randint(0, live[s])
            c.rewind(s, keep)
            live[s] = keep
        elif live:
            batch = rng.sample(list(live), rng.randint(1, len(live)))
            counts = [rng.choice([1, 1, 7, 64, 90]) for _ in batch]
            try:
                c.begin_step(batch, counts)
            except CacheError as e:
                assert "context_exceeded" in str(e) or "cache full" in str(e)
                continue
            c.end_step(batch, counts)
            for s, n in zip(batch, counts):
                live[s] += n
        c.check()
        assert {s: c.length(s) for s in live} == live
        for g in c.kv_groups:
            assert g.table.held_pages() == sum((n + PAGE_TOKENS - 1) // PAGE_TOKENS for n in live.values())
            for s, n in live.items():
                row = g.table.rows[s]
                assert len(row) == (n + PAGE_TOKENS - 1) // PAGE_TOKENS or (len(row) >= (n + PAGE_TOKENS - 1) // PAGE_TOKENS)
                assert g.block_host[s, :len(row)].tolist() == row and all(p >= 0 for p in row[:(n + PAGE_TOKENS - 1) // PAGE_TOKENS])
    for s in list(live):
        c.release(s)
    assert all(g.table.pool.n_free == g.table.pool.capacity for g in c.kv_groups) and c.slots.n_held == 0
