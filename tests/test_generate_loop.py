"""Decisions of the generation loop, on the CPU, against a toy stepper whose next token is a
function of the whole history of its sequence (as crates/bfi-runtime/src/engine/decode_tests.rs
does): a mixed-up slot, a lost token or a wrong step shows as a different output."""
import pytest

from builderforce_inference_b200.engine.generate import generate_batch, plan_batches, token_budget
from builderforce_inference_b200.sampling import SampleParams, uniform_draw

VOCAB = 50


def next_token(history):
    h = 17
    for t in history:
        h = (h * 31 + t + 1) % 1000003
    return h % VOCAB


def expected(prompt, budget, stop=()):
    out, hist = [], list(prompt)
    while len(out) < budget:
        t = next_token(hist)
        if t in stop:
            return out, "stop"
        out.append(t)
        hist.append(t)
    return out, "length"


class ToyStepper:
    page_tokens = 64

    def __init__(self, max_seq_len=256, n_pages=64, n_slots=4):
        self.max_seq_len, self.n_pages = max_seq_len, n_pages
        self.free = list(range(n_slots - 1, -1, -1))
        self.hist = {}
        self.log = []            # ("prefill", n_seqs) / ("decode", n_seqs)
        self.max_live = 0

    def acquire(self):
        s = self.free.pop()
        self.hist[s] = []
        self.max_live = max(self.max_live, len(self.hist))
        return s

    def release(self, slot):
        assert slot in self.hist, "slot released twice"
        del self.hist[slot]
        self.free.append(slot)

    def prefill(self, slots, prompts):
        self.log.append(("prefill", len(slots)))
        for s, p in zip(slots, prompts):
            assert self.hist[s] == [], "slot not empty at prefill"
            self.hist[s] = list(p)
        return list(slots)

    def decode(self, slots, tokens):
        self.log.append(("decode", len(slots)))
        for s, t in zip(slots, tokens):
            self.hist[s].append(t)
            assert len(self.hist[s]) <= self.max_seq_len
        return list(slots)

    def sample(self, handle, params, requests, steps, histories):
        return [next_token(self.hist[s]) for s in handle]


def test_budget_rules():
    assert token_budget(10, 5, 100) == 5
    assert token_budget(10, 0, 100) == 90            # 0: what the context still holds (mod.rs:353-357)
    assert token_budget(98, 5, 100) == 2
    assert token_budget(100, 5, 100) == 0
    with pytest.raises(ValueError, match="context_exceeded"):
        token_budget(101, 5, 100)


def test_unequal_prompts_share_steps_and_shorter_ones_end_earlier():
    st = ToyStepper(n_slots=4)
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9], [10, 11]]
    # budgets differ through the context limit: max_seq_len 12 -> 9, 11, 7, 10; cap by max_tokens 8
    st.max_seq_len = 12
    rep = generate_batch(st, prompts, SampleParams(max_tokens=8), max_batch=4)
    want = [expected(p, min(8, 12 - len(p))) for p in prompts]
    assert [(r.tokens, r.finish_reason) for r in rep.results] == want
    # one prefill for all four; shared steps = the longest sequence's, not the sum (mod.rs:664-691)
    assert st.log[0] == ("prefill", 4)
    assert rep.shared_steps == 7 and len(st.log) == 8
    assert [n for k, n in st.log[1:]] == [4, 4, 4, 4, 4, 4, 3]
    assert st.hist == {} and sorted(st.free) == [0, 1, 2, 3]
    assert rep.generated_tokens == sum(len(w[0]) for w in want)


def test_stop_token_is_not_appended_and_frees_the_slot_at_once():
    prompts = [[3, 1, 4], [1, 5, 9, 2], [6, 5]]
    free_run = [expected(p, 12)[0] for p in prompts]
    stop = {free_run[0][4], free_run[2][0]}
    st = ToyStepper()
    rep = generate_batch(st, prompts, SampleParams(max_tokens=12), stop_ids=stop, max_batch=3)
    for p, r in zip(prompts, rep.results):
        toks, why = expected(p, 12, stop)
        assert (r.tokens, r.finish_reason) == (toks, why)
        assert not set(r.tokens) & stop
    assert rep.results[2].tokens == [] and rep.results[2].finish_reason == "stop"
    assert st.log[1] == ("decode", 2)              # the third request never takes a decode step
    assert st.hist == {}


def test_the_last_token_is_not_forwarded():
    st = ToyStepper()
    rep = generate_batch(st, [[1, 2]], SampleParams(max_tokens=3))
    assert len(rep.results[0].tokens) == 3
    assert st.log == [("prefill", 1), ("decode", 1), ("decode", 1)]
    st = ToyStepper()
    rep = generate_batch(st, [[1, 2]], SampleParams(max_tokens=1))
    assert st.log == [("prefill", 1)] and rep.shared_steps == 0


def test_batches_follow_one_another_and_reuse_slots():
    st = ToyStepper(n_slots=2)
    prompts = [[i + 1, i + 2] for i in range(5)]
    rep = generate_batch(st, prompts, SampleParams(max_tokens=4), max_batch=2)
    assert rep.batches == 3 and st.max_live == 2
    assert [k for k, _ in st.log if k == "prefill"] == ["prefill"] * 3
    assert [r.tokens for r in rep.results] == [expected(p, 4)[0] for p in prompts]


def test_batches_respect_the_cache_size():
    # each request may hold 10 + 99 tokens -> 2 pages; 5 pages fit two requests
    assert plan_batches([10] * 5, [100] * 5, max_batch=64, page_tokens=64, n_pages=5) == [[0, 1], [2, 3], [4]]
    assert plan_batches([10, 200, 10], [10, 10, 10], 64, 64, 4) == [[0], [1], [2]]
    with pytest.raises(ValueError, match="cache pages"):
        plan_batches([1000], [10], 64, 64, 4)


def test_full_context_and_empty_prompt():
    st = ToyStepper(max_seq_len=8)
    rep = generate_batch(st, [[1] * 8, [2] * 6], SampleParams(max_tokens=0))
    assert rep.results[0].tokens == [] and rep.results[0].finish_reason == "length"
    assert rep.results[1].tokens == expected([2] * 6, 2)[0]
    assert st.log[0] == ("prefill", 1)
    with pytest.raises(ValueError, match="empty prompt"):
        generate_batch(ToyStepper(), [[]], SampleParams())
    with pytest.raises(ValueError, match="context_exceeded"):
        generate_batch(ToyStepper(max_seq_len=4), [[1] * 5], SampleParams())


def test_slots_are_released_when_a_step_fails():
    class Failing(ToyStepper):
        def decode(self, slots, tokens):
            raise RuntimeError("boom")
    st = Failing()
    with pytest.raises(RuntimeError, match="boom"):
        generate_batch(st, [[1], [2]], SampleParams(max_tokens=5))
    assert st.hist == {}


def test_sample_params_and_draws():
    SampleParams().validate()
    assert SampleParams().max_tokens == 256 and SampleParams().greedy       # sample.rs:33-49
    for bad in (dict(max_tokens=-1), dict(repeat_penalty=0.0), dict(top_p=0.0), dict(min_p=1.5), dict(top_k=-1)):
        with pytest.raises(ValueError):
            SampleParams(**bad).validate()
    us = [uniform_draw(3, r, s) for r in range(4) for s in range(50)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) == len(us)
    assert uniform_draw(3, 1, 2) == uniform_draw(3, 1, 2) != uniform_draw(4, 1, 2)
    assert abs(sum(us) / len(us) - 0.5) < 0.1


def test_the_step_index_arrays_are_packed_in_the_layout_the_kernels_read():
    """``pack_meta`` against the layout written out plainly: ids, positions, slots (padded with 0, 0,
    -1), cu_seqlens (padded with its last offset), sequence slots and starts (padded with -1 and
    0), the page count, the wanted rows."""
    import numpy as np
    from builderforce_inference_b200.engine.engine import pack_meta
    rng = np.random.default_rng(5)
    for n_real_seq, n_seq, pad_tok in ((1, 1, 0), (3, 4, 5), (8, 16, 8), (5, 5, 0)):
        counts = rng.integers(1, 7, n_real_seq)
        cu = [0] + list(np.cumsum(counts))
        k = int(cu[-1])
        n_tok = k + pad_tok
        tok = rng.integers(0, 1000, k).tolist()
        pos = rng.integers(0, 500, k).astype(np.int32)
        slot_of = rng.integers(0, 9, k).tolist()
        seq_slots = rng.integers(0, 9, n_real_seq).tolist()
        seq_starts = rng.integers(0, 400, n_real_seq).tolist()
        want = rng.integers(0, k, 3).tolist()
        plain = np.concatenate([
            tok, np.zeros(pad_tok), pos, np.zeros(pad_tok), slot_of, np.full(pad_tok, -1),
            cu, np.full(n_seq - n_real_seq, cu[-1]), seq_slots, np.full(n_seq - n_real_seq, -1),
            seq_starts, np.zeros(n_seq - n_real_seq), [77], want]).astype(np.int32)
        dst = np.full(plain.shape[0] + 3, 12345, dtype=np.int32)
        n = pack_meta(dst, tok, pos, slot_of, cu, n_tok, n_seq, seq_slots, seq_starts, 77, want)
        assert n == plain.shape[0]
        assert (dst[:n] == plain).all() and (dst[n:] == 12345).all()


def test_pinned_staging_buffers_are_bounded_whatever_the_step_sizes():
    """Many distinct step sizes must not grow page-locked memory: buffers are kept per power-of-two
    capacity, four in rotation each."""
    import numpy as np
    from builderforce_inference_b200.engine.engine import PINNED_RING, PinnedRings
    made = []

    def make(cap):
        made.append(cap)
        return np.empty(cap, dtype=np.int32)

    rings = PinnedRings(make)
    sizes = list(range(1, 5000, 7))
    for n in sizes * 3:
        entry = rings.take(n)
        assert len(entry[0]) >= n
        assert len(entry[0]) == PinnedRings.capacity_for(n)
    capacities = {PinnedRings.capacity_for(n) for n in sizes}
    assert rings.n_buffers() == len(made) == PINNED_RING * len(capacities)
    assert len(capacities) <= 8
    # a ring hands its buffers out in rotation
    first = [id(rings.take(100)[0]) for _ in range(PINNED_RING)]
    assert len(set(first)) == PINNED_RING
    assert [id(rings.take(100)[0]) for _ in range(PINNED_RING)] == first


def test_page_buckets_of_single_token_steps():
    from builderforce_inference_b200.engine.engine import pages_bucket
    assert [pages_bucket(n, 64) for n in (1, 2, 4, 5, 16, 17, 64)] == [1, 4, 4, 16, 16, 64, 64]
    assert pages_bucket(33, 40) == 64 and pages_bucket(40, 40) == 64       # the last bucket holds the limit
    assert pages_bucket(3, 2) == 4 and pages_bucket(1, 1) == 1


def test_page_ranges_of_the_decode_attention():
    """Into how many page ranges a step's sequences are cut: never more than a sequence can have
    pages or the merge kernel takes (32), enough blocks to fill the SMs when the pages allow it, and
    no range much longer than 24 pages unless the cap of 32 forces it."""
    from builderforce_inference_b200.kernels.fast_ops import DECODE_PAGES_PER_BLOCK, decode_splits
    for n_sm in (148, 132, 16):
        for n_seqs in (1, 2, 8, 33, 64, 256):
            for n_kv, group in ((8, 4), (1, 16), (2, 20), (4, 1)):
                for max_pages in (1, 2, 4, 16, 64, 512, 2048):
                    s = decode_splits(n_seqs, n_kv, group, max_pages, n_sm)
                    assert 1 <= s <= min(32, max_pages)
                    blocks = n_seqs * n_kv * ((group + 15) // 16)
                    if s < min(32, max_pages):          # not at a cap: the GPU is filled and ranges are short
                        assert blocks * s >= 2 * n_sm
                        assert -(-max_pages // s) <= DECODE_PAGES_PER_BLOCK
    assert decode_splits(8, 8, 4, 64, 148) == 6 and decode_splits(64, 8, 4, 64, 148) == 3
    assert decode_splits(1, 8, 4, 64, 148) == 32 and decode_splits(64, 8, 4, 16, 148) == 1


class AheadToyStepper(ToyStepper):
    """The toy stepper with the one-step-ahead interface: a ticket is the list of ids "on the
    device"; the loop may read it only through ``sample_wait``."""

    pipelined = True

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.waited = 0

    def sample_start(self, handle, params, requests, steps):
        return {"ids": [next_token(self.hist[s]) for s in handle], "read": False}

    def sample_wait(self, ticket):
        assert not ticket["read"], "a ticket is read once"
        ticket["read"] = True
        self.waited += 1
        return list(ticket["ids"])

    def decode_sampled(self, slots, ticket, rows):
        assert not ticket["read"], "the next step must be launched before the host reads the ids"
        return self.decode(slots, [ticket["ids"][r] for r in rows])


@pytest.mark.parametrize("max_tokens,n_stop", [(8, 0), (12, 2), (1, 0), (2, 1), (30, 3)])
def test_one_step_ahead_gives_the_plain_loops_results(max_tokens, n_stop):
    """The loop that launches step k+1 before it has read token k returns what the plain loop
    returns: same tokens, finish reasons, count of shared steps; every slot is given back; a
    sequence that met its stop token takes at most one step too many."""
    prompts = [[3, 1, 4], [1, 5, 9, 2], [6, 5], [3, 5, 8, 9, 7, 9], [2]]
    free_run = [expected(p, 30)[0] for p in prompts]
    stop = {free_run[i][min(i + 1, max_tokens - 1)] for i in range(n_stop)}
    plain, ahead = ToyStepper(max_seq_len=64), AheadToyStepper(max_seq_len=64)
    a = generate_batch(plain, prompts, SampleParams(max_tokens=max_tokens), stop_ids=stop, max_batch=3)
    b = generate_batch(ahead, prompts, SampleParams(max_tokens=max_tokens), stop_ids=stop, max_batch=3)
    assert [(r.tokens, r.finish_reason) for r in b.results] == [(r.tokens, r.finish_reason) for r in a.results]
    for p, r in zip(prompts, b.results):
        assert (r.tokens, r.finish_reason) == expected(p, max_tokens, stop)
    assert (b.shared_steps, b.generated_tokens, b.batches) == (a.shared_steps, a.generated_tokens, a.batches)
    assert ahead.hist == {} and sorted(ahead.free) == [0, 1, 2, 3]
    n_plain = sum(1 for k, _ in plain.log if k == "decode")
    n_ahead = sum(1 for k, _ in ahead.log if k == "decode")
    assert n_plain <= n_ahead <= n_plain + (2 if n_stop else 0)      # at most one extra step per batch
    if not n_stop:
        assert [n for _, n in ahead.log] == [n for _, n in plain.log]


def test_penalties_keep_the_plain_loop():
    st = AheadToyStepper()
    generate_batch(st, [[1, 2, 3]], SampleParams(max_tokens=4, repeat_penalty=1.2), max_batch=1)
    assert st.waited == 0 and len(st.log) == 4
