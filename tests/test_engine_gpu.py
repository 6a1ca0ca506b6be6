"""The engine against the plain implementation, in float32 and bfloat16: each request alone and
whole; with the last 32 tokens one by one; in batches of unequal lengths whose shorter requests
end earlier, one batch after another so that slots and pages are used again; long decoding; the
first tokens of a sequence; a poisoned cache; cut prompts; windows."""
import pytest
import torch

from helpers import CONFIGS, model_folder, plain_logits, random_prompts, rel_err, store_dtype, tol

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def load(name, dtype, **kw):
    from builderforce_inference_b200.engine.engine import Engine
    kw.setdefault("max_tokens", 4096)
    return Engine.load(model_folder(name, store_dtype(dtype)), dtype=dtype, **kw)


def S(slot, tokens, want):
    from builderforce_inference_b200.engine.engine import SequenceStep
    return SequenceStep(slot, tokens, want)


def check(got, ref, dtype, what=""):
    err = rel_err(got, ref)
    assert err < tol(dtype), f"{what}: rel err {err:.3e} over {tol(dtype):.0e}"
    return err


def first_bad_row(got, ref, dtype):
    for i in range(got.shape[0]):
        if rel_err(got[i:i + 1], ref[i:i + 1]) >= tol(dtype):
            return i
    return None


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_each_request_alone_and_whole(name, dtype):
    eng = load(name, dtype)
    folder = model_folder(name, store_dtype(dtype))
    lens = [1, 2, 5, 17, 33, 64, 65, 100]
    for p in random_prompts(CONFIGS[name]["vocab_size"], lens):
        s = eng.acquire()
        got = eng.step([S(s, p, list(range(len(p))))]).cpu()
        ref = plain_logits(folder, p)
        assert got.shape == ref.shape
        bad = first_bad_row(got, ref, dtype)
        assert bad is None, f"len {len(p)}: first wrong position {bad}"
        eng.release(s)
    eng.cache.check()


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "E", "F"])
def test_last_32_tokens_one_by_one(name, dtype, graphs):
    eng = load(name, dtype, use_graphs=graphs)
    folder = model_folder(name, store_dtype(dtype))
    for p in random_prompts(CONFIGS[name]["vocab_size"], [33, 40, 96, 120], seed=8):
        ref = plain_logits(folder, p)
        k = len(p) - 32
        s = eng.acquire()
        rows = [eng.step([S(s, p[:k], list(range(k)))]).cpu().clone()]
        for t in range(k, len(p)):
            rows.append(eng.step([S(s, [p[t]], [0])]).cpu().clone())
        got = torch.cat(rows)
        bad = first_bad_row(got, ref, dtype)
        assert bad is None, f"len {len(p)}: first wrong position {bad} (prompt end at {k})"
        eng.release(s)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "E", "F"])
def test_unequal_batches_one_after_another(name, dtype, graphs):
    """Batches start together (one step with every prompt prefix), then one token each; shorter
    requests end earlier and give their slot back; the next batch reuses slots and pages that
    still hold the previous batch's rows."""
    eng = load(name, dtype, use_graphs=graphs, max_tokens=64 * 12)
    folder = model_folder(name, store_dtype(dtype))
    vocab = CONFIGS[name]["vocab_size"]
    batches = [[5, 11, 17], [1, 7, 32, 64], [100, 3], [70, 70, 2, 9, 31]]
    seen_slots = []
    for bi, lens in enumerate(batches):
        prompts = random_prompts(vocab, lens, seed=20 + bi)
        refs = [plain_logits(folder, p) for p in prompts]
        n_pref = [max(1, n - 3 - 2 * i) for i, n in enumerate(lens)]
        slots = [eng.acquire() for _ in prompts]
        seen_slots.append(list(slots))
        lg = eng.step([S(s, p[:k], list(range(k))) for s, p, k in zip(slots, prompts, n_pref)]).cpu().clone()
        got = [[] for _ in prompts]
        o = 0
        for i, k in enumerate(n_pref):
            got[i].append(lg[o:o + k])
            o += k
        pos = list(n_pref)
        live = [i for i in range(len(prompts)) if pos[i] < lens[i]]
        for i in range(len(prompts)):
            if i not in live:
                eng.release(slots[i])
        while live:
            lg = eng.step([S(slots[i], [prompts[i][pos[i]]], [0]) for i in live]).cpu().clone()
            for j, i in enumerate(live):
                got[i].append(lg[j:j + 1])
                pos[i] += 1
            for i in list(live):
                if pos[i] == lens[i]:
                    eng.release(slots[i])
                    live.remove(i)
        for i, ref in enumerate(refs):
            g = torch.cat(got[i])
            bad = first_bad_row(g, ref, dtype)
            assert bad is None, f"batch {bi} request {i} (len {lens[i]}, prefix {n_pref[i]}): first wrong position {bad}"
        eng.cache.check()
        assert eng.cache.slots.n_held == 0
    assert set(seen_slots[1]) & set(seen_slots[0]), "slots were not reused"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["D", "E"])
def test_long_decoding(name, dtype):
    """Hundreds of single-token steps across many page edges, two sequences of different phase."""
    eng = load(name, dtype)
    folder = model_folder(name, store_dtype(dtype))
    pa, pb = random_prompts(CONFIGS[name]["vocab_size"], [400, 333], seed=31)
    ra, rb = plain_logits(folder, pa), plain_logits(folder, pb)
    a, b = eng.acquire(), eng.acquire()
    lg = eng.step([S(a, pa[:10], [9]), S(b, pb[:50], [49])]).cpu()
    assert rel_err(lg[0:1], ra[9:10]) < tol(dtype) and rel_err(lg[1:2], rb[49:50]) < tol(dtype)
    ia, ib = 10, 50
    worst = 0.0
    while ia < len(pa) or ib < len(pb):
        seqs, who = [], []
        if ia < len(pa):
            seqs.append(S(a, [pa[ia]], [0])); who.append(("a", ia)); ia += 1
        if ib < len(pb):
            seqs.append(S(b, [pb[ib]], [0])); who.append(("b", ib)); ib += 1
        lg = eng.step(seqs).cpu()
        for j, (w, i) in enumerate(who):
            ref = ra if w == "a" else rb
            e = rel_err(lg[j:j + 1], ref[i:i + 1])
            assert e < tol(dtype), f"sequence {w} position {i}: rel err {e:.3e}"
            worst = max(worst, e)
    eng.release(a)
    eng.release(b)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(dtype):
    """Position 0 and 1: a one-token prompt, then its first decoded tokens, alone and beside a
    longer neighbour."""
    name = "B"
    eng = load(name, dtype)
    folder = model_folder(name, store_dtype(dtype))
    p, q = random_prompts(CONFIGS[name]["vocab_size"], [4, 40], seed=2)
    ref, refq = plain_logits(folder, p), plain_logits(folder, q)
    s = eng.acquire()
    rows = [eng.step([S(s, [p[0]], [0])]).cpu().clone()]
    for t in p[1:]:
        rows.append(eng.step([S(s, [t], [0])]).cpu().clone())
    check(torch.cat(rows), ref, dtype, "alone")
    eng.release(s)
    s, n = eng.acquire(), eng.acquire()
    lg = eng.step([S(s, [p[0]], [0]), S(n, q[:37], [36])]).cpu().clone()
    check(lg[0:1], ref[0:1], dtype, "position 0 beside a neighbour")
    check(lg[1:2], refq[36:37], dtype, "neighbour")
    for i in range(1, 4):
        lg = eng.step([S(n, [q[36 + i]], [0]), S(s, [p[i]], [0])]).cpu().clone()
        check(lg[1:2], ref[i:i + 1], dtype, f"position {i}")
        check(lg[0:1], refq[36 + i:37 + i], dtype, f"neighbour {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "E", "F"])
def test_poisoned_cache_and_stale_rows_do_not_matter(name, dtype):
    """Every page is filled with NaN before use: rows at or past a sequence's length, and rows a
    freed slot left behind, are never read.  E and F have the head sizes of the bfloat16 decode
    and prompt attention kernels (64 with a window of 70, and 128); their prompts are long enough
    for the tensor-core prompt kernel (128 tokens and more in one step)."""
    long = name != "A"
    n1, n2, k2, singles = (330, 300, 140, 20) if long else (70, 45, 20, 10)
    eng = load(name, dtype, max_tokens=64 * (8 if long else 4))
    folder = model_folder(name, store_dtype(dtype))
    eng.cache.poison()
    p1, p2 = random_prompts(CONFIGS[name]["vocab_size"], [n1, n2], seed=4)
    s = eng.acquire()
    check(eng.step([S(s, p1, list(range(n1)))]).cpu(), plain_logits(folder, p1), dtype, "first use")
    eng.release(s)
    s2 = eng.acquire()
    assert s2 == s
    got = [eng.step([S(s2, p2[:k2], list(range(k2)))]).cpu().clone()]
    for t in p2[k2:k2 + singles]:
        got.append(eng.step([S(s2, [t], [0])]).cpu().clone())
    rest = p2[k2 + singles:]                    # a continuation (140 tokens for E and F) over the stale rows
    got.append(eng.step([S(s2, rest, list(range(len(rest))))]).cpu().clone())
    check(torch.cat(got), plain_logits(folder, p2), dtype, "reused slot over stale rows")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["E", "F"])
def test_long_continuations_through_the_fast_attention(name, dtype):
    """Pieces of 128 tokens and more that continue a cached prefix (the tensor-core prompt kernel
    with a start above zero), through the engine's own cache: for E the windowed layer (70 keys)
    has by then given back the pages behind its window, so the kernel meets their -1 entries; a
    neighbour of another phase shares the steps; single tokens in between."""
    folder = model_folder(name, store_dtype(dtype))
    p, q = random_prompts(CONFIGS[name]["vocab_size"], [500, 260], seed=16)
    rp, rq = plain_logits(folder, p), plain_logits(folder, q)
    eng = load(name, dtype)
    eng.cache.poison()
    a, b = eng.acquire(), eng.acquire()
    cuts_a, cuts_b = [0, 1, 70, 200, 201, 372, 500], [0, 130, 131, 260]
    ga, gb = [], []
    for step in range(6):
        seqs = []
        if step + 1 < len(cuts_a):
            ta = p[cuts_a[step]:cuts_a[step + 1]]
            seqs.append(S(a, ta, list(range(len(ta)))))
        if step + 1 < len(cuts_b):
            tb = q[cuts_b[step]:cuts_b[step + 1]]
            seqs.append(S(b, tb, list(range(len(tb)))))
        lg = eng.step(seqs).cpu().clone()
        if step + 1 < len(cuts_a):
            ga.append(lg[:len(ta)])
            lg = lg[len(ta):]
        if step + 1 < len(cuts_b):
            gb.append(lg)
    bad = first_bad_row(torch.cat(ga), rp, dtype)
    assert bad is None, f"request a: first wrong position {bad} (pieces start at {cuts_a})"
    bad = first_bad_row(torch.cat(gb), rq, dtype)
    assert bad is None, f"request b: first wrong position {bad} (pieces start at {cuts_b})"
    if CONFIGS[name].get("use_sliding_window"):
        win = [g for g in eng.cache.kv_groups if g.need.window is not None][0]
        assert win.table.rows[a][:6] == [-1] * 6          # pages behind the window went back
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_rewind_and_redo(name, dtype):
    """A sequence wound back to a shorter prefix and continued gives what the whole gives
    (crates/bfi-models/src/session.rs:50-62); the pages past the mark are free meanwhile."""
    from builderforce_inference_b200.engine.engine import StepError
    folder = model_folder(name, store_dtype(dtype))
    n = 120 if name == "A" else 200
    p, other = random_prompts(CONFIGS[name]["vocab_size"], [n, n], seed=12)
    ref = plain_logits(folder, p)
    eng = load(name, dtype, max_tokens=64 * 8)
    eng.cache.poison()
    s = eng.acquire()
    k = n - 50
    eng.step([S(s, p[:k], [])])
    for t in other[:7]:                                  # tokens that will be wound back
        eng.step([S(s, [t], [0])])
    held = eng.cache.kv_groups[0].table.held_pages()
    eng.rewind(s, 40)
    assert eng.length(s) == 40 and eng.cache.kv_groups[0].table.held_pages() == 1 < held
    got = eng.step([S(s, p[40:k], list(range(k - 40)))]).cpu().clone()
    check(got, ref[40:k], dtype, "redo after rewind")
    rows = [eng.step([S(s, [t], [0])]).cpu().clone() for t in p[k:k + 5]]
    eng.rewind(s, k + 2)
    rows = rows[:2] + [eng.step([S(s, [t], [0])]).cpu().clone() for t in p[k + 2:]]
    check(torch.cat(rows), ref[k:], dtype, "single tokens after a rewind")
    eng.rewind(s, 0)
    check(eng.step([S(s, p[:33], list(range(33)))]).cpu(), ref[:33], dtype, "from the start again")
    with pytest.raises(StepError, match="cannot keep"):
        eng.rewind(s, 34)
    eng.release(s)
    eng.cache.check()
    windowed = load("C", dtype)
    s = windowed.acquire()
    windowed.step([S(s, [1, 2, 3], [])])
    with pytest.raises(StepError, match="rewind unsupported"):
        windowed.rewind(s, 1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C"])
def test_prompts_cut_into_pieces_give_the_same_logits(name, dtype):
    """A step may continue a cached prefix with several tokens, and the engine itself cuts long
    steps into micro-batches: neither changes a logit beyond rounding."""
    folder = model_folder(name, store_dtype(dtype))
    p, q = random_prompts(CONFIGS[name]["vocab_size"], [150, 90], seed=6)
    rp, rq = plain_logits(folder, p), plain_logits(folder, q)
    eng = load(name, dtype)
    a, b = eng.acquire(), eng.acquire()
    cuts_a, cuts_b = [0, 1, 64, 65, 130, 150], [0, 33, 34, 90]
    ga, gb = [], []
    for step in range(5):
        seqs = []
        if step + 1 < len(cuts_a):
            ta = p[cuts_a[step]:cuts_a[step + 1]]
            seqs.append(S(a, ta, list(range(len(ta)))))
        if step + 1 < len(cuts_b):
            tb = q[cuts_b[step]:cuts_b[step + 1]]
            seqs.append(S(b, tb, list(range(len(tb)))))
        lg = eng.step(seqs).cpu().clone()
        if step + 1 < len(cuts_a):
            ga.append(lg[:len(ta)])
            lg = lg[len(ta):]
        if step + 1 < len(cuts_b):
            gb.append(lg)
    check(torch.cat(ga), rp, dtype, "pieces, request a")
    check(torch.cat(gb), rq, dtype, "pieces, request b")
    small = load(name, dtype, prefill_chunk_tokens=64)
    a, b = small.acquire(), small.acquire()
    lg = small.step([S(a, p, list(range(150))), S(b, q, [89, 0, 45])]).cpu()
    check(lg[:150], rp, dtype, "micro-batches, request a")
    check(lg[150:], rq[[89, 0, 45]], dtype, "micro-batches, wanted places in the given order")


def test_logits_do_not_depend_on_the_batch_or_the_slot():
    """The same request alone, in a crowd, in another slot and through a padded captured step."""
    name, dtype = "B", "float32"
    folder = model_folder(name, store_dtype(dtype))
    p = random_prompts(CONFIGS[name]["vocab_size"], [48], seed=9)[0]
    others = random_prompts(CONFIGS[name]["vocab_size"], [5, 90, 64, 33, 12], seed=10)
    outs = []
    for crowd, graphs in ((0, False), (3, False), (5, True), (2, True)):
        eng = load(name, dtype, use_graphs=graphs)
        pre = [eng.acquire() for _ in range(crowd)]
        s = eng.acquire()
        seqs = [S(x, o[:-1], []) for x, o in zip(pre, others)] + [S(s, p[:40], [])]
        assert eng.step(seqs).shape[0] == 0
        rows = []
        for i in range(40, 48):
            seqs = [S(x, [o[-1]], []) for x, o in zip(pre[:crowd if i == 40 else 0], others)] + [S(s, [p[i]], [0])]
            rows.append(eng.step(seqs).cpu().clone())
        outs.append(torch.cat(rows))
    ref = plain_logits(folder, p)[40:]
    for o in outs:
        assert rel_err(o, ref) < 1e-5
        assert rel_err(o, outs[0]) < 2e-6


def test_refusals_come_before_any_launch():
    from builderforce_inference_b200.engine.engine import StepError
    eng = load("A", "float32", max_tokens=128)
    s = eng.acquire()
    with pytest.raises(StepError, match="empty token list"):
        eng.step([S(s, [], [])])
    with pytest.raises(StepError, match="out of range"):
        eng.step([S(s, [1, 256], [0])])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([S(s, [1, 2], [2])])
    with pytest.raises(StepError, match="context_exceeded"):
        eng.step([S(s, [1] * 129, [0])])
    with pytest.raises(StepError, match="not held"):
        eng.step([S(s + 1, [1], [0])])
    assert eng.length(s) == 0
    eng.step([S(s, [1] * 128, [127])])
    with pytest.raises(StepError, match="context_exceeded"):
        eng.step([S(s, [1], [0])])
    eng.release(s)
    eng.cache.check()


def test_a_32bit_checkpoint_runs_in_a_bfloat16_engine():
    """A tensor stored in 32-bit stays so; the kernels take the mixed pair."""
    name = "A"
    folder = model_folder(name, torch.float32)
    from builderforce_inference_b200.engine.engine import Engine
    eng = Engine.load(folder, dtype="bfloat16", max_tokens=256)
    assert eng.decoder.embedding.dtype == torch.float32
    p = random_prompts(CONFIGS[name]["vocab_size"], [40])[0]
    s = eng.acquire()
    got = eng.step([S(s, p, list(range(40)))]).cpu()
    assert rel_err(got, plain_logits(folder, p)) < tol("bfloat16")


@pytest.mark.parametrize("dtype", DTYPES)
def test_benchmark_layer_sizes_against_plain(dtype):
    """Two layers at the Qwen3-4B sizes: a prompt whole (300 tokens: the many-token kernels), its
    last 12 tokens one by one (the few-row kernels), and an unequal batch of 40 (the kernels in
    between), all against the plain implementation."""
    name = "WIDE"
    folder = model_folder(name, store_dtype(dtype))
    eng = load(name, dtype, max_tokens=64 * 64)
    prompts = random_prompts(CONFIGS[name]["vocab_size"], [300, 130, 77], seed=41)
    refs = [plain_logits(folder, p) for p in prompts]
    s = eng.acquire()
    got = eng.step([S(s, prompts[0], list(range(300)))]).cpu()
    bad = first_bad_row(got, refs[0], dtype)
    assert bad is None, f"whole prompt: first wrong position {bad}, rel err {rel_err(got, refs[0]):.3e}"
    eng.release(s)
    s = eng.acquire()
    rows = [eng.step([S(s, prompts[0][:288], [287])]).cpu().clone()]
    for t in range(288, 300):
        rows.append(eng.step([S(s, [prompts[0][t]], [0])]).cpu().clone())
    check(torch.cat(rows), refs[0][287:], dtype, "last tokens one by one")
    eng.release(s)
    # 40 sequences decode together: 3 real requests and copies of the third at other phases
    slots = [eng.acquire() for _ in range(40)]
    pre = [290, 120, 70] + [10 + i for i in range(37)]
    src = [0, 1, 2] + [2] * 37
    eng.step([S(sl, prompts[i][:k], []) for sl, i, k in zip(slots, src, pre)])
    for step in range(5):
        lg = eng.step([S(sl, [prompts[i][k + step]], [0]) for sl, i, k in zip(slots, src, pre)]).cpu()
        for j in (0, 1, 2, 3, 20, 39):
            e = rel_err(lg[j:j + 1], refs[src[j]][pre[j] + step:pre[j] + step + 1])
            assert e < tol(dtype), f"batch of 40, row {j}, step {step}: rel err {e:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_benchmark_lengths_against_plain(dtype):
    """Two layers at the Qwen3-4B widths at the lengths the benchmark runs: a 2,048-token prompt
    whole (16 tiles of 128 tokens per head); the same cut 1,000 + 1,048 (a long continuation);
    single tokens at positions 4,088 to 4,095 alone (64 pages, the most page ranges per sequence)
    and inside unequal batches of 8 and of 40.  Every sequence is a prefix of one 4,096-token
    prompt, so one run of the plain implementation serves them all."""
    name = "WIDE"
    folder = model_folder(name, store_dtype(dtype))
    full = random_prompts(CONFIGS[name]["vocab_size"], [4096], seed=77)[0]
    ref = plain_logits(folder, full)
    eng = load(name, dtype, max_tokens=64 * 600, prefill_chunk_tokens=4096)
    eng.cache.poison()
    s = eng.acquire()
    got = eng.step([S(s, full[:2048], list(range(2048)))]).cpu()
    bad = first_bad_row(got, ref[:2048], dtype)
    assert bad is None, f"2,048 tokens whole: first wrong position {bad}"
    eng.release(s)
    s = eng.acquire()
    got = [eng.step([S(s, full[:1000], list(range(990, 1000)))]).cpu().clone()]
    got.append(eng.step([S(s, full[1000:2048], list(range(1048)))]).cpu().clone())
    bad = first_bad_row(torch.cat(got), ref[990:2048], dtype)
    assert bad is None, f"1,000 + 1,048: first wrong position {990 + bad}"
    # go on to 4,088 (a continuation of 2,040 tokens) and decode the last 8 alone
    eng.step([S(s, full[2048:4088], [])])
    rows = [eng.step([S(s, [full[t]], [0])]).cpu().clone() for t in range(4088, 4096)]
    check(torch.cat(rows), ref[4088:], dtype, "positions 4,088..4,095 alone")
    eng.release(s)
    for batch in (8, 40):
        lens = [4088] + [1 + (i * 397) % 700 for i in range(1, batch - 1)] + [2047]
        slots = [eng.acquire() for _ in lens]
        eng.step([S(sl, full[:n], []) for sl, n in zip(slots, lens)])
        for step in range(8):
            lg = eng.step([S(sl, [full[n + step]], [0]) for sl, n in zip(slots, lens)]).cpu()
            for j in (0, 1, batch // 2, batch - 1):
                e = rel_err(lg[j:j + 1], ref[lens[j] + step:lens[j] + step + 1])
                assert e < tol(dtype), f"batch of {batch}, row {j} (position {lens[j] + step}): rel err {e:.3e}"
        for sl in slots:
            eng.release(sl)
    eng.cache.check()


@pytest.mark.parametrize("graphs", [False, True])
def test_a_step_fed_from_device_ids_equals_the_same_step_from_host_ids(graphs):
    name, dtype = "B", "float32"
    folder = model_folder(name, store_dtype(dtype))
    prompts = random_prompts(CONFIGS[name]["vocab_size"], [20, 3, 41], seed=33)
    nxt = [7, 300, 123]
    outs = []
    for fed_on_device in (False, True):
        eng = load(name, dtype, use_graphs=graphs)
        slots = [eng.acquire() for _ in prompts]
        eng.step([S(s, p, []) for s, p in zip(slots, prompts)])
        if fed_on_device:
            ids = torch.tensor(nxt, dtype=torch.int32, device="cuda:0")
            outs.append(eng.step_sampled(slots, ids).cpu().clone())
            outs.append(eng.step_sampled(slots[:2], ids[1:].contiguous()).cpu().clone())
        else:
            outs.append(eng.step([S(s, [t], [0]) for s, t in zip(slots, nxt)]).cpu().clone())
            outs.append(eng.step([S(s, [t], [0]) for s, t in zip(slots[:2], nxt[1:])]).cpu().clone())
        assert [eng.length(s) for s in slots] == [22, 5, 42]
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])
    ref = plain_logits(folder, prompts[0] + [nxt[0], nxt[1]])
    assert rel_err(outs[3][0:1], ref[-1:]) < tol(dtype)
