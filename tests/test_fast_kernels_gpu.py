"""The bfloat16 kernels written for speed, each alone against a plain float32 reference of the
same operation on the same bfloat16 inputs."""
import math

import pytest
import torch

from helpers import rel_err
from plain import qwen3_plain as P
from builderforce_inference_b200.kernels.library import KernelError
from test_kernels_gpu import DEV, Pages, gen, plain_paged_attention

pytestmark = pytest.mark.gpu


def fast():
    from builderforce_inference_b200.kernels import fast_ops
    return fast_ops


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("n,k", [(38, 64), (130, 136), (2560, 1024), (9730, 520)])
def test_skinny_gemm_store(m, n, k):
    a = torch.randn(m, k, generator=gen(m)).bfloat16()
    w = (torch.randn(n, k, generator=gen(n)) * 0.1).bfloat16()
    ref = P.linear(w.float(), a.float())
    for odt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):
        out = torch.full((m, n), float("nan"), dtype=odt, device=DEV)
        assert fast().skinny_gemm(a.to(DEV), w.to(DEV), out, 0)
        assert rel_err(out.float(), ref) < tol


@pytest.mark.parametrize("m", [1, 5, 24, 64])
def test_skinny_gemm_epilogues(m):
    n, k = 304, 2560
    a = torch.randn(m, k, generator=gen(m)).bfloat16()
    w = (torch.randn(n, k, generator=gen(3)) * 0.05).bfloat16()
    res = torch.randn(m, n, generator=gen(4))
    out = res.clone().to(DEV)
    assert fast().skinny_gemm(a.to(DEV), w.to(DEV), out, 1)
    assert rel_err(out, res + P.linear(w.float(), a.float())) < 2e-5
    gate, up = w[0::2].float(), w[1::2].float()          # rows interleaved gate/up
    out2 = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert fast().skinny_gemm(a.to(DEV), w.to(DEV), out2, 2)
    assert rel_err(out2.float(), P.swiglu(P.linear(gate, a.float()), P.linear(up, a.float()))) < 1e-2


def test_skinny_gemm_declines_what_it_cannot_do():
    a = torch.randn(4, 20, device=DEV).bfloat16()
    w = torch.randn(8, 20, device=DEV).bfloat16()
    out = torch.empty(4, 8, dtype=torch.float32, device=DEV)
    assert not fast().skinny_gemm(a, w, out, 0)                       # K not a multiple of 8
    assert not fast().linear_bf16(a, w, out, 0)                       # nor does the tensor-core kernel take it
    a = torch.randn(65, 64, device=DEV).bfloat16()
    w = torch.randn(8, 64, device=DEV).bfloat16()
    assert not fast().skinny_gemm(a, w, torch.empty(65, 8, dtype=torch.float32, device=DEV), 0)   # too many rows
    # the dispatcher then takes another kernel and the result is still right
    from builderforce_inference_b200.kernels.linear import linear
    out = torch.empty(65, 8, dtype=torch.float32, device=DEV)
    linear(a, w, out)
    assert rel_err(out, a.float().cpu() @ w.float().cpu().t()) < 2e-5
    a = torch.randn(70, 20, device=DEV).bfloat16()
    w = torch.randn(9, 20, device=DEV).bfloat16()
    out = torch.empty(70, 9, dtype=torch.float32, device=DEV)
    linear(a, w, out)                                                  # K = 20: only the general kernel takes it
    assert rel_err(out, a.float().cpu() @ w.float().cpu().t()) < 2e-5


@pytest.mark.parametrize("n,k,stages,ksplit", [(256, 512, 2, 1), (300, 1000, 6, 3), (128, 64, 12, 1)])
def test_weight_stream_reads_a_matrix_and_trips_no_wait(n, k, stages, ksplit):
    """The measuring kernel of the few-row products' rings: it computes nothing, so what there is
    to check is that every size runs through and no bounded wait runs out."""
    assert tc_status_clear() == 0
    w = torch.randn(n, k, generator=gen(n)).bfloat16().to(DEV)
    for _ in range(3):
        assert fast().weight_stream(w, stages=stages, ksplit=ksplit)
    torch.cuda.synchronize()
    assert tc_status_clear() == 0
    with pytest.raises(KernelError):
        fast().weight_stream(w.float())


class Ctx:
    """The few fields of a step context the decode attention reads."""

    def __init__(self, slots, starts):
        from builderforce_inference_b200.engine.context import Workspace
        i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
        self.n_seqs = self.n_tokens = len(slots)
        self.max_seq_tokens = 1
        self.seq_slot, self.seq_start = i32(slots), i32(starts)
        self.total_pages = i32([sum(s // 64 + 1 for s, sl in zip(starts, slots) if sl >= 0)])
        self.workspace = Workspace(torch.device(DEV))


@pytest.mark.parametrize("n_q,n_kv,d", [(8, 2, 64), (4, 4, 64), (32, 8, 128), (16, 1, 128), (6, 3, 128), (40, 2, 64)])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_decode(n_q, n_kv, d, window, monkeypatch):
    starts = [0, 1, 62, 63, 64, 65, 127, 128, 300, 511, 700]
    slots = list(range(len(starts)))
    slots[3] = -1                                        # a padding row: its output stays untouched
    pages = Pages(len(starts), 768, n_kv, d, torch.bfloat16, window=window, seed=d + n_q)
    g = gen(n_q + d)
    scale = 1.0 / math.sqrt(d)
    qs, refs = [], []
    for slot, start in zip(slots, starts):
        n = start + 1
        k = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        v = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        q = torch.randn(1, n_q, d, generator=g).bfloat16().float()
        if slot >= 0:
            pages.write(slot, 0, k, v)
        qs.append(q.reshape(1, n_q * d))
        refs.append(plain_paged_attention(q, k, v, start, window, scale).reshape(1, n_q * d))
    q_all = torch.cat(qs).bfloat16().to(DEV)
    ref = torch.cat(refs)
    for forced in (None, 1, 2, 5, 12):
        ctx = Ctx(slots, starts)
        if forced is not None:
            monkeypatch.setattr(fast(), "decode_splits", lambda *a, f=forced: f)
        out = torch.full((len(starts), n_q * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert fast().attention_decode_bf16(ctx, q_all, out, pages.view, n_q, scale)
        got = out.float().cpu()
        assert torch.isnan(got[3]).all()
        keep = [i for i in range(len(starts)) if i != 3]
        assert rel_err(got[keep], ref[keep]) < 1e-2, forced


def test_attention_decode_finds_a_far_key_and_respects_the_window_edge():
    n_q, n_kv, d, n = 8, 2, 128, 1500
    g = gen(1)
    q = torch.randn(1, n_q, d, generator=g)
    q = q / q.norm(dim=-1, keepdim=True)
    v = torch.randn(n, n_kv, d, generator=g)
    scale = 1.0 / math.sqrt(d)
    for window, target, inside in ((None, 0, True), (None, 64, True), (None, 1087, True), (None, 1499, True),
                                   (200, 1300, True), (200, 1299, False), (64, 1436, True), (64, 1435, False)):
        pages = Pages(1, n, n_kv, d, torch.bfloat16, window=window)
        k = torch.randn(n, n_kv, d, generator=g) * 0.05
        for h in range(n_kv):
            k[target, h] = q[0, h * 4] * 40.0 * math.sqrt(d)
        pages.write(0, 0, k, v)
        out = torch.empty(1, n_q * d, dtype=torch.bfloat16, device=DEV)
        assert fast().attention_decode_bf16(Ctx([0], [n - 1]), q.reshape(1, -1).bfloat16().to(DEV), out, pages.view,
                                            n_q, scale)
        got = out.float().cpu().reshape(n_q, d)
        kq, vq = pages.read(0, n)
        ref = plain_paged_attention(q.bfloat16().float(), kq, vq, n - 1, window, scale).reshape(n_q, d)
        assert rel_err(got, ref) < 1e-2
        for h in range(n_kv):
            close = bool((got[h * 4] - vq[target, h]).abs().max() < 0.05)
            assert close == inside, (window, target)


def test_attention_decode_declines_other_head_sizes():
    pages = Pages(1, 64, 1, 48, torch.bfloat16)
    q = torch.zeros(1, 48, dtype=torch.bfloat16, device=DEV)
    assert not fast().attention_decode_bf16(Ctx([0], [3]), q, torch.empty_like(q), pages.view, 1, 0.1)


@pytest.mark.parametrize("m", [1, 8, 24, 64])
def test_skinny_gemm_splits_k_between_blocks_and_stays_deterministic(m):
    """Few row tiles and a long K: blocks share K and the last to arrive adds their partial sums in
    a fixed order, so two runs agree to the bit and the counters are left at zero."""
    n, k = 2560, 4096
    a = torch.randn(m, k, generator=gen(m)).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=gen(5)) * 0.05).bfloat16().to(DEV)
    assert fast()._skinny_scratch_need(m, n, k)[0] > 0          # this shape does split
    res = torch.randn(m, n, generator=gen(6))
    outs = []
    for _ in range(3):
        out = res.clone().to(DEV)
        assert fast().skinny_gemm(a, w, out, 1)
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert rel_err(outs[0], res + P.linear(w.float().cpu(), a.float().cpu())) < 2e-5
    assert int(fast()._split_scratch.counters[a.device].abs().sum()) == 0


# ------------------------------------------------------------------ tcgen05 / TMA matrix product
def tc_check(m, n, k, epi, seed=0):
    g = gen(seed + m + n)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    ref = P.linear(w.float(), a.float())
    if epi == 1:
        res = torch.randn(m, n, generator=g)
        out = res.clone().to(DEV)
        ref = res + ref
    elif epi == 2:
        out = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
        ref = P.swiglu(ref[:, 0::2], ref[:, 1::2])
    else:
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    assert fast().gemm_tcgen05(a.to(DEV), w.to(DEV), out, epi)
    torch.cuda.synchronize()
    assert int(fast().tc_status(torch.device(DEV))[0].item()) == 0, "a bounded wait ran out"
    assert rel_err(out.float(), ref) < (1e-2 if epi == 2 else 3e-5), (m, n, k, epi)


@pytest.mark.parametrize("m", [1, 9, 16, 17, 33, 64, 65, 128, 129, 300, 1000])
@pytest.mark.parametrize("n,k", [(128, 64), (130, 136), (2560, 1024), (72, 200), (640, 2568)])
def test_gemm_tcgen05_any_size(m, n, k):
    """Token counts around every tile size, widths that are no multiple of 128 (ragged last tile),
    K that is no multiple of 64 (zero-filled tail) and small enough to leave splits empty."""
    tc_check(m, n, k, 0)


@pytest.mark.parametrize("m,n,k", [(12, 2560, 4096), (64, 2560, 9728), (40, 6144, 2560), (200, 384, 4096), (2048, 2560, 512)])
@pytest.mark.parametrize("epi", [0, 1, 2])
def test_gemm_tcgen05_epilogues_with_and_without_split(m, n, k, epi):
    """Few row tiles make the blocks of a tile a cluster that splits K; the sum is added in split
    order out of the blocks' shared memory, so two runs agree to the bit."""
    tc_check(m, n, k, epi)
    g = gen(1)
    a = torch.randn(m, k, generator=g).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16().to(DEV)
    outs = []
    for _ in range(2):
        out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
        assert fast().gemm_tcgen05(a, w, out, 0)
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1])


def test_gemm_tcgen05_strided_operands_and_refusals():
    big = torch.randn(50, 4096, generator=gen(2)).bfloat16().to(DEV)
    a = big[:, 1024:1024 + 512]                                    # row stride 4096, 512 columns
    w = (torch.randn(300, 512, generator=gen(3)) * 0.05).bfloat16().to(DEV)
    out_big = torch.zeros(50, 1000, dtype=torch.float32, device=DEV)
    out = out_big[:, 100:400]
    assert fast().gemm_tcgen05(a, w, out, 0)
    assert rel_err(out, a.float().cpu() @ w.float().cpu().t()) < 3e-5
    assert float(out_big[:, :100].abs().sum()) == 0 and float(out_big[:, 400:].abs().sum()) == 0
    assert not fast().gemm_tcgen05(big[:, 3:3 + 64], w[:, :64], torch.zeros(50, 300, device=DEV), 0)   # unaligned base
    assert not fast().gemm_tcgen05(big[:, :20], w[:, :20], torch.zeros(50, 300, device=DEV), 0)        # K % 8 != 0


# ------------------------------------------------------------------ tensor-core prompt attention
class PrefillCtx:
    def __init__(self, seqs):
        i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
        cu = [0]
        for _, _, t in seqs:
            cu.append(cu[-1] + t)
        self.n_seqs, self.n_tokens = len(seqs), cu[-1]
        self.max_seq_tokens = max(t for _, _, t in seqs)
        self.cu_seqlens, self.seq_slot, self.seq_start = i32(cu), i32([s for s, _, _ in seqs]), i32([st for _, st, _ in seqs])


def prefill_kernel(name):
    return fast().attention_prefill_bf16 if name == "mma" else fast().attention_prefill_tcgen05_bf16


def tc_status_clear():
    st = fast().tc_status(torch.device(DEV))
    words = st.tolist()
    st.zero_()
    assert words[1] == 0 and words[2] == 0, "the prompt attention left its ticket counters standing"
    return words[0]


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
@pytest.mark.parametrize("n_q,n_kv,d", [(8, 2, 64), (4, 4, 128), (6, 1, 128), (3, 3, 64)])
@pytest.mark.parametrize("window", [None, 70])
def test_attention_prefill(n_q, n_kv, d, window, kernel):
    """Whole prompts, continuations of a cached prefix and single tokens in one launch, lengths around
    the 16-token warp rows, the 64- and 128-token blocks and the 64-key pages; one padding sequence."""
    seqs = [(2, 0, 33), (0, 0, 1), (3, 95, 1), (1, 31, 34), (-1, 0, 5), (4, 64, 64), (5, 0, 200), (6, 63, 130), (7, 10, 17)]
    pages = Pages(8, 400, n_kv, d, torch.bfloat16, window=window, seed=d + n_q)
    g = gen(n_q * 10 + d)
    scale = 1.0 / math.sqrt(d)
    qs, refs = [], []
    for slot, start, t in seqs:
        n = start + t
        k = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        v = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        qq = torch.randn(t, n_q, d, generator=g).bfloat16().float()
        if slot >= 0:
            pages.write(slot, 0, k, v)
        qs.append(qq.reshape(t, n_q * d))
        refs.append(plain_paged_attention(qq, k, v, start, window, scale).reshape(t, n_q * d))
    q_all = torch.cat(qs).bfloat16().to(DEV)
    out = torch.full(q_all.shape, float("nan"), dtype=torch.bfloat16, device=DEV)
    assert prefill_kernel(kernel)(PrefillCtx(seqs), q_all, out, pages.view, n_q, scale)
    got, ref = out.float().cpu(), torch.cat(refs)
    assert tc_status_clear() == 0
    o = 0
    for slot, start, t in seqs:
        if slot < 0:
            assert torch.isnan(got[o:o + t]).all()
        else:
            assert rel_err(got[o:o + t], ref[o:o + t]) < 1e-2, (slot, start, t)
        o += t


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
def test_attention_prefill_far_key_and_causality(kernel):
    """A dominating key far back must be found by late queries and must not leak to earlier ones."""
    n_q, n_kv, d, n = 4, 2, 128, 600
    g = gen(5)
    scale = 1.0 / math.sqrt(d)
    q = torch.randn(n, n_q, d, generator=g)
    q = q / q.norm(dim=-1, keepdim=True)
    v = torch.randn(n, n_kv, d, generator=g)
    k = torch.randn(n, n_kv, d, generator=g) * 0.05
    target = 257
    k[target, 0] = q[500, 0] * 40.0 * math.sqrt(d)       # query 500, head 0 must find key 257
    k[target, 1] = q[100, 2] * 40.0 * math.sqrt(d)       # query 100 (head 2) lies before the key: must not see it
    pages = Pages(1, n, n_kv, d, torch.bfloat16)
    pages.write(0, 0, k, v)
    out = torch.empty(n, n_q * d, dtype=torch.bfloat16, device=DEV)
    assert prefill_kernel(kernel)(PrefillCtx([(0, 0, n)]), q.reshape(n, -1).bfloat16().to(DEV), out, pages.view, n_q, scale)
    got = out.float().cpu().reshape(n, n_q, d)
    kq, vq = pages.read(0, n)
    ref = plain_paged_attention(q.bfloat16().float(), kq, vq, 0, None, scale)
    assert rel_err(got, ref) < 1e-2
    assert (got[500, 0] - vq[target, 0]).abs().max() < 0.05
    assert (got[100, 2] - vq[target, 1]).abs().max() > 0.2


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("window", [None, 200])
def test_attention_prefill_tcgen05_long_and_ragged(d, window):
    """Several 128-token blocks per sequence, prefixes that end inside a page, a last page that is
    partly unwritten (the cache is full of NaN there), pages before the window given back."""
    n_q, n_kv = 6, 2
    seqs = [(0, 0, 700), (1, 333, 400), (2, 1000, 129), (3, 64, 128), (4, 5, 255)]
    pages = Pages(5, 1200, n_kv, d, torch.bfloat16, window=window, seed=d)
    g = gen(d + 1)
    scale = 1.0 / math.sqrt(d)
    qs, refs = [], []
    for slot, start, t in seqs:
        n = start + t
        k = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        v = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        qq = torch.randn(t, n_q, d, generator=g).bfloat16().float()
        pages.write(slot, 0, k, v)
        if window is not None:
            # pages wholly before the window of the step's first new token are no longer held
            table = pages.table.clone()
            table[slot, :max(0, start - window + 1) // 64] = -1
            pages.table = table
        qs.append(qq.reshape(t, n_q * d))
        refs.append(plain_paged_attention(qq, k, v, start, window, scale).reshape(t, n_q * d))
    pages.view.block_table.copy_(pages.table)
    q_all = torch.cat(qs).bfloat16().to(DEV)
    out = torch.full(q_all.shape, float("nan"), dtype=torch.bfloat16, device=DEV)
    assert fast().attention_prefill_tcgen05_bf16(PrefillCtx(seqs), q_all, out, pages.view, n_q, scale)
    got, ref = out.float().cpu(), torch.cat(refs)
    assert tc_status_clear() == 0
    o = 0
    for slot, start, t in seqs:
        assert rel_err(got[o:o + t], ref[o:o + t]) < 1e-2, (slot, start, t)
        o += t


@pytest.mark.parametrize("window", [None, 150])
def test_attention_prefill_tcgen05_many_items_per_block(window):
    """Far more (sequence, head, 128-token tile) items than SMs, of unequal sizes, so that every
    block runs through many items: its rings, score and output buffers and the shared ticket
    counter carry on from one item into the next; some sequences are padding."""
    n_q, n_kv, d = 8, 4, 128
    g = gen(77)
    lens = torch.randint(1, 640, (44,), generator=g).tolist()
    starts = torch.randint(0, 130, (44,), generator=g).tolist()
    seqs, slot = [], 0
    for i, (start, t) in enumerate(zip(starts, lens)):
        if i % 9 == 4:
            seqs.append((-1, 0, t))
        else:
            seqs.append((slot, start if i % 3 else 0, t))
            slot += 1
    pages = Pages(slot, 800, n_kv, d, torch.bfloat16, window=window, seed=5)
    scale = 1.0 / math.sqrt(d)
    qs, refs = [], []
    for sl, start, t in seqs:
        n = start + t
        k = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        v = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        qq = torch.randn(t, n_q, d, generator=g).bfloat16().float()
        if sl >= 0:
            pages.write(sl, 0, k, v)
        qs.append(qq.reshape(t, n_q * d))
        refs.append(plain_paged_attention(qq, k, v, start, window, scale).reshape(t, n_q * d))
    q_all = torch.cat(qs).bfloat16().to(DEV)
    ref = torch.cat(refs)
    for _ in range(2):                                   # the second launch finds the counters as the first left them
        out = torch.full(q_all.shape, float("nan"), dtype=torch.bfloat16, device=DEV)
        assert fast().attention_prefill_tcgen05_bf16(PrefillCtx(seqs), q_all, out, pages.view, n_q, scale)
        got = out.float().cpu()
        assert tc_status_clear() == 0
        o = 0
        for sl, start, t in seqs:
            if sl < 0:
                assert torch.isnan(got[o:o + t]).all()
            else:
                assert rel_err(got[o:o + t], ref[o:o + t]) < 1e-2, (sl, start, t)
            o += t


def test_attention_prefill_tcgen05_more_sequences_than_its_table_holds():
    """Above 512 sequences the kernel reads the sequences' numbers from global memory instead of
    its shared-memory table."""
    n_q, n_kv, d = 2, 1, 64
    seqs = [(i, 0, 1 + i % 3) for i in range(530)] + [(530, 7, 131)]
    pages = Pages(531, 192, n_kv, d, torch.bfloat16, seed=9)
    g = gen(31)
    scale = 1.0 / math.sqrt(d)
    qs, refs = [], []
    for sl, start, t in seqs:
        n = start + t
        k = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        v = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        qq = torch.randn(t, n_q, d, generator=g).bfloat16().float()
        pages.write(sl, 0, k, v)
        qs.append(qq.reshape(t, n_q * d))
        refs.append(plain_paged_attention(qq, k, v, start, None, scale).reshape(t, n_q * d))
    q_all = torch.cat(qs).bfloat16().to(DEV)
    out = torch.full(q_all.shape, float("nan"), dtype=torch.bfloat16, device=DEV)
    assert fast().attention_prefill_tcgen05_bf16(PrefillCtx(seqs), q_all, out, pages.view, n_q, scale)
    assert tc_status_clear() == 0
    assert rel_err(out.float().cpu(), torch.cat(refs)) < 1e-2


def test_attention_prefill_tcgen05_rising_scores():
    """Scores that grow from key to key by far more than the kernel lets a stale maximum lag (2^8):
    the running maximum must be raised, and the output rescaled, tile after tile."""
    n_q, n_kv, d, n = 2, 1, 128, 640
    g = gen(9)
    scale = 1.0 / math.sqrt(d)
    u = torch.randn(d, generator=g)
    u = u / u.norm()
    q = (u * 8.0 * math.sqrt(d)).repeat(n, n_q, 1) + 0.1 * torch.randn(n, n_q, d, generator=g)
    ramp = torch.linspace(-4.0, 12.0, n).reshape(n, 1, 1)                # q.k*scale runs from about -32 to 96
    k = ramp * u.reshape(1, 1, d) + 0.05 * torch.randn(n, n_kv, d, generator=g)
    v = torch.randn(n, n_kv, d, generator=g)
    pages = Pages(1, n, n_kv, d, torch.bfloat16)
    pages.write(0, 0, k, v)
    out = torch.empty(n, n_q * d, dtype=torch.bfloat16, device=DEV)
    assert fast().attention_prefill_tcgen05_bf16(PrefillCtx([(0, 0, n)]), q.reshape(n, -1).bfloat16().to(DEV), out, pages.view,
                                                 n_q, scale)
    assert tc_status_clear() == 0
    kq, vq = pages.read(0, n)
    ref = plain_paged_attention(q.bfloat16().float(), kq, vq, 0, None, scale)
    got = out.float().cpu().reshape(n, n_q, d)
    assert torch.isfinite(got).all()
    assert rel_err(got, ref) < 1e-2


@pytest.mark.parametrize("m", [128, 129, 255, 1000, 2100])
@pytest.mark.parametrize("n,k,epi", [(256, 64, 0), (130, 136, 0), (2568, 1024, 1), (304, 2560, 2), (6144, 2560, 0), (72, 200, 2)])
def test_gemm_tcgen05_many_tokens(m, n, k, epi):
    """128 tokens or more take the persistent kernel (tokens on the lanes, two accumulators in
    tensor memory); ragged token and feature tiles, K tails, every epilogue."""
    tc_check(m, n, k, epi, seed=7)


@pytest.mark.parametrize("halves", [1, 2])
@pytest.mark.parametrize("tile_n", [128, 144, 176, 240, 256])
@pytest.mark.parametrize("m,n,k,epi", [(300, 2560, 512, 1), (129, 1000, 200, 0), (640, 2000, 1024, 2), (1500, 700, 4096, 0)])
def test_gemm_tcgen05_many_tokens_every_tile(tile_n, halves, m, n, k, epi):
    """The persistent kernel's tile (128 or 256 tokens x 128..256 features) is chosen per product;
    every tile gives the same result, with several tiles per block and ragged edges."""
    import ctypes
    from builderforce_inference_b200.kernels.library import library
    lib = library("fast").lib
    # the override holds for the next call of the product only: nothing to put back
    lib.bfi_gemm_tcgen05_tune_next(ctypes.c_int(0), ctypes.c_int(tile_n), ctypes.c_int(halves))
    tc_check(m, n, k, epi, seed=tile_n + halves)
    assert tc_status_clear() == 0


@pytest.mark.parametrize("m,n,k", [(300, 2560, 512), (129, 1000, 200), (1500, 704, 1024)])
@pytest.mark.parametrize("epi,out_dtype", [(0, torch.bfloat16), (2, torch.float32), (2, torch.bfloat16), (0, torch.float32)])
def test_gemm_tcgen05_many_tokens_every_output_type(m, n, k, epi, out_dtype):
    """The many-row kernel's values leave as whole rows through a staging tile: every kind of
    output (stored or gated, bfloat16 or float32) with whole groups, a ragged last group and rows
    past the last token."""
    g = gen(m + n + epi)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    ref = P.linear(w.float(), a.float())
    if epi == 2:
        ref = P.swiglu(ref[:, 0::2], ref[:, 1::2])
    out = torch.full(tuple(ref.shape), float("nan"), dtype=out_dtype, device=DEV)
    assert fast().gemm_tcgen05(a.to(DEV), w.to(DEV), out, epi)
    torch.cuda.synchronize()
    assert tc_status_clear() == 0
    assert rel_err(out.float(), ref) < (1e-2 if out_dtype == torch.bfloat16 or epi == 2 else 3e-5)


def test_gemm_tcgen05_many_tokens_unaligned_output_rows():
    """An output whose rows are not 16-byte aligned takes the scalar stores and is still right."""
    m, n, k = 300, 200, 512
    a = torch.randn(m, k, generator=gen(1)).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=gen(2)) * 0.05).bfloat16().to(DEV)
    big = torch.zeros(m, 333, dtype=torch.bfloat16, device=DEV)
    out = big[:, 7:207]
    assert fast().gemm_tcgen05(a, w, out, 0)
    assert rel_err(out.float(), a.float().cpu() @ w.float().cpu().t()) < 1e-2
    assert float(big[:, :7].abs().sum()) == 0 and float(big[:, 207:].abs().sum()) == 0
