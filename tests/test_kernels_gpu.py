"""Each kernel alone against a plain float32 reference of the same operation, at sizes other than
the engine's: widths and vocabularies that are no power of two, head sizes in steps of 16, any
grouping of heads, ragged tiles, page and tile boundaries, windows."""
import math

import pytest
import torch

from helpers import rel_err
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops():
    from builderforce_inference_b200.kernels import ops as o
    return o


def gen(seed=0):
    return torch.Generator().manual_seed(seed)


def dt_tol(dt):
    return 2e-6 if dt == torch.float32 else 1.2e-2


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_embed_rows(dt):
    table = torch.randn(301, 72, generator=gen()).to(dt)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = torch.empty(5, 72, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().embed_rows(table.to(DEV), ids.to(DEV), out, status)
    assert torch.equal(out.cpu(), P.embedding(table.float(), ids.tolist()))
    assert status.item() == 0
    bad = torch.tensor([3, 301], dtype=torch.int32, device=DEV)
    ops().embed_rows(table.to(DEV), bad, out[:2], status)
    assert status.item() & ops().STATUS_BAD_TOKEN and out[1].abs().sum().item() == 0


# ------------------------------------------------------------------ RMS norm
@pytest.mark.parametrize("width", [16, 72, 1000, 2560, 5121])
@pytest.mark.parametrize("wdt,odt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.float32, torch.bfloat16)])
def test_rmsnorm(width, wdt, odt):
    x = torch.randn(7, width, generator=gen(width)) * 3.0
    w = (1 + 0.1 * torch.randn(width, generator=gen(1))).to(wdt)
    eps = 1e-5
    out = torch.empty(7, width, dtype=odt, device=DEV)
    ops().rmsnorm(x.to(DEV), w.to(DEV), eps, out)
    ref = P.rms_norm(x, w.float(), eps)
    assert rel_err(out.float(), ref) < dt_tol(odt)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, width, dtype=odt, device=DEV)
    ops().rmsnorm(x.to(DEV), w.to(DEV), eps, out2, rows)
    assert rel_err(out2.float(), ref[[6, 0, 3]]) < dt_tol(odt)


def test_rmsnorm_eps_matters_and_sits_inside_the_root():
    x = torch.full((1, 32), 1e-3)
    w = torch.ones(32)
    out = torch.empty(1, 32, dtype=torch.float32, device=DEV)
    ops().rmsnorm(x.to(DEV), w.to(DEV), 1e-2, out)
    assert abs(out[0, 0].item() - 1e-3 / math.sqrt(1e-6 + 1e-2)) < 1e-7


# ------------------------------------------------------------------ SiLU * mul
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
def test_silu_mul(dt, interleaved):
    g = torch.randn(5, 200, generator=gen(2)) * 4
    u = torch.randn(5, 200, generator=gen(3))
    g[0, 0], g[0, 1] = 60.0, -60.0                      # the overflow-safe branches
    gq, uq = g.to(dt), u.to(dt)
    gu = torch.stack([gq, uq], dim=2).reshape(5, 400) if interleaved else torch.cat([gq, uq], dim=1)
    out = torch.empty(5, 200, dtype=dt, device=DEV)
    ops().silu_mul(gu.to(DEV).contiguous(), out, interleaved)
    assert rel_err(out.float(), P.swiglu(gq.float(), uq.float())) < dt_tol(dt)


# ------------------------------------------------------------------ matrix products, CUDA cores
@pytest.mark.parametrize("m", [1, 2, 3, 5, 9, 16, 17, 70, 130])
@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16)])
def test_gemm_simt_store(m, adt, wdt):
    n, k = 137, 150
    a = torch.randn(m, k, generator=gen(m)).to(adt)
    w = (torch.randn(n, k, generator=gen(9)) * 0.1).to(wdt)
    ref = P.linear(w.float(), a.float())
    for odt in (torch.float32, torch.bfloat16):
        out = torch.empty(m, n, dtype=odt, device=DEV)
        ops().gemm_simt(a.to(DEV), w.to(DEV), out, ops().EPI_STORE)
        assert rel_err(out.float(), ref) < (2e-6 if odt == torch.float32 else 1e-2)


@pytest.mark.parametrize("m", [1, 4, 11, 65])
def test_gemm_simt_accumulates_into_the_residual_and_gates(m):
    n, k = 72, 200
    a = torch.randn(m, k, generator=gen(m))
    w = torch.randn(n, k, generator=gen(4)) * 0.1
    res = torch.randn(m, n, generator=gen(5))
    out = res.clone().to(DEV)
    ops().gemm_simt(a.to(DEV), w.to(DEV), out, ops().EPI_ACCUMULATE)
    assert rel_err(out, res + P.linear(w, a)) < 2e-6
    # gated epilogue over interleaved rows: row 2j = gate_j, row 2j+1 = up_j
    gate, up = w[:36], w[36:]
    wi = torch.stack([gate, up], dim=1).reshape(72, k)
    out2 = torch.empty(m, 36, dtype=torch.float32, device=DEV)
    ops().gemm_simt(a.to(DEV), wi.to(DEV).contiguous(), out2, ops().EPI_SWIGLU)
    assert rel_err(out2, P.swiglu(P.linear(gate, a), P.linear(up, a))) < 2e-6


def test_gemm_simt_strided_rows_and_refusals():
    from builderforce_inference_b200.kernels.library import KernelError
    big = torch.randn(9, 300, generator=gen(1)).to(DEV)
    a = big[:, 20:120]                                   # row stride 300, 100 columns
    w = torch.randn(33, 100, generator=gen(2)).to(DEV)
    out = torch.empty(9, 33, dtype=torch.float32, device=DEV)
    ops().gemm_simt(a, w, out)
    assert rel_err(out, a.cpu() @ w.cpu().t()) < 2e-6
    with pytest.raises(KernelError):
        ops().gemm_simt(a, torch.randn(33, 99, device=DEV), out)
    with pytest.raises(KernelError):
        ops().gemm_simt(a, w, torch.empty(9, 33, dtype=torch.bfloat16, device=DEV), ops().EPI_ACCUMULATE)
    with pytest.raises(KernelError):
        ops().gemm_simt(a.cpu(), w.cpu(), out.cpu())      # no CPU path


# ------------------------------------------------------------------ cache helpers for the attention kernels
class Pages:
    """A hand-made paged cache for kernel tests: ``n_slots`` sequences, pages handed out in a
    scrambled order so that a wrong page lookup cannot go unnoticed."""

    def __init__(self, n_slots, max_len, n_kv, d, dt, window=None, seed=0):
        from builderforce_inference_b200.cache import KVView
        blocks = (max_len + 63) // 64
        n_pages = n_slots * blocks + 3
        perm = torch.randperm(n_pages, generator=gen(seed)).tolist()
        self.table = torch.full((n_slots, blocks), -1, dtype=torch.int32)
        it = iter(perm)
        for s in range(n_slots):
            for b in range(blocks):
                self.table[s, b] = next(it)
        self.k = torch.full((n_pages, n_kv, 64, d), float("nan"), dtype=dt, device=DEV)
        self.v = torch.full((n_pages, n_kv, 64, d), float("nan"), dtype=dt, device=DEV)
        self.view = KVView(self.k, self.v, self.table.to(DEV), n_kv, d, window)
        self.n_kv, self.d = n_kv, d

    def write(self, slot, pos0, k, v):
        """k, v: [T, n_kv, d] placed at positions pos0.. of the slot."""
        for t in range(k.shape[0]):
            p = pos0 + t
            page = int(self.table[slot, p // 64])
            self.k[page, :, p % 64, :] = k[t].to(self.k.dtype).to(DEV)
            self.v[page, :, p % 64, :] = v[t].to(self.v.dtype).to(DEV)

    def read(self, slot, n):
        k = torch.stack([self.k[int(self.table[slot, p // 64]), :, p % 64, :] for p in range(n)])
        v = torch.stack([self.v[int(self.table[slot, p // 64]), :, p % 64, :] for p in range(n)])
        return k.float().cpu(), v.float().cpu()


def plain_paged_attention(q, k_all, v_all, start, window, scale):
    """q [T,hq,d] at positions start..; k_all, v_all [start+T, hkv, d]."""
    d = q.shape[-1]
    n = k_all.shape[0]
    qq = torch.zeros(n, q.shape[1], d)
    qq[start:] = q
    out = P.attention(qq * (scale * math.sqrt(d)), k_all, v_all, window)
    return out[start:]


def run_attention(q, pages, seqs, n_q, scale, dt):
    """seqs: list of (slot, start, T); q packed [sum T, n_q*d]."""
    cu = [0]
    for _, _, t in seqs:
        cu.append(cu[-1] + t)
    out = torch.full((cu[-1], q.shape[1]), float("nan"), dtype=dt, device=DEV)
    i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    ops().attention_paged(q.to(dt).to(DEV), q.shape[1], out, pages.view, i32(cu), i32([s for s, _, _ in seqs]),
                          i32([st for _, st, _ in seqs]), len(seqs), max(t for _, _, t in seqs), n_q, scale)
    return out.float().cpu()


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d", [(4, 2, 16), (6, 1, 48), (5, 5, 32), (8, 2, 128), (3, 3, 80), (16, 1, 64)])
def test_attention_paged_mixed_batch(dt, n_q, n_kv, d):
    """Whole prompts, a continuation of a cached prefix and single tokens in one launch, with
    lengths around tile (32) and page (64) edges."""
    seqs = [(2, 0, 33), (0, 0, 1), (3, 95, 1), (1, 31, 34), (4, 64, 1), (5, 0, 70), (6, 63, 2)]
    pages = Pages(7, 200, n_kv, d, dt, seed=d)
    g = gen(n_q * 100 + d)
    scale = 1.0 / math.sqrt(d)
    qs, refs = [], []
    for slot, start, t in seqs:
        n = start + t
        k = torch.randn(n, n_kv, d, generator=g).to(dt).float()
        v = torch.randn(n, n_kv, d, generator=g).to(dt).float()
        q = torch.randn(t, n_q, d, generator=g).to(dt).float()
        pages.write(slot, 0, k, v)
        qs.append(q.reshape(t, n_q * d))
        refs.append(plain_paged_attention(q, k, v, start, None, scale).reshape(t, n_q * d))
    got = run_attention(torch.cat(qs), pages, seqs, n_q, scale, dt)
    assert rel_err(got, torch.cat(refs)) < (3e-6 if dt == torch.float32 else 1e-2)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_among_hundreds(dt):
    """Random keys would hide a skipped tile: one key per query head is made to dominate, at
    places that exercise the first and last row of pages and tiles, and the output must be that
    key's value."""
    n_q, n_kv, d, n = 4, 2, 32, 700
    g = gen(7)
    pages = Pages(1, n, n_kv, d, dt)
    k = torch.randn(n, n_kv, d, generator=g) * 0.05
    v = torch.randn(n, n_kv, d, generator=g)
    q = torch.randn(1, n_q, d, generator=g)
    q = q / q.norm(dim=-1, keepdim=True)
    for target in (0, 31, 32, 63, 64, 65, 383, 384, 640, 698, 699):
        kk = k.clone()
        for h in range(n_kv):
            kk[target, h] = q[0, h * 2] * 40.0 * math.sqrt(d)        # score 40 for the group's first head
        pages.write(0, 0, kk, v)
        got = run_attention(q.reshape(1, -1), pages, [(0, n - 1, 1)], n_q, 1.0 / math.sqrt(d), dt)
        got = got.reshape(n_q, d)
        kq, vq = pages.read(0, n)
        ref = plain_paged_attention(q.to(dt).float(), kq, vq, n - 1, None, 1.0 / math.sqrt(d)).reshape(n_q, d)
        assert rel_err(got, ref) < (3e-6 if dt == torch.float32 else 1e-2), target
        for h in range(n_kv):
            assert (got[h * 2] - vq[target, h]).abs().max() < 0.05, (target, h)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [1, 5, 32, 40, 64, 100])
def test_attention_window_edges(dt, window):
    """The key at pos-window+1 counts, the key at pos-window does not: a dominating key is put at
    each and the output must follow."""
    n_q, n_kv, d, n = 2, 1, 16, 230
    g = gen(window)
    v = torch.randn(n, n_kv, d, generator=g)
    q = torch.randn(1, n_q, d, generator=g)
    q = q / q.norm(dim=-1, keepdim=True)
    scale = 1.0 / math.sqrt(d)
    pos = n - 1
    for target, inside in ((pos - window + 1, True), (pos - window, False)):
        if target < 0:
            continue
        pages = Pages(1, n, n_kv, d, dt, window=window)
        k = torch.randn(n, n_kv, d, generator=g) * 0.05
        k[target, 0] = q[0, 0] * 40.0 * math.sqrt(d)
        pages.write(0, 0, k, v)
        got = run_attention(q.reshape(1, -1), pages, [(0, pos, 1)], n_q, scale, dt).reshape(n_q, d)
        kq, vq = pages.read(0, n)
        ref = plain_paged_attention(q.to(dt).float(), kq, vq, pos, window, scale).reshape(n_q, d)
        assert rel_err(got, ref) < (3e-6 if dt == torch.float32 else 1e-2)
        close = (got[0] - vq[target, 0]).abs().max() < 0.05
        assert bool(close) == inside, (window, target, inside)
    # a whole prompt under the same window, every row against the plain implementation
    pages = Pages(1, n, n_kv, d, dt, window=window)
    k = torch.randn(n, n_kv, d, generator=g).to(dt).float()
    qq = torch.randn(n, n_q, d, generator=g).to(dt).float()
    pages.write(0, 0, k, v)
    got = run_attention(qq.reshape(n, -1), pages, [(0, 0, n)], n_q, scale, dt)
    _, vq = pages.read(0, n)
    assert rel_err(got, P.attention(qq, k, vq, window).reshape(n, -1)) < (3e-6 if dt == torch.float32 else 1e-2)


def test_attention_never_reads_past_a_sequence_or_a_padding_row():
    """Rows past the length are NaN in ``Pages``; a padding sequence (slot -1) leaves its output
    untouched."""
    n_q, n_kv, d = 4, 2, 16
    pages = Pages(2, 128, n_kv, d, torch.float32)
    g = gen(3)
    k, v = torch.randn(50, n_kv, d, generator=g), torch.randn(50, n_kv, d, generator=g)
    pages.write(1, 0, k, v)
    q = torch.randn(2, n_q * d, generator=g)
    got = run_attention(q, pages, [(1, 49, 1), (-1, 0, 1)], n_q, 0.25, torch.float32)
    assert torch.isfinite(got[0]).all() and torch.isnan(got[1]).all()


# ------------------------------------------------------------------ q/k norm + rotation + cache write
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d,theta", [(4, 2, 16, 1e4), (6, 3, 48, 1e6), (2, 1, 128, 5e5), (3, 3, 80, 1e4), (5, 5, 64, 1e4), (8, 2, 128, 1e6)])
def test_qk_norm_rope_cache(dt, n_q, n_kv, d, theta):
    from builderforce_inference_b200.parts.rotary import rotary_table
    g = gen(d)
    seqs = [(1, 60, 7), (0, 0, 3), (2, 127, 1)]                 # (slot, start, T): crosses a page edge
    pages = Pages(3, 200, n_kv, d, dt)
    t_all = sum(t for _, _, t in seqs)
    qkv = (torch.randn(t_all, (n_q + 2 * n_kv) * d, generator=g) * 2).to(dt)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(dt)
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(dt)
    eps = 1e-5
    pos, slot = [], []
    for s, st, t in seqs:
        pos += list(range(st, st + t))
        slot += [s] * t
    table = rotary_table(theta, d, 256, DEV)
    dev = qkv.to(DEV).clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    ops().qk_norm_rope_cache(dev, n_q, n_kv, d, qw.to(DEV), kw.to(DEV), eps, table, d, i32(pos), i32(slot),
                             pages.view, ops().FLAG_WRITE_CACHE, status)
    assert status.item() == 0
    x = qkv.float()
    q = x[:, :n_q * d].reshape(t_all, n_q, d)
    k = x[:, n_q * d:(n_q + n_kv) * d].reshape(t_all, n_kv, d)
    v = x[:, (n_q + n_kv) * d:].reshape(t_all, n_kv, d)
    q_ref = P.rope_neox(P.rms_norm(q, qw.float(), eps), pos, theta)
    k_ref = P.rope_neox(P.rms_norm(k, kw.float(), eps), pos, theta)
    tol = 3e-6 if dt == torch.float32 else 1e-2
    assert rel_err(dev[:, :n_q * d].float().reshape(t_all, n_q, d), q_ref) < tol
    # k and v in the buffer are untouched; the cache holds the transformed k and the plain v
    assert torch.equal(dev[:, n_q * d:].cpu(), qkv[:, n_q * d:])
    row = 0
    for s, st, t in seqs:
        for i in range(t):
            p = st + i
            page = int(pages.table[s, p // 64])
            assert rel_err(pages.k[page, :, p % 64, :].float(), k_ref[row]) < tol
            assert torch.equal(pages.v[page, :, p % 64, :].float().cpu(), v[row].to(dt).float())
            row += 1
    # everything else in the cache is still untouched (NaN)
    assert int(torch.isfinite(pages.k.float()).sum().item()) == t_all * n_kv * d
    # padding rows (slot -1) are skipped; a position outside the table is recorded, not read
    dev2 = qkv.to(DEV).clone()
    ops().qk_norm_rope_cache(dev2, n_q, n_kv, d, qw.to(DEV), kw.to(DEV), eps, table, d, i32(pos),
                             i32([-1] * t_all), pages.view, ops().FLAG_WRITE_CACHE, status)
    assert torch.equal(dev2.cpu(), qkv) and status.item() == 0
    ops().qk_norm_rope_cache(dev2, n_q, n_kv, d, qw.to(DEV), kw.to(DEV), eps, table, d, i32([999] * t_all),
                             i32(slot), pages.view, 0, status)
    assert status.item() & ops().STATUS_BAD_POSITION


@pytest.mark.parametrize("n_q,n_kv,d", [(5, 5, 64), (6, 3, 128), (32, 8, 128), (3, 1, 64)])
def test_qk_norm_rope_cache_many_tokens(n_q, n_kv, d):
    """Hundreds of tokens take the variant in which a warp handles several heads of a token; head
    counts that do not fill a warp's share, padding tokens in between, a token without a page."""
    from builderforce_inference_b200.parts.rotary import rotary_table
    g = gen(d + n_q)
    theta, eps, n = 1e6, 1e-6, 700
    pages = Pages(2, 1024, n_kv, d, torch.bfloat16)
    qkv = (torch.randn(n, (n_q + 2 * n_kv) * d, generator=g) * 2).bfloat16()
    qw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    kw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    pos = list(range(100, 100 + n))
    slot = [1] * n
    for i in (0, 13, 699):
        slot[i] = -1                                     # padding tokens
    table = rotary_table(theta, d, 1024, DEV)
    dev = qkv.to(DEV).clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    ops().qk_norm_rope_cache(dev, n_q, n_kv, d, qw.to(DEV), kw.to(DEV), eps, table, d, i32(pos), i32(slot),
                             pages.view, ops().FLAG_WRITE_CACHE, status)
    assert status.item() == 0
    x = qkv.float()
    q = x[:, :n_q * d].reshape(n, n_q, d)
    k = x[:, n_q * d:(n_q + n_kv) * d].reshape(n, n_kv, d)
    v = x[:, (n_q + n_kv) * d:].reshape(n, n_kv, d)
    q_ref = P.rope_neox(P.rms_norm(q, qw.float(), eps), pos, theta)
    k_ref = P.rope_neox(P.rms_norm(k, kw.float(), eps), pos, theta)
    live = [i for i in range(n) if slot[i] >= 0]
    got_q = dev[:, :n_q * d].float().cpu().reshape(n, n_q, d)
    assert rel_err(got_q[live], q_ref[live]) < 1e-2
    dead = [i for i in range(n) if slot[i] < 0]
    assert torch.equal(dev.cpu()[dead], qkv[dead])      # padding rows untouched
    assert torch.equal(dev[:, n_q * d:].cpu(), qkv[:, n_q * d:])
    k_got, v_got = pages.read(1, 100 + n)
    assert rel_err(k_got[100:][live], k_ref[live]) < 1e-2
    assert torch.equal(v_got[100:][live], v[live])
    assert int(torch.isfinite(pages.k.float()).sum().item()) == len(live) * n_kv * d
    # a live token whose page the sequence does not hold is recorded
    pages.view.block_table[1, 5] = -1
    ops().qk_norm_rope_cache(qkv.to(DEV).clone(), n_q, n_kv, d, qw.to(DEV), kw.to(DEV), eps, table, d, i32(pos), i32(slot),
                             pages.view, ops().FLAG_WRITE_CACHE, status)
    assert status.item() & ops().STATUS_NO_PAGE


def test_rotation_table_against_the_formula():
    from builderforce_inference_b200.parts.rotary import rotary_table
    t = rotary_table(1e6, 128, 4096, "cpu")
    for pos, i in ((0, 0), (1, 0), (4095, 0), (4095, 63), (777, 31)):
        ang = pos / (1e6 ** (2 * i / 128))
        assert abs(t[pos, i, 0].item() - math.cos(ang)) < 1e-7
        assert abs(t[pos, i, 1].item() - math.sin(ang)) < 1e-7


# ------------------------------------------------------------------ sampling
def test_argmax_lowest_index_wins_and_any_vocabulary():
    for vocab in (5, 301, 4096, 151936):
        x = torch.randn(3, vocab, generator=gen(vocab))
        x[0, vocab // 2] = 50.0
        x[0, vocab - 1] = 50.0
        x[1, 0] = 60.0
        x[2, :] = -float("inf")
        out = torch.empty(3, dtype=torch.int32, device=DEV)
        ops().argmax_rows(x.to(DEV), out)
        assert out.tolist() == [vocab // 2, 0, 0]
        assert out.tolist()[:2] == [P.argmax_first(r.tolist()) for r in x[:2]]
        # with scratch, many blocks search each row; same answers, ties across chunks included
        scratch = torch.empty(2 * 3 * (vocab // 8192 + 1), dtype=torch.int32, device=DEV)
        out.fill_(-1)
        ops().argmax_rows(x.to(DEV), out, scratch)
        assert out.tolist() == [vocab // 2, 0, 0]


@pytest.mark.parametrize("vocab", [37, 384, 5000])
def test_temperature_sampling_follows_the_plain_cdf(vocab):
    g = gen(vocab)
    rows = 24
    x = torch.randn(rows, vocab, generator=g) * 2
    temp = 0.8
    us = torch.rand(rows, generator=g).tolist()
    us[0], us[1] = 0.0, 0.9999999
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops().sample_rows(x.to(DEV), torch.full((rows,), temp, device=DEV), torch.tensor(us, device=DEV), out)
    for r in range(rows):
        p = torch.softmax(x[r].double() / temp, dim=0)
        cdf = torch.cumsum(p, 0)
        tok = out[r].item()
        lo = cdf[tok - 1].item() if tok > 0 else 0.0
        assert lo - 1e-5 <= us[r] <= cdf[tok].item() + 1e-5, (r, tok, us[r], lo, cdf[tok].item())
        kind, pairs = P.target(x[r].tolist(), [], P.PlainSampleParams(temperature=temp))
        plain_tok = P.draw(pairs, us[r])
        assert tok == plain_tok or abs(us[r] - lo) < 1e-5 or abs(us[r] - cdf[tok].item()) < 1e-5


def _sorted_sample(x, us, temp, probs=None, **kw):
    rows, vocab = x.shape
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    probs = torch.empty(rows * vocab, device=DEV) if probs is None else probs
    ops().sample_sorted_rows(x.to(DEV), torch.full((rows,), temp, device=DEV), torch.tensor(us, device=DEV), out, probs, **kw)
    return out.tolist()


@pytest.mark.parametrize("vocab", [37, 384, 5000])
@pytest.mark.parametrize("cuts", [dict(top_k=12), dict(top_p=0.8), dict(top_k=50, top_p=0.6), dict(top_p=0.95, min_p=0.02),
                                  dict(top_k=1), dict(top_p=0.0), dict(top_k=3, min_p=0.9)])
def test_top_k_top_p_sampling_follows_the_plain_order(vocab, cuts):
    """The kept set and the draw in the reference's order (probability descending, index ascending)
    against the plain sampler, which sorts; a uniform number may differ only on the edge of an interval."""
    g = gen(vocab + len(cuts))
    rows, temp = 24, 0.9
    x = torch.randn(rows, vocab, generator=g) * 2
    us = torch.rand(rows, generator=g).tolist()
    us[0], us[1] = 0.0, 0.9999999
    got = _sorted_sample(x, us, temp, **cuts)
    for r in range(rows):
        kind, pairs = P.target(x[r].tolist(), [], P.PlainSampleParams(temperature=temp, **cuts))
        assert kind == "weights"
        assert got[r] in [i for i, _ in pairs], (r, "a token outside the kept set")
        total = sum(w for _, w in pairs)
        cum = 0.0
        for i, w in pairs:
            lo, cum = cum, cum + w
            if i == got[r]:
                assert lo - 1e-5 * total <= us[r] * total <= cum + 1e-5 * total, (r, got[r], us[r])


def test_top_k_top_p_sampling_with_ties_penalties_and_a_large_vocabulary():
    # ties: equal logits are ordered by index, so top_k = 3 over five equal maxima keeps the first three
    vocab = 64
    x = torch.full((1, vocab), -5.0)
    for i in (40, 7, 22, 9, 63):
        x[0, i] = 3.0
    for u, want in ((0.0, 7), (0.34, 9), (0.67, 22), (0.999, 22)):
        assert _sorted_sample(x, [u], 1.0, top_k=3) == [want]
        kind, pairs = P.target(x[0].tolist(), [], P.PlainSampleParams(temperature=1.0, top_k=3))
        assert [i for i, _ in pairs] == [7, 9, 22] and P.draw(pairs, u) == want
    # top_p over the same ties: 0.5 of the mass needs three of the five (each holds a fifth, nearly)
    assert _sorted_sample(x, [0.999], 1.0, top_p=0.5) == [22]
    # penalties first: the seen maximum falls behind
    y = torch.zeros(1, vocab)
    y[0, 3], y[0, 9] = 5.0, 4.0
    seen = torch.tensor([3, 40], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 2], dtype=torch.int32, device=DEV)
    work = torch.empty(vocab, device=DEV)
    assert _sorted_sample(y, [0.0], 1.0, top_k=1, repeat_penalty=2.0, seen=seen, seen_cu=cu, work=work) == [9]
    # min_p above 1 empties the set: the reference answers with the argmax of the unpenalised logits
    assert _sorted_sample(y, [0.5], 1.0, top_k=5, min_p=1.5, repeat_penalty=2.0, seen=seen, seen_cu=cu, work=work) == [3]
    # the benchmark's vocabulary, peaked and flat rows
    g = gen(77)
    big = torch.randn(4, 151936, generator=g)
    big[0] *= 6.0
    us = [0.3, 0.77, 0.05, 0.999]
    got = _sorted_sample(big, us, 0.8, top_k=40, top_p=0.9)
    for r in range(4):
        kind, pairs = P.target(big[r].tolist(), [], P.PlainSampleParams(temperature=0.8, top_k=40, top_p=0.9))
        total = sum(w for _, w in pairs)
        cum = 0.0
        hit = False
        for i, w in pairs:
            lo, cum = cum, cum + w
            if i == got[r]:
                hit = lo - 1e-5 * total <= us[r] * total <= cum + 1e-5 * total
        assert hit, (r, got[r])
    # the same call twice: fixed-point masses make the answer independent of the order of the additions
    assert got == _sorted_sample(big, us, 0.8, top_k=40, top_p=0.9)


def test_sampling_penalties_and_min_p():
    vocab = 50
    x = torch.zeros(2, vocab)
    x[0, 3], x[0, 9] = 5.0, 4.0          # seen id 3 is pushed below id 9
    x[1, 7], x[1, 8] = 2.0, 1.9
    seen = torch.tensor([3, 40, 8], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 2, 3], dtype=torch.int32, device=DEV)
    work = torch.empty(2 * vocab, device=DEV)
    out = torch.empty(2, dtype=torch.int32, device=DEV)
    zero = torch.zeros(2, device=DEV)
    ops().sample_rows(x.to(DEV), zero, zero, out, 2.0, 0.0, 0.0, seen, cu, work)
    assert out.tolist() == [9, 7]
    ops().sample_rows(x.to(DEV), zero, zero, out, 1.0, 1.5, 0.0, seen, cu, work)
    assert out.tolist() == [9, 7]
    assert P.target(x[0].tolist(), [3, 40], P.PlainSampleParams(repeat_penalty=2.0)) == ("token", 9)
    # min_p 0.5 at temperature 1 keeps ids whose probability is at least half the best one's:
    # with u near 1 the draw must land on the last kept id, never in the tail
    y = torch.full((1, vocab), -3.0)
    y[0, 10], y[0, 30] = 2.0, 1.5
    one = torch.ones(1, device=DEV)
    for u, want in ((0.0, 10), (0.99, 30)):
        ops().sample_rows(y.to(DEV), one, torch.tensor([u], device=DEV), out[:1], 1.0, 0.0, 0.5)
        assert out[0].item() == want
        kind, pairs = P.target(y[0].tolist(), [], P.PlainSampleParams(temperature=1.0, min_p=0.5))
        assert P.draw(pairs, u) == want
