"""The bfloat16 kernels written for speed, each alone against a plain float32 reference of the
same operation on the same bfloat16 inputs."""
import math

import pytest
import torch

from helpers import rel_err
from plain import qwen3_plain as P
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
        assert fast().linear_bf16(a.to(DEV), w.to(DEV), out, 0)
        assert rel_err(out.float(), ref) < tol


@pytest.mark.parametrize("m", [1, 5, 24, 64])
def test_skinny_gemm_epilogues(m):
    n, k = 304, 2560
    a = torch.randn(m, k, generator=gen(m)).bfloat16()
    w = (torch.randn(n, k, generator=gen(3)) * 0.05).bfloat16()
    res = torch.randn(m, n, generator=gen(4))
    out = res.clone().to(DEV)
    assert fast().linear_bf16(a.to(DEV), w.to(DEV), out, 1)
    assert rel_err(out, res + P.linear(w.float(), a.float())) < 2e-5
    gate, up = w[0::2].float(), w[1::2].float()          # rows interleaved gate/up
    out2 = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert fast().linear_bf16(a.to(DEV), w.to(DEV), out2, 2)
    assert rel_err(out2.float(), P.swiglu(P.linear(gate, a.float()), P.linear(up, a.float()))) < 1e-2


def test_skinny_gemm_declines_what_it_cannot_do():
    a = torch.randn(4, 20, device=DEV).bfloat16()
    w = torch.randn(8, 20, device=DEV).bfloat16()
    out = torch.empty(4, 8, dtype=torch.float32, device=DEV)
    assert not fast().linear_bf16(a, w, out, 0)                       # K not a multiple of 8
    a = torch.randn(65, 64, device=DEV).bfloat16()
    w = torch.randn(8, 64, device=DEV).bfloat16()
    assert not fast().linear_bf16(a, w, torch.empty(65, 8, dtype=torch.float32, device=DEV), 0)   # too many rows
    # the dispatcher then takes the general kernel and the result is still right
    from builderforce_inference_b200.kernels.linear import linear
    out = torch.empty(65, 8, dtype=torch.float32, device=DEV)
    linear(a, w, out)
    assert rel_err(out, a.float().cpu() @ w.float().cpu().t()) < 2e-5


class Ctx:
    """The few fields of a step context the decode attention reads."""

    def __init__(self, slots, starts):
        from builderforce_inference_b200.engine.context import Workspace
        i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
        self.n_seqs = self.n_tokens = len(slots)
        self.max_seq_tokens = 1
        self.seq_slot, self.seq_start = i32(slots), i32(starts)
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
        if forced is not None:
            monkeypatch.setattr(fast(), "decode_splits", lambda *a, f=forced: f)
        out = torch.full((len(starts), n_q * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert fast().attention_decode_bf16(Ctx(slots, starts), q_all, out, pages.view, n_q, scale)
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
        assert fast().linear_bf16(a, w, out, 1)
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert rel_err(outs[0], res + P.linear(w.float().cpu(), a.float().cpu())) < 2e-5
    assert int(fast()._split_scratch.counters[a.device].abs().sum()) == 0
