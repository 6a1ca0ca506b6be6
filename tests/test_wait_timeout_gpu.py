"""A bounded wait that runs out.  Every wait on an mbarrier in the tcgen05 kernels gives up after
a number of polls, records a time-out in the status word, lets copies in flight land, frees the
block's tensor memory and returns; the host turns the status into an error.  Here the wait is made
to run out in the only harmless way: the probe entry points launch the same kernels with a limit
of a few thousand polls and a producer that issues nothing, so the consumers wait for data that
never comes and give up within milliseconds.  Nothing faults, traps or spins without a bound.
The reference's counterpart is its health check of a device path that went dead
(crates/bfi-core/src/resident/health.rs:26-168)."""
import math
import time

import pytest
import torch

from helpers import CONFIGS, model_folder, plain_logits, random_prompts, rel_err, tol
from test_fast_kernels_gpu import PrefillCtx, fast, tc_check, tc_status_clear
from test_kernels_gpu import DEV, Pages, gen, plain_paged_attention

pytestmark = pytest.mark.gpu
TIMEOUT_BIT = 8
POLLS = 2000


def timed(fn):
    from builderforce_inference_b200.kernels.library import library
    library("fast")                                   # built and loaded before the clock starts
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    assert fn()
    torch.cuda.synchronize()
    return time.perf_counter() - t0


@pytest.mark.parametrize("m,n,k", [(8, 128, 256), (16, 640, 2560), (200, 300, 512)])
def test_matrix_product_wait_runs_out_and_the_next_launch_is_right(m, n, k):
    """One block with 8 rows (the kernel the decode step runs), a clustered split-K grid, and the
    persistent many-row kernel."""
    assert tc_status_clear() == 0
    a = torch.randn(m, k, generator=gen(1)).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=gen(2)) * 0.05).bfloat16().to(DEV)
    out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    took = timed(lambda: fast().gemm_tcgen05_wait_probe(a, w, out, 0, POLLS, True))
    assert took < 2.0, f"the launch took {took:.2f} s to give up"
    assert tc_status_clear() & TIMEOUT_BIT
    # a short limit alone (producer at work) must not trip anything when the data does arrive:
    # with 65536 polls per wait this product still completes
    assert fast().gemm_tcgen05_wait_probe(a, w, out, 0, 65536, False)
    torch.cuda.synchronize()
    assert tc_status_clear() == 0
    assert rel_err(out, a.float().cpu() @ w.float().cpu().t()) < 3e-5
    # the ordinary entry point afterwards: tensor memory was freed and the barriers start afresh
    for _ in range(3):
        tc_check(m, n, k, 1, seed=5)
    assert tc_status_clear() == 0


@pytest.mark.parametrize("d", [64, 128])
def test_prompt_attention_wait_runs_out_and_the_next_launch_is_right(d):
    n_q, n_kv, n = 4, 2, 300
    assert tc_status_clear() == 0
    g = gen(d)
    scale = 1.0 / math.sqrt(d)
    k = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
    v = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
    q = torch.randn(n, n_q, d, generator=g).bfloat16().float()
    pages = Pages(1, n, n_kv, d, torch.bfloat16, seed=3)
    pages.write(0, 0, k, v)
    ctx = PrefillCtx([(0, 0, n)])
    q_dev = q.reshape(n, n_q * d).bfloat16().to(DEV)
    out = torch.full((n, n_q * d), 7.0, dtype=torch.bfloat16, device=DEV)
    took = timed(lambda: fast().attention_prefill_tcgen05_wait_probe(ctx, q_dev, out, pages.view, n_q, scale, POLLS, True))
    assert took < 2.0, f"the launch took {took:.2f} s to give up"
    assert tc_status_clear() & TIMEOUT_BIT            # and the ticket counters are back at zero
    assert float(out.float().min()) == 7.0 and float(out.float().max()) == 7.0      # nothing was written
    ref = plain_paged_attention(q, k, v, 0, None, scale).reshape(n, n_q * d)
    for _ in range(2):
        assert fast().attention_prefill_tcgen05_bf16(ctx, q_dev, out, pages.view, n_q, scale)
        torch.cuda.synchronize()
        assert tc_status_clear() == 0
        assert rel_err(out.float().cpu(), ref) < 1e-2


@pytest.mark.parametrize("d,forced", [(64, 1), (128, 1), (128, 4)])
def test_decode_attention_wait_runs_out_and_the_next_launch_is_right(d, forced, monkeypatch):
    """The pages of the decode attention come by TMA onto an mbarrier per stage: with a thread that
    asks for no page every block's first wait runs out."""
    from test_fast_kernels_gpu import Ctx
    n_q, n_kv = 8, 2
    starts = [5, 130, 700]
    assert tc_status_clear() == 0
    g = gen(d + forced)
    scale = 1.0 / math.sqrt(d)
    pages = Pages(len(starts), 768, n_kv, d, torch.bfloat16, seed=4)
    qs, refs = [], []
    for slot, start in enumerate(starts):
        n = start + 1
        k = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        v = torch.randn(n, n_kv, d, generator=g).bfloat16().float()
        q = torch.randn(1, n_q, d, generator=g).bfloat16().float()
        pages.write(slot, 0, k, v)
        qs.append(q.reshape(1, n_q * d))
        refs.append(plain_paged_attention(q, k, v, start, None, scale).reshape(1, n_q * d))
    q_all, ref = torch.cat(qs).bfloat16().to(DEV), torch.cat(refs)
    monkeypatch.setattr(fast(), "decode_splits", lambda *a: forced)
    ctx = Ctx(list(range(len(starts))), starts)
    out = torch.full((len(starts), n_q * d), 7.0, dtype=torch.bfloat16, device=DEV)
    took = timed(lambda: fast().attention_decode_wait_probe(ctx, q_all, out, pages.view, n_q, scale, POLLS, True))
    assert took < 2.0, f"the launch took {took:.2f} s to give up"
    assert tc_status_clear() & TIMEOUT_BIT
    if forced == 1:                                   # no second kernel: nothing was written
        assert float(out.float().min()) == 7.0 and float(out.float().max()) == 7.0
    # a short limit alone, with the pages asked for, trips nothing
    assert fast().attention_decode_wait_probe(ctx, q_all, out, pages.view, n_q, scale, 65536, False)
    torch.cuda.synchronize()
    assert tc_status_clear() == 0
    assert rel_err(out.float().cpu(), ref) < 1e-2
    for _ in range(2):
        out.fill_(7.0)
        assert fast().attention_decode_bf16(ctx, q_all, out, pages.view, n_q, scale)
        torch.cuda.synchronize()
        assert tc_status_clear() == 0
        assert rel_err(out.float().cpu(), ref) < 1e-2


def test_the_engine_reports_a_timed_out_wait_and_goes_on():
    """The status word the probes set is the one ``Engine.check_status`` reads: the step that
    follows a time-out raises ``StepError``, the word is cleared, and later steps are right."""
    from builderforce_inference_b200.engine.engine import Engine, SequenceStep, StepError
    name, dtype = "F", "bfloat16"
    folder = model_folder(name, torch.bfloat16)
    eng = Engine.load(folder, dtype=dtype, max_tokens=1024)
    p = random_prompts(CONFIGS[name]["vocab_size"], [200], seed=2)[0]
    ref = plain_logits(folder, p)
    s = eng.acquire()
    got = eng.step([SequenceStep(s, p[:150], list(range(150)))]).cpu()
    assert rel_err(got, ref[:150]) < tol(dtype)
    a = torch.randn(8, 256, generator=gen(1)).bfloat16().to(DEV)
    w = torch.randn(128, 256, generator=gen(2)).bfloat16().to(DEV)
    out = torch.zeros(8, 128, dtype=torch.float32, device=DEV)
    assert fast().gemm_tcgen05_wait_probe(a, w, out, 0, POLLS, True)
    with pytest.raises(StepError, match="bounded wait"):
        eng.step([SequenceStep(s, [p[150]], [0])])
    # the step itself ran (the time-out was the probe's); the sequence goes on from there
    assert eng.length(s) == 151
    rows = [eng.step([SequenceStep(s, [t], [0])]).cpu().clone() for t in p[151:160]]
    assert rel_err(torch.cat(rows), ref[151:160]) < tol(dtype)
    got = eng.step([SequenceStep(s, p[160:], list(range(40)))]).cpu()
    assert rel_err(got, ref[160:]) < tol(dtype)
