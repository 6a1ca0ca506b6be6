"""The matrix product for callers that may not allocate device memory.

Some hosts of this library cannot give a kernel a scratch buffer: they handed every byte of device
memory to their own arena at start-up, or they run inside another runtime's callback where the
CUDA allocator must not be called, or they work to a fixed memory plan.  For them the library
exports ``bfi_skinny_gemm_bf16_static``, whose scratch (partial sums and counters of the split over
K) is a 4 MiB array inside the library itself.  This test calls that function through its exported
C symbol, twice in a row on the same array, and checks it against the ordinary entry point, which
takes its scratch from the caller.  It lives in a file of its own that pytest collects last.
"""
import ctypes
from ctypes import c_int, c_long, c_void_p

import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lib():
    from builderforce_inference_b200.kernels.library import library
    lib = library("fast").lib
    lib.bfi_skinny_gemm_bf16_static.restype = c_int
    lib.bfi_last_error.restype = ctypes.c_char_p
    return lib


def _static(lib, a, w, out, epilogue):
    code = {torch.float32: 0, torch.bfloat16: 1}[out.dtype]
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.bfi_skinny_gemm_bf16_static(
        c_void_p(a.data_ptr()), c_long(a.stride(0)), c_void_p(w.data_ptr()), c_long(w.stride(0)),
        c_void_p(out.data_ptr()), c_int(code), c_long(out.stride(0)), c_int(a.shape[0]), c_int(w.shape[0]),
        c_int(a.shape[1]), c_int(epilogue), stream)


@pytest.mark.parametrize("m", [1, 8, 40])
def test_static_scratch_matches_the_ordinary_entry_point_twice_in_a_row(m):
    from builderforce_inference_b200.kernels import fast_ops
    lib = _lib()
    g = torch.Generator().manual_seed(m)
    n, k = 2560, 4096                                     # few row tiles, long K: the plan splits K
    assert fast_ops._skinny_scratch_need(m, n, k)[0] > 0
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16().to(DEV)
    for call in range(2):                                 # the second call finds the first one's leftovers
        a = torch.randn(m, k, generator=g).bfloat16().to(DEV)
        res = torch.randn(m, n, generator=g).to(DEV)
        want = res.clone()
        assert fast_ops.skinny_gemm(a, w, want, 1)
        got = res.clone()
        assert _static(lib, a, w, got, 1) == 0, lib.bfi_last_error()
        torch.cuda.synchronize()
        assert rel_err(got, want) < 2e-5, call
        assert rel_err(got, res.cpu() + a.float().cpu() @ w.float().cpu().t()) < 2e-5
    # a shape that does not split needs no scratch and runs as well
    w2 = (torch.randn(6144, 512, generator=g) * 0.05).bfloat16().to(DEV)
    a2 = torch.randn(m, 512, generator=g).bfloat16().to(DEV)
    want = torch.empty(m, 6144, dtype=torch.bfloat16, device=DEV)
    got = torch.empty_like(want)
    assert fast_ops.skinny_gemm(a2, w2, want, 0)
    assert _static(lib, a2, w2, got, 0) == 0
    torch.cuda.synchronize()
    assert rel_err(got.float(), want.float()) < 1e-2


def test_static_scratch_refuses_what_it_cannot_hold():
    from builderforce_inference_b200.kernels import fast_ops
    lib = _lib()
    m, n, k = 64, 4784, 8192
    a = torch.zeros(m, k, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(n, k, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    assert _static(lib, a[:, :20], w[:, :20], out, 0) == 2          # K not a multiple of 8: declined
    # the library's own plans stay within the array; a plan forced to split K six ways over 299
    # tiles of 64 rows does not, and is refused before anything is launched
    out.fill_(7.0)
    lib.bfi_skinny_tune_next(c_int(0), c_int(0), c_int(6))          # holds for the next call only
    assert _static(lib, a, w, out, 0) == 1
    assert b"needs" in lib.bfi_last_error()
    torch.cuda.synchronize()
    assert float(out.min()) == 7.0 and float(out.max()) == 7.0
    # a wrong argument is refused before anything is put on the stream as well
    assert _static(lib, a, w, out, 7) == 1 and b"epilogue" in lib.bfi_last_error()
    # the override is gone: the same shape now runs with the library's own plan
    assert _static(lib, a, w, out, 0) == 0
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0


def test_static_scratch_entry_point_allocates_nothing():
    """Device memory in use, as the driver counts it, is the same before and after a call (the
    first call on a device has already looked the array's address up and loaded the kernels)."""
    from builderforce_inference_b200.kernels import fast_ops
    lib = _lib()
    m, n, k = 8, 2560, 4096
    assert fast_ops._skinny_scratch_need(m, n, k)[0] > 0
    a = torch.randn(m, k).bfloat16().to(DEV)
    w = torch.randn(n, k).bfloat16().to(DEV)
    out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    assert _static(lib, a, w, out, 1) == 0
    torch.cuda.synchronize()

    def free_bytes():
        return torch.cuda.mem_get_info()[0]             # cudaMemGetInfo: what the driver has left

    before, torch_before = free_bytes(), torch.cuda.memory_allocated()
    for _ in range(3):
        assert _static(lib, a, w, out, 1) == 0
    torch.cuda.synchronize()
    assert free_bytes() == before and torch.cuda.memory_allocated() == torch_before
