"""The matrix product for callers that cannot allocate device memory (mhb_gemm_simt_noalloc).

Some users of the kernel library cannot call cudaMalloc when they need a product: they run while
a stream is being captured into a CUDA graph, or they have given all free device memory to a page
pool, or they are plug-ins that are handed device pointers and may not own memory.  For them the
split-K scratch lives in a fixed 8 MiB array inside the library.  This test calls the entry
point through its exported C symbol (ctypes, raw device pointers), twice in a row, and compares
with the existing entry point (mhb_gemm_simt, one pass, no scratch) at the tolerance the other
product tests use.  The second call is smaller than the first, so the array still holds the
first call's partial sums where the second call does not write: a product that read stale
scratch would show.  Collected last, so a run that stops at the first failure has already run
everything else.
"""
import ctypes
import math
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_FLOATS = 2 * 1024 * 1024


def lib():
    from mini_hisparse_b200.kernels import build

    handle = build.load("gemm_simt")
    handle.mhb_gemm_simt_noalloc.restype = c_int
    return handle


def existing(handle, a, w, out):
    rc = handle.mhb_gemm_simt(
        c_void_p(a.data_ptr()), c_int(0 if a.dtype == torch.float32 else 1), c_void_p(w.data_ptr()),
        c_int(0 if w.dtype == torch.float32 else 1), c_void_p(out.data_ptr()), c_int(0), c_void_p(0),
        c_int(a.shape[0]), c_int(w.shape[0]), c_int(a.shape[1]), c_longlong(a.stride(0)),
        c_longlong(w.stride(0)), c_longlong(out.stride(0)), c_int(1), c_longlong(0),
        c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, handle.mhb_last_error().decode()


def no_alloc(handle, a, w, out, nsplit):
    return handle.mhb_gemm_simt_noalloc(
        c_void_p(a.data_ptr()), c_int(0 if a.dtype == torch.float32 else 1), c_void_p(w.data_ptr()),
        c_int(0 if w.dtype == torch.float32 else 1), c_void_p(out.data_ptr()), c_int(a.shape[0]),
        c_int(w.shape[0]), c_int(a.shape[1]), c_longlong(a.stride(0)), c_longlong(w.stride(0)),
        c_longlong(out.stride(0)), c_int(nsplit), c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_product_matches_existing_entry_point_twice():
    handle = lib()
    g = torch.Generator().manual_seed(5)
    # the last two: more splits than K has elements (the empty ones must add zeros), and one split
    cases = [((130, 333, 1000), torch.float32, 7), ((9, 77, 520), torch.bfloat16, 4), ((5, 40, 16), torch.float32, 20),
             ((33, 20, 100), torch.float32, 1)]
    for (M, N, K), dtype, nsplit in cases:            # two calls in a row, the second one smaller
        a = torch.randn(M, K, generator=g).to(dtype).to(DEV)
        w = torch.randn(N, K, generator=g).to(dtype).to(DEV)
        want = torch.empty(M, N, device=DEV)
        got = torch.full((M, N + 3), float("nan"), device=DEV)        # a row stride that is not N
        existing(handle, a, w, want)
        before = torch.cuda.memory_allocated()
        rc = no_alloc(handle, a, w, got, nsplit)
        assert rc == 0, handle.mhb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before               # nothing came from torch's allocator
        torch.testing.assert_close(got[:, :N], want, atol=2e-5 * math.sqrt(K), rtol=2e-5)
        torch.testing.assert_close(want, a.float() @ w.float().T, atol=2e-5 * math.sqrt(K), rtol=2e-5)
        assert bool(got[:, N:].isnan().all())                          # nothing outside the output


def test_no_alloc_product_refuses_what_does_not_fit():
    handle = lib()
    M, N, K, nsplit = 1024, 1024, 64, 3                               # 3 Mi floats > 2 Mi
    a = torch.zeros(M, K, device=DEV)
    w = torch.zeros(N, K, device=DEV)
    out = torch.full((M, N), 7.0, device=DEV)
    rc = no_alloc(handle, a, w, out, nsplit)
    assert rc != 0
    msg = handle.mhb_last_error().decode()
    assert "scratch" in msg and str(SCRATCH_FLOATS) in msg
    torch.cuda.synchronize()
    assert float(out.min()) == 7.0                                    # nothing was launched
    small = torch.zeros(4, 8, device=DEV)
    assert no_alloc(handle, small, small, out, 70000) != 0 and "65535" in handle.mhb_last_error().decode()
    narrow = torch.full((4, 2), 7.0, device=DEV)                      # a row stride of 2 for 4 columns
    assert no_alloc(handle, small, small, narrow, 1) != 0 and "row stride" in handle.mhb_last_error().decode()
    torch.cuda.synchronize()
    assert float(narrow.min()) == 7.0
