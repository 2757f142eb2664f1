"""GPU test of myea_b200_gemm_nt_static, the contraction entry point for hosts that cannot allocate device memory in
the call path (the operand-panel scratch is a fixed array inside the library image instead of cudaMalloc'ed memory).

The file name sorts last on purpose: if this test fails, a run that stops at the first failure has already run
everything else.  The result must equal the handle-free reference entry point myea_b200_gemm_nt (same kernels, scratch
from cudaMalloc) within the tolerance of the other GEMM tests, on two calls in a row with different shapes and data
(the shared array keeps the first call's panels; the second call must not see them), then the size limit is checked.
Device buffers for A, B, C are the caller's: here they come from torch."""
import ctypes as C

import numpy as np
import pytest

from myea_b200 import capi

pytestmark = pytest.mark.gpu
TOL = 2e-5


def _both(lib, torch, M, N, K, accumulate, seed):
    rng = np.random.default_rng(seed)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((N, K)).astype(np.float32)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    want = C0.copy()
    ms = C.c_float(0)
    assert lib.myea_b200_gemm_nt(0, 0, M, N, K, A.ctypes.data, B.ctypes.data, want.ctypes.data, accumulate, C.byref(ms), 0) == 0
    dA, dB, dC = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), torch.from_numpy(C0).cuda()
    torch.cuda.synchronize()
    msg = C.create_string_buffer(256)
    rc = lib.myea_b200_gemm_nt_static(0, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), accumulate, None, msg, 256)
    assert rc == 0, msg.value
    got = dC.cpu().numpy()
    exact = A.astype(np.float64) @ B.astype(np.float64).T + (C0 if accumulate else 0)
    scale = np.abs(exact).max()
    assert np.abs(got - want).max() / scale < TOL          # against the existing entry point
    assert np.abs(got - exact).max() / scale < TOL         # and against float64


def test_static_scratch_matches_allocating_entry_point_twice():
    torch = pytest.importorskip("torch")
    lib = capi.load()
    _both(lib, torch, 300, 520, 1000, accumulate=0, seed=1)   # fills most of a panel region, ragged in every dimension
    _both(lib, torch, 129, 70, 45, accumulate=1, seed=2)      # smaller second call over the first call's leftovers


def test_static_scratch_reaches_the_wide_kernel_and_allocates_nothing():
    """a shape that takes the 256 x 256 persistent kernel yet fits the fixed array (about 4.7 M of 8 Mi floats); this entry
    point has no partial-sum workspace, so that kernel computes whole tiles only.  A second, warm call must leave the
    device's free memory exactly where it was."""
    torch = pytest.importorskip("torch")
    lib = capi.load()
    M, N, K = 512, 640, 2048
    _both(lib, torch, M, N, K, accumulate=0, seed=3)
    rng = np.random.default_rng(4)
    dA = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda()
    dB = torch.from_numpy(rng.standard_normal((N, K)).astype(np.float32)).cuda()
    dC = torch.zeros((M, N), device="cuda")
    msg = C.create_string_buffer(256)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert lib.myea_b200_gemm_nt_static(0, M, N, K, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 0, None, msg, 256) == 0, msg.value
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.cuda.current_device() == 0


def test_static_scratch_refuses_oversized_problems():
    torch = pytest.importorskip("torch")
    lib = capi.load()
    x = torch.zeros(16, device="cuda")
    msg = C.create_string_buffer(256)
    rc = lib.myea_b200_gemm_nt_static(0, 4096, 4096, 4096, x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, None, msg, 256)
    assert rc == -1 and b"too large" in msg.value
    assert lib.myea_b200_gemm_nt_static(0, 4, 4, 0, x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, None, msg, 256) == -1
