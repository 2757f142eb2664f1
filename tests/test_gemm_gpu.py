"""GPU tests of the dense contraction alone (myea_b200_gemm_nt): split-precision tcgen05 against a float64 product.
Shapes cover single tiles, ragged edges in all three dimensions (TMA zero fill, guarded epilogue), K tails that are
not a multiple of the 32-float stage, accumulate mode, long K, and the FP32 FMA engine."""
import ctypes as C

import numpy as np
import pytest

from myea_b200 import capi

pytestmark = pytest.mark.gpu


TILE_SINGLE, TILE_PAIR, TILE_WIDE, TILE_WIDE_WHOLE = 128 << 8, 2 << 8, 3 << 8, 4 << 8   # forced tile shapes (engine bits 8..16)
A_TRANSPOSED, B_TRANSPOSED = 1 << 17, 1 << 18                                            # operand handed over as [K][rows]


def _gemm(M, N, K, engine=0, accumulate=0, seed=0, positive=False, return_out=False):
    lib = capi.load()
    rng = np.random.default_rng(seed)
    gen = (lambda s: rng.uniform(0, 1, s)) if positive else rng.standard_normal
    A, B = gen((M, K)).astype(np.float32), gen((N, K)).astype(np.float32)
    C0 = rng.standard_normal((M, N)).astype(np.float32) if accumulate else np.zeros((M, N), np.float32)
    out = C0.copy()
    ms = C.c_float(0)
    Ain = np.ascontiguousarray(A.T) if engine & A_TRANSPOSED else A
    Bin = np.ascontiguousarray(B.T) if engine & B_TRANSPOSED else B
    rc = lib.myea_b200_gemm_nt(0, engine, M, N, K, Ain.ctypes.data, Bin.ctypes.data, out.ctypes.data, accumulate, C.byref(ms), 0)
    assert rc == 0
    want = A.astype(np.float64) @ B.astype(np.float64).T + (C0 if accumulate else 0)
    err = float(np.abs(out - want).max() / np.abs(want).max())
    return (err, out) if return_out else err


@pytest.mark.parametrize("shape", [(128, 128, 32), (128, 256, 64), (1, 1, 1), (5, 3, 7), (100, 10, 256), (129, 130, 33),
                                   (300, 520, 100), (256, 64, 128), (512, 512, 512), (127, 1000, 2048)])
def test_tcgen05_matches_float64(shape):
    assert _gemm(*shape) < 2e-5


@pytest.mark.parametrize("shape", [(64, 64, 16), (5, 3, 7), (300, 520, 100)])
def test_fma_engine_matches_float64(shape):
    assert _gemm(*shape, engine=1) < 2e-5


def test_accumulate_into_c():
    assert _gemm(256, 384, 512, accumulate=1) < 2e-5


def test_long_k_stays_accurate():
    # the multi-accumulator layout keeps a 16384-long sum within 3e-5 even for all-positive data (worst case for the
    # tensor core's truncating accumulate); zero-mean data is an order of magnitude better
    assert _gemm(256, 256, 16384) < 3e-5
    assert _gemm(256, 256, 16384, positive=True) < 1e-4


def test_forced_256_wide_tile():
    assert _gemm(256, 512, 1024, engine=(256 << 8)) < 5e-5


@pytest.mark.parametrize("tile", [TILE_SINGLE, TILE_PAIR, TILE_WIDE, TILE_WIDE_WHOLE])
@pytest.mark.parametrize("shape", [(256, 256, 64), (300, 520, 100), (1000, 777, 333), (129, 130, 33)])
def test_every_tile_shape(tile, shape):
    assert _gemm(*shape, engine=tile) < 2e-5


@pytest.mark.parametrize("shape", [(300, 520, 4096), (1024, 512, 2048), (2048, 1024, 1024), (640, 896, 8200), (2048, 2048, 8192)])
def test_tiles_split_along_k_are_exact_and_repeatable(shape):
    """fewer tiles than SM pairs: the 256 x 256 kernel cuts the K chunks of the tiles into equal runs (stream-K); the
    partial sums are added in a fixed order, so two runs agree bit for bit"""
    e1, o1 = _gemm(*shape, engine=TILE_WIDE, return_out=True)
    e2, o2 = _gemm(*shape, engine=TILE_WIDE, return_out=True)
    e3 = _gemm(*shape, engine=TILE_WIDE_WHOLE)
    assert e1 < 2e-5 and e3 < 2e-5
    assert np.array_equal(o1, o2)
    assert _gemm(*shape, engine=TILE_WIDE, accumulate=1) < 2e-5


@pytest.mark.parametrize("flags", [A_TRANSPOSED, B_TRANSPOSED, A_TRANSPOSED | B_TRANSPOSED])
@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 1000), (1000, 3000, 777), (130, 129, 136)])
def test_operands_read_through_their_columns(flags, shape):
    """MN-major operands of the 256 x 256 kernel: the source is [K][rows] and is not transposed on the way"""
    assert _gemm(*shape, engine=TILE_WIDE | flags) < 2e-5
    assert _gemm(*shape, engine=1 | TILE_WIDE | flags) < 2e-5   # the FP32 FMA engine on the same panels


@pytest.mark.parametrize("tile", [TILE_SINGLE, TILE_PAIR, TILE_WIDE])
@pytest.mark.parametrize("shape", [(256, 256, 64), (300, 520, 100), (1024, 512, 2048)])
def test_fused_activation_derivative_epilogue(tile, shape):
    """bit 19: C = (A B^T) .* relu'(C_in) - the epilogue of the error-propagation product, staged through shared memory"""
    M, N, K = shape
    lib = capi.load()
    rng = np.random.default_rng(5)
    A, B = rng.standard_normal((M, K)).astype(np.float32), rng.standard_normal((N, K)).astype(np.float32)
    pre = rng.standard_normal((M, N)).astype(np.float32)
    out = pre.copy()
    rc = lib.myea_b200_gemm_nt(0, tile | (1 << 19), M, N, K, A.ctypes.data, B.ctypes.data, out.ctypes.data, 0, None, 0)
    assert rc == 0
    want = (A.astype(np.float64) @ B.astype(np.float64).T) * (pre >= 0)
    assert float(np.abs(out - want).max() / np.abs(want).max()) < 2e-5


def test_invalid_arguments():
    lib = capi.load()
    assert lib.myea_b200_gemm_nt(0, 0, 0, 4, 4, None, None, None, 0, None, 0) == -1
