"""Self-check and timing of the dense contraction through the C ABI (myea_b200_gemm_nt).

    python -m myea_b200.gemm_check M N K [--repeats R] [--engine 0|1] [--bn 128|256]

Prints the maximum error against a float64 product (relative to the largest output) and, with --repeats, the mean
device time of one contraction including its two operand-split kernels.  Host buffers in, host buffers out."""
import argparse
import ctypes as C

import numpy as np

from . import capi


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("M", type=int)
    ap.add_argument("N", type=int)
    ap.add_argument("K", type=int)
    ap.add_argument("--repeats", type=int, default=0)
    ap.add_argument("--engine", type=int, default=0)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    lib = capi.load()
    rng = np.random.default_rng(a.seed)
    A = rng.standard_normal((a.M, a.K), dtype=np.float32)
    B = rng.standard_normal((a.N, a.K), dtype=np.float32)
    out = np.zeros((a.M, a.N), np.float32)
    ms = C.c_float(0)
    rc = lib.myea_b200_gemm_nt(0, a.engine | (a.bn << 8), a.M, a.N, a.K, A.ctypes.data, B.ctypes.data, out.ctypes.data, 0, C.byref(ms), a.repeats)
    if rc != 0:
        raise SystemExit("myea_b200_gemm_nt failed with status %d" % rc)
    if a.M * a.N * a.K <= 2 ** 34:
        want = A.astype(np.float64) @ B.astype(np.float64).T
        print("max error / max |C| = %.3e" % (np.abs(out - want).max() / np.abs(want).max()))
    if a.repeats > 0:
        print("%.4f ms per contraction, %.1f TFLOP/s (2*M*N*K)" % (ms.value, 2.0 * a.M * a.N * a.K / (ms.value * 1e-3) / 1e12))


if __name__ == "__main__":
    main()
