"""GPU tests at the benchmark configurations' FULL sizes.  The reference would need minutes to hours per step there, so
these check size-independent properties of one training step instead of comparing with it: identities between tensors
the library returns (loss = sum of squared output errors; the weight derivative of a layer = error^T x input, recomputed
in float64 from the downloaded errors and activations; bias derivative = column sums; the Adam update formula),
linearity of the contraction, and equivariance of a recurrent network under a permutation of the batch."""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err
from myea_b200 import capi, workloads
from myea_b200.net import Net

pytestmark = pytest.mark.gpu
TOL = 1e-4


def test_c2_full_size_step_identities():
    wl = workloads.c2_wide_mlp()                       # 8 x 4096 + BN + ReLU + dropout -> 1024, batch 4096
    gpu = Net(wl.desc, wl.opt)
    X, Y = wl.batch()
    wl.materialize(gpu)
    p0 = gpu.get(capi.BUF_PARAMETERS)
    gpu.reset_loss(); gpu.forward(X); gpu.compute_error(Y); gpu.backward(); gpu.update_derivative_weight()
    n_layers = len(wl.layers)
    out = gpu.outputs(n_layers - 1)[0].astype(np.float64)            # [4096, 1024], linear output
    delta = out - Y[0].astype(np.float64)
    s, cnt, _ = gpu.loss()
    assert cnt == delta.size
    assert abs(s - (delta * delta).sum()) <= 1e-5 * s
    assert rel_err(gpu.errors(n_layers - 1)[0], delta) < 1e-6
    g = gpu.get(capi.BUF_DERIVATIVES)
    li = gpu.layer_index(n_layers - 1)
    a_prev = gpu.outputs(n_layers - 2)[0].astype(np.float64)         # [4096, 4096], after ReLU and dropout
    dW = g[li.first_connection_index:li.last_connection_index].reshape(wl.n_out, -1)
    assert rel_err(dW, delta.T @ a_prev) < TOL
    db = g[li.first_bias_connection_index:li.last_bias_connection_index]
    assert rel_err(db, delta.sum(axis=0)) < TOL
    # a hidden layer: 512 of its 4096 neurons (the error w.r.t. the summation, i.e. behind the normalization backward)
    l = n_layers - 2
    lh = gpu.layer_index(l)
    d_h = gpu.errors(l)[0][:, :512].astype(np.float64)
    a_h = gpu.outputs(l - 1)[0].astype(np.float64)
    dW_h = g[lh.first_connection_index:lh.last_connection_index].reshape(4096, 4096)[:512]
    assert rel_err(dW_h, d_h.T @ a_h) < TOL
    # half of the dropout mask is zero, and the kept activations are non-negative (ReLU): a_prev has >= 50 % zeros
    assert (a_prev == 0).mean() > 0.5 and a_prev.min() >= 0
    # Adam, first step: w -= lr_t * m / (sqrt(v) + eps) with m = (1 - b1) g, v = (1 - b2) g^2
    gpu.update_parameter()
    p1 = gpu.get(capi.BUF_PARAMETERS)
    o = wl.opt
    sl = slice(li.first_connection_index, li.first_connection_index + (1 << 20))
    gg = g[sl].astype(np.float32)
    m, v = np.float32(1 - o.adam_beta1) * gg, np.float32(1 - o.adam_beta2) * gg * gg
    lr_t = np.float32(o.adam_learning_rate) * np.sqrt(np.float32(1 - o.adam_beta2)) / np.float32(1 - o.adam_beta1)
    want = p0[sl] - lr_t * m / (np.sqrt(v) + np.float32(o.adam_epsilon))
    assert rel_err(p1[sl], want) < 1e-6
    assert np.all(gpu.get(capi.BUF_DERIVATIVES)[sl] == 0)            # the update zeroes the derivatives
    gpu.close()


def test_contraction_is_linear_and_exact_at_4096_cubed():
    lib = capi.load()
    M = N = K = 4096
    rng = np.random.default_rng(0)
    A = rng.standard_normal((M, K), dtype=np.float32)
    B1, B2 = rng.standard_normal((N, K), dtype=np.float32), rng.standard_normal((N, K), dtype=np.float32)

    def gemm(B):
        out = np.zeros((M, N), np.float32)
        assert lib.myea_b200_gemm_nt(0, 0, M, N, K, A.ctypes.data, B.ctypes.data, out.ctypes.data, 0, None, 0) == 0
        return out

    c1, c2, c12 = gemm(B1), gemm(B2), gemm(B1 + B2)
    assert rel_err(c12, c1.astype(np.float64) + c2) < 1e-5
    rows = slice(1000, 1128)
    want = A[rows].astype(np.float64) @ B1.astype(np.float64).T
    assert rel_err(c1[rows], want) < 1e-5
    # two runs agree bit for bit (the split tiles are summed in a fixed order)
    assert np.array_equal(c1, gemm(B1))


def test_c3_full_size_forward_is_equivariant_under_batch_permutation():
    wl = workloads.c3_lstm()                          # 2 x LSTM(1024), T = 64, batch 256
    gpu = Net(wl.desc, wl.opt)
    X, Y = wl.batch()
    wl.materialize(gpu)
    last = len(wl.layers) - 1
    gpu.forward(X)
    out = gpu.outputs(last).copy()
    assert np.isfinite(out).all() and np.abs(out).max() > 0
    perm = np.random.default_rng(4).permutation(wl.B)
    gpu.forward(np.ascontiguousarray(X[:, perm]))
    assert rel_err(gpu.outputs(last), out[:, perm]) < 1e-6
    # one full step at this size: loss identity and the output layer's weight derivative from the downloaded tensors
    gpu.reset_loss(); gpu.forward(X); gpu.compute_error(Y); gpu.backward(); gpu.update_derivative_weight()
    T = wl.T
    delta = out[T - 1].astype(np.float64) - Y[T - 1]                 # only the last time step is scored (time delays = T - 1)
    s, cnt, _ = gpu.loss()
    assert cnt == delta.size and abs(s - (delta * delta).sum()) <= 1e-5 * s
    li = gpu.layer_index(last)
    g = gpu.get(capi.BUF_DERIVATIVES)
    h2 = gpu.outputs(last - 1)[T - 1].astype(np.float64)             # second LSTM layer's output at the last step
    dW = g[li.first_connection_index:li.last_connection_index].reshape(wl.n_out, -1)
    assert rel_err(dW, delta.T @ h2) < TOL
    gpu.close()
