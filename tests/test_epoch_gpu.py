"""GPU tests of the epoch loop (myea_b200_dataset_set / train_epoch / evaluate): the same shuffled order, mini-batch by
mini-batch, through the compiled reference's step functions (what Dataset_Mini_Batch::Training_Loop does) must give
the same parameters, mean loss and evaluation loss.  Tolerance 1e-4 max relative error per tensor."""
import ctypes as C

import numpy as np
import pytest

import cases
from conftest import rel_err
from myea_b200 import capi
from myea_b200.net import Net
from oracle import myea_oracle, ref

pytestmark = pytest.mark.gpu
TOL = 1e-4


def _oracle(wl):
    return ref.RefNet(wl.desc, wl.opt, threads=1) if ref.available() else myea_oracle.OracleNet(wl.desc, wl.opt)


def _dataset(wl, n, seed=3):
    rng = np.random.default_rng(seed)
    T = max(1, int(wl.desc.number_recurrent_depth))
    X = rng.standard_normal((n, T, wl.n_in)).astype(np.float32)
    if wl.one_hot:
        Y = np.zeros((n, T, wl.n_out), np.float32)
        lab = rng.integers(0, wl.n_out, (n, T))
        for i in range(n):
            for t in range(T):
                Y[i, t, lab[i, t]] = 1.0
    else:
        Y = rng.standard_normal((n, T, wl.n_out)).astype(np.float32)
    return X, Y


def _reference_loss(wl, s, n):
    return s / (n // wl.n_out) if wl.one_hot else s / n


@pytest.mark.parametrize("name,sub_batches", [("mlp_relu_gd", 1), ("mlp_selu_momentum", 2), ("c2_small", 1), ("lstm1_all_steps_adam", 1)])
def test_epochs_match_the_reference_step_loop(name, sub_batches):
    wl = cases.CASES[name]()
    B, mini = wl.B, wl.B * sub_batches
    n = mini * 3
    X, Y = _dataset(wl, n)
    gpu, cpu = Net(wl.desc, wl.opt), _oracle(wl)
    wl.materialize(gpu); wl.materialize(cpu)
    gpu.dataset_set(X.reshape(n, -1), Y.reshape(n, -1))
    rng = np.random.default_rng(11)
    for epoch in range(2):
        order = rng.permutation(n)
        loss_gpu, acc_gpu = gpu.train_epoch(order, mini)
        losses, acc_cpu = [], 0.0
        for mb in range(n // mini):
            cpu.reset_loss()
            for sub in range(sub_batches):
                idx = order[mb * mini + sub * B: mb * mini + (sub + 1) * B]
                xb = np.ascontiguousarray(X[idx].transpose(1, 0, 2))   # [T][B][in]
                yb = np.ascontiguousarray(Y[idx].transpose(1, 0, 2))
                cpu.forward(xb); cpu.compute_error(yb); cpu.backward(); cpu.update_derivative_weight()
            s, cnt, a = cpu.loss()
            losses.append(_reference_loss(wl, s, cnt)); acc_cpu += a
            cpu.update_parameter(training_size=n)   # (the batch size only enters the normalized weight decay, which these cases do not use)
        assert abs(loss_gpu - np.mean(losses)) <= 1e-4 * abs(np.mean(losses)) + 1e-6
        assert acc_gpu == acc_cpu
        assert rel_err(gpu.get(capi.BUF_PARAMETERS), cpu.get(capi.BUF_PARAMETERS)) < TOL
    # evaluation pass: inference-mode forward over the first 2 batches
    m = 2 * B
    loss_e, ls, nl, acc = gpu.evaluate(m)
    cpu.reset_loss()
    for k in range(2):
        xb = np.ascontiguousarray(X[k * B:(k + 1) * B].transpose(1, 0, 2)); yb = np.ascontiguousarray(Y[k * B:(k + 1) * B].transpose(1, 0, 2))
        cpu.forward(xb, training=False); cpu.compute_error(yb)
    s, cnt, a = cpu.loss()
    assert nl == cnt and acc == a and abs(ls - s) <= 1e-4 * abs(s) + 1e-6
    assert abs(loss_e - _reference_loss(wl, s, cnt)) <= 1e-4 * abs(loss_e) + 1e-6
    gpu.close(); cpu.close()


def test_epoch_with_device_drawn_masks_runs_and_is_repeatable():
    wl = cases.CASES["c2_small"]()
    n = wl.B * 4
    X, Y = _dataset(wl, n)
    out = []
    for _ in range(2):
        gpu = Net(wl.desc, wl.opt)
        wl.materialize(gpu)
        gpu.dataset_set(X.reshape(n, -1), Y.reshape(n, -1))
        loss, _ = gpu.train_epoch(np.arange(n), wl.B, mask_seed=77, first_step=5)
        out.append((loss, gpu.get(capi.BUF_PARAMETERS)))
        gpu.close()
    assert out[0][0] == out[1][0] and np.array_equal(out[0][1], out[1][1])


@pytest.mark.parametrize("name", ["mlp_relu_gd", "c2_small", "lstm1_all_steps_adam", "lstm2_zoneout_clip"])
def test_short_last_batches_match_the_reference(name):
    """the last sub-batch of a mini-batch and the last mini-batch of the epoch may be shorter than the allocated batch
    (Dataset::Train_Batch_BP, Dataset.cpp:667-691); BN statistics are then those of the short batch; recurrent
    networks keep the allocated batch as the pitch of a time step"""
    wl = cases.CASES[name]()
    B = wl.B
    mini = B + B // 2                 # one full sub-batch + a half one
    n = 2 * mini + B // 3 + 1         # two whole mini-batches + a short one
    X, Y = _dataset(wl, n)
    gpu, cpu = Net(wl.desc, wl.opt), _oracle(wl)
    wl.materialize(gpu); wl.materialize(cpu)
    gpu.dataset_set(X.reshape(n, -1), Y.reshape(n, -1))
    order = np.random.default_rng(2).permutation(n)
    loss_gpu, acc_gpu = gpu.train_epoch(order, mini)
    losses, acc_cpu = [], 0.0
    for first in range(0, n, mini):
        size = min(mini, n - first)
        cpu.reset_loss()
        for done in range(0, size, B):
            b = min(B, size - done)
            idx = order[first + done: first + done + b]
            cpu.forward(np.ascontiguousarray(X[idx].transpose(1, 0, 2)), batch=b)
            cpu.compute_error(np.ascontiguousarray(Y[idx].transpose(1, 0, 2)))
            cpu.backward(); cpu.update_derivative_weight()
        s, cnt, a = cpu.loss()
        losses.append(_reference_loss(wl, s, cnt)); acc_cpu += a
        cpu.update_parameter(training_size=n, batch=size)
    assert abs(loss_gpu - np.mean(losses)) <= 1e-4 * abs(np.mean(losses)) + 1e-6
    assert acc_gpu == acc_cpu
    assert rel_err(gpu.get(capi.BUF_PARAMETERS), cpu.get(capi.BUF_PARAMETERS)) < TOL
    # evaluation over a number of examples that is not a multiple of the batch
    m = B + 3
    loss_e, ls, nl, acc = gpu.evaluate(m)
    cpu.reset_loss()
    for first in range(0, m, B):
        b = min(B, m - first)
        cpu.forward(np.ascontiguousarray(X[first:first + b].transpose(1, 0, 2)), training=False, batch=b)
        cpu.compute_error(np.ascontiguousarray(Y[first:first + b].transpose(1, 0, 2)))
    s, cnt, a = cpu.loss()
    assert nl == cnt and acc == a and abs(ls - s) <= 1e-4 * abs(s) + 1e-6
    gpu.close(); cpu.close()


def test_bad_requests_are_refused_not_mangled():
    wl = cases.CASES["lstm1_all_steps_adam"]()
    gpu = Net(wl.desc, wl.opt)
    wl.materialize(gpu)
    n = wl.B * 2 + 1
    X, Y = _dataset(wl, n)
    gpu.dataset_set(X.reshape(n, -1), Y.reshape(n, -1))
    loss, acc = C.c_double(), C.c_double()
    bad = np.array([0, n + 5] * wl.B, dtype=np.uint64)[:wl.B * 2]      # an index past the dataset
    assert gpu.lib.myea_b200_train_epoch(gpu.h, bad.ctypes.data, bad.size, wl.B, C.byref(wl.opt), 0, 0, C.byref(loss), C.byref(acc)) == -1
    assert gpu.lib.myea_b200_evaluate(gpu.h, None, n + 1, None, None, None, None) == -1      # more examples than the dataset holds
    x = np.zeros((wl.desc.number_recurrent_depth, wl.B + 1, wl.n_in), np.float32)
    assert gpu.lib.myea_b200_forward(gpu.h, wl.B + 1, x.ctypes.data, 1) == -1                # batch above the allocated one
    gpu.close()
