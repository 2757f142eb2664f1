"""GPU parity tests: every case of tests/cases.py runs through the C ABI on cuda:0 and is compared with the oracle
(the compiled reference when oracle/_ref is present, else the numpy restatement) and with the committed golden vectors.
Tolerance: 1e-4 max relative error per tensor (max |a-b| / max |b|) on derivatives, updated parameters and moments;
sizes, index map, loss-term counts and accuracy hit counts bit-exact."""
import os

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


def _seeded_shake(wl):
    """ShakeDrop draws for an oracle that does not draw its own (the numpy restatement): seeded, one dict per step"""
    rng = np.random.default_rng(99)
    steps = []
    for _ in range(cases.STEPS):
        d = {}
        for l, L in enumerate(wl.layers):
            if L.type_layer == capi.LAYER_RESIDUAL and L.type_dropout == capi.DROP_SHAKEDROP:
                w = int(wl.layers[l + int(L.unit_parameters[0])].unit_parameters[0])
                d[l] = ((rng.random(wl.B) < L.dropout_values[0]).astype(np.uint8), rng.uniform(-1, 1, (wl.B, w)).astype(np.float32),
                        rng.uniform(0, 1, (wl.B, w)).astype(np.float32))
        steps.append(d)
    return steps


def _compare(out, want, tol=TOL):
    assert list(out["sizes"]) == [int(x) for x in want["sizes"]]
    assert np.array_equal(np.asarray(out["index_map"], np.int64), np.asarray(want["index_map"], np.int64))
    for k in ("grad0", "grad1", "param0", "param1", "output_last", "m"):
        assert rel_err(out[k], want[k]) < tol, (k, rel_err(out[k], want[k]))
    for k in ("rprop_steps", "rprop_delta"):        # iRPROP+: step sizes and last weight changes are exact multiples, not approximations
        if k in out:
            assert np.array_equal(np.asarray(out[k], np.float32), np.asarray(want[k], np.float32)), k
    for k in ("loss0", "loss1"):
        assert abs(out[k][0] - want[k][0]) <= 1e-4 * abs(want[k][0]) + 1e-6
        assert out[k][1] == want[k][1]
        assert out[k][2] == want[k][2]
    if "norm_mean_avg" in want:
        assert rel_err(out["norm_mean_avg"], want["norm_mean_avg"]) < tol
        assert rel_err(out["norm_sigma_avg"], want["norm_sigma_avg"]) < tol


@pytest.mark.parametrize("name", sorted(cases.CASES) + sorted(cases.CASES_ORACLE_ONLY))
def test_step_matches_oracle(name):
    wl = (cases.CASES.get(name) or cases.CASES_ORACLE_ONLY[name])()
    gpu, cpu = Net(wl.desc, wl.opt), _oracle(wl)
    want = cases.run_steps(cpu, wl, shake=_seeded_shake(wl))
    out = cases.run_steps(gpu, wl, shake=want["shake"] if want["shake"] and want["shake"][0] else _seeded_shake(wl))
    gpu.synchronize()
    assert gpu.launches() > 0
    _compare(out, want)
    gpu.close(); cpu.close()


@pytest.mark.parametrize("af", [capi.AF_THRESHOLD, capi.AF_THRESHOLD_SYMMETRIC, capi.AF_GAUSSIAN_STEPWISE])
def test_activations_without_a_derivative_run_forward(af):
    """the threshold functions and the stepwise Gaussian (a constant 0 in the reference) have no entry in the reference's
    derivative switch; their forward values are checked against the restatement, inference mode"""
    wl = cases._mlp_variant("af_%d" % af, [16, 12], af, capi.opt(capi.OPT_GD, gd_lr=0.01), B=9, n_in=10, n_out=4)
    gpu, cpu = Net(wl.desc, wl.opt), myea_oracle.OracleNet(wl.desc, wl.opt)
    X, _ = wl.batch()
    for net in (gpu, cpu):
        wl.materialize(net)
        net.forward(X, training=False)
    for l in range(1, len(wl.layers)):
        a, b = np.asarray(gpu.outputs(l), np.float32).ravel(), np.asarray(cpu.outputs(l), np.float32).ravel()
        assert (np.abs(a - b) > 1e-4).mean() < 0.02, l      # a summation within rounding of the threshold may land on either side
    gpu.close()


@pytest.mark.parametrize("dropout", [capi.DROP_NONE, capi.DROP_BERNOULLI_INVERTED, capi.DROP_BERNOULLI])
def test_autoencoder_pre_training_matches_the_reference(dropout):
    """Set__Pre_Training_Level 1, 2 and back to 0 on a 10-7-4-7-10 autoencoder, two steps each: derivatives, losses, the
    answering layer's outputs and the updated parameters against the compiled reference (the restatement without it)"""
    wl = cases.autoencoder_case(dropout)
    gpu, cpu = Net(wl.desc, wl.opt), _oracle(wl)
    out, want = cases.run_pre_training(gpu, wl), cases.run_pre_training(cpu, wl)
    assert gpu.launches() > 0
    for k in want:
        if k.endswith("loss"):
            assert abs(out[k][0] - want[k][0]) <= 1e-4 * abs(want[k][0]) + 1e-6 and out[k][1] == want[k][1] and out[k][2] == want[k][2], k
        else:
            assert rel_err(out[k], want[k]) < TOL, (k, rel_err(out[k], want[k]))
    gpu.close(); cpu.close()


@pytest.mark.parametrize("name", sorted(cases.CASES_WITHOUT_REFERENCE))
def test_step_matches_restatement_where_the_reference_cannot_serve(name):
    """bidirectional LSTM, and normalized layers beside LSTM layers (the reference crashes while it builds such a network):
    checked against the numpy restatement (parity against the reference binary is unpinned here)"""
    wl = cases.CASES_WITHOUT_REFERENCE[name]()
    gpu, cpu = Net(wl.desc, wl.opt), myea_oracle.OracleNet(wl.desc, wl.opt)
    out, want = cases.run_steps(gpu, wl), cases.run_steps(cpu, wl)
    _compare(out, want)
    for l in range(1, len(wl.layers)):
        assert rel_err(gpu.outputs(l), cpu.outputs(l)) < TOL
    gpu.close()


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_step_matches_golden(name, golden_dir):
    path = os.path.join(golden_dir, name + ".npz")
    if not os.path.exists(path):
        pytest.skip("no golden fixture")
    gold = np.load(path)
    wl = cases.CASES[name]()
    gpu = Net(wl.desc, wl.opt)
    out = cases.run_steps(gpu, wl, shake=cases.shake_from_golden(gold))
    _compare(out, {k: gold[k] for k in gold.files})
    gpu.close()


@pytest.mark.parametrize("name", ["c1_small", "c2_small"])
def test_fp32_fma_engine_matches_too(name, monkeypatch):
    """the second GEMM engine (plain FP32 FMA) gives the same step: isolates tensor-core issues from everything else"""
    monkeypatch.setenv("MYEA_B200_GEMM_ENGINE", "1")
    wl = cases.CASES[name]()
    gpu, cpu = Net(wl.desc, wl.opt), _oracle(wl)
    _compare(cases.run_steps(gpu, wl), cases.run_steps(cpu, wl))
    gpu.close(); cpu.close()


def test_layer_errors_and_outputs_match_per_layer():
    wl = cases.CASES["c2_small"]()
    gpu, cpu = Net(wl.desc, wl.opt), _oracle(wl)
    X, Y = wl.batch()
    for net in (gpu, cpu):
        wl.materialize(net)
        net.forward(X); net.compute_error(Y); net.backward()
    for l in range(1, len(wl.layers)):
        assert rel_err(gpu.outputs(l), cpu.outputs(l)) < TOL
        assert rel_err(gpu.errors(l), cpu.errors(l)) < TOL
    gpu.close(); cpu.close()


def test_inference_forward_matches():
    wl = cases.CASES["mlp_bernoulli_amsbound_clip"]()
    gpu, cpu = Net(wl.desc, wl.opt), _oracle(wl)
    X, _ = wl.batch()
    for net in (gpu, cpu):
        wl.materialize(net)
        net.forward(X, training=False)
    last = len(wl.layers) - 1
    assert rel_err(gpu.outputs(last), cpu.outputs(last)) < TOL
    gpu.close(); cpu.close()


def test_derivatives_accumulate_over_sub_batches():
    """Update_Derivative_Weight adds into the derivative buffer; two passes before the update give twice the derivative"""
    wl = cases.CASES["c1_small"]()
    gpu = Net(wl.desc, wl.opt)
    wl.materialize(gpu)
    X, Y = wl.batch()
    gpu.forward(X); gpu.compute_error(Y); gpu.backward(); gpu.update_derivative_weight()
    g1 = gpu.get(capi.BUF_DERIVATIVES)
    gpu.forward(X); gpu.compute_error(Y); gpu.backward(); gpu.update_derivative_weight()
    g2 = gpu.get(capi.BUF_DERIVATIVES)
    assert rel_err(g2, 2.0 * g1) < 1e-6
    gpu.update_parameter()
    assert not gpu.get(capi.BUF_DERIVATIVES).any()       # the optimizer zeroes the derivatives
    gpu.close()


def test_bad_calls_return_status_not_crash():
    wl = cases.CASES["c1_small"]()
    gpu = Net(wl.desc, wl.opt)
    lib = gpu.lib
    X, _ = wl.batch()
    assert lib.myea_b200_forward(gpu.h, wl.B + 1, X.ctypes.data, 1) == -1          # more rows than were allocated
    assert lib.myea_b200_forward(gpu.h, wl.B - 1, X.ctypes.data, 1) == 0           # fewer rows: fine for a feed-forward network
    assert lib.myea_b200_backward(gpu.h, wl.B) == -1                                # not the batch in flight
    assert lib.myea_b200_set_mask_bernoulli(gpu.h, 1, X.ctypes.data, 3) == -1      # layer without a mask
    assert b"mask" in lib.myea_b200_last_error(gpu.h)
    gpu.close()
