"""CPU tests: the numpy restatement (oracle/myea_oracle.py) against the golden vectors produced by the unmodified
reference, and against the compiled reference itself when oracle/_ref is present."""
import os

import numpy as np
import pytest

import cases
from conftest import rel_err
from oracle import myea_oracle, ref

TOL = 5e-5   # float32 summation-order noise between numpy and the reference's scalar loops (the adaptive optimizers amplify it)


def _load(golden_dir, name):
    path = os.path.join(golden_dir, name + ".npz")
    if not os.path.exists(path):
        pytest.skip("no golden fixture for %s" % name)
    return np.load(path)


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_oracle_matches_golden(name, golden_dir):
    gold = _load(golden_dir, name)
    wl = cases.CASES[name]()
    net = myea_oracle.OracleNet(wl.desc, wl.opt)
    out = cases.run_steps(net, wl, shake=cases.shake_from_golden(gold))
    assert list(out["sizes"]) == list(gold["sizes"])                      # integer work: bit-exact
    assert np.array_equal(np.asarray(out["index_map"], np.int64), gold["index_map"])
    for k in ("grad0", "grad1", "param0", "param1", "output_last", "m"):
        assert rel_err(out[k], gold[k]) < TOL, k
    for k in ("rprop_steps", "rprop_delta"):                              # iRPROP+: exact multiples of the initial step
        if k in out:
            assert np.array_equal(np.asarray(out[k], np.float32), gold[k]), k
    for k in ("loss0", "loss1"):
        assert abs(out[k][0] - gold[k][0]) <= 1e-4 * abs(gold[k][0]) + 1e-6
        assert out[k][1] == gold[k][1]                                    # number of loss terms: exact
        assert out[k][2] == gold[k][2]                                    # accuracy hit count: exact
    if "norm_mean_avg" in gold.files:
        assert rel_err(out["norm_mean_avg"], gold["norm_mean_avg"]) < TOL
        assert rel_err(out["norm_sigma_avg"], gold["norm_sigma_avg"]) < TOL


@pytest.mark.parametrize("name,dropout", [("autoencoder_pre_training", cases.capi.DROP_NONE),
                                          ("autoencoder_pre_training_dropout", cases.capi.DROP_BERNOULLI_INVERTED)])
def test_oracle_pre_training_matches_golden(name, dropout, golden_dir):
    """autoencoder pre-training: levels 1 and 2, then the whole network, against the reference's vectors"""
    gold = _load(golden_dir, name)
    wl = cases.autoencoder_case(dropout)
    out = cases.run_pre_training(myea_oracle.OracleNet(wl.desc, wl.opt), wl)
    assert sorted(out) == sorted(gold.files)
    for k in gold.files:
        if k.endswith("loss"):
            assert abs(out[k][0] - gold[k][0]) <= 1e-4 * abs(gold[k][0]) + 1e-6 and out[k][1] == gold[k][1] and out[k][2] == gold[k][2], k
        else:
            assert rel_err(out[k], gold[k]) < TOL, k


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_golden_inputs_unchanged(name, golden_dir):
    """the seeded inputs the fixtures were generated from are still what the workload builders produce"""
    gold = _load(golden_dir, name)
    wl = cases.CASES[name]()
    net = myea_oracle.OracleNet(wl.desc, wl.opt)
    X, Y = wl.batch()
    p = wl.parameters(net)
    chk = np.array([np.abs(X).sum(dtype=np.float64), np.abs(Y).sum(dtype=np.float64), np.abs(p).sum(dtype=np.float64)])
    assert np.allclose(chk, gold["input_checksum"], rtol=1e-12)


@pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not present")
@pytest.mark.parametrize("name", ["c1_small", "c2_small", "mlp_brn_elu_adabound_wd"])
def test_reference_reproduces_golden(name, golden_dir):
    """the compiled reference is deterministic: a fresh run gives the committed vectors bit for bit (1 thread)"""
    gold = _load(golden_dir, name)
    wl = cases.CASES[name]()
    net = ref.RefNet(wl.desc, wl.opt, threads=1)
    out = cases.run_steps(net, wl)
    net.close()
    for k in ("grad0", "param1"):
        assert np.array_equal(np.asarray(out[k], np.float32), gold[k]), k


@pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not present")
def test_reference_openmp_equals_loop():
    """OpenMP slices merged = Loop result up to summation order (the bench's CPU baseline uses the OpenMP path)"""
    wl = cases.CASES["c2_small"]()
    a = ref.RefNet(wl.desc, wl.opt, threads=1)
    b = ref.RefNet(wl.desc, wl.opt, threads=4)
    oa, ob = cases.run_steps(a, wl), cases.run_steps(b, wl)
    a.close(); b.close()
    assert rel_err(ob["grad0"], oa["grad0"]) < 1e-5
    assert rel_err(ob["param1"], oa["param1"]) < 1e-5
