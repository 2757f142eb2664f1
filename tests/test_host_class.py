"""The host-side mirror of the reference's `class Neural_Network` (myea_b200/host): its example program drives config 1
through Compile / Set__* / Forward_Pass / Compute__Error / Backward_Pass / Update_Derivative_Weight / Update_Parameter
exactly as the reference's harness does.  On a GPU the loss on the fixed batch must fall step after step; without a GPU
the program must fail loudly (there is no CPU path)."""
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "myea_b200", "host", "train_mlp")


def _has_gpu():
    import torch
    return torch.cuda.is_available()


def test_example_is_built():
    assert os.path.exists(EXE), "build with: python -c 'import __graft_entry__ as g; g.build()'"


def test_fails_loudly_without_gpu():
    if _has_gpu():
        pytest.skip("a GPU is present")
    r = subprocess.run([EXE, "2"], capture_output=True, text=True, timeout=120)
    assert r.returncode != 0 and "ERROR" in r.stderr


@pytest.mark.gpu
def test_trains_config_1_through_the_reference_api():
    r = subprocess.run([EXE, "12"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    losses = [float(x) for x in re.findall(r"loss ([0-9.]+)", r.stdout)]
    assert len(losses) == 12
    assert 0.15 < losses[0] < 0.6                      # mean of -t*log(y) over 10 outputs, near ln(10)/10 at the start
    assert all(b < a for a, b in zip(losses, losses[1:]))


@pytest.mark.gpu
def test_checkpoint_round_trip_through_the_reference_api(tmp_path):
    """Save_Dimension_Parameters / Save_General_Parameters / Load of the host class: the trained network written in
    the reference's text format and read into a second object answers the batch identically"""
    prefix = str(tmp_path / "mlp")
    r = subprocess.run([EXE, "4", prefix], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "checkpoint round trip: identical" in r.stdout
    head = open(prefix + ".nn", "rb").read(200)
    assert head.startswith(b"|===| DIMENSION |===|\r\ntype_network 3\r\nnumber_layers 4\r\n")
    assert b"type_optimizer_function 2\r\n" in open(prefix + ".net", "rb").read()


@pytest.mark.gpu
def test_parameters_match_the_reference_class_driven_through_the_same_calls(tmp_path):
    """the example program and the reference's own `class Neural_Network` (compiled from its sources, oracle/_ref) make
    the same member calls - Compile, Set__*, then per step Reset__Loss, Forward_Pass, Compute__Error, Backward_Pass,
    Update_Derivative_Weight, Update_Parameter - on the same parameters, inputs and targets read from files; the
    trained parameters agree to 1e-4 (max |a - b| / max |b|).  Momentum descent: a linear update, so that the bound
    holds for every parameter (Adam's first steps turn rounding noise of a zero derivative into a full step)."""
    import sys
    sys.path.insert(0, ROOT)
    from myea_b200 import capi
    from oracle import ref
    if not ref.available():
        pytest.skip("the compiled reference is not here")
    B, sizes, steps = 128, (64, 256, 256, 10), 6
    rng = np.random.default_rng(5)
    layers = [capi.fc(64), capi.fc(256, capi.AF_TANH), capi.fc(256, capi.AF_TANH), capi.fc(10, capi.AF_SOFTMAX)]
    desc = capi.net(layers, B, loss=capi.LOSS_CE, accuracy=capi.ACC_CE)
    opt = capi.opt(capi.OPT_GD)
    opt.learning_rate, opt.learning_momentum = 0.01, 0.9          # the class defaults the example leaves in place
    cpu = ref.RefNet(desc, opt, threads=1)
    P = cpu.sizes()[0]
    params = np.zeros(P, np.float32)
    for l in range(1, 4):
        ix = cpu.layer_index(l)
        bound = (5.0 / 3.0 if l < 3 else 1.0) * np.sqrt(6.0 / (sizes[l - 1] + sizes[l]))
        a, b = int(ix.first_connection_index), int(ix.last_connection_index)
        params[a:b] = rng.uniform(-bound, bound, b - a)
    X = rng.uniform(-1, 1, (B, 64)).astype(np.float32)
    Y = np.zeros((B, 10), np.float32)
    Y[np.arange(B), rng.integers(0, 10, B)] = 1.0
    params.tofile(tmp_path / "parameters.f32"); X.tofile(tmp_path / "inputs.f32"); Y.tofile(tmp_path / "targets.f32")
    r = subprocess.run([EXE, str(steps), "", str(tmp_path), str(capi.OPT_GD)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    got = np.fromfile(tmp_path / "parameters_out.f32", np.float32)
    cpu.set(capi.BUF_PARAMETERS, params)
    losses = []
    for _ in range(steps):
        cpu.reset_loss()
        cpu.forward(X[None]); cpu.compute_error(Y[None]); cpu.backward(); cpu.update_derivative_weight()
        s, n, _ = cpu.loss()
        losses.append(s / n)
        cpu.update_parameter(training_size=B)
    want = cpu.get(capi.BUF_PARAMETERS)
    assert got.shape == want.shape
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-4
    mine = [float(x) for x in re.findall(r"loss ([0-9.]+)", r.stdout)]
    assert np.allclose(mine, losses, rtol=1e-4)
    cpu.close()
