"""The host-side mirror of the reference's `class Neural_Network` (myea_b200/host): its example program drives config 1
through Compile / Set__* / Forward_Pass / Compute__Error / Backward_Pass / Update_Derivative_Weight / Update_Parameter
exactly as the reference's harness does.  On a GPU the loss on the fixed batch must fall step after step; without a GPU
the program must fail loudly (there is no CPU path)."""
import os
import re
import subprocess

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
