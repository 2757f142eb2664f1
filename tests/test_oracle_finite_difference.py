"""CPU test: the numpy restatement's hand-written backward pass against float64 finite differences of its own forward
pass, on the layer the compiled reference cannot check (bidirectional LSTM) and, as a control, on a unidirectional LSTM
that IS pinned against the reference.  The reference's derivative is d/dw of 0.5 * sum (prediction - target)^2 over the
scored steps (delta = prediction - target for a linear output); zoneout is off because the reference's backward pass
ignores the zoneout masks."""
import numpy as np
import pytest

import cases
from myea_b200 import capi
from oracle import myea_oracle


def _objective(net, X, Y):
    net.reset_loss()
    net.forward(X)
    net.compute_error(Y)
    return 0.5 * net.loss()[0]


@pytest.mark.parametrize("name", ["bilstm_no_zoneout_amsgrad", "lstm1_all_steps_adam"])
def test_backward_matches_finite_differences(name):
    make = cases.CASES_WITHOUT_REFERENCE.get(name) or cases.CASES[name]
    wl = make()
    net = myea_oracle.OracleNet(wl.desc, wl.opt, dtype=np.float64)
    wl.materialize(net)
    X, Y = wl.batch()
    net.forward(X); net.compute_error(Y); net.backward(); net.update_derivative_weight()
    grad = net.buf[capi.BUF_DERIVATIVES].copy()
    p = net.buf[capi.BUF_PARAMETERS]
    rng = np.random.default_rng(3)
    used = np.flatnonzero(grad != 0)
    picks = rng.choice(used, size=min(60, used.size), replace=False)
    eps = 1e-6
    for i in picks:
        keep = p[i]
        p[i] = keep + eps
        up = _objective(net, X, Y)
        p[i] = keep - eps
        down = _objective(net, X, Y)
        p[i] = keep
        fd = (up - down) / (2 * eps)
        assert abs(fd - grad[i]) <= 1e-5 * max(1.0, abs(grad[i])), (i, fd, grad[i])
