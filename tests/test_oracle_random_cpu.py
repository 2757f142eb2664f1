"""The numpy restatement against the compiled reference on seeded random feed-forward architectures (CPU only): random
depth and widths, sigmoidal activation functions, batch normalization / renormalization, Bernoulli and inverted dropout,
average / max pooling, residual blocks of equal and unequal width with and without ShakeDrop (the reference's draws
replayed), gradient descent with and without momentum / Nesterov / clip / weight decay; two training steps.

What is compared: derivatives, updated parameters, the last layer's outputs, running averages, loss.  Bars: every
network within 5e-3 of max|reference| (tiny batch deviations of normalized units amplify fp32 rounding: a chain of
saturating layers leaves a unit almost constant over the 24 rows, and sigma^2 + epsilon then carries a per-cent error
on either side), and at least 85 % of the networks within 5e-5.  A difference in meaning - a wrong formula, a wrong
index - shows as an error of order one.  Optimizers that take the SIGN of a derivative (Adam-type first steps, iRPROP+)
and activation functions with kinks are left to the pinned cases: on random networks a derivative that is zero on one
side and 1e-12 on the other decides a whole step."""
import numpy as np
import pytest

import cases
from conftest import rel_err
from myea_b200 import capi, workloads
from oracle import myea_oracle, ref
from test_checkpoint_random_cpu import _random_network

pytestmark = pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not present")

SMOOTH = [capi.AF_TANH, capi.AF_SIGMOID, capi.AF_ELLIOT, capi.AF_ELLIOT_SYMMETRIC, capi.AF_GAUSSIAN, capi.AF_GAUSSIAN_SYMMETRIC, capi.AF_ISRU,
          capi.AF_ISRLU]
SEEDS = range(48)


def _errors(seed):
    desc, opt, layers = _random_network(seed, activations=SMOOTH, optimizers=[capi.OPT_GD], batch=24)
    n_in, n_out = int(layers[0].unit_parameters[0]), int(layers[-1].unit_parameters[0])
    one_hot = layers[-1].type_activation_function == capi.AF_SOFTMAX

    def workload():
        w = workloads.Workload("random%d" % seed, desc, opt, n_in, n_out, one_hot, layers)
        w.seed = seed
        return w

    net = ref.RefNet(desc, opt, threads=1)
    try:
        want = cases.run_steps(net, workload(), steps=2)
    finally:
        net.close()
    got = cases.run_steps(myea_oracle.OracleNet(desc, opt), workload(), steps=2, shake=want["shake"])
    assert got["index_map"] == want["index_map"] and got["sizes"] == want["sizes"]
    for it in (0, 1):
        assert got["loss%d" % it][1] == want["loss%d" % it][1]              # how many values were scored
    keys = [k for k in ("grad0", "param0", "grad1", "param1", "output_last", "norm_mean_avg", "norm_sigma_avg", "m") if k in want]
    return max(rel_err(got[k], want[k]) for k in keys)


@pytest.fixture(scope="module")
def errors():
    return {seed: _errors(seed) for seed in SEEDS}


def test_every_random_network_within_the_conditioning_bar(errors):
    worst = max(errors, key=errors.get)
    assert errors[worst] < 5e-3, "seed %d: %.2e" % (worst, errors[worst])


def test_most_random_networks_at_rounding_level(errors):
    tight = sum(e < 5e-5 for e in errors.values())
    assert tight >= 0.85 * len(errors), sorted(errors.items(), key=lambda kv: -kv[1])[:8]


def random_recurrent_case(seed):
    """(descriptor, optimizer settings, layers) of a seeded random recurrent network for a numerics comparison: the
    layer list of the checkpoint test's generator (LSTM layers of 1 - 3 cells per block with and without zoneout,
    independently recurrent layers, fully connected layers), sigmoidal activation functions, gradient descent with or
    without momentum and clip, a batch of 6 sequences of 2 - 5 time steps"""
    from test_checkpoint_random_cpu import _random_recurrent_network
    desc, opt = _random_recurrent_network(seed)
    layers = [desc.layers[l] for l in range(desc.number_layers)]
    for L in layers:
        if L.type_layer == capi.LAYER_FC and L.type_activation_function != capi.AF_LINEAR:
            L.type_activation_function = [capi.AF_TANH, capi.AF_SIGMOID, capi.AF_ELLIOT_SYMMETRIC, capi.AF_ISRU][seed % 4]
        if L.type_layer == capi.LAYER_FC_IND_RNN:
            L.type_activation_function = capi.AF_TANH
    opt = capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9 if seed % 2 else 0.0, clip=opt.clip_gradient if opt.use_clip_gradient else None)
    desc = capi.net(layers, batch=6, T=int(desc.number_recurrent_depth), loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE,
                    time_delays=int(desc.number_time_delays), clip_gradient=float(desc.clip_gradient))
    return desc, opt, layers


def recurrent_errors(seed, make_net):
    desc, opt, layers = random_recurrent_case(seed)
    n_in, n_out = int(layers[0].unit_parameters[0]), int(layers[-1].unit_parameters[0])

    def workload():
        w = workloads.Workload("recurrent%d" % seed, desc, opt, n_in, n_out, False, layers)
        w.seed = seed
        return w

    net = ref.RefNet(desc, opt, threads=1)
    try:
        want = cases.run_steps(net, workload(), steps=2)
    finally:
        net.close()
    other = make_net(desc, opt)
    try:
        got = cases.run_steps(other, workload(), steps=2)
    finally:
        if hasattr(other, "close"):
            other.close()
    assert got["index_map"] == want["index_map"] and list(got["sizes"]) == list(want["sizes"])
    for it in (0, 1):
        assert got["loss%d" % it][1] == want["loss%d" % it][1]
    return max(rel_err(got[k], want[k]) for k in ("grad0", "param0", "grad1", "param1", "output_last", "m"))


@pytest.mark.parametrize("seed", range(40))
def test_random_recurrent_network(seed):
    assert recurrent_errors(seed, myea_oracle.OracleNet) < 2e-5


def random_autoencoder_case(seed):
    """(workload, coded layers on the way in) of a seeded random autoencoder: 3, 5 or 7 layers of units with mirrored
    widths, sigmoidal activation functions (and ELU, Gaussian), no / Bernoulli / inverted dropout on the encoding side"""
    rng = np.random.default_rng(900 + seed)
    smooth = [capi.AF_TANH, capi.AF_SIGMOID, capi.AF_ELLIOT_SYMMETRIC, capi.AF_ISRU, capi.AF_ELU, capi.AF_GAUSSIAN]
    depth = int(rng.integers(1, 4))
    widths = [int(rng.integers(6, 16))]
    for _ in range(depth):
        widths.append(int(rng.integers(3, widths[-1] + 1)))
    full = widths + widths[-2::-1]
    layers = [capi.fc(full[0])]
    for i, w in enumerate(full[1:-1], 1):
        drop = int(rng.choice([capi.DROP_NONE, capi.DROP_BERNOULLI, capi.DROP_BERNOULLI_INVERTED])) if i <= depth else capi.DROP_NONE
        layers.append(capi.fc(w, int(rng.choice(smooth)), dropout=drop, p=(float(np.float32(rng.uniform(0.5, 0.9))), 0.0, 0.0) if drop else (0.0, 0.0, 0.0)))
    layers.append(capi.fc(full[-1], capi.AF_LINEAR))
    desc = capi.net(layers, int(rng.integers(4, 12)), loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE)
    desc.type_network = capi.NET_AUTOENCODER
    wl = workloads.Workload("autoencoder%d" % seed, desc, capi.opt(capi.OPT_GD, gd_lr=0.05, momentum=0.9 if seed % 2 else 0.0), full[0], full[-1], False, layers)
    wl.seed = seed
    return wl, depth


def autoencoder_errors(seed, make_net):
    """every pre-training level of the network in turn, then the whole network (level 0), two steps each"""
    wl, depth = random_autoencoder_case(seed)
    levels = tuple(range(1, depth + 1)) + (0,)
    net = ref.RefNet(wl.desc, wl.opt, threads=1)
    try:
        want = cases.run_pre_training(net, wl, levels=levels)
    finally:
        net.close()
    wl, _ = random_autoencoder_case(seed)
    other = make_net(wl.desc, wl.opt)
    try:
        got = cases.run_pre_training(other, wl, levels=levels)
    finally:
        if hasattr(other, "close"):
            other.close()
    for k in want:
        if k.endswith("loss"):
            assert got[k][1] == want[k][1], k
    return max(rel_err(got[k], want[k]) for k in want if not k.endswith("loss"))


@pytest.mark.parametrize("seed", range(40))
def test_random_autoencoder_pre_training(seed):
    assert autoencoder_errors(seed, myea_oracle.OracleNet) < 2e-5


WIDE = [136, 200, 257, 264, 300, 384]


def wide_errors(seed, make_net):
    """the feed-forward generator at layer widths of 136 - 384 units and batches of 136 - 200 rows: sizes at which the
    CUDA path takes its CTA-pair and 256 x 256 contraction kernels, shared operand panels and the kernels that write
    panels while they produce; widths that are no multiple of 8 take the plain paths.  (One reference thread: the
    harness replays the reference's ShakeDrop draws from the generator of thread 0.)"""
    desc, opt, layers = _random_network(seed, activations=SMOOTH, optimizers=[capi.OPT_GD], batch=[136, 160, 200][seed % 3], widths=WIDE)
    opt.learning_rate = 1e-4     # derivatives are sums over the rows
    n_in, n_out = int(layers[0].unit_parameters[0]), int(layers[-1].unit_parameters[0])
    one_hot = layers[-1].type_activation_function == capi.AF_SOFTMAX

    def workload():
        w = workloads.Workload("wide%d" % seed, desc, opt, n_in, n_out, one_hot, layers)
        w.seed = seed
        return w

    net = ref.RefNet(desc, opt, threads=1)
    try:
        want = cases.run_steps(net, workload(), steps=2)
    finally:
        net.close()
    other = make_net(desc, opt)
    try:
        got = cases.run_steps(other, workload(), steps=2, shake=want["shake"])
    finally:
        if hasattr(other, "close"):
            other.close()
    assert got["index_map"] == want["index_map"] and list(got["sizes"]) == list(want["sizes"])
    for it in (0, 1):
        assert got["loss%d" % it][1] == want["loss%d" % it][1]
    keys = [k for k in ("grad0", "param0", "grad1", "param1", "output_last", "norm_mean_avg", "norm_sigma_avg", "m") if k in want]
    return max(rel_err(got[k], want[k]) for k in keys)


@pytest.mark.parametrize("seed", range(24))
def test_random_wide_network(seed):
    assert wide_errors(seed, myea_oracle.OracleNet) < 1e-4
