"""The CUDA path against the compiled reference on seeded random feed-forward architectures (the generator and the bars
of tests/test_oracle_random_cpu.py): random depth and widths, sigmoidal activation functions, batch normalization /
renormalization, Bernoulli and inverted dropout, average / max pooling, residual blocks of equal and unequal width with
and without ShakeDrop (the reference's draws replayed), gradient descent with momentum / Nesterov / clip / weight decay;
two training steps through the C ABI on cuda:0.  Every network within 1e-2 of max|reference| (ill-conditioned batch
deviations, see the CPU test; measured worst: 3.6e-3 on the network where the restatement itself is 2.4e-3 from the
reference), at least 80 % within the 1e-4 parity tolerance (measured: 43 of 48).  A difference in meaning shows as an
error of order one."""
import pytest

import cases
from conftest import rel_err
from myea_b200 import capi, workloads
from myea_b200.net import Net
from oracle import ref
from test_checkpoint_random_cpu import _random_network
from test_oracle_random_cpu import SMOOTH, SEEDS

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not present")]


def _errors(seed):
    desc, opt, layers = _random_network(seed, activations=SMOOTH, optimizers=[capi.OPT_GD], batch=24)
    n_in, n_out = int(layers[0].unit_parameters[0]), int(layers[-1].unit_parameters[0])
    one_hot = layers[-1].type_activation_function == capi.AF_SOFTMAX

    def workload():
        w = workloads.Workload("random%d" % seed, desc, opt, n_in, n_out, one_hot, layers)
        w.seed = seed
        return w

    cpu = ref.RefNet(desc, opt, threads=1)
    try:
        want = cases.run_steps(cpu, workload(), steps=2)
    finally:
        cpu.close()
    gpu = Net(desc, opt)
    try:
        got = cases.run_steps(gpu, workload(), steps=2, shake=want["shake"])
        gpu.synchronize()
        assert gpu.launches() > 0
    finally:
        gpu.close()
    assert got["index_map"] == want["index_map"] and list(got["sizes"]) == list(want["sizes"])
    for it in (0, 1):
        assert got["loss%d" % it][1] == want["loss%d" % it][1]
    keys = [k for k in ("grad0", "param0", "grad1", "param1", "output_last", "norm_mean_avg", "norm_sigma_avg", "m") if k in want]
    return max(rel_err(got[k], want[k]) for k in keys)


@pytest.fixture(scope="module")
def errors():
    return {seed: _errors(seed) for seed in SEEDS}


def test_every_random_network_within_the_conditioning_bar(errors):
    worst = max(errors, key=errors.get)
    assert errors[worst] < 1e-2, "seed %d: %.2e" % (worst, errors[worst])


def test_most_random_networks_within_the_parity_tolerance(errors):
    tight = sum(e < 1e-4 for e in errors.values())
    assert tight >= 0.80 * len(errors), sorted(errors.items(), key=lambda kv: -kv[1])[:8]


@pytest.mark.parametrize("seed", range(40))
def test_random_recurrent_network(seed):
    """LSTM layers of 1 - 3 cells per block with and without zoneout, independently recurrent layers and fully connected
    layers between them, 2 - 5 time steps: within the 1e-4 parity tolerance of the compiled reference"""
    from test_oracle_random_cpu import recurrent_errors
    assert recurrent_errors(seed, Net) < 1e-4


@pytest.mark.parametrize("seed", range(40))
def test_random_autoencoder_pre_training(seed):
    """autoencoders of 3, 5 or 7 layers with mirrored widths: every pre-training level in turn, then the whole network"""
    from test_oracle_random_cpu import autoencoder_errors
    assert autoencoder_errors(seed, Net) < 1e-4


def test_random_wide_networks():
    """layer widths of 136 - 384 units, batches of 136 - 200 rows (CTA-pair and 256 x 256 contraction kernels, shared
    operand panels, producers that write panels; widths that are no multiple of 8 on the plain paths)"""
    from test_oracle_random_cpu import wide_errors
    errors = {seed: wide_errors(seed, Net) for seed in range(24)}
    print(sorted(errors.items(), key=lambda kv: -kv[1]))
    worst = max(errors, key=errors.get)
    assert errors[worst] < 1e-4, "seed %d: %.2e" % (worst, errors[worst])
