"""Checkpoint writer against the compiled reference's writer on seeded random feed-forward architectures (CPU only):
random depth and widths, every activation function, batch normalization / renormalization, Bernoulli and inverted
dropout, average / max pooling layers, residual blocks of equal and unequal width (zero-padded identity) with and
without ShakeDrop.  Both writers must produce the same bytes for `.nn` and `.net`, and the files written here must
parse back to the arrays they were written from.  Text and integer work: exact equality."""
import numpy as np
import pytest

from myea_b200 import capi, checkpoint
from oracle import ref

pytestmark = pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not present")

ACTIVATIONS = [getattr(capi, n) for n in dir(capi) if n.startswith("AF_") and n not in ("AF_NONE", "AF_SOFTMAX")]
OPTIMIZERS = [capi.OPT_ADAM, capi.OPT_AMSGRAD, capi.OPT_ADABOUND, capi.OPT_AMSBOUND, capi.OPT_GD, capi.OPT_NOSADAM, capi.OPT_IRPROP_PLUS]


def _random_network(seed, activations=None, optimizers=None, batch=None, widths=None):
    """(descriptor, optimizer settings, layer list) of a seeded random feed-forward network; `widths`: the layer widths
    to draw from (default: 3 .. 24)"""
    activations, optimizers = activations or ACTIVATIONS, optimizers or OPTIMIZERS
    rng = np.random.default_rng(seed)
    width = (lambda: int(rng.choice(widths))) if widths else (lambda: int(rng.integers(3, 25)))
    layers = [capi.fc(width())]
    prev = layers[0].unit_parameters[0]
    norm_of_net = int(rng.choice([capi.NORM_BN, capi.NORM_BRN]))   # the reference refuses both kinds in one network
    for _ in range(int(rng.integers(2, 6))):
        kind = rng.choice(["fc", "fc", "fc", "pool", "block"])
        af = int(rng.choice(activations))
        norm = int(rng.choice([capi.NORM_NONE, norm_of_net]))
        drop = int(rng.choice([capi.DROP_NONE, capi.DROP_BERNOULLI, capi.DROP_BERNOULLI_INVERTED]))
        p = (float(np.float32(rng.uniform(0.3, 0.9))), 0.0, 0.0) if drop != capi.DROP_NONE else (0.0, 0.0, 0.0)
        if kind == "fc":
            prev = width()
            layers.append(capi.fc(prev, af, norm, drop, p))
        elif kind == "pool" and prev >= 4 and layers[-1].type_layer == capi.LAYER_FC:
            kernel, stride = int(rng.integers(2, 4)), int(rng.integers(1, 3))
            which = capi.LAYER_MAX_POOLING if rng.random() < 0.5 else capi.LAYER_AVERAGE_POOLING
            layers.append(capi.pooling(which, kernel, stride, padding=int(rng.integers(0, 2)), ceil_mode=bool(rng.random() < 0.5)))
            layers.append(capi.fc(width(), af))      # a fully connected layer reads the pooled units
            prev = layers[-1].unit_parameters[0]
        elif kind == "block" and layers[-1].type_layer == capi.LAYER_FC:
            inner = prev if rng.random() < 0.5 else width()
            shake = rng.random() < 0.5
            layers.append(capi.residual(2, capi.DROP_SHAKEDROP if shake else capi.DROP_NONE, (0.5, 0.0, 0.0) if shake else (0.0, 0.0, 0.0)))
            layers.append(capi.fc(inner, af))
            layers.append(capi.fc(inner, af, norm))
            layers.append(capi.fc(width(), af))      # a plain layer closes the stretch after a block
            prev = layers[-1].unit_parameters[0]
    softmax = rng.random() < 0.5
    layers.append(capi.fc(width(), capi.AF_SOFTMAX if softmax else capi.AF_LINEAR))
    desc = capi.net(layers, batch=batch or int(rng.integers(2, 9)), loss=capi.LOSS_CE if softmax else capi.LOSS_MSE,
                    accuracy=capi.ACC_CE if softmax else capi.ACC_DISTANCE)
    kind = int(rng.choice(optimizers))
    opt = capi.opt(kind, lr=float(np.float32(rng.uniform(1e-4, 1e-2))), weight_decay=float(np.float32(rng.choice([0.0, 1e-4]))),
                   clip=float(np.float32(rng.uniform(0.5, 2.0))) if rng.random() < 0.3 else None,
                   momentum=float(np.float32(rng.choice([0.0, 0.9]))), nesterov=bool(rng.random() < 0.3))
    return desc, opt, layers


@pytest.mark.parametrize("seed", range(40))
def test_random_architecture_files_equal_the_reference_writers(seed, tmp_path):
    desc, opt, layers = _random_network(seed)
    net = ref.RefNet(desc, opt, threads=1)
    try:
        P, _, _, units = net.sizes()
        rng = np.random.default_rng(1000 + seed)
        net.set(capi.BUF_PARAMETERS, rng.standard_normal(P).astype(np.float32))
        if units:
            net.set(capi.BUF_NORM_MEAN_AVERAGE, rng.standard_normal(units).astype(np.float32))
            net.set(capi.BUF_NORM_VARIANCE_AVERAGE, (rng.random(units) + 0.5).astype(np.float32))
        params = net.get(capi.BUF_PARAMETERS).copy()
        mean = net.get(capi.BUF_NORM_MEAN_AVERAGE)[:units].copy() if units else None
        sigma = net.get(capi.BUF_NORM_VARIANCE_AVERAGE)[:units].copy() if units else None
        r_nn, r_net, m_nn, m_net = [tmp_path / f for f in ("r.nn", "r.net", "m.nn", "m.net")]
        net.save(r_nn, r_net)
    finally:
        net.close()
    checkpoint.format_files(desc, opt, params, mean, sigma, m_nn, m_net)
    assert m_nn.read_bytes() == r_nn.read_bytes()
    assert m_net.read_bytes() == r_net.read_bytes()
    # and what was written parses back: same layer list, same arrays wherever the file carries them
    got_desc, got_opt, p, m, s = checkpoint.parse(m_nn, m_net, batch=desc.batch_size)
    assert got_desc.number_layers == desc.number_layers
    for l in range(desc.number_layers):
        assert got_desc.layers[l].type_layer == desc.layers[l].type_layer
        assert got_desc.layers[l].type_normalization == desc.layers[l].type_normalization
        assert got_desc.layers[l].type_dropout == desc.layers[l].type_dropout
    again_nn, again_net = tmp_path / "again.nn", tmp_path / "again.net"
    checkpoint.format_files(got_desc, got_opt, p, m, s, again_nn, again_net)
    assert again_nn.read_bytes() == m_nn.read_bytes()
    assert again_net.read_bytes() == m_net.read_bytes()


def _random_recurrent_network(seed):
    """LSTM layers (1 - 3 cells per block, zoneout or not), independently recurrent layers and fully connected layers
    between them; every layer above an LSTM layer is at least as wide as the LSTM has cells (the reference shifts an
    LSTM layer's bias base by its cell count)"""
    rng = np.random.default_rng(500 + seed)
    layers = [capi.fc(int(rng.integers(3, 12)))]
    widest = 0
    for _ in range(int(rng.integers(1, 4))):
        kind = rng.choice(["lstm", "lstm", "ind", "fc"])
        if kind == "lstm":
            blocks, cells = int(rng.integers(2, 7)), int(rng.integers(1, 4))
            zone = rng.random() < 0.5
            layers.append(capi.lstm(blocks, cells, dropout=capi.DROP_ZONEOUT if zone else capi.DROP_NONE,
                                    p=(float(np.float32(rng.uniform(0.05, 0.4))), float(np.float32(rng.uniform(0.05, 0.4))), 0.0) if zone else (0.0, 0.0, 0.0)))
            widest = max(widest, blocks * cells)
        elif kind == "ind":
            layers.append(capi.fc_ind_rnn(max(widest, int(rng.integers(3, 16))), int(rng.choice([capi.AF_RELU, capi.AF_TANH]))))
        else:
            layers.append(capi.fc(max(widest, int(rng.integers(3, 16))), int(rng.choice(ACTIVATIONS))))
    layers.append(capi.fc(max(widest, int(rng.integers(2, 10))), capi.AF_LINEAR))
    T = int(rng.integers(2, 6))
    clip = float(np.float32(rng.choice([0.5, 1.0, 4.0, 12.0]))) if rng.random() < 0.5 else None
    # the descriptor carries the object's clip_gradient member (the bound of independently recurrent weights follows it)
    desc = capi.net(layers, batch=int(rng.integers(2, 7)), T=T, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE, time_delays=int(rng.integers(0, T)),
                    clip_gradient=clip or 0.0)
    opt = capi.opt(int(rng.choice(OPTIMIZERS)), lr=float(np.float32(rng.uniform(1e-4, 1e-2))), clip=clip)
    return desc, opt


@pytest.mark.parametrize("seed", range(24))
def test_random_recurrent_architecture_files_equal_the_reference_writers(seed, tmp_path):
    desc, opt = _random_recurrent_network(seed)
    net = ref.RefNet(desc, opt, threads=1)
    try:
        P = net.sizes()[0]
        net.set(capi.BUF_PARAMETERS, np.random.default_rng(2000 + seed).standard_normal(P).astype(np.float32))
        params = net.get(capi.BUF_PARAMETERS).copy()
        r_nn, r_net, m_nn, m_net = [tmp_path / f for f in ("r.nn", "r.net", "m.nn", "m.net")]
        net.save(r_nn, r_net)
    finally:
        net.close()
    checkpoint.format_files(desc, opt, params, None, None, m_nn, m_net)
    assert m_nn.read_bytes() == r_nn.read_bytes()
    assert m_net.read_bytes() == r_net.read_bytes()
    got_desc, got_opt, p, m, s = checkpoint.parse(m_nn, m_net, batch=desc.batch_size)
    again_nn, again_net = tmp_path / "again.nn", tmp_path / "again.net"
    checkpoint.format_files(got_desc, got_opt, p, m, s, again_nn, again_net)
    assert again_nn.read_bytes() == m_nn.read_bytes()
    assert again_net.read_bytes() == m_net.read_bytes()
    # the dimension file alone (no general file to state clip_gradient): the bound of the independently recurrent
    # layers still comes back bit for bit
    alone_desc, _, p, m, s = checkpoint.parse(m_nn, None, batch=desc.batch_size)
    alone_nn = tmp_path / "alone.nn"
    checkpoint.format_files(alone_desc, got_opt, p, m, s, alone_nn, None)
    assert alone_nn.read_bytes() == m_nn.read_bytes()
