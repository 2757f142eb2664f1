"""Checkpoint files in the reference's text format (Save_Dimension_Parameters, Neural_Network__Save.cpp:204;
Save_General_Parameters, Save.cpp:23; Load, Neural_Network__Load.cpp:2323) through the host-only halves of the product
library's entry points, on the CPU:

  * the writer reproduces, byte for byte, the files the unmodified reference wrote for four trained networks
    (tests/golden/checkpoint, made by tests/golden/make_checkpoint_golden.py) from the parameters and running
    statistics the training fixtures hold for the same state,
  * the reader returns the description and every array from those reference-written files exactly,
  * write -> read -> write is the identity for every case, wide and oracle-only ones included,
  * where the compiled reference is present: both writers agree byte for byte on every case, the reference's own
    Load accepts the files written here and ends with bit-identical parameters, layer settings and optimizer
    settings, and files the reference writes load here.

Integer and text work: the bar is exact equality everywhere (floats round-trip through "%.16g")."""
import gzip
import os
import tempfile

import numpy as np
import pytest

import cases
from myea_b200 import capi, checkpoint
from oracle import ref

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FIXTURES = ["mlp_brn_elu_adabound_wd", "mlp_tanh_nesterov_ce", "lstm2_zoneout_clip", "res_bn_tanh_adam_noshake"]
ALL = sorted(cases.CASES) + sorted(cases.CASES_ORACLE_ONLY)


def _case(name):
    return (cases.CASES.get(name) or cases.CASES_ORACLE_ONLY[name])()


def _fixture(name):
    with gzip.open(os.path.join(GOLD, "checkpoint", name + ".nn.gz"), "rb") as f:
        nn = f.read()
    with open(os.path.join(GOLD, "checkpoint", name + ".net"), "rb") as f:
        general = f.read()
    return nn, general


def _trained_state(name):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    P, _, _, units = [int(v) for v in g["sizes"]]
    mean = g["norm_mean_avg"] if units else None      # units x time steps values
    sigma = g["norm_sigma_avg"] if units else None
    return g["param1"][:P], mean, sigma


def _saved_mask(desc, index_of, P):
    """parameters the file carries: everything except (a) the cell-input bias slots of LSTM layers, which the
    reference's writer skips (it lists 3 * blocks values from the index already shifted by the cell count) and (b) the
    scale / shift slots the reference allocates for layers that are not normalized (input, residual, output layers
    and plain hidden ones once any layer is normalized), which no code reads"""
    keep = np.ones(P, bool)
    for l in range(desc.number_layers):
        li = index_of(l)
        if desc.layers[l].type_layer == capi.LAYER_LSTM:
            cells = int(li.number_outputs)
            keep[int(li.first_bias_connection_index) - cells:int(li.first_bias_connection_index)] = False
        if desc.layers[l].type_normalization == capi.NORM_NONE and int(li.number_units_norm):
            keep[int(li.scale_index):int(li.scale_index) + int(li.number_units_norm)] = False
            keep[int(li.shift_index):int(li.shift_index) + int(li.number_units_norm)] = False
    return keep


def _desc_tuple(d, general=True):
    net = (d.number_layers, d.type_network, d.number_recurrent_depth, d.number_time_delays)
    if general:
        net += (d.type_loss_function, d.type_accuracy_function)
    layers = []
    for l in range(d.number_layers):
        L = d.layers[l]
        drop = tuple(L.dropout_values) if L.type_dropout != capi.DROP_NONE else (0.0, 0.0, 0.0)
        layers.append((L.type_layer, L.use_bidirectional, L.unit_parameters[0], L.unit_parameters[1] if L.type_layer == capi.LAYER_LSTM else 0,
                       L.type_normalization, L.type_dropout, drop))
    return net, layers


@pytest.mark.parametrize("name", FIXTURES)
def test_writer_reproduces_reference_files(name, tmp_path):
    wl = _case(name)
    params, mean, sigma = _trained_state(name)
    nn, general = tmp_path / "a.nn", tmp_path / "a.net"
    checkpoint.format_files(wl.desc, wl.opt, params, mean, sigma, nn, general)
    want_nn, want_general = _fixture(name)
    assert nn.read_bytes() == want_nn
    assert general.read_bytes() == want_general


@pytest.mark.parametrize("name", FIXTURES)
def test_reader_on_reference_files(name, tmp_path):
    wl = _case(name)
    want_nn, want_general = _fixture(name)
    nn, general = tmp_path / "r.nn", tmp_path / "r.net"
    nn.write_bytes(want_nn)
    general.write_bytes(want_general)
    desc, opt, params, mean, sigma = checkpoint.parse(nn, general, batch=wl.desc.batch_size)
    assert _desc_tuple(desc) == _desc_tuple(wl.desc)
    assert desc.batch_size == wl.desc.batch_size
    want, want_mean, want_sigma = _trained_state(name)
    g = np.load(os.path.join(GOLD, name + ".npz"))

    class Index:
        def __init__(self, row):
            (self.first_connection_index, self.last_connection_index, self.first_bias_connection_index, self.last_bias_connection_index,
             self.scale_index, self.shift_index, self.number_inputs, self.number_outputs, self.block_stride, self.number_units_norm) = [int(v) for v in row]

    keep = _saved_mask(desc, lambda l: Index(g["index_map"][l]), want.size)
    assert params.size == want.size
    assert np.array_equal(params[keep], want[keep])
    if want_mean is not None:
        # running statistics exist in the file for normalized layers only; the others hold the allocation values 0 / 1
        for l in range(1, desc.number_layers):
            if desc.layers[l].type_normalization != capi.NORM_NONE:
                li = Index(g["index_map"][l])
                lo = li.scale_index - (want.size - 2 * mean.size)
                assert np.array_equal(mean[lo:lo + li.number_units_norm], want_mean[lo:lo + li.number_units_norm])
                assert np.array_equal(sigma[lo:lo + li.number_units_norm], want_sigma[lo:lo + li.number_units_norm])
    # optimizer settings
    for f in ("type_optimizer_function", "use_adam_bias_correction", "learning_rate", "learning_momentum", "use_nesterov", "adam_learning_rate",
              "adam_beta1", "adam_beta2", "adam_epsilon", "learning_rate_final", "learning_gamma", "regularization__weight_decay",
              "use_normalized_weight_decay", "use_clip_gradient", "regularization__max_norm_constraints"):
        assert getattr(opt, f) == getattr(wl.opt, f), f
    # and the reader's arrays written again give the reference's bytes back
    again = tmp_path / "again.nn"
    checkpoint.format_files(desc, opt, params, mean, sigma, again, None)
    if not (~keep).any():
        assert again.read_bytes() == want_nn


@pytest.mark.parametrize("name", ALL)
def test_write_read_write_identity(name, tmp_path):
    wl = _case(name)
    rng = np.random.default_rng(11)
    a, b = tmp_path / "a.nn", tmp_path / "b.nn"
    ga, gb = tmp_path / "a.net", tmp_path / "b.net"
    # sizes come from a first parse of a file written with zeros
    checkpoint.format_files(wl.desc, wl.opt, np.zeros(1 << 22, np.float32), np.zeros(1 << 16, np.float32), np.zeros(1 << 16, np.float32), a, ga)
    desc, opt, p0, m0, s0 = checkpoint.parse(a, ga, batch=wl.desc.batch_size)
    params = rng.standard_normal(p0.size).astype(np.float32)
    params[::7] = np.float32(1e-30) * params[::7]          # tiny, huge and exactly representable values all survive the text
    params[1::13] = np.float32(3e30)
    mean = rng.standard_normal(m0.size).astype(np.float32)
    sigma = rng.random(s0.size).astype(np.float32) + 0.5
    checkpoint.format_files(wl.desc, wl.opt, params, mean, sigma, a, ga)
    desc, opt, p1, m1, s1 = checkpoint.parse(a, ga, batch=wl.desc.batch_size)
    checkpoint.format_files(desc, opt, p1, m1, s1, b, gb)
    assert a.read_bytes() == b.read_bytes()
    assert ga.read_bytes() == gb.read_bytes()
    assert _desc_tuple(desc) == _desc_tuple(wl.desc)


def test_reader_rejects_damaged_files(tmp_path):
    want_nn, want_general = _fixture("mlp_tanh_nesterov_ce")
    general = tmp_path / "g.net"
    general.write_bytes(want_general)
    cut = tmp_path / "cut.nn"
    cut.write_bytes(want_nn[:len(want_nn) // 2])
    with pytest.raises(RuntimeError):
        checkpoint.parse(cut, general)
    swapped = tmp_path / "swapped.nn"
    swapped.write_bytes(want_nn.replace(b"total_parameters ", b"total_parameters 1", 1))
    with pytest.raises(RuntimeError, match="totals"):
        checkpoint.parse(swapped, general)
    with pytest.raises(RuntimeError):
        checkpoint.parse(tmp_path / "missing.nn", general)
    with pytest.raises(RuntimeError):
        checkpoint.parse(general, general)          # a `.net` file where the `.nn` file belongs
    bidirectional = tmp_path / "bi.nn"
    lstm_nn, _ = _fixture("lstm2_zoneout_clip")
    bidirectional.write_bytes(lstm_nn.replace(b"use_bidirectional 0", b"use_bidirectional 1", 1))
    with pytest.raises(RuntimeError, match="-4"):
        checkpoint.parse(bidirectional, None)


needs_ref = pytest.mark.skipif(not ref.available(), reason="compiled reference (oracle/_ref) not present")


@needs_ref
@pytest.mark.parametrize("name", ALL)
def test_both_writers_agree_and_reference_loads_ours(name, tmp_path):
    wl = _case(name)
    net = ref.RefNet(wl.desc, wl.opt, threads=1)
    try:
        wl.materialize(net)
        params = net.get(capi.BUF_PARAMETERS).copy()
        units = net.sizes()[3]
        rng = np.random.default_rng(5)
        averages = units * max(1, int(wl.desc.number_recurrent_depth))    # one set per time step
        if units:                                    # non-trivial running statistics in the reference object itself
            net.set(capi.BUF_NORM_MEAN_AVERAGE, rng.standard_normal(averages).astype(np.float32))
            net.set(capi.BUF_NORM_VARIANCE_AVERAGE, (rng.random(averages) + 0.5).astype(np.float32))
        mean = net.get(capi.BUF_NORM_MEAN_AVERAGE)[:averages].copy() if units else None
        sigma = net.get(capi.BUF_NORM_VARIANCE_AVERAGE)[:averages].copy() if units else None
        r_nn, r_net, m_nn, m_net = [tmp_path / f for f in ("r.nn", "r.net", "m.nn", "m.net")]
        net.save(r_nn, r_net)
        checkpoint.format_files(wl.desc, wl.opt, params, mean, sigma, m_nn, m_net)
        assert m_nn.read_bytes() == r_nn.read_bytes()
        assert m_net.read_bytes() == r_net.read_bytes()
        keep = _saved_mask(wl.desc, net.layer_index, params.size)
    finally:
        net.close()
    # the reference's own loader on the files written here.  For networks with LSTM layers it rejects every file, its
    # own included: its writer omits `use_layer_normalization_before_activation` for those layers (Save.cpp:636-644)
    # and its reader insists on it (Load.cpp:5459); identical bytes are all that can be shown there.
    recurrent = any(wl.desc.layers[l].type_layer == capi.LAYER_LSTM for l in range(wl.desc.number_layers))
    if recurrent:
        with pytest.raises(RuntimeError):
            ref.RefNet.load(r_nn, r_net)
        desc, opt, p, m, s = checkpoint.parse(r_nn, r_net, batch=wl.desc.batch_size)
        assert np.array_equal(p[keep], params[keep])
        return
    loaded = ref.RefNet.load(m_nn, m_net)
    try:
        assert loaded.sizes() == (params.size,) + _totals(wl) + (units,)
        got = loaded.get(capi.BUF_PARAMETERS)
        assert np.array_equal(got[keep], params[keep])
        for l in range(1, wl.desc.number_layers):
            want, have = wl.desc.layers[l], loaded.layer_state(l)
            assert (have.type_layer, have.type_normalization, have.type_dropout) == (want.type_layer, want.type_normalization, want.type_dropout)
            if want.type_layer == capi.LAYER_FC and not _first_in_block(wl.desc, l):
                assert have.type_activation_function == want.type_activation_function
            if want.type_dropout != capi.DROP_NONE:
                assert tuple(have.dropout_values) == tuple(want.dropout_values)
        v, u = loaded.general_state()
        o = wl.opt
        assert u[0] == o.type_optimizer_function and u[1] == wl.desc.type_loss_function and u[2] == wl.desc.type_accuracy_function
        assert u[3] == o.use_nesterov and u[4] == o.use_clip_gradient and u[5] == wl.desc.type_network
        assert u[6] == wl.desc.number_recurrent_depth and u[7] == wl.desc.number_time_delays
        assert [np.float32(x) for x in v[:7]] == [np.float32(x) for x in (o.learning_rate, o.learning_momentum, o.adam_learning_rate, o.adam_beta1,
                                                                         o.adam_beta2, o.adam_epsilon, o.regularization__weight_decay)]
    finally:
        loaded.close()
    # and the reference's files parse here to the same arrays
    desc, opt, p, m, s = checkpoint.parse(r_nn, r_net, batch=wl.desc.batch_size)
    assert np.array_equal(p[keep], params[keep])
    assert _desc_tuple(desc) == _desc_tuple(wl.desc)


def _totals(wl):
    """(total_weights, total_bias) as the file written here states them"""
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "t.nn")
        checkpoint.format_files(wl.desc, wl.opt, np.zeros(1 << 22, np.float32), np.zeros(1 << 16, np.float32), np.zeros(1 << 16, np.float32), path, None)
        head = open(path, "rb").read(2000).split(b"\r\n")
    kv = dict(line.split(b" ", 1) for line in head if line.startswith(b"total_"))
    return int(kv[b"total_weights"]), int(kv[b"total_bias"])


def _first_in_block(desc, l):
    return desc.layers[l - 1].type_layer == capi.LAYER_RESIDUAL
