"""GPU tests of the device-side mask generation (myea_b200_generate_masks): every array bit for bit against the numpy
restatement of the counter-based generator, repeatability, and a training step that uses generated masks against the
compiled reference given the same (downloaded) masks."""
import numpy as np
import pytest

import cases
from conftest import rel_err
from myea_b200 import capi
from myea_b200.net import Net
from oracle import philox, ref

pytestmark = pytest.mark.gpu
SEED, STEP = 0x1234567890ABCDEF, 41


def _expected(wl, layer, L, T):
    """{kind: array} for one layer, from the restatement"""
    out = {}
    if L.type_layer == capi.LAYER_FC and L.type_dropout in (capi.DROP_BERNOULLI, capi.DROP_BERNOULLI_INVERTED):
        n = T * int(L.unit_parameters[0])
        out[capi.MASK_BERNOULLI] = philox.bernoulli_mask(SEED, STEP, layer, n, L.dropout_values[0])
    if L.type_layer == capi.LAYER_LSTM and L.type_dropout == capi.DROP_ZONEOUT:
        n = T * int(L.unit_parameters[0]) * (2 if L.use_bidirectional else 1)
        out[capi.MASK_ZONEOUT_STATE], out[capi.MASK_ZONEOUT_OUTPUT] = philox.zoneout_masks(SEED, STEP, layer, n, L.dropout_values[0], L.dropout_values[1])
    if L.type_layer == capi.LAYER_RESIDUAL and L.type_dropout == capi.DROP_SHAKEDROP:
        width = int(wl.layers[layer + int(L.unit_parameters[0])].unit_parameters[0])
        m, a, b = philox.shakedrop(SEED, STEP, layer, wl.B, width, L.dropout_values[0])
        out[capi.MASK_SHAKEDROP], out[capi.MASK_SHAKEDROP_ALPHA], out[capi.MASK_SHAKEDROP_BETA] = m, a.ravel(), b.ravel()
    return out


@pytest.mark.parametrize("name", ["c2_small", "mlp_bernoulli_amsbound_clip", "lstm2_zoneout_clip", "c5_small", "c4_small"])
def test_generated_arrays_match_the_restatement_bit_for_bit(name):
    wl = (cases.CASES.get(name) or cases.CASES_WITHOUT_REFERENCE[name])()
    gpu = Net(wl.desc, wl.opt)
    gpu.generate_masks(SEED, STEP)
    T = int(wl.desc.number_recurrent_depth) if hasattr(wl.desc, "number_recurrent_depth") else 1
    checked = 0
    for layer, L in enumerate(wl.layers):
        for kind, want in _expected(wl, layer, L, max(T, 1)).items():
            got = gpu.download_mask(layer, kind, want.shape)
            assert got.dtype == want.dtype and np.array_equal(got, want), (layer, kind)
            checked += 1
    assert checked > 0
    # the same coordinates give the same arrays; the next step gives different ones
    first = {(l, k): gpu.download_mask(l, k, w.shape) for l, L in enumerate(wl.layers) for k, w in _expected(wl, l, L, max(T, 1)).items()}
    gpu.generate_masks(SEED, STEP + 1)
    assert any(not np.array_equal(v, gpu.download_mask(l, k, v.shape)) for (l, k), v in first.items())
    gpu.generate_masks(SEED, STEP)
    assert all(np.array_equal(v, gpu.download_mask(l, k, v.shape)) for (l, k), v in first.items())
    gpu.close()


@pytest.mark.skipif(not ref.available(), reason="compiled reference not present")
def test_step_with_generated_masks_matches_reference_given_the_same_masks():
    wl = cases.CASES["c2_small"]()
    gpu, cpu = Net(wl.desc, wl.opt), ref.RefNet(wl.desc, wl.opt, threads=1)
    X, Y = wl.batch()
    wl.materialize(gpu); wl.materialize(cpu)
    gpu.generate_masks(SEED, STEP)
    for layer, L in enumerate(wl.layers):
        if L.type_dropout == capi.DROP_BERNOULLI_INVERTED:
            cpu.set_mask_bernoulli(layer, gpu.download_mask(layer, capi.MASK_BERNOULLI, (int(L.unit_parameters[0]),)))
    for net in (gpu, cpu):
        net.reset_loss(); net.forward(X); net.compute_error(Y); net.backward(); net.update_derivative_weight()
    assert rel_err(gpu.get(capi.BUF_DERIVATIVES), cpu.get(capi.BUF_DERIVATIVES)) < 1e-4
    gpu.close(); cpu.close()


def test_bad_arguments():
    wl = cases.CASES["c1_small"]()
    gpu = Net(wl.desc, wl.opt)
    gpu.generate_masks(1, 2)   # a network without masks: nothing to do, no error
    buf = np.zeros(4, np.uint8)
    assert gpu.lib.myea_b200_download_mask(gpu.h, 1, capi.MASK_BERNOULLI, buf.ctypes.data, 4) == -1
    assert gpu.lib.myea_b200_download_mask(gpu.h, 99, capi.MASK_BERNOULLI, buf.ctypes.data, 4) == -1
    gpu.close()
