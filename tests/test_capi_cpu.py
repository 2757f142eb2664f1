"""CPU tests of the boundary: the C-ABI library loads without a GPU, exports every symbol the header declares, the
ctypes structs have the header's layout, and compute entry points fail loudly (no CPU fallback) without a device."""
import ctypes as C
import os
import re

import pytest

from myea_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header():
    with open(os.path.join(ROOT, "include", "myea_b200.h")) as f:
        return f.read()


def test_library_is_built():
    assert os.path.exists(capi.LIB_PATH), "build with: python -c 'import __graft_entry__ as g; g.build()'"


def test_every_declared_symbol_is_exported():
    declared = sorted(set(re.findall(r"\b(myea_b200_[a-z0-9_]+)\s*\(", _header())))
    assert declared == capi.exported_symbols()
    lib = C.CDLL(capi.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name


def test_struct_layouts_match_header():
    # sizes implied by the header's field lists on an LP64 ABI
    assert C.sizeof(capi.LayerDesc) == 4 + 4 + 5 * 8 + 4 * 4 + 3 * 4 + 4
    assert C.sizeof(capi.NetDesc) == 4 + 4 + 8 * 3 + 4 * 2 + 4 * 5 + 4 + capi.MAX_LAYERS * C.sizeof(capi.LayerDesc)
    assert C.sizeof(capi.OptDesc) == 27 * 4
    assert C.sizeof(capi.LayerIndex) == 10 * 8


def test_enumerators_match_header():
    h = _header()
    for macro, value in (("MYEA_LAYER_FULLY_CONNECTED", capi.LAYER_FC), ("MYEA_LAYER_LSTM", capi.LAYER_LSTM),
                         ("MYEA_LAYER_RESIDUAL", capi.LAYER_RESIDUAL), ("MYEA_AF_TANH", capi.AF_TANH), ("MYEA_AF_RELU", capi.AF_RELU),
                         ("MYEA_AF_SOFTMAX", capi.AF_SOFTMAX), ("MYEA_OPT_ADAM", capi.OPT_ADAM), ("MYEA_OPT_AMSGRAD", capi.OPT_AMSGRAD),
                         ("MYEA_OPT_ADABOUND", capi.OPT_ADABOUND), ("MYEA_OPT_NOSADAM", capi.OPT_NOSADAM), ("MYEA_OPT_IRPROP_PLUS", capi.OPT_IRPROP_PLUS), ("MYEA_LOSS_MSE", capi.LOSS_MSE), ("MYEA_DROPOUT_ZONEOUT", capi.DROP_ZONEOUT),
                         ("MYEA_AF_COSINE", capi.AF_COSINE), ("MYEA_AF_ELLIOT_SYMMETRIC", capi.AF_ELLIOT_SYMMETRIC), ("MYEA_AF_GAUSSIAN_STEPWISE", capi.AF_GAUSSIAN_STEPWISE),
                         ("MYEA_AF_ISRLU", capi.AF_ISRLU), ("MYEA_AF_LINEAR_PIECE_SYMMETRIC", capi.AF_LINEAR_PIECE_SYMMETRIC), ("MYEA_AF_PARAMETRIC_RELU", capi.AF_PARAMETRIC_RELU),
                         ("MYEA_AF_SIGMOID_STEPWISE", capi.AF_SIGMOID_STEPWISE), ("MYEA_AF_SINE_SYMMETRIC", capi.AF_SINE_SYMMETRIC), ("MYEA_AF_TANH_STEPWISE", capi.AF_TANH_STEPWISE),
                         ("MYEA_AF_THRESHOLD_SYMMETRIC", capi.AF_THRESHOLD_SYMMETRIC)):
        m = re.search(r"#define\s+%s\s+(\d+)u?" % macro, h)
        assert m and int(m.group(1)) == value, macro


def test_create_without_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = capi.load()
    d = capi.net([capi.fc(4), capi.fc(3)], batch=2)
    h = C.c_void_p()
    rc = lib.myea_b200_create(C.byref(h), C.byref(d), 0)
    assert rc != 0 and not h        # MYEA_E_CUDA: there is no CPU path to fall back to


def test_invalid_arguments_are_rejected_without_touching_a_device():
    lib = capi.load()
    h = C.c_void_p()
    assert lib.myea_b200_create(C.byref(h), None, 0) == -1
    d = capi.net([capi.fc(4)], batch=2)    # a single layer is not a network
    assert lib.myea_b200_create(C.byref(h), C.byref(d), 0) == -1
    assert lib.myea_b200_forward(None, 1, None, 1) == -1
    assert lib.myea_b200_update_parameter(None, 1, 1, None) == -1
