"""Test infrastructure, not product code.

numpy-friendly wrapper over oracle/_ref/libmyea_ref.so: the reference's own CPU implementation of the training
step, compiled unmodified by oracle/build_ref.sh and driven through oracle/ref_harness.cpp.  Method names mirror
myea_b200.net.Net so that a parity test can run the same script against both.
Only tests/, __graft_entry__.smoke() and the CPU-baseline leg of bench.py may import this module.
"""
import ctypes as C
import os

import numpy as np

from myea_b200 import capi

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libmyea_ref.so")
LIB_PATH_F64 = os.path.join(HERE, "_ref", "libmyea_ref_f64.so")   # the reference built with its COMPILE_DOUBLE switch
_LIBS = {}


def available(double=False):
    return os.path.exists(LIB_PATH_F64 if double else LIB_PATH)


def _lib(double=False):
    if double not in _LIBS:
        lib = C.CDLL(LIB_PATH_F64 if double else LIB_PATH)
        lib.ref_scalar_bytes.restype = C.c_int
        scalar = C.c_double if lib.ref_scalar_bytes() == 8 else C.c_float
        lib.scalar, lib.np_scalar = scalar, (np.float64 if scalar is C.c_double else np.float32)
        lib.ref_create.restype = C.c_void_p
        lib.ref_create.argtypes = [C.POINTER(capi.NetDesc), C.POINTER(capi.OptDesc), C.c_int]
        lib.ref_destroy.argtypes = [C.c_void_p]
        lib.ref_threads.argtypes = [C.c_void_p]
        lib.ref_sizes.argtypes = [C.c_void_p] + [C.POINTER(C.c_uint64)] * 4
        lib.ref_layer_index.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(capi.LayerIndex)]
        lib.ref_buffer.restype = C.POINTER(scalar)
        lib.ref_buffer.argtypes = [C.c_void_p, C.c_int]
        lib.ref_set_mask_bernoulli.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64]
        lib.ref_set_pre_training_level.argtypes = [C.c_void_p, C.c_uint64]
        lib.ref_set_mask_zoneout.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint64]
        lib.ref_set_training.argtypes = [C.c_void_p, C.c_int]
        lib.ref_load_batch.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]
        lib.ref_run.argtypes = [C.c_void_p, C.c_uint64, C.c_int]
        lib.ref_merge_derivatives.argtypes = [C.c_void_p]
        lib.ref_update_parameter.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(capi.OptDesc)]
        lib.ref_reset_loss.argtypes = [C.c_void_p]
        lib.ref_get_loss.argtypes = [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.POINTER(C.c_double)]
        lib.ref_get_outputs.argtypes = [C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p]
        lib.ref_get_errors.argtypes = [C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p]
        lib.ref_shakedrop_replay.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.ref_save.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p]
        lib.ref_load.restype = C.c_void_p
        lib.ref_load.argtypes = [C.c_char_p, C.c_char_p]
        lib.ref_layer_state.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(capi.LayerDesc)]
        lib.ref_general_state.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_uint64)]
        lib.ref_time_steps.restype = C.c_double
        lib.ref_time_steps.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_int, C.c_int]
        _LIBS[double] = lib
    return _LIBS[double]


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class RefNet:
    def __init__(self, desc, opt, threads=1, double=False):
        """double=True: the COMPILE_DOUBLE build of the same sources; buffers, outputs and errors are float64 arrays then"""
        self.lib = _lib(double)
        self.desc, self.opt = desc, opt
        self.h = self.lib.ref_create(C.byref(desc), C.byref(opt), threads)
        if not self.h:
            raise RuntimeError("reference Compile / Set__* failed for this descriptor")
        self.T = int(desc.number_recurrent_depth)
        self.B = int(desc.batch_size)
        self.P, self.W, self.n_bias, self.n_norm = self.sizes()
        self.threads = self.lib.ref_threads(self.h)

    @classmethod
    def load(cls, path_dimension, path_general):
        """the reference's own Load (Neural_Network__Load.cpp:2323) into a fresh object (buffers and state queries only)"""
        self = cls.__new__(cls)
        self.lib = _lib()
        self.h = self.lib.ref_load(str(path_dimension).encode(), str(path_general).encode())
        if not self.h:
            raise RuntimeError("the reference's Load rejected the files")
        self.P, self.W, self.n_bias, self.n_norm = self.sizes()
        self.T = self.B = 1
        self.threads = 1
        return self

    def save(self, path_dimension, path_general=None):
        """the reference's own Save_Dimension_Parameters / Save_General_Parameters (Neural_Network__Save.cpp:204, :23)"""
        if self.lib.ref_save(self.h, str(path_dimension).encode(), None if path_general is None else str(path_general).encode()) != 0:
            raise RuntimeError("the reference's Save_* failed")

    def layer_state(self, layer):
        d = capi.LayerDesc()
        if self.lib.ref_layer_state(self.h, layer, C.byref(d)) != 0:
            raise IndexError(layer)
        return d

    def general_state(self):
        v, u = (C.c_float * 12)(), (C.c_uint64 * 8)()
        self.lib.ref_general_state(self.h, v, u)
        return list(v), list(u)

    def close(self):
        if self.h:
            self.lib.ref_destroy(self.h)
            self.h = None

    def sizes(self):
        v = [C.c_uint64() for _ in range(4)]
        self.lib.ref_sizes(self.h, *[C.byref(x) for x in v])
        return tuple(int(x.value) for x in v)

    def layer_index(self, layer):
        li = capi.LayerIndex()
        if self.lib.ref_layer_index(self.h, layer, C.byref(li)) != 0:
            raise RuntimeError("bad layer")
        return li

    def _buf(self, which, count):
        p = self.lib.ref_buffer(self.h, which)
        if not p:
            raise RuntimeError("reference buffer %d is not allocated" % which)
        return np.ctypeslib.as_array(p, shape=(count,))

    def _count(self, which):
        return self.n_norm * self.T if which in (capi.BUF_NORM_MEAN_AVERAGE, capi.BUF_NORM_VARIANCE_AVERAGE) else self.P

    def get(self, which):
        return self._buf(which, self._count(which)).copy()

    def set(self, which, arr):
        a = np.ascontiguousarray(arr, dtype=self.lib.np_scalar).ravel()
        self._buf(which, a.size)[:] = a

    def set_mask_bernoulli(self, layer, mask):
        m = np.ascontiguousarray(mask, dtype=np.uint8).ravel()
        if self.lib.ref_set_mask_bernoulli(self.h, layer, m.ctypes.data, m.size) != 0:
            raise RuntimeError("layer %d has no Bernoulli mask" % layer)

    def set_mask_zoneout(self, layer, state, output):
        s = np.ascontiguousarray(state, dtype=np.uint8).ravel()
        o = np.ascontiguousarray(output, dtype=np.uint8).ravel()
        if self.lib.ref_set_mask_zoneout(self.h, layer, s.ctypes.data, o.ctypes.data, s.size) != 0:
            raise RuntimeError("layer %d has no zoneout mask" % layer)

    def forward(self, X, training=True, batch=None):
        X = _f32(X)
        self.active_B = int(batch or self.B)   # Forward_Pass(batch_size_received, ...): any batch up to the allocated one
        self.lib.ref_set_training(self.h, 1 if training else 0)
        self.lib.ref_load_batch(self.h, self.active_B, X.ctypes.data, None)
        self.lib.ref_run(self.h, self.active_B, 1)

    def compute_error(self, Y):
        Y = _f32(Y)
        b = getattr(self, "active_B", self.B)
        self.lib.ref_load_batch(self.h, b, None, Y.ctypes.data)
        self.lib.ref_run(self.h, b, 2)

    def backward(self):
        self.lib.ref_run(self.h, getattr(self, "active_B", self.B), 4)

    def update_derivative_weight(self):
        self.lib.ref_run(self.h, getattr(self, "active_B", self.B), 8)
        self.lib.ref_merge_derivatives(self.h)

    def update_parameter(self, training_size=None, opt=None, batch=None):
        o = opt or self.opt
        self.lib.ref_update_parameter(self.h, batch or self.B, training_size or self.B, C.byref(o))

    def reset_loss(self):
        self.lib.ref_reset_loss(self.h)

    def loss(self):
        s, n, a = C.c_double(), C.c_uint64(), C.c_double()
        self.lib.ref_get_loss(self.h, C.byref(s), C.byref(n), C.byref(a))
        return s.value, int(n.value), a.value

    def outputs(self, layer):
        w = int(self.layer_index(layer).number_outputs)
        out = np.empty((self.T, self.B, w), self.lib.np_scalar)
        self.lib.ref_get_outputs(self.h, layer, self.B, out.ctypes.data)
        return out

    def errors(self, layer):
        w = int(self.layer_index(layer).number_outputs)
        out = np.empty((self.T, self.B, w), self.lib.np_scalar)
        if self.lib.ref_get_errors(self.h, layer, self.B, out.ctypes.data) != 0:
            raise RuntimeError("layer %d has no error buffer" % layer)
        return out

    def set_pre_training_level(self, level):
        if self.lib.ref_set_pre_training_level(self.h, int(level)) != 0:
            raise RuntimeError("Set__Pre_Training_Level(%d) failed" % level)

    def next_shakedrop(self):
        """{residual layer: (mask[B], alpha[B, width], beta[B, width])} the reference will draw in its NEXT training step.
        Copies of the generators of thread 0 are replayed: an object that is to be compared row by row with another
        implementation is created with threads=1 (with more threads every thread draws for its own rows)."""
        layers = [l for l in range(1, int(self.desc.number_layers))
                  if self.desc.layers[l].type_layer == capi.LAYER_RESIDUAL and self.desc.layers[l].type_dropout == capi.DROP_SHAKEDROP]
        if not layers:
            return {}
        widths = [int(self.layer_index(l).number_outputs) for l in layers]
        total = sum(self.B * w for w in widths)
        masks = np.zeros(len(layers) * self.B, np.uint8)
        alpha, beta = np.zeros(total, np.float32), np.zeros(total, np.float32)
        n = self.lib.ref_shakedrop_replay(self.h, self.B, masks.ctypes.data, alpha.ctypes.data, beta.ctypes.data)
        if n != len(layers):
            raise RuntimeError("ShakeDrop replay found %d blocks, expected %d" % (n, len(layers)))
        out, off = {}, 0
        for k, (l, w) in enumerate(zip(layers, widths)):
            out[l] = (masks[k * self.B:(k + 1) * self.B].copy(), alpha[off:off + self.B * w].reshape(self.B, w).copy(),
                      beta[off:off + self.B * w].reshape(self.B, w).copy())
            off += self.B * w
        return out

    def time_steps(self, X, Y, warmup, steps, training_size=None):
        """milliseconds for `steps` whole training steps on (X, Y)"""
        X, Y = _f32(X), _f32(Y)
        self.lib.ref_set_training(self.h, 1)
        self.lib.ref_load_batch(self.h, self.B, X.ctypes.data, Y.ctypes.data)
        return self.lib.ref_time_steps(self.h, self.B, training_size or self.B, warmup, steps)
