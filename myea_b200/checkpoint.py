"""Host-only halves of the checkpoint entry points: the reference's `.nn` (Save_Dimension_Parameters,
Neural_Network__Save.cpp:204) and `.net` (Save_General_Parameters, Save.cpp:23) text files written from and parsed
into plain arrays.  They run in the product library but touch no GPU, so tools and CPU-side tests can convert
checkpoints without a device.  Net.save / Net.load are the device-resident forms."""
import ctypes as C

import numpy as np

from . import capi


def _f32(a, n):
    a = np.ascontiguousarray(a if a is not None else np.zeros(max(n, 1)), dtype=np.float32)
    return a


def format_files(desc, opt, parameters, mean_average=None, variance_average=None, path_dimension=None, path_general=None):
    lib = capi.load()
    if path_dimension is not None:
        p = _f32(parameters, 0)
        m, s = _f32(mean_average, 1), _f32(variance_average, 1)
        rc = lib.myea_b200_checkpoint_format_dimension(C.byref(desc), p.ctypes.data, m.ctypes.data, s.ctypes.data, str(path_dimension).encode())
        if rc != 0:
            raise RuntimeError("checkpoint_format_dimension failed (%d)" % rc)
    if path_general is not None:
        rc = lib.myea_b200_checkpoint_format_general(C.byref(desc), C.byref(opt), str(path_general).encode())
        if rc != 0:
            raise RuntimeError("checkpoint_format_general failed (%d)" % rc)


def parse(path_dimension, path_general=None, batch=1, arrays=True):
    """-> (NetDesc, OptDesc, parameters, mean_average, variance_average); the arrays are None with arrays=False"""
    lib = capi.load()
    desc, opt = capi.NetDesc(), capi.OptDesc()
    P, U = C.c_uint64(), C.c_uint64()
    pg = None if path_general is None else str(path_general).encode()

    def call(p, cap, m, s, ncap):
        rc = lib.myea_b200_checkpoint_parse(str(path_dimension).encode(), pg, int(batch), C.byref(desc), C.byref(opt), p, cap, m, s, ncap,
                                            C.byref(P), C.byref(U))
        if rc != 0:
            raise RuntimeError("checkpoint_parse failed (%d): %s" % (rc, lib.myea_b200_checkpoint_last_error().decode()))

    call(None, 0, None, None, 0)
    if not arrays:
        return desc, opt, None, None, None
    params = np.zeros(P.value, np.float32)
    n = U.value * max(1, int(desc.number_recurrent_depth))      # running averages: one set per time step, [layer][T][units]
    mean, sigma = np.zeros(max(n, 1), np.float32), np.zeros(max(n, 1), np.float32)
    call(params.ctypes.data, P.value, mean.ctypes.data, sigma.ctypes.data, n)
    return desc, opt, params, mean[:n], sigma[:n]
