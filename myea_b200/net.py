"""numpy-facing wrapper over the C ABI (include/myea_b200.h): one `Net` = one `Neural_Network` object of the
reference on one GPU.  Method names follow the reference's member functions (Forward_Pass -> forward, Compute__Error ->
compute_error, Backward_Pass -> backward, Update_Derivative_Weight -> update_derivative_weight, Update_Parameter ->
update_parameter); every method is a thin call into libmyea_b200.so and raises RuntimeError with the library's
message when the status is not MYEA_OK.  There is no CPU path: without the library or without a GPU it raises.
"""
import ctypes as C

import numpy as np

from . import capi


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Net:
    def __init__(self, desc, opt=None, device=0):
        self.lib = capi.load()
        self.desc, self.opt = desc, opt
        self.h = C.c_void_p()
        rc = self.lib.myea_b200_create(C.byref(self.h), C.byref(desc), device)
        if rc != 0:
            msg = self.lib.myea_b200_last_error(self.h).decode() if self.h else "no CUDA device / invalid descriptor"
            if self.h:
                self.lib.myea_b200_destroy(self.h)
                self.h = None
            raise RuntimeError("myea_b200_create failed (%d): %s" % (rc, msg))
        self.T = int(desc.number_recurrent_depth)
        self.B = int(desc.batch_size)
        self.P, self.W, self.n_bias, self.n_norm = self.sizes()

    @classmethod
    def load(cls, path_dimension, path_general, batch, device=0):
        """Neural_Network::Load (Neural_Network__Load.cpp:2323): the network the reference's `.nn` / `.net` files describe,
        built for `batch` rows with parameters and normalization averages uploaded; .opt holds the optimizer settings"""
        self = cls.__new__(cls)
        self.lib = capi.load()
        self.h = C.c_void_p()
        opt = capi.OptDesc()
        rc = self.lib.myea_b200_load(C.byref(self.h), str(path_dimension).encode(), str(path_general).encode(), int(batch), device, C.byref(opt))
        if rc != 0:
            msg = self.lib.myea_b200_checkpoint_last_error().decode() or (self.lib.myea_b200_last_error(self.h).decode() if self.h else "")
            if self.h:
                self.lib.myea_b200_destroy(self.h)
            self.h = None
            raise RuntimeError("myea_b200_load failed (%d): %s" % (rc, msg))
        from . import checkpoint
        self.desc = checkpoint.parse(path_dimension, path_general, batch, arrays=False)[0]
        self.opt = opt
        self.T = int(self.desc.number_recurrent_depth)
        self.B = int(batch)
        self.P, self.W, self.n_bias, self.n_norm = self.sizes()
        return self

    def save(self, path_dimension, path_general=None, opt=None):
        """Save_Dimension_Parameters / Save_General_Parameters (Neural_Network__Save.cpp:204, :23)"""
        self._ck(self.lib.myea_b200_save_dimension_parameters(self.h, str(path_dimension).encode()), "save_dimension_parameters")
        if path_general is not None:
            self._ck(self.lib.myea_b200_save_general_parameters(self.h, C.byref(opt or self.opt), str(path_general).encode()), "save_general_parameters")

    def _ck(self, rc, what):
        if rc != 0:
            raise RuntimeError("%s failed (%d): %s" % (what, rc, self.lib.myea_b200_last_error(self.h).decode()))

    def close(self):
        if self.h:
            self.lib.myea_b200_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sizes(self):
        v = [C.c_uint64() for _ in range(4)]
        self._ck(self.lib.myea_b200_sizes(self.h, *[C.byref(x) for x in v]), "sizes")
        return tuple(int(x.value) for x in v)

    def layer_index(self, layer):
        li = capi.LayerIndex()
        self._ck(self.lib.myea_b200_layer_index(self.h, layer, C.byref(li)), "layer_index")
        return li

    def _count(self, which):
        return self.n_norm * self.T if which in (capi.BUF_NORM_MEAN_AVERAGE, capi.BUF_NORM_VARIANCE_AVERAGE) else self.P

    def get(self, which):
        out = np.empty(self._count(which), np.float32)
        self._ck(self.lib.myea_b200_download(self.h, which, out.ctypes.data, 0, out.size), "download")
        return out

    def set(self, which, arr):
        a = _f32(arr).ravel()
        self._ck(self.lib.myea_b200_upload(self.h, which, a.ctypes.data, 0, a.size), "upload")

    def set_mask_bernoulli(self, layer, mask):
        m = np.ascontiguousarray(mask, dtype=np.uint8).ravel()
        self._ck(self.lib.myea_b200_set_mask_bernoulli(self.h, layer, m.ctypes.data, m.size), "set_mask_bernoulli")

    def set_mask_zoneout(self, layer, state, output):
        s = np.ascontiguousarray(state, dtype=np.uint8).ravel()
        o = np.ascontiguousarray(output, dtype=np.uint8).ravel()
        self._ck(self.lib.myea_b200_set_mask_zoneout(self.h, layer, s.ctypes.data, o.ctypes.data, s.size), "set_mask_zoneout")

    def set_pre_training_level(self, level):
        """0 = the whole network; k >= 1 = train hidden layer k and its mirror image as one autoencoder pair"""
        self._ck(self.lib.myea_b200_set_pre_training_level(self.h, int(level)), "set_pre_training_level")

    def set_shakedrop(self, layer, mask, alpha, beta):
        m = np.ascontiguousarray(mask, dtype=np.uint8).ravel()
        a, b = _f32(alpha), _f32(beta)
        self._ck(self.lib.myea_b200_set_shakedrop(self.h, layer, m.ctypes.data, a.ctypes.data, b.ctypes.data, m.size), "set_shakedrop")

    def dataset_set(self, X, Y):
        """X: [N, T*inputs], Y: [N, T*outputs] example-major rows; kept on the device"""
        X, Y = _f32(X), _f32(Y)
        self._ck(self.lib.myea_b200_dataset_set(self.h, X.shape[0], X.ctypes.data, Y.ctypes.data), "dataset_set")

    def train_epoch(self, order, mini_batch, opt=None, mask_seed=0, first_step=0):
        order = np.ascontiguousarray(order, dtype=np.uint64)
        loss, acc = C.c_double(), C.c_double()
        self._ck(self.lib.myea_b200_train_epoch(self.h, order.ctypes.data, order.size, mini_batch, C.byref(opt or self.opt), mask_seed, first_step,
                                                C.byref(loss), C.byref(acc)), "train_epoch")
        return loss.value, acc.value

    def evaluate(self, n, order=None):
        o = None if order is None else np.ascontiguousarray(order, dtype=np.uint64)
        loss, ls, nl, acc = C.c_double(), C.c_double(), C.c_uint64(), C.c_double()
        self._ck(self.lib.myea_b200_evaluate(self.h, None if o is None else o.ctypes.data, n, C.byref(loss), C.byref(ls), C.byref(nl), C.byref(acc)),
                 "evaluate")
        return loss.value, ls.value, nl.value, acc.value

    def generate_masks(self, seed, step):
        """fills every dropout / zoneout / ShakeDrop array on the device from the counter-based generator"""
        self._ck(self.lib.myea_b200_generate_masks(self.h, int(seed), int(step)), "generate_masks")

    def download_mask(self, layer, kind, shape):
        out = np.zeros(shape, np.float32 if kind in (capi.MASK_SHAKEDROP_ALPHA, capi.MASK_SHAKEDROP_BETA) else np.uint8)
        self._ck(self.lib.myea_b200_download_mask(self.h, layer, kind, out.ctypes.data, out.nbytes), "download_mask")
        return out

    def forward(self, X, training=True, batch=None):
        """X: [T, batch, inputs]; `batch` below the allocated batch size is allowed for feed-forward networks"""
        X = _f32(X)
        self.active_B = int(batch or self.B)
        self._ck(self.lib.myea_b200_forward(self.h, self.active_B, X.ctypes.data, 1 if training else 0), "forward")

    def compute_error(self, Y):
        Y = _f32(Y)
        self._ck(self.lib.myea_b200_compute_error(self.h, getattr(self, "active_B", self.B), Y.ctypes.data), "compute_error")

    def backward(self):
        self._ck(self.lib.myea_b200_backward(self.h, getattr(self, "active_B", self.B)), "backward")

    def update_derivative_weight(self):
        self._ck(self.lib.myea_b200_update_derivative_weight(self.h, getattr(self, "active_B", self.B)), "update_derivative_weight")

    def update_parameter(self, training_size=None, opt=None, batch=None):
        o = opt or self.opt
        self._ck(self.lib.myea_b200_update_parameter(self.h, batch or self.B, training_size or self.B, C.byref(o)), "update_parameter")

    def clear_training_arrays(self):
        self._ck(self.lib.myea_b200_clear_training_arrays(self.h), "clear_training_arrays")

    def reset_loss(self):
        self._ck(self.lib.myea_b200_reset_loss(self.h), "reset_loss")

    def loss(self):
        s, n, a = C.c_double(), C.c_uint64(), C.c_double()
        self._ck(self.lib.myea_b200_get_loss(self.h, C.byref(s), C.byref(n), C.byref(a)), "get_loss")
        return s.value, int(n.value), a.value

    def outputs(self, layer):
        w = int(self.layer_index(layer).number_outputs)
        out = np.empty((self.T, self.B, w), np.float32)
        self._ck(self.lib.myea_b200_get_outputs(self.h, layer, out.ctypes.data, out.size), "get_outputs")
        return out

    def errors(self, layer):
        w = int(self.layer_index(layer).number_outputs)
        out = np.empty((self.T, self.B, w), np.float32)
        self._ck(self.lib.myea_b200_get_errors(self.h, layer, out.ctypes.data, out.size), "get_errors")
        return out

    def synchronize(self):
        self._ck(self.lib.myea_b200_synchronize(self.h), "synchronize")

    def launches(self):
        return int(self.lib.myea_b200_kernel_launches(self.h))

    def profile(self, enable):
        self._ck(self.lib.myea_b200_profile(self.h, 1 if enable else 0), "profile")

    def profile_read(self, reset=True):
        ms = (C.c_double * capi.TIMER_CLASSES)()
        ln = (C.c_uint64 * capi.TIMER_CLASSES)()
        fl = (C.c_double * 1)()
        self._ck(self.lib.myea_b200_profile_read(self.h, ms, ln, fl, 1 if reset else 0), "profile_read")
        return list(ms), [int(x) for x in ln], fl[0]
