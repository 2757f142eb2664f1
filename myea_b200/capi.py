"""ctypes view of include/myea_b200.h: the descriptor structs, the enumerator values and the library loader.

Nothing here computes; it is the Python-side declaration of the C ABI that the parity tests and bench.py call.
The product library is required: `load()` raises if `libmyea_b200.so` is missing (there is no CPU fallback).
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmyea_b200.so")

MAX_LAYERS = 64

# enumerators (values of the reference's enums, see include/myea_b200.h)
NET_AUTOENCODER = 1
LAYER_FC, LAYER_LSTM, LAYER_RESIDUAL = 4, 8, 10
LAYER_AVERAGE_POOLING, LAYER_MAX_POOLING = 1, 9
LAYER_FC_IND_RNN = 5
NET_FEEDFORWARD, NET_RECURRENT = 3, 4
AF_ELU, AF_LINEAR, AF_LEAKY_RELU, AF_RELU, AF_SELU, AF_SIGMOID, AF_SOFTMAX, AF_TANH = 3, 11, 14, 16, 17, 18, 22, 23
(AF_COSINE, AF_COSINE_SYMMETRIC, AF_ELLIOT, AF_ELLIOT_SYMMETRIC, AF_GAUSSIAN, AF_GAUSSIAN_STEPWISE, AF_GAUSSIAN_SYMMETRIC, AF_ISRU, AF_ISRLU,
 AF_LINEAR_PIECE, AF_LINEAR_PIECE_SYMMETRIC, AF_PARAMETRIC_RELU, AF_SINE, AF_SIGMOID_STEPWISE, AF_SINE_SYMMETRIC, AF_TANH_STEPWISE, AF_THRESHOLD,
 AF_THRESHOLD_SYMMETRIC) = 1, 2, 4, 5, 6, 7, 8, 9, 10, 12, 13, 15, 19, 20, 21, 24, 25, 26
NORM_NONE, NORM_BN, NORM_BRN = 0, 1, 2
MASK_BERNOULLI, MASK_ZONEOUT_STATE, MASK_ZONEOUT_OUTPUT, MASK_SHAKEDROP, MASK_SHAKEDROP_ALPHA, MASK_SHAKEDROP_BETA = range(6)
DROP_NONE, DROP_BERNOULLI, DROP_BERNOULLI_INVERTED, DROP_SHAKEDROP, DROP_ZONEOUT = 0, 2, 3, 5, 7
LOSS_CE, LOSS_MSE = 2, 10
ACC_NONE, ACC_CE, ACC_DISTANCE = 0, 1, 3
OPT_ADABOUND, OPT_ADAM, OPT_AMSBOUND, OPT_AMSGRAD, OPT_GD, OPT_IRPROP_PLUS, OPT_NOSADAM = 1, 2, 4, 5, 6, 8, 9
(BUF_PARAMETERS, BUF_DERIVATIVES, BUF_FIRST_MOMENT, BUF_SECOND_MOMENT, BUF_SECOND_MOMENT_HAT, BUF_MASK_REGULARIZED,
 BUF_NORM_MEAN_AVERAGE, BUF_NORM_VARIANCE_AVERAGE, BUF_PREVIOUS_DELTA, BUF_PREVIOUS_DERIVATIVES, BUF_PREVIOUS_STEPS) = range(11)
TIMER_CLASSES = 8


class LayerDesc(C.Structure):
    _fields_ = [("type_layer", C.c_uint32), ("use_bidirectional", C.c_uint32), ("unit_parameters", C.c_uint64 * 5),
                ("type_activation_function", C.c_uint32), ("type_normalization", C.c_uint32),
                ("use_layer_normalization_before_activation", C.c_uint32), ("type_dropout", C.c_uint32),
                ("dropout_values", C.c_float * 3), ("reserved", C.c_uint32)]


class NetDesc(C.Structure):
    _fields_ = [("number_layers", C.c_uint32), ("type_network", C.c_uint32), ("number_recurrent_depth", C.c_uint64),
                ("number_time_delays", C.c_uint64), ("batch_size", C.c_uint64), ("type_loss_function", C.c_uint32),
                ("type_accuracy_function", C.c_uint32), ("accuracy_variance", C.c_float),
                ("normalization_momentum_average", C.c_float), ("normalization_epsilon", C.c_float),
                ("batch_renormalization_r_correction_maximum", C.c_float),
                ("batch_renormalization_d_correction_maximum", C.c_float), ("clip_gradient", C.c_float),
                ("layers", LayerDesc * MAX_LAYERS)]


class OptDesc(C.Structure):
    _fields_ = [("type_optimizer_function", C.c_uint32), ("use_adam_bias_correction", C.c_uint32),
                ("learning_rate", C.c_float), ("learning_momentum", C.c_float), ("use_nesterov", C.c_uint32),
                ("adam_learning_rate", C.c_float), ("adam_beta1", C.c_float), ("adam_beta2", C.c_float),
                ("adam_epsilon", C.c_float), ("learning_rate_final", C.c_float), ("learning_gamma", C.c_float),
                ("regularization__weight_decay", C.c_float), ("use_normalized_weight_decay", C.c_uint32),
                ("use_clip_gradient", C.c_uint32), ("clip_gradient", C.c_float), ("epoch_time_step", C.c_float),
                ("adam_gamma", C.c_float), ("regularization__max_norm_constraints", C.c_float),
                ("rprop_increase_factor", C.c_float), ("rprop_decrease_factor", C.c_float), ("rprop_delta_min", C.c_float),
                ("rprop_delta_max", C.c_float), ("rprop_delta_zero", C.c_float), ("loss_rprop", C.c_float), ("previous_loss_rprop", C.c_float),
                ("regularization__l1", C.c_float), ("regularization__l2", C.c_float)]


class LayerIndex(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in
                ("first_connection_index", "last_connection_index", "first_bias_connection_index",
                 "last_bias_connection_index", "scale_index", "shift_index", "number_inputs", "number_outputs",
                 "block_stride", "number_units_norm")]

    def as_tuple(self):
        return tuple(getattr(self, n) for n, _ in self._fields_)


def fc(units, af=AF_LINEAR, norm=NORM_NONE, dropout=DROP_NONE, p=(0.0, 0.0, 0.0), norm_before=True):
    d = LayerDesc()
    d.type_layer = LAYER_FC
    d.unit_parameters[0] = units
    d.type_activation_function = af
    d.type_normalization = norm
    d.use_layer_normalization_before_activation = 1 if norm_before else 0
    d.type_dropout = dropout
    for i in range(3):
        d.dropout_values[i] = p[i]
    return d


def fc_ind_rnn(units, af=AF_RELU, norm=NORM_NONE, dropout=DROP_NONE, p=(0.0, 0.0, 0.0)):
    """independently recurrent fully connected layer: y_t = f(W x_t + b + u * y_{t-1}), one recurrent weight per unit"""
    d = fc(units, af, norm, dropout, p)
    d.type_layer = LAYER_FC_IND_RNN
    return d


def pooling(kind, kernel, stride, padding=0, dilation=1, ceil_mode=False):
    """average (LAYER_AVERAGE_POOLING) or max (LAYER_MAX_POOLING) pooling over the units of the layer before"""
    d = LayerDesc()
    d.type_layer = kind
    for i, v in enumerate((kernel, stride, padding, dilation, 1 if ceil_mode else 0)):
        d.unit_parameters[i] = v
    return d


def lstm(blocks, cells_per_block=1, bidirectional=False, dropout=DROP_NONE, p=(0.0, 0.0, 0.0)):
    d = LayerDesc()
    d.type_layer = LAYER_LSTM
    d.use_bidirectional = 1 if bidirectional else 0
    d.unit_parameters[0] = blocks
    d.unit_parameters[1] = cells_per_block
    d.use_layer_normalization_before_activation = 1
    d.type_dropout = dropout
    for i in range(3):
        d.dropout_values[i] = p[i]
    return d


def residual(block_depth, dropout=DROP_NONE, p=(0.0, 0.0, 0.0), normalization=NORM_NONE):
    d = LayerDesc()
    d.type_layer = LAYER_RESIDUAL
    d.unit_parameters[0] = block_depth
    d.type_normalization = normalization   # of the block's output, before ShakeDrop and the skip add
    d.use_layer_normalization_before_activation = 1
    d.type_dropout = dropout
    for i in range(3):
        d.dropout_values[i] = p[i]
    return d


def net(layers, batch, T=1, loss=LOSS_MSE, accuracy=ACC_NONE, time_delays=0, momentum=0.0, epsilon=0.0, r_max=0.0,
        d_max=0.0, clip_gradient=0.0):
    """Network descriptor. momentum/epsilon/r_max/d_max of 0 keep the reference defaults
    (0.999, 1e-5, 1, 0: Data.hpp:2966-2969)."""
    d = NetDesc()
    d.number_layers = len(layers)
    d.type_network = NET_RECURRENT if T > 1 or any(l.type_layer in (LAYER_LSTM, LAYER_FC_IND_RNN) for l in layers) else NET_FEEDFORWARD
    d.number_recurrent_depth = T
    d.number_time_delays = time_delays
    d.batch_size = batch
    d.type_loss_function = loss
    d.type_accuracy_function = accuracy
    d.normalization_momentum_average = momentum
    d.normalization_epsilon = epsilon
    d.batch_renormalization_r_correction_maximum = r_max
    d.batch_renormalization_d_correction_maximum = d_max
    d.clip_gradient = clip_gradient   # only shapes the recurrent-weight bounds of independently recurrent layers; 0 = class default 1
    for i, l in enumerate(layers):
        d.layers[i] = l
    return d


def opt(kind=OPT_ADAM, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, bias_correction=True, final_lr=0.1, gamma=1e-3,
        weight_decay=0.0, normalized_wd=True, clip=None, gd_lr=0.01, momentum=0.0, nesterov=False, epoch=1.0, nosadam_gamma=0.1,
        max_norm=0.0, rprop=(0.0, 0.0, 0.0, 0.0, 0.0), l1=0.0, l2=0.0):
    """rprop: (increase factor, decrease factor, delta min, delta max, delta zero) of iRPROP+, 0 = class default"""
    o = OptDesc()
    o.type_optimizer_function = kind
    o.use_adam_bias_correction = 1 if bias_correction else 0
    o.learning_rate = gd_lr
    o.learning_momentum = momentum
    o.use_nesterov = 1 if nesterov else 0
    o.adam_learning_rate, o.adam_beta1, o.adam_beta2, o.adam_epsilon = lr, beta1, beta2, eps
    o.learning_rate_final, o.learning_gamma = final_lr, gamma
    o.regularization__weight_decay = weight_decay
    o.use_normalized_weight_decay = 1 if normalized_wd else 0
    o.use_clip_gradient = 0 if clip is None else 1
    o.clip_gradient = 1.0 if clip is None else clip
    o.epoch_time_step = epoch
    o.adam_gamma = nosadam_gamma
    o.regularization__max_norm_constraints = max_norm
    o.regularization__l1, o.regularization__l2 = l1, l2
    (o.rprop_increase_factor, o.rprop_decrease_factor, o.rprop_delta_min, o.rprop_delta_max, o.rprop_delta_zero) = rprop
    return o


_LIB = None

_PROTOS = {
    "myea_b200_create": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(NetDesc), C.c_int]),
    "myea_b200_destroy": (None, [C.c_void_p]),
    "myea_b200_set_pre_training_level": (C.c_int, [C.c_void_p, C.c_uint64]),
    "myea_b200_last_error": (C.c_char_p, [C.c_void_p]),
    "myea_b200_sizes": (C.c_int, [C.c_void_p] + [C.POINTER(C.c_uint64)] * 4),
    "myea_b200_layer_index": (C.c_int, [C.c_void_p, C.c_uint32, C.POINTER(LayerIndex)]),
    "myea_b200_dataset_set": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]),
    "myea_b200_train_epoch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(OptDesc), C.c_uint64, C.c_uint64,
                                        C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "myea_b200_evaluate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_uint64),
                                     C.POINTER(C.c_double)]),
    "myea_b200_save_dimension_parameters": (C.c_int, [C.c_void_p, C.c_char_p]),
    "myea_b200_save_general_parameters": (C.c_int, [C.c_void_p, C.POINTER(OptDesc), C.c_char_p]),
    "myea_b200_load": (C.c_int, [C.POINTER(C.c_void_p), C.c_char_p, C.c_char_p, C.c_uint64, C.c_int, C.POINTER(OptDesc)]),
    "myea_b200_checkpoint_format_dimension": (C.c_int, [C.POINTER(NetDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p]),
    "myea_b200_checkpoint_format_general": (C.c_int, [C.POINTER(NetDesc), C.POINTER(OptDesc), C.c_char_p]),
    "myea_b200_checkpoint_parse": (C.c_int, [C.c_char_p, C.c_char_p, C.c_uint64, C.POINTER(NetDesc), C.POINTER(OptDesc), C.c_void_p, C.c_uint64,
                                             C.c_void_p, C.c_void_p, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "myea_b200_checkpoint_last_error": (C.c_char_p, []),
    "myea_b200_generate_masks": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64]),
    "myea_b200_download_mask": (C.c_int, [C.c_void_p, C.c_uint32, C.c_int, C.c_void_p, C.c_uint64]),
    "myea_b200_upload": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_uint64, C.c_uint64]),
    "myea_b200_download": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_uint64, C.c_uint64]),
    "myea_b200_set_mask_bernoulli": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64]),
    "myea_b200_set_mask_zoneout": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint64]),
    "myea_b200_set_shakedrop": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64]),
    "myea_b200_forward": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_int]),
    "myea_b200_forward_device": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_int]),
    "myea_b200_compute_error": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "myea_b200_compute_error_device": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "myea_b200_reset_loss": (C.c_int, [C.c_void_p]),
    "myea_b200_get_loss": (C.c_int, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.POINTER(C.c_double)]),
    "myea_b200_backward": (C.c_int, [C.c_void_p, C.c_uint64]),
    "myea_b200_update_derivative_weight": (C.c_int, [C.c_void_p, C.c_uint64]),
    "myea_b200_update_parameter": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(OptDesc)]),
    "myea_b200_clear_training_arrays": (C.c_int, [C.c_void_p]),
    "myea_b200_get_outputs": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64]),
    "myea_b200_get_errors": (C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64]),
    "myea_b200_comm_unique_id": (C.c_int, [C.c_void_p]),
    "myea_b200_comm_init": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "myea_b200_synchronize": (C.c_int, [C.c_void_p]),
    "myea_b200_stream": (C.c_void_p, [C.c_void_p]),
    "myea_b200_kernel_launches": (C.c_uint64, [C.c_void_p]),
    "myea_b200_gemm_nt": (C.c_int, [C.c_int, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_int, C.POINTER(C.c_float), C.c_int]),
    "myea_b200_gemm_nt_static": (C.c_int, [C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p,
                                           C.c_int, C.c_void_p, C.c_char_p, C.c_size_t]),
    "myea_b200_profile": (C.c_int, [C.c_void_p, C.c_int]),
    "myea_b200_profile_read": (C.c_int, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_uint64),
                                         C.POINTER(C.c_double), C.c_int]),
}


def exported_symbols():
    """Names of every entry point include/myea_b200.h declares."""
    return sorted(_PROTOS)


def load(path=None):
    """dlopen the product library and attach prototypes. Raises OSError when it has not been built."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise OSError("%s is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                      "(the CUDA library is the product; there is no CPU fallback)" % p)
    lib = C.CDLL(p, mode=C.RTLD_GLOBAL)
    for name, (res, args) in _PROTOS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _LIB = lib
    return lib
