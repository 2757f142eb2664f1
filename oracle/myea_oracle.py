"""Test infrastructure, not product code.

numpy restatement of the reference's training step (MyEA `class Neural_Network`, CPU "Loop" variants), used as the
parity checker where the compiled reference (oracle/_ref) cannot travel or cannot serve (bidirectional LSTM).  Only
tests/, __graft_entry__.smoke() and the CPU-baseline leg of bench.py may import it.

Pinned: tests/test_oracle_golden.py checks this module against tests/golden/*.npz, which were produced by running the
unmodified reference (oracle/_ref, built by oracle/build_ref.sh) through tests/golden/make_golden.py.  The
bidirectional LSTM has no usable reference run (the reference's own bidirectional wiring overlaps the two
directions' buffers); for that layer this module composes the reference's unidirectional routines, and parity of
that case is pinned only against this restatement plus a float64 finite-difference check: "parity unpinned" for
bidirectional LSTM against the reference binary.

Each routine cites the reference file:line it follows (paths relative to
Neural_Network_Library_Windows/Source_Files/Neural_Network/).  Arithmetic is float32 unless `dtype=np.float64` is
passed to OracleNet (tie-breaker / finite differences).  Same method set as oracle.ref.RefNet and myea_b200.net.Net.
"""
import math

import numpy as np

from myea_b200 import capi

F = np.float32


# ---------------------------------------------------------------------------------------------------------------
# activation functions: Header_Files/Neural_Network/Activation_Functions.hpp:34-183, Neural_Network.cpp:3157-3204
# ---------------------------------------------------------------------------------------------------------------
_STEP_SIGMOID = ((-2.64665246, -1.47221947, -0.549306154, 0.549306154, 1.47221935, 2.64665294),
                 (0.00499999989, 0.0500000007, 0.25, 0.75, 0.949999988, 0.995000005), 0.0, 1.0)
_STEP_TANH = ((-2.64665294, -1.47221935, -0.549306154, 0.549306154, 1.47221935, 2.64665294),
              (-0.99000001, -0.899999976, -0.5, 0.5, 0.899999976, 0.99000001), -1.0, 1.0)


def _stepwise(z, table):
    """AF_STEPWISE_real (Activation_Functions.hpp:28-31): linear between six points, constant outside"""
    dt = z.dtype.type
    v, r, lo, hi = table
    v, r = [dt(np.float32(x)) for x in v], [dt(np.float32(x)) for x in r]
    out = np.full_like(z, dt(hi))
    for k in range(4, -1, -1):
        seg = (((r[k + 1] - r[k]) * (z - v[k])) / (v[k + 1] - v[k])) + r[k]
        out = np.where(z < v[k + 1], seg, out)
    return np.where(z < v[0], dt(lo), out)


def af_fire(af, z):
    """AF_FIRE (Activation_Functions.hpp:124-196)"""
    dt = z.dtype.type
    if af == capi.AF_TANH:
        with np.errstate(over="ignore"):      # e^(+big) = inf gives the limit -1, as in the reference's float arithmetic
            return dt(2) / (dt(1) + np.exp(dt(-2) * z)) - dt(1)
    if af == capi.AF_SIGMOID:
        with np.errstate(over="ignore"):
            return dt(1) / (dt(1) + np.exp(-z))
    if af == capi.AF_RELU:
        return np.where(z < 0, dt(0), z)
    if af in (capi.AF_LEAKY_RELU, capi.AF_PARAMETRIC_RELU):
        return np.where(z < 0, dt(0.01) * z, z)
    if af == capi.AF_ELU:
        return np.where(z < 0, np.exp(np.minimum(z, 0)) - dt(1), z)
    if af == capi.AF_SELU:
        a, s = dt(1.6732632423543772848170429916717), dt(1.0507009873554804934193349852946)
        return s * np.where(z <= 0, a * np.exp(np.minimum(z, 0)) - a, z)
    if af == capi.AF_LINEAR_PIECE:
        return np.where(z < 0, dt(0), np.where(z > 1, dt(1), z))
    if af == capi.AF_LINEAR_PIECE_SYMMETRIC:
        return np.where(z < -1, dt(-1), np.where(z > 1, dt(1), z))
    if af == capi.AF_SIGMOID_STEPWISE:
        return _stepwise(z, _STEP_SIGMOID)
    if af == capi.AF_TANH_STEPWISE:
        return _stepwise(z, _STEP_TANH)
    if af == capi.AF_THRESHOLD:
        return np.where(z < 0, dt(0), dt(1)).astype(z.dtype)
    if af == capi.AF_THRESHOLD_SYMMETRIC:
        return np.where(z < 0, dt(-1), dt(1)).astype(z.dtype)
    if af == capi.AF_GAUSSIAN:
        return np.exp(-z * z)
    if af == capi.AF_GAUSSIAN_SYMMETRIC:
        return np.exp(-z * z) * dt(2) - dt(1)
    if af == capi.AF_GAUSSIAN_STEPWISE:
        return np.zeros_like(z)
    if af == capi.AF_ELLIOT:
        return (z / dt(2)) / (dt(1) + np.abs(z)) + dt(0.5)
    if af == capi.AF_ELLIOT_SYMMETRIC:
        return z / (dt(1) + np.abs(z))
    if af == capi.AF_SINE:
        return np.sin(z) / dt(2) + dt(0.5)
    if af == capi.AF_SINE_SYMMETRIC:
        return np.sin(z)
    if af == capi.AF_COSINE:
        return np.cos(z) / dt(2) + dt(0.5)
    if af == capi.AF_COSINE_SYMMETRIC:
        return np.cos(z)
    if af == capi.AF_ISRU:
        return z * (dt(1) / np.sqrt(dt(1) + z * z))
    if af == capi.AF_ISRLU:
        return np.where(z < 0, z * (dt(1) / np.sqrt(dt(1) + z * z)), z)
    return z  # linear


def af_derive(af, z, y):
    """Activation_Function_Derive (Neural_Network.cpp:3157-3199), steepness 1; functions outside its switch get the value"""
    dt = y.dtype.type
    one = np.ones_like(y)
    if af in (capi.AF_TANH, capi.AF_TANH_STEPWISE):
        return dt(1) - y * y
    if af in (capi.AF_SIGMOID, capi.AF_SIGMOID_STEPWISE):
        return y * (dt(1) - y)
    if af == capi.AF_RELU:
        return np.where(z < 0, dt(0), one)
    if af in (capi.AF_LEAKY_RELU, capi.AF_PARAMETRIC_RELU):
        return np.where(z < 0, dt(0.01), one)
    if af == capi.AF_ELU:          # steepness * alpha * y below zero, y = e^z - 1 (not alpha * e^z)
        return np.where(z < 0, y, one)
    if af == capi.AF_SELU:
        a, s = dt(1.6732632423543772848170429916717), dt(1.0507009873554804934193349852946)
        return s * np.where(z <= 0, y + a, one)
    if af == capi.AF_GAUSSIAN:
        return dt(-2) * z * y
    if af == capi.AF_GAUSSIAN_SYMMETRIC:
        return dt(-2) * z * (y + dt(1))
    if af == capi.AF_ELLIOT:
        return dt(1) / (dt(2) * (dt(1) + np.abs(z)) * (dt(1) + np.abs(z)))
    if af == capi.AF_ELLIOT_SYMMETRIC:
        return dt(1) / ((dt(1) + np.abs(z)) * (dt(1) + np.abs(z)))
    if af == capi.AF_SINE:
        return np.cos(z) / dt(2)
    if af == capi.AF_SINE_SYMMETRIC:
        return np.cos(z)
    if af == capi.AF_COSINE:
        return -np.sin(z) / dt(2)
    if af == capi.AF_COSINE_SYMMETRIC:
        return -np.sin(z)
    if af in (capi.AF_ISRU, capi.AF_ISRLU):
        zs = np.where(z == 0, dt(1), z)
        q = np.where(z == 0, dt(1), y / zs)
        cube = q * q * q
        return cube if af == capi.AF_ISRU else np.where(z < 0, cube, one)
    if af in (capi.AF_THRESHOLD, capi.AF_THRESHOLD_SYMMETRIC, capi.AF_GAUSSIAN_STEPWISE):
        return y
    return one  # linear, linear piece, softmax


# ---------------------------------------------------------------------------------------------------------------
# index map: Neural_Network__Prepare_Connections.cpp:20-252, Neural_Network__Compile.cpp:426-785,
# normalized-unit slots Neural_Network__Allocate.cpp:2378-2460
# ---------------------------------------------------------------------------------------------------------------
class _Layer:
    pass


def build_index_map(desc):
    n = int(desc.number_layers)
    Ls = []
    for l in range(n):
        d = desc.layers[l]
        L = _Layer()
        L.d, L.type = d, int(d.type_layer)
        L.n_out = 0
        L.ind_rnn = L.type == capi.LAYER_FC_IND_RNN   # a fully connected layer plus one recurrent weight per unit
        if L.ind_rnn:
            L.type = capi.LAYER_FC
        if L.type == capi.LAYER_FC:
            L.n_out = int(d.unit_parameters[0])
        elif L.type == capi.LAYER_LSTM:
            L.n_out = int(d.unit_parameters[0]) * max(1, int(d.unit_parameters[1])) * (2 if d.use_bidirectional else 1)
        elif L.type in (capi.LAYER_AVERAGE_POOLING, capi.LAYER_MAX_POOLING):
            # Assign__Post__Layer (Neural_Network__Compile.cpp:250-271): the average ignores the dilation, the maximum counts it
            k, s_, p_, dil, ceil_mode = (int(d.unit_parameters[i]) for i in range(5))
            n_prev = Ls[l - 1].n_out
            span = n_prev + 2 * p_ - k if L.type == capi.LAYER_AVERAGE_POOLING else n_prev + 2 * p_ - dil * (k - 1) - 1
            q = span / s_ + 1.0
            L.n_out = int(math.ceil(q) if ceil_mode else math.floor(q))
        L.depth = int(d.unit_parameters[0]) if L.type == capi.LAYER_RESIDUAL else 0
        L.idx = dict(first_connection_index=0, last_connection_index=0, first_bias_connection_index=0,
                     last_bias_connection_index=0, scale_index=0, shift_index=0, number_inputs=0, number_outputs=0,
                     block_stride=0, number_units_norm=0)
        Ls.append(L)
    # a residual layer is as wide as the wider of its shortcut and its block's last layer (zero-padded identity,
    # Assign__Post__Layers, Neural_Network__Compile.cpp:222-424); the shortcut is the layer before, or the residual layer
    # of the block that ends there
    for l in range(1, n):
        if Ls[l].type == capi.LAYER_RESIDUAL:
            feeder = l - 1
            for q in range(1, l):
                if Ls[q].type == capi.LAYER_RESIDUAL and q + Ls[q].depth == l - 1:
                    feeder = q
            Ls[l].n_out = max(Ls[feeder].n_out, Ls[l + Ls[l].depth].n_out)
    for l in range(1, n):
        Ls[l].input_layer, Ls[l].n_in = l - 1, Ls[l - 1].n_out
    for l in range(1, n):
        if Ls[l].type == capi.LAYER_RESIDUAL:
            Ls[l + 1].input_layer, Ls[l + 1].n_in = l - 1, Ls[l - 1].n_out
            after = l + Ls[l].depth + 1
            if after < n:
                Ls[after].input_layer, Ls[after].n_in = l, Ls[l].n_out
    tw = 0
    for l in range(1, n):
        L = Ls[l]
        L.idx["number_inputs"], L.idx["number_outputs"] = (L.n_in if L.type in (capi.LAYER_FC, capi.LAYER_LSTM) else 0), L.n_out
        if L.type == capi.LAYER_FC:
            L.idx["first_connection_index"] = tw
            tw += L.n_out * L.n_in
            if L.ind_rnn:
                tw += L.n_out       # the units' self connections (Prepare__Connections__FC_Ind_RNN, …Prepare_Connections.cpp:45-78)
            L.idx["last_connection_index"] = tw
        elif L.type == capi.LAYER_LSTM:
            dirs = 2 if L.d.use_bidirectional else 1
            cpb = max(1, int(L.d.unit_parameters[1]))
            blocks = int(L.d.unit_parameters[0])
            cells = blocks * cpb
            L.idx["block_stride"] = cpb * (L.n_in + cells) + 3 * L.n_in + 3 * cells + 3 * cpb
            L.idx["first_connection_index"] = tw
            tw += dirs * blocks * L.idx["block_stride"]
            L.idx["last_connection_index"] = tw
    Ls[0].idx["number_outputs"] = Ls[0].n_out
    tb = 0
    for l in range(1, n):
        L = Ls[l]
        if L.type == capi.LAYER_FC:
            L.idx["first_bias_connection_index"] = tw + tb
            tb += L.n_out
            L.idx["last_bias_connection_index"] = tw + tb
        elif L.type == capi.LAYER_LSTM:
            dirs = 2 if L.d.use_bidirectional else 1
            cells, blocks = L.n_out, int(L.d.unit_parameters[0]) * dirs
            L.idx["first_bias_connection_index"] = tw + tb + cells   # shifted by the cell count, as the reference does
            tb += cells + 3 * blocks
            L.idx["last_bias_connection_index"] = tw + tb
    P = tw + tb
    units = 0
    if any(int(desc.layers[l].type_normalization) != capi.NORM_NONE for l in range(1, n)):
        # units a layer normalizes (Prepare__Normalized__Layer / __Residual_Layer, Neural_Network__Layer_Normalization.cpp:43-154):
        # its outputs; inside a residual block its input; for a residual layer the outputs of the block's last layer
        off, own = [], []
        in_block = set()
        for l in range(1, n):
            if Ls[l].type == capi.LAYER_RESIDUAL:
                in_block.update(range(l + 1, l + Ls[l].depth + 1))
        for l in range(n):
            off.append(units)
            if Ls[l].type in (capi.LAYER_AVERAGE_POOLING, capi.LAYER_MAX_POOLING):
                own.append(0)
            elif Ls[l].type == capi.LAYER_LSTM:   # three per cell and six per block, counted although the layer does not normalize
                own.append(3 * Ls[l].n_out + 6 * int(Ls[l].d.unit_parameters[0]) * (2 if Ls[l].d.use_bidirectional else 1))
            else:
                own.append(Ls[l + Ls[l].depth].n_out if Ls[l].type == capi.LAYER_RESIDUAL else (Ls[l].n_in if l in in_block else Ls[l].n_out))
            units += own[l]
        for l in range(n):
            Ls[l].idx["scale_index"] = P + off[l]
            Ls[l].idx["shift_index"] = P + units + off[l]
            Ls[l].idx["number_units_norm"] = own[l]
            Ls[l].norm_off = off[l]
        P += 2 * units
    return Ls, P, tw, tb, units


class OracleNet:
    def __init__(self, desc, opt, threads=1, dtype=np.float32):
        self.desc, self.opt, self.dt = desc, opt, dtype
        self.T, self.B = int(desc.number_recurrent_depth), int(desc.batch_size)
        self.layers, self.P, self.W, self.n_bias, self.n_norm = build_index_map(desc)
        z = lambda k: np.zeros(k, dtype)
        self.buf = {capi.BUF_PARAMETERS: z(self.P), capi.BUF_DERIVATIVES: z(self.P), capi.BUF_FIRST_MOMENT: z(self.P),
                    capi.BUF_SECOND_MOMENT: z(self.P), capi.BUF_SECOND_MOMENT_HAT: z(self.P), capi.BUF_MASK_REGULARIZED: z(self.P),
                    capi.BUF_PREVIOUS_DELTA: z(self.P), capi.BUF_NORM_MEAN_AVERAGE: z(self.n_norm * self.T),
                    capi.BUF_NORM_VARIANCE_AVERAGE: np.ones(self.n_norm * self.T, dtype)}
        self.masks, self.zone, self.shake = {}, {}, {}
        # sharded batch: `allreduce(array) -> array summed over the ranks` and the number of ranks (tests/test_sharding_cpu.py)
        self.allreduce, self.world = None, 1
        self.time_step = dtype(0)
        self.loss_sum, self.n_loss, self.acc_sum = 0.0, 0, 0.0
        self.training = True
        self.momentum = dtype(desc.normalization_momentum_average if desc.normalization_momentum_average > 0 else 0.999)
        self.eps = dtype(desc.normalization_epsilon if desc.normalization_epsilon > 0 else 1e-5)
        self.r_max = dtype(desc.batch_renormalization_r_correction_maximum if desc.batch_renormalization_r_correction_maximum > 0 else 1.0)
        self.d_max = dtype(desc.batch_renormalization_d_correction_maximum if desc.batch_renormalization_d_correction_maximum > 0 else 0.0)

    # ---- bookkeeping ----------------------------------------------------------------------------------------
    def close(self):
        pass

    def sizes(self):
        return self.P, self.W, self.n_bias, self.n_norm

    def layer_index(self, l):
        li = capi.LayerIndex()
        for k, v in self.layers[l].idx.items():
            setattr(li, k, v)
        return li

    _ALIAS = {capi.BUF_PREVIOUS_DERIVATIVES: capi.BUF_FIRST_MOMENT, capi.BUF_PREVIOUS_STEPS: capi.BUF_SECOND_MOMENT}

    def get(self, which):
        return self.buf[self._ALIAS.get(which, which)].astype(np.float32).copy()

    def set(self, which, arr):
        a = np.asarray(arr).ravel()
        self.buf[self._ALIAS.get(which, which)][:a.size] = a.astype(self.dt)

    def set_mask_bernoulli(self, l, mask):
        self.masks[l] = np.asarray(mask).reshape(self.T, -1).astype(bool)

    def set_mask_zoneout(self, l, state, output):
        self.zone[l] = (np.asarray(state).reshape(self.T, -1).astype(bool), np.asarray(output).reshape(self.T, -1).astype(bool))

    def set_shakedrop(self, l, mask, alpha, beta):
        self.shake[l] = (np.asarray(mask).astype(bool), np.asarray(alpha, self.dt), np.asarray(beta, self.dt))

    def reset_loss(self):
        self.loss_sum, self.n_loss, self.acc_sum = 0.0, 0, 0.0

    def loss(self):
        return float(self.loss_sum), int(self.n_loss), float(self.acc_sum)

    def outputs(self, l):
        return np.asarray(self.layers[l].values, np.float32).reshape(self.T, self.B, -1)

    def errors(self, l):
        L = self.layers[l]
        e = L.dh if L.type == capi.LAYER_LSTM else L.errors
        return np.asarray(e, np.float32).reshape(self.T, self.B, -1)

    def _p(self):
        return self.buf[capi.BUF_PARAMETERS]

    def _g(self):
        return self.buf[capi.BUF_DERIVATIVES]

    # ---- fully connected layer ---------------------------------------------------------------------------------
    def _fc_weights(self, L):
        i = L.idx
        return self._p()[i["first_connection_index"]:i["first_connection_index"] + L.n_out * L.n_in].reshape(L.n_out, L.n_in)

    def _norm_steps(self, rows):
        """row ranges of the time steps inside a [T * rows-per-step, H] array (one step for a feed-forward network)"""
        T = self.T if rows % self.T == 0 and self.T > 1 else 1
        n = rows // T
        return [(t, slice(t * n, (t + 1) * n)) for t in range(T)]

    def _norm_forward(self, L, z):
        """Forward_Pass__Batch_Normalization__Training / __Batch_Renormalization__Training
        (Neural_Network__Forward_Pass__Loop.cpp:4673-4853); inference :4644-4671.  The 'variance' is the standard
        deviation sqrt(E[x^2]-mean^2+eps); r and d use the already updated running averages.  Every time step has
        statistics and running averages of its own ([layer][T][units] arrays), gamma and beta are shared."""
        dt = self.dt
        H = L.idx["number_units_norm"]
        gamma = self._p()[L.idx["scale_index"]:L.idx["scale_index"] + H]
        beta = self._p()[L.idx["shift_index"]:L.idx["shift_index"] + H]
        L.xhat = np.zeros_like(z)
        L.stats = {}
        for t, rows in self._norm_steps(z.shape[0]):
            o = L.norm_off * self.T + t * H
            ma = self.buf[capi.BUF_NORM_MEAN_AVERAGE][o:o + H]
            sa = self.buf[capi.BUF_NORM_VARIANCE_AVERAGE][o:o + H]
            zt = z[rows]
            if self.training:
                s1, s2 = zt.sum(0, dtype=dt), (zt * zt).sum(0, dtype=dt)
                if self.allreduce is not None:   # the statistics are those of the whole batch, whichever rank holds which rows
                    s1, s2 = self.allreduce(s1), self.allreduce(s2)
                inv = dt(1) / dt(zt.shape[0] * self.world)
                mean = s1 * inv
                sigma = np.sqrt(s2 * inv - mean * mean + self.eps)
                ma += self.momentum * (mean - ma)
                sa += self.momentum * (sigma - sa)
                r, d = np.ones(H, dt), np.zeros(H, dt)
                if int(L.d.type_normalization) == capi.NORM_BRN:
                    r = np.clip(sigma / sa, dt(1) / self.r_max, self.r_max)
                    d = np.clip((mean - ma) / sa, -self.d_max, self.d_max)
                L.stats[t] = (mean, sigma, r, d)
                L.xhat[rows] = (zt - mean) / sigma * r + d
            else:
                L.xhat[rows] = (zt - ma) / sa
        return gamma * L.xhat + beta

    def _norm_backward(self, L, z, delta):
        """Backward_Pass__Batch_Normalization / __Batch_Renormalization (Neural_Network__Backward_Pass__Loop.cpp:1380-1628),
        time step by time step; the derivatives of gamma and beta add up over the steps"""
        dt = self.dt
        H = L.idx["number_units_norm"]
        gamma = self._p()[L.idx["scale_index"]:L.idx["scale_index"] + H]
        self._g()[L.idx["scale_index"]:L.idx["scale_index"] + H] += (delta * L.xhat).sum(0, dtype=dt)
        self._g()[L.idx["shift_index"]:L.idx["shift_index"] + H] += delta.sum(0, dtype=dt)
        out = np.zeros_like(delta)
        for t, rows in self._norm_steps(z.shape[0]):
            mean, sigma, r, _ = L.stats[t]
            zt = z[rows]
            B = dt(zt.shape[0] * self.world)
            dh = delta[rows] * gamma
            d_mean = (dh * (-r / sigma)).sum(0, dtype=dt)
            d_sigma = (dh * (zt - mean) * (-r / (sigma * sigma))).sum(0, dtype=dt)
            if self.allreduce is not None:       # scale / shift derivatives stay local (summed with the other derivatives later)
                d_mean, d_sigma = self.allreduce(d_mean), self.allreduce(d_sigma)
            out[rows] = dh * (r / sigma) + d_sigma * ((zt - mean) / (B * sigma)) + d_mean * (dt(1) / B)
        return out

    def _dropout(self, l, y):
        """Bernoulli / inverted Bernoulli dropout of layer l on rows y of ONE time step `self._t` (mask row per step)"""
        L = self.layers[l]
        dt = self.dt
        drop = int(L.d.type_dropout)
        if drop in (capi.DROP_BERNOULLI, capi.DROP_BERNOULLI_INVERTED):
            p = dt(L.d.dropout_values[0])
            if self.training:
                m = np.asarray(self.masks[l]).reshape(-1, y.shape[1])[self._t]
                y = np.where(m, y * (dt(1) / p) if drop == capi.DROP_BERNOULLI_INVERTED else y, dt(0))
            elif drop == capi.DROP_BERNOULLI:
                y = y * p
        return y

    def _ind_rnn_forward(self, l, pre):
        """Forward_Pass__FC_Ind_RNN__Loop (Neural_Network__Recurrent_Forward_Pass__Loop.cpp:813-860): per time step
        pre_t = z'_t + u * y_{t-1}, y_t = f(pre_t), dropout in place on y_t (what the next step then sees)"""
        L = self.layers[l]
        dt = self.dt
        i = L.idx
        u = self._p()[i["first_connection_index"] + L.n_out * L.n_in:i["last_connection_index"]]
        af = int(L.d.type_activation_function)
        n = pre.shape[0] // self.T
        L.pre = np.array(pre, dt)
        y = np.zeros_like(L.pre)
        for t in range(self.T):
            rows = slice(t * n, (t + 1) * n)
            if t > 0:
                L.pre[rows] = L.pre[rows] + u * y[(t - 1) * n:t * n]
            self._t = t
            y[rows] = self._dropout(l, af_fire(af, L.pre[rows]))
        L.values = y.astype(dt)
        return L.values

    def _ind_rnn_backward(self, L, D):
        """Backward_Pass__FC__DF_Ind_RNN__Loop (Neural_Network__Backward_Pass__Loop.cpp:1296-1372):
        dAF_t = D_t * f' + u * f' * dAF_{t+1}, backwards in time"""
        dt = self.dt
        i = L.idx
        u = self._p()[i["first_connection_index"] + L.n_out * L.n_in:i["last_connection_index"]]
        f = af_derive(int(L.d.type_activation_function), L.pre, L.values)
        n = D.shape[0] // self.T
        dAF = np.zeros_like(D)
        for t in range(self.T - 1, -1, -1):
            rows = slice(t * n, (t + 1) * n)
            dAF[rows] = D[rows] * f[rows]
            if t + 1 < self.T:
                dAF[rows] = dAF[rows] + u * f[rows] * dAF[(t + 1) * n:(t + 2) * n]
        L.dAF = dAF.astype(dt)
        return L.dAF

    def _pooling_windows(self, L):
        """padded positions j * stride + k * dilation read by output j, and which of them fall inside the input"""
        k, s_, p_, dil = (int(L.d.unit_parameters[i]) for i in range(4))
        pos = np.arange(L.n_out)[:, None] * s_ + np.arange(k)[None, :] * dil      # [n_out, kernel]
        inside = (pos >= p_) & (pos < L.n_in + p_)
        return pos, inside, p_, k

    def _pooling_forward(self, L, x):
        """Forward_Pass__Average_Pooling__Loop / __Max_Pooling__Loop (Neural_Network__Forward_Pass__Loop.cpp:4537-4582,
        :5069-5136): the average divides by the kernel size whatever falls outside the input; the maximum takes 0 for a
        position outside and keeps the first of equal values"""
        dt = self.dt
        pos, inside, pad, k = self._pooling_windows(L)
        idx = np.clip(pos - pad, 0, L.n_in - 1)
        win = x[:, idx]                                                            # [rows, n_out, kernel]
        if L.type == capi.LAYER_AVERAGE_POOLING:
            out = np.zeros((x.shape[0], L.n_out), dt)
            for kk in range(k):                                                    # summed in kernel order
                out += np.where(inside[None, :, kk], win[:, :, kk], dt(0))
            L.values = out * (dt(1) / dt(k))
        else:
            top = np.full((x.shape[0], L.n_out), -np.finfo(np.float32).max, dt)
            best = np.zeros((x.shape[0], L.n_out), np.int64)
            for kk in range(k):
                v = np.where(inside[None, :, kk], win[:, :, kk], dt(0))
                take = np.where(inside[None, :, kk], top < v, top < 0)
                best = np.where(take, pos[None, :, kk], best)
                top = np.where(take, v, top)
            L.values, L.winner = top, best
        L.pool_in = x.shape[1]
        return L.values

    def _pooling_backward(self, L):
        """Backward_Pass__Average_Pooling__Loop / __Max_Pooling__Loop (Neural_Network__Backward_Pass__Loop.cpp:1004-1040,
        :1139-1175): error on the layer's inputs"""
        dt = self.dt
        pos, inside, pad, k = self._pooling_windows(L)
        d = L.errors
        D = np.zeros((d.shape[0], L.n_in), dt)
        if L.type == capi.LAYER_AVERAGE_POOLING:
            share = d * (dt(1) / dt(k))
            for j in range(L.n_out):
                for kk in range(k):
                    if inside[j, kk]:
                        D[:, pos[j, kk] - pad] += share[:, j]
        else:
            rows = np.arange(d.shape[0])
            for j in range(L.n_out):
                w = L.winner[:, j]
                ok = (w >= pad) & (w < L.n_in + pad)
                np.add.at(D, (rows[ok], w[ok] - pad), d[ok, j])
        return D

    def _fc_forward(self, l, x):
        """Forward_Pass__FC (Neural_Network__Forward_Pass__Loop.cpp:350-790): weights, bias (only without
        normalization), normalization, activation, dropout applied in place on the output (:4917-4990)."""
        L = self.layers[l]
        dt = self.dt
        z = x @ self._fc_weights(L).T
        norm = int(L.d.type_normalization) != capi.NORM_NONE
        if not norm:
            z = z + self._p()[L.idx["first_bias_connection_index"]:L.idx["first_bias_connection_index"] + L.n_out]
        L.z = z
        pre = self._norm_forward(L, z) if norm else z
        if L.ind_rnn:
            return self._ind_rnn_forward(l, pre)
        L.pre = pre
        af = int(L.d.type_activation_function)
        if af == capi.AF_SOFTMAX:
            e = np.exp(pre - pre.max(1, keepdims=True))
            y = e * (dt(1) / e.sum(1, keepdims=True, dtype=dt))
        else:
            y = af_fire(af, pre)
        drop = int(L.d.type_dropout)
        drop_training = self.training if getattr(self, "_drop_training", None) is None else self._drop_training
        if drop in (capi.DROP_BERNOULLI, capi.DROP_BERNOULLI_INVERTED):
            p = dt(L.d.dropout_values[0])
            if drop_training:
                # one mask row per time step (…Forward_Pass__Loop.cpp:4947-4970); rows of y are time-major
                m = np.repeat(np.asarray(self.masks[l]).reshape(-1, y.shape[1])[:max(1, y.shape[0] // self.active_B)], self.active_B, axis=0)
                y = np.where(m, y * (dt(1) / p) if drop == capi.DROP_BERNOULLI_INVERTED else y, dt(0))
            elif drop == capi.DROP_BERNOULLI:
                y = y * p
        L.values = y.astype(dt)
        return L.values

    # ---- step functions ------------------------------------------------------------------------------------------
    def set_pre_training_level(self, level):
        """Set__Pre_Training_Level (Neural_Network__Indexing.cpp:20-51): 0 = the whole network, k >= 1 = hidden layer k and its
        mirror image n - k are trained as one autoencoder pair"""
        self.pre_training_level = int(level)

    def _forward_pre_training(self):
        """FF__Forward_Pass_Batch__Pre_Training__Loop (Neural_Network__Forward_Pass__Loop.cpp:205-326): layers before the
        coded one in inference behaviour (Forward_Pass__Encode__FC :794-1018; the layer feeding the coded layer keeps its
        training dropout), the coded layer (:1020-1479) and the decoded layer (:1481-) in training behaviour with dropout
        reduced to its inference scaling; the decoded layer reads the coded layer's output"""
        k, n = self.pre_training_level, len(self.layers)
        state = self.training
        for l in range(1, k):
            self.training = False
            self._drop_training = state and l == k - 1
            self._fc_forward(l, self.layers[self.layers[l].input_layer].values)
        self.training = state
        self._drop_training = False
        self._fc_forward(k, self.layers[self.layers[k].input_layer].values)
        self._fc_forward(n - k, self.layers[k].values)
        self._drop_training = None

    def forward(self, X, training=True, batch=None):
        self.training = training
        self.active_B = int(batch or self.B)   # Forward_Pass(batch_size_received, ...): any batch up to the allocated one (T = 1)
        X = np.asarray(X, self.dt).reshape(self.T * self.active_B, -1)
        self.layers[0].values = X
        n = len(self.layers)
        if getattr(self, "pre_training_level", 0):
            return self._forward_pre_training()
        l = 1
        while l < n:
            L = self.layers[l]
            x = self.layers[L.input_layer].values
            if L.type == capi.LAYER_FC:
                self._fc_forward(l, x)
                l += 1
            elif L.type == capi.LAYER_LSTM:
                from oracle import myea_oracle_lstm
                myea_oracle_lstm.forward(self, l, x)
                l += 1
            elif L.type in (capi.LAYER_AVERAGE_POOLING, capi.LAYER_MAX_POOLING):
                self._pooling_forward(L, x)
                l += 1
            else:
                from oracle import myea_oracle_residual
                myea_oracle_residual.forward(self, l)
                l += L.depth + 1

    def compute_error(self, Y):
        """FF__Compute__Error / RNN__Compute__Error (Neural_Network__Compute__Error__Loop.cpp:20-209,
        Neural_Network__Recurrent_Compute__Error__Loop.cpp): delta = f'(pre, y) * (y - desired) whatever the loss; steps
        before number_time_delays are not scored and get zero error."""
        dt = self.dt
        L = self.layers[-1]
        k = getattr(self, "pre_training_level", 0)
        if k:   # the decoded layer answers; above level 1 it is compared with what the coded layer read (FF__Compute__Error :120)
            L = self.layers[len(self.layers) - k]
            if k > 1:
                Y = self.layers[k - 1].values
        Y = np.asarray(Y, dt).reshape(self.T * getattr(self, "active_B", self.B), -1)
        t0 = min(int(self.desc.number_time_delays), self.T) if self.T > 1 else 0
        skip = t0 * getattr(self, "active_B", self.B)
        y, t, pre = L.values[skip:], Y[skip:], L.pre[skip:]
        diff = y - t
        af = int(L.d.type_activation_function)
        L.errors = np.zeros_like(L.values)
        L.errors[skip:] = af_derive(af, pre, y) * diff
        loss = int(self.desc.type_loss_function)
        if loss == capi.LOSS_MSE:
            self.loss_sum += float((diff * diff).sum(dtype=np.float64))
        elif loss == capi.LOSS_CE:
            o = np.where(y != 0, y, np.maximum(y, dt(1e-6)))
            if L.n_out == 1:
                self.loss_sum += float((-(t * np.log(o) + (1 - t) * np.log(1 - o))).sum(dtype=np.float64))
            else:
                self.loss_sum += float((-(t * np.log(o))).sum(dtype=np.float64))
        self.n_loss += diff.size
        acc = int(self.desc.type_accuracy_function)
        if acc == capi.ACC_DISTANCE:
            var = self.desc.accuracy_variance if self.desc.accuracy_variance > 0 else 0.49
            self.acc_sum += float((np.abs(diff) <= dt(var)).sum())
        elif acc == capi.ACC_CE:
            H = L.n_out
            want = np.where((t == 1).any(1), (t == 1).argmax(1), H)
            got = H - 1 - y[:, ::-1].argmax(1)   # the LAST maximum wins (>= in the reference's scan)
            self.acc_sum += float((want == got).sum())

    def backward(self):
        """FF__Backward_Pass_Batch (Neural_Network__Backward_Pass__Loop.cpp:80-209): error to the previous layer
        (:1079-1114), activation derivative (:1259-1294), normalization backward."""
        n = len(self.layers)
        k = getattr(self, "pre_training_level", 0)
        if k:   # FF__Backward_Pass_Batch__Pre_Training__Loop (…Backward_Pass__Loop.cpp:211-296): decoded -> coded layer, no further
            K, D = self.layers[k], self.layers[n - k]
            K.errors = (D.errors @ self._fc_weights(D)) * af_derive(int(K.d.type_activation_function), K.pre, K.values)
            return
        l = n - 1
        while l >= 1:
            N = self.layers[l]
            if N.type == capi.LAYER_RESIDUAL:
                from oracle import myea_oracle_residual
                l = myea_oracle_residual.backward(self, l)
                continue
            p = N.input_layer
            if p < 1:
                break
            Pl = self.layers[p]
            if N.type == capi.LAYER_FC:
                D = N.errors @ self._fc_weights(N)
            elif N.type in (capi.LAYER_AVERAGE_POOLING, capi.LAYER_MAX_POOLING):
                D = self._pooling_backward(N)
            else:
                from oracle import myea_oracle_lstm
                D = myea_oracle_lstm.error_to_input(self, l)
            if Pl.type == capi.LAYER_FC:
                da = self._ind_rnn_backward(Pl, D) if Pl.ind_rnn else D * af_derive(int(Pl.d.type_activation_function), Pl.pre, Pl.values)
                Pl.errors = self._norm_backward(Pl, Pl.z, da) if int(Pl.d.type_normalization) != capi.NORM_NONE else da
            elif Pl.type == capi.LAYER_LSTM:
                from oracle import myea_oracle_lstm
                Pl.dh = D
                myea_oracle_lstm.backward(self, p)
            else:
                Pl.errors = D
            l = p

    def update_derivative_weight(self):
        """Update_Derivative_Weight__FC + bias (Neural_Network__Update_Derivative_Weight__Loop.cpp): sums over the batch,
        never divided by the batch size."""
        k = getattr(self, "pre_training_level", 0)
        trained = (k, len(self.layers) - k) if k else range(1, len(self.layers))
        for l in trained:
            L = self.layers[l]
            if L.type == capi.LAYER_FC:
                x = getattr(L, "dw_input", None)
                if k and l == len(self.layers) - k:   # the decoded layer read the coded layer's output
                    x = self.layers[k].values
                elif x is None:
                    x = self.layers[L.input_layer].values
                i = L.idx
                self._g()[i["first_connection_index"]:i["first_connection_index"] + L.n_out * L.n_in] += (L.errors.T @ x).ravel()
                if L.ind_rnn and self.T > 1:   # Update_Derivative_Weight__FC_Ind_RNN: dAF of step t with the output of step t - 1
                    n = L.values.shape[0] // self.T
                    self._g()[i["first_connection_index"] + L.n_out * L.n_in:i["last_connection_index"]] += (L.dAF[n:] * L.values[:-n]).sum(0, dtype=self.dt)
                if int(L.d.type_normalization) == capi.NORM_NONE:
                    self._g()[i["first_bias_connection_index"]:i["first_bias_connection_index"] + L.n_out] += L.errors.sum(0, dtype=self.dt)
            elif L.type == capi.LAYER_LSTM:
                from oracle import myea_oracle_lstm
                myea_oracle_lstm.update_derivative_weight(self, l)

    def update_parameter(self, training_size=None, opt=None, batch=None):
        """Update_Parameter (Neural_Network.cpp:4719-4900): clip (Neural_Network__Clip_Gradient.cpp:82-94), optimizer
        (Neural_Network__Adam.cpp:39-95, __AMSGrad.cpp, __AdaBound.cpp, __AMSBound.cpp, __Gradient_Descent*.cpp,
        __Nesterov_Accelerated_Gradient.cpp), derivatives reset to zero.  Update_Parameter's own L2 call is a no-op in
        the reference (argument order), only the decoupled weight decay inside the optimizers acts."""
        o = opt or self.opt
        dt = self.dt
        N = training_size or self.B
        g, w = self._g(), self._p()
        if self.allreduce is not None:       # Merge_Derivatives_Parameters across ranks
            g[:] = self.allreduce(g)
        if o.use_clip_gradient:
            norm = np.sqrt((g * g).sum(dtype=dt))
            if norm >= dt(o.clip_gradient):
                g *= dt(o.clip_gradient) / norm
        self.time_step = dt(self.time_step + 1)
        t = self.time_step
        wd = dt(o.regularization__weight_decay)
        if wd != 0 and o.use_normalized_weight_decay:
            wd = wd * np.sqrt(dt(batch or self.B) / (dt(N) * dt(o.epoch_time_step if o.epoch_time_step > 0 else 1.0)))
        decay = self.buf[capi.BUF_MASK_REGULARIZED] * wd * w if wd != 0 else 0
        kind = int(o.type_optimizer_function)
        b1, b2, eps = dt(o.adam_beta1), dt(o.adam_beta2), dt(o.adam_epsilon)
        if kind == capi.OPT_NOSADAM:
            # Neural_Network__NosAdam.cpp:97-160: beta2_t = B / (B + t^-gamma), then B += t^-gamma; bias correction with the fixed beta2
            pw = np.power(t, -dt(o.adam_gamma if o.adam_gamma > 0 else 0.1), dtype=dt)
            prev = dt(getattr(self, "nosadam_previous_beta2", 0.0))
            b2t = prev / (prev + pw)
            self.nosadam_previous_beta2 = dt(prev + pw)
            lr = dt(o.adam_learning_rate)
            lr_t = lr * np.sqrt(dt(1) - np.power(b2, t, dtype=dt)) / (dt(1) - np.power(b1, t, dtype=dt)) if o.use_adam_bias_correction else lr
            m, v = self.buf[capi.BUF_FIRST_MOMENT], self.buf[capi.BUF_SECOND_MOMENT]
            m[:] = b1 * m + (dt(1) - b1) * g
            v[:] = b2t * v + (dt(1) - b2t) * g * g
            w -= lr_t * m / (np.sqrt(v) + eps) + decay
        elif kind in (capi.OPT_ADAM, capi.OPT_AMSGRAD, capi.OPT_ADABOUND, capi.OPT_AMSBOUND):
            lr = dt(o.adam_learning_rate)
            lr_t = lr * np.sqrt(dt(1) - np.power(b2, t, dtype=dt)) / (dt(1) - np.power(b1, t, dtype=dt)) if o.use_adam_bias_correction else lr
            m, v = self.buf[capi.BUF_FIRST_MOMENT], self.buf[capi.BUF_SECOND_MOMENT]
            m[:] = b1 * m + (dt(1) - b1) * g
            v[:] = b2 * v + (dt(1) - b2) * g * g
            vv = v
            if kind in (capi.OPT_AMSGRAD, capi.OPT_AMSBOUND):
                vh = self.buf[capi.BUF_SECOND_MOMENT_HAT]
                vh[:] = np.maximum(vh, v)
                vv = vh
            if kind in (capi.OPT_ADAM, capi.OPT_AMSGRAD):
                w -= lr_t * m / (np.sqrt(vv) + eps) + decay
            else:
                lo = dt(o.learning_rate_final) * (dt(1) - dt(1) / (dt(o.learning_gamma) * t + dt(1)))
                hi = dt(o.learning_rate_final) * (dt(1) + dt(1) / (dt(o.learning_gamma) * t))
                w -= np.clip(lr_t / (np.sqrt(vv) + eps), lo, hi) * m + decay
        elif kind == capi.OPT_IRPROP_PLUS:
            # Update_Parameter__iRPROP_plus__Loop (Neural_Network__iRPROP_plus.cpp:30-120); the first-moment buffer holds
            # the previous derivatives, the second-moment buffer the previous steps (0 = rprop_delta_zero, what
            # Clear_Optimizer, Train.cpp:163-190, writes there); no decay term on this path
            d = lambda v, dflt: dt(v) if v > 0 else dt(dflt)
            inc, dec = d(o.rprop_increase_factor, 1.2), d(o.rprop_decrease_factor, 0.5)
            dmin, dmax, dzero = d(o.rprop_delta_min, 1e-6), d(o.rprop_delta_max, 50.0), d(o.rprop_delta_zero, 0.1)
            pd, step, prev = self.buf[capi.BUF_FIRST_MOMENT], self.buf[capi.BUF_SECOND_MOMENT], self.buf[capi.BUF_PREVIOUS_DELTA]
            step[step == 0] = dzero
            same = pd * g
            up, down = same > 0, same < 0
            sign = (g > 0).astype(dt) - (g < 0).astype(dt)
            step[up] = np.minimum(step[up] * inc, dmax)
            step[down] = np.maximum(step[down] * dec, dmin)
            if o.loss_rprop > o.previous_loss_rprop:
                w[down] -= prev[down]
            prev[~down] = -sign[~down] * step[~down]
            w[~down] += prev[~down]
            pd[:] = np.where(down, dt(0), g)
        else:
            lr, mom = dt(o.learning_rate), dt(o.learning_momentum)
            if mom == 0:
                w -= lr * g + decay
            else:
                prev = self.buf[capi.BUF_PREVIOUS_DELTA]
                prev[:] = lr * g + mom * prev
                if o.use_nesterov:
                    w -= mom * prev - lr * g + decay
                else:
                    w -= prev + decay
        # independently recurrent layers: recurrent weights kept inside +-(MAG / k)^(1/T) (…Constraint_Recurrent_Weight.cpp:43-80,
        # :317-334), MAG = clip(clip_gradient, 2, 10), k = 0.9^(T/10) for symmetric activation functions, else 1
        for L in self.layers[1:]:
            if getattr(L, "ind_rnn", False):
                cg = float(self.desc.clip_gradient) or 1.0
                mag = np.float32(min(max(cg, 2.0), 10.0))
                sym = int(L.d.type_activation_function) in (capi.AF_COSINE_SYMMETRIC, capi.AF_ELLIOT_SYMMETRIC, capi.AF_GAUSSIAN_SYMMETRIC,
                                                            capi.AF_LINEAR_PIECE_SYMMETRIC, capi.AF_SINE_SYMMETRIC, capi.AF_TANH, capi.AF_TANH_STEPWISE,
                                                            capi.AF_THRESHOLD_SYMMETRIC)
                t = np.float32(self.T)
                b = np.power(mag / np.power(np.float32(0.9), t / np.float32(10)), np.float32(1) / t) if sym else np.power(mag, np.float32(1) / t)
                a0 = L.idx["first_connection_index"] + L.n_out * L.n_in
                np.clip(w[a0:L.idx["last_connection_index"]], -dt(b), dt(b), out=w[a0:L.idx["last_connection_index"]])
        c = dt(o.regularization__max_norm_constraints)
        if c != 0:   # …Max_Norm_Constraints.cpp:147-165 + Euclidean_Norm__Loop :48-88: one weight row per neuron of every FC layer
            for L in self.layers[1:]:
                if L.type != capi.LAYER_FC:
                    continue
                W = self._fc_weights(L)   # a view into the parameter buffer
                norms = np.sqrt((W * W).sum(axis=1, dtype=dt))
                big = norms >= c
                W[big] *= (c / norms[big])[:, None]
            # LSTM blocks (…Max_Norm_Constraints.cpp:167-310): every run of weights is its own vector - per cell the input and
            # the recurrent weights of the cell input, per block those of the three gates and the three peephole runs.  A
            # run that starts at parameter 0 is passed over (`first_index > start_index` with start 0).
            for L in self.layers[1:]:
                if L.type != capi.LAYER_LSTM:
                    continue
                dirs = 2 if L.d.use_bidirectional else 1
                cpb, K, I, S = max(1, int(L.d.unit_parameters[1])), int(L.d.unit_parameters[0]), L.n_in, L.idx["block_stride"]
                C = K * cpb
                p = self._p()
                for k in range(dirs * K):
                    base = L.idx["first_connection_index"] + k * S
                    runs = []
                    for j in range(cpb):
                        runs += [(base + j * (I + C), I), (base + j * (I + C) + I, C)]
                    g0 = base + cpb * (I + C)
                    runs += [(g0 + g * I, I) for g in range(3)] + [(g0 + 3 * I + g * C, C) for g in range(3)]
                    runs += [(g0 + 3 * I + 3 * C + g * cpb, cpb) for g in range(3)]
                    for a, n in runs:
                        if a == 0:
                            continue
                        v = p[a:a + n]
                        norm = np.sqrt((v * v).sum(dtype=dt))
                        if norm >= c:
                            v *= c / norm
        g[:] = 0
