"""The five benchmark / parity workloads as descriptors plus seeded synthetic tensors.

Each builder returns a `Workload`: network descriptor, optimizer descriptor and a `materialize(net_like)` routine that
writes the SAME seeded parameters, masks and coefficients into any object with the Net / RefNet method set, so the
CUDA path and the oracle start from identical state.  `scale` shrinks widths / batch / depth for parity tests; 1.0 is
the full size the throughput metric is quoted on.

Weights: Glorot-uniform, bound = gain * sqrt(6 / (fan_in + fan_out)) with the reference's gains (tanh 5/3, ReLU
sqrt(2), others 1: Neural_Network__Initialization__Glorot.cpp:22-110); biases 0; gamma 1, beta 0, running mean 0 and
running deviation 1.  LSTM recurrent matrices are orthogonal (QR of a seeded Gaussian) because the reference's own
orthogonal initializer is not implemented for LSTM layers; peepholes use the Glorot range; biases 0.
"""
import math

import numpy as np

from . import capi


class Workload:
    def __init__(self, name, desc, opt, n_in, n_out, one_hot, layers):
        self.name, self.desc, self.opt = name, desc, opt
        self.n_in, self.n_out, self.one_hot = n_in, n_out, one_hot
        self.layers = layers
        self.T = int(desc.number_recurrent_depth)
        self.B = int(desc.batch_size)
        self.input_dist = "normal"
        self.seed = 0
        self.flops_per_step = 0.0   # algorithmic GEMM flops of one full step (fwd + bwd data + bwd weight)

    # ---- synthetic batch -------------------------------------------------------------------------------------
    def batch(self, seed=None, rows=None):
        """inputs [T, B, n_in], targets [T, B, n_out]"""
        rng = np.random.default_rng(self.seed + 1000 if seed is None else seed)
        B = rows or self.B
        if self.input_dist == "uniform":
            X = rng.uniform(-1.0, 1.0, (self.T, B, self.n_in)).astype(np.float32)
        else:
            X = rng.standard_normal((self.T, B, self.n_in), dtype=np.float32)
        if self.one_hot:
            Y = np.zeros((self.T, B, self.n_out), np.float32)
            lab = rng.integers(0, self.n_out, (self.T, B))
            for t in range(self.T):
                Y[t, np.arange(B), lab[t]] = 1.0
        else:
            Y = rng.standard_normal((self.T, B, self.n_out), dtype=np.float32)
        return X, Y

    # ---- parameters ------------------------------------------------------------------------------------------
    def parameters(self, net):
        """flat [P] parameter vector for `net` (anything with sizes() and layer_index())"""
        rng = np.random.default_rng(self.seed)
        P, W, nb, nn = net.sizes()
        p = np.zeros(P, np.float32)
        for l in range(1, len(self.layers)):
            L = self.layers[l]
            li = net.layer_index(l)
            n_in, n_out = int(li.number_inputs), int(li.number_outputs)
            if L.type_layer in (capi.LAYER_FC, capi.LAYER_FC_IND_RNN):
                gain = {capi.AF_TANH: 5.0 / 3.0, capi.AF_RELU: math.sqrt(2.0)}.get(L.type_activation_function, 1.0)
                bound = gain * math.sqrt(6.0 / (n_in + n_out))
                a, b = int(li.first_connection_index), int(li.last_connection_index)
                p[a:b] = rng.uniform(-bound, bound, b - a)
                if L.type_layer == capi.LAYER_FC_IND_RNN:     # the units' recurrent weights close the layer's range
                    p[b - n_out:b] = rng.uniform(0.2, 0.9, n_out)
            elif L.type_layer == capi.LAYER_LSTM:
                dirs = 2 if L.use_bidirectional else 1
                C = n_out // dirs
                stride = int(li.block_stride)
                base = int(li.first_connection_index)
                bound_in = math.sqrt(6.0 / (n_in + C))
                if int(L.unit_parameters[1]) > 1:   # several cells per block: uniform values over the layer's whole range
                    a, b = base, int(li.last_connection_index)
                    p[a:b] = rng.uniform(-bound_in, bound_in, b - a)
                    continue
                for d in range(dirs):
                    blk = np.zeros((C, stride), np.float32)   # one row per block (1 cell per block)
                    # [W_z,in | W_z,rec | W_i,in W_f,in W_o,in | W_i,rec W_f,rec W_o,rec | p_i p_f p_o]
                    o = 0
                    blk[:, o:o + n_in] = rng.uniform(-bound_in, bound_in, (C, n_in)); o += n_in
                    blk[:, o:o + C] = _orthogonal(rng, C); o += C
                    for _ in range(3):
                        blk[:, o:o + n_in] = rng.uniform(-bound_in, bound_in, (C, n_in)); o += n_in
                    for _ in range(3):
                        blk[:, o:o + C] = _orthogonal(rng, C); o += C
                    blk[:, o:o + 3] = rng.uniform(-bound_in, bound_in, (C, 3))
                    p[base + d * C * stride: base + (d + 1) * C * stride] = blk.ravel()
        if nn:
            p[W + nb: W + nb + nn] = 1.0
        return p

    def materialize(self, net):
        """write parameters, running statistics, regularization mask, dropout / zoneout masks into `net`"""
        rng = np.random.default_rng(self.seed + 7)
        P, W, nb, nn = net.sizes()
        net.set(capi.BUF_PARAMETERS, self.parameters(net))
        if nn:
            net.set(capi.BUF_NORM_MEAN_AVERAGE, np.zeros(nn * self.T, np.float32))      # one set of averages per time step
            net.set(capi.BUF_NORM_VARIANCE_AVERAGE, np.ones(nn * self.T, np.float32))
        if self.opt.regularization__weight_decay != 0.0:
            m = np.zeros(P, np.float32)
            m[:W] = 1.0   # weights 1, biases and gamma / beta 0 (Neural_Network__Indexing.cpp:50-76)
            net.set(capi.BUF_MASK_REGULARIZED, m)
        for l in range(1, len(self.layers)):
            L = self.layers[l]
            width = int(net.layer_index(l).number_outputs)
            if L.type_dropout in (capi.DROP_BERNOULLI, capi.DROP_BERNOULLI_INVERTED):
                net.set_mask_bernoulli(l, (rng.random(self.T * width) < L.dropout_values[0]).astype(np.uint8))
            elif L.type_dropout == capi.DROP_ZONEOUT:
                n = self.T * width   # a bidirectional layer's width already counts both directions
                net.set_mask_zoneout(l, (rng.random(n) >= L.dropout_values[0]).astype(np.uint8),
                                     (rng.random(n) >= L.dropout_values[1]).astype(np.uint8))
            elif L.type_dropout == capi.DROP_SHAKEDROP:
                # drawn for every kind of net so that the seeded stream stays aligned; the compiled reference draws its
                # own coefficients while it runs (tests read them back and impose them on the other side)
                mask = (rng.random(self.B) < L.dropout_values[0]).astype(np.uint8)
                alpha = rng.uniform(-1.0, 1.0, (self.B, width)).astype(np.float32)
                beta = rng.uniform(0.0, 1.0, (self.B, width)).astype(np.float32)
                if hasattr(net, "set_shakedrop"):
                    net.set_shakedrop(l, mask, alpha, beta)


def _orthogonal(rng, n):
    q, r = np.linalg.qr(rng.standard_normal((n, n)))
    return (q * np.sign(np.diag(r))).astype(np.float32)


def _s(x, scale, lo=4, mult=1):
    v = max(lo, int(round(x * scale)))
    return (v + mult - 1) // mult * mult


def _mlp_flops(widths, B):
    f = 0.0
    for i in range(1, len(widths)):
        f += 2.0 * B * widths[i - 1] * widths[i] * (3 if i > 1 else 2)   # no input error for the first layer
    return f


def c1_mlp(scale=1.0, batch=None):
    """config 1: MLP 64-256-256-10, tanh / softmax, cross-entropy, batch 128, Adam"""
    w = [_s(64, scale), _s(256, scale), _s(256, scale), 10]
    B = batch or _s(128, scale)
    layers = [capi.fc(w[0]), capi.fc(w[1], capi.AF_TANH), capi.fc(w[2], capi.AF_TANH), capi.fc(w[3], capi.AF_SOFTMAX)]
    wl = Workload("C1 MLP 64-256-256-10", capi.net(layers, B, loss=capi.LOSS_CE, accuracy=capi.ACC_CE), capi.opt(capi.OPT_ADAM),
                  w[0], w[3], True, layers)
    wl.input_dist = "uniform"
    wl.flops_per_step = _mlp_flops(w, B)
    return wl


def c2_wide_mlp(scale=1.0, batch=None, hidden_layers=8):
    """config 2: 8 x FC 4096 + BatchNorm (before ReLU) + ReLU + inverted dropout 0.5, FC 4096 -> 1024 linear, MSE, batch 4096"""
    H, O = _s(4096, scale, mult=4), _s(1024, scale, mult=4)
    B = batch or _s(4096, scale)
    layers = [capi.fc(H)]
    for _ in range(hidden_layers):
        layers.append(capi.fc(H, capi.AF_RELU, capi.NORM_BN, capi.DROP_BERNOULLI_INVERTED, (0.5, 0.0, 0.0)))
    layers.append(capi.fc(O, capi.AF_LINEAR))
    wl = Workload("C2 wide MLP 8x4096 BN ReLU dropout", capi.net(layers, B, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE),
                  capi.opt(capi.OPT_ADAM), H, O, False, layers)
    wl.flops_per_step = _mlp_flops([H] * (hidden_layers + 1) + [O], B)
    return wl


def c3_lstm(scale=1.0, batch=None, T=None):
    """config 3: 2-layer LSTM with peepholes, input 512, hidden 1024, T 64, batch 256, MSE on the last step, AMSGrad"""
    I, H = _s(512, scale), _s(1024, scale)
    T = T or _s(64, scale, lo=3)
    B = batch or _s(256, scale)
    layers = [capi.fc(I), capi.lstm(H), capi.lstm(H), capi.fc(H, capi.AF_LINEAR)]
    wl = Workload("C3 2xLSTM(1024) peephole", capi.net(layers, B, T=T, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE,
                                                         time_delays=T - 1), capi.opt(capi.OPT_AMSGRAD), I, H, False, layers)
    rows = float(T * B)
    f = 2.0 * rows * 4 * H * (I + H) * 2          # layer 1: forward + weight derivative (no input error)
    f += 2.0 * rows * 4 * H * H                    # layer 1: recurrent error propagation
    f += 2.0 * rows * 4 * H * (H + H) * 3          # layer 2: forward, error propagation (recurrent + to layer 1), weights
    f += 2.0 * rows * H * H * 3                    # output layer
    wl.flops_per_step = f
    return wl


def c4_residual(scale=1.0, batch=None, blocks=6):
    """config 4: FC 1024->2048, 6 residual blocks [FC 2048, BRN + ELU + FC 2048] with ShakeDrop 0.5, softmax 1000, AdaBound, wd 1e-4"""
    I, H, O = _s(1024, scale, mult=4), _s(2048, scale, mult=4), _s(1000, scale, lo=5)
    B = batch or _s(2048, scale)
    layers = [capi.fc(I), capi.fc(H, capi.AF_ELU)]
    for _ in range(blocks):
        layers += [capi.residual(2, capi.DROP_SHAKEDROP, (0.5, 0.0, 0.0)), capi.fc(H, capi.AF_ELU),
                   capi.fc(H, capi.AF_ELU, capi.NORM_BRN)]
    layers.append(capi.fc(O, capi.AF_SOFTMAX))
    wl = Workload("C4 residual MLP BRN ELU ShakeDrop", capi.net(layers, B, loss=capi.LOSS_CE, accuracy=capi.ACC_CE, r_max=3.0, d_max=5.0),
                  capi.opt(capi.OPT_ADABOUND, final_lr=0.1, weight_decay=1e-4), I, O, True, layers)
    wl.input_dist = "uniform"
    wl.flops_per_step = _mlp_flops([I] + [H] * (2 * blocks + 1) + [O], B)
    return wl


def c5_bilstm(scale=1.0, batch=None, T=None, out=None):
    """config 5: bidirectional LSTM, input 1024, hidden 2048 per direction, T 128, batch 1024, zoneout 0.1, clip 1.0, Adam"""
    I, H = _s(1024, scale), _s(2048, scale)
    O = out or _s(1024, scale)
    T = T or _s(128, scale, lo=3)
    B = batch or _s(1024, scale)
    layers = [capi.fc(I), capi.lstm(H, bidirectional=True, dropout=capi.DROP_ZONEOUT, p=(0.1, 0.1, 0.0)), capi.fc(O, capi.AF_LINEAR)]
    wl = Workload("C5 BiLSTM(2048) zoneout clip", capi.net(layers, B, T=T, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE),
                  capi.opt(capi.OPT_ADAM, clip=1.0), I, O, False, layers)
    rows = float(T * B)
    wl.flops_per_step = 2 * (2.0 * rows * 4 * H * (I + H) * 2 + 2.0 * rows * 4 * H * H) + 2.0 * rows * 2 * H * O * 3
    return wl


BUILDERS = {"c1": c1_mlp, "c2": c2_wide_mlp, "c3": c3_lstm, "c4": c4_residual, "c5": c5_bilstm}
