"""Parity cases shared by the golden-fixture generator, the CPU tests and the GPU tests: reduced-shape versions of the
five benchmark configurations plus targeted variants (every optimizer, plain Bernoulli dropout, batch renormalization,
clipping, weight decay, ragged widths that are not multiples of any tile)."""
import numpy as np

from myea_b200 import capi, workloads


def _mlp_variant(name, hidden, af, opt, B=24, n_in=13, n_out=5, norm=capi.NORM_NONE, drop=capi.DROP_NONE, p=0.6, loss=capi.LOSS_MSE,
                 out_af=capi.AF_LINEAR, **kw):
    layers = [capi.fc(n_in)] + [capi.fc(h, af, norm, drop, (p, 0, 0)) for h in hidden] + [capi.fc(n_out, out_af)]
    acc = capi.ACC_CE if loss == capi.LOSS_CE else capi.ACC_DISTANCE
    wl = workloads.Workload(name, capi.net(layers, B, loss=loss, accuracy=acc, **kw), opt, n_in, n_out, loss == capi.LOSS_CE, layers)
    return wl


CASES = {
    "c1_small": lambda: workloads.c1_mlp(scale=0.25),
    "c2_small": lambda: workloads.c2_wide_mlp(scale=1.0 / 64, batch=48, hidden_layers=3),
    "mlp_ragged_tanh_adam": lambda: _mlp_variant("ragged", [37, 19], capi.AF_TANH, capi.opt(capi.OPT_ADAM), B=21, n_in=11, n_out=3),
    "mlp_sigmoid_amsgrad": lambda: _mlp_variant("amsgrad", [20], capi.AF_SIGMOID, capi.opt(capi.OPT_AMSGRAD), out_af=capi.AF_SIGMOID),
    "mlp_brn_elu_adabound_wd": lambda: _mlp_variant("brn", [28, 28], capi.AF_ELU, capi.opt(capi.OPT_ADABOUND, weight_decay=1e-3), norm=capi.NORM_BRN,
                                                    r_max=3.0, d_max=5.0, momentum=0.9),
    "mlp_bernoulli_amsbound_clip": lambda: _mlp_variant("amsbound", [32], capi.AF_LEAKY_RELU, capi.opt(capi.OPT_AMSBOUND, clip=0.5), drop=capi.DROP_BERNOULLI),
    # every width and the batch above 128 (and ragged): the three contractions of each layer run on the 256 x 256
    # tensor-core kernel from operand panels shared between the forward and the backward readings
    "mlp_wide_bn_dropout_adam": lambda: _mlp_variant("wide", [144, 132], capi.AF_RELU, capi.opt(capi.OPT_ADAM), B=130, n_in=136, n_out=129,
                                                     norm=capi.NORM_BN, drop=capi.DROP_BERNOULLI_INVERTED, p=0.5),
    "mlp_tanh_nosadam": lambda: _mlp_variant("nosadam", [20, 12], capi.AF_TANH, capi.opt(capi.OPT_NOSADAM, nosadam_gamma=0.1)),
    # descent with a large rate so that rows do cross the bound and get rescaled
    "mlp_relu_momentum_max_norm": lambda: _mlp_variant("maxnorm", [16, 16], capi.AF_RELU, capi.opt(capi.OPT_GD, gd_lr=0.05, momentum=0.9, max_norm=0.8)),
    # sign-based steps of 0.1 from the first update on: a derivative's sign, not its size, decides, so the case keeps to
    # tanh units (no exactly-zero derivatives that a rounding difference could push to either side)
    "mlp_tanh_irprop_plus": lambda: _mlp_variant("irprop", [20, 12], capi.AF_TANH, capi.opt(capi.OPT_IRPROP_PLUS)),
    "mlp_relu_gd": lambda: _mlp_variant("gd", [16, 16], capi.AF_RELU, capi.opt(capi.OPT_GD, gd_lr=0.01)),
    "mlp_selu_momentum": lambda: _mlp_variant("mom", [16], capi.AF_SELU, capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9)),
    "mlp_tanh_nesterov_ce": lambda: _mlp_variant("nag", [16], capi.AF_TANH, capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9, nesterov=True),
                                                 loss=capi.LOSS_CE, out_af=capi.AF_SOFTMAX, n_out=6),
}

STEPS = 2


def run_steps(net, wl, steps=STEPS, shake=None):
    """the reference's training sequence (Dataset.cpp:637-691, 7654-7690) on one seeded batch; returns what a parity
    check compares.  `shake`: per-step ShakeDrop draws {layer: (mask, alpha, beta)} to impose (a list, one dict per
    step); the compiled reference draws its own and reports them (they come back under the key "shake")."""
    X, Y = wl.batch()
    wl.materialize(net)
    out = {"shake": []}
    for it in range(steps):
        if hasattr(net, "next_shakedrop"):
            out["shake"].append(net.next_shakedrop())
        elif shake is not None:
            for layer, (m, a, b) in shake[it].items():
                net.set_shakedrop(layer, m, a, b)
        net.reset_loss()
        net.forward(X)
        net.compute_error(Y)
        net.backward()
        net.update_derivative_weight()
        out["grad%d" % it] = net.get(capi.BUF_DERIVATIVES)
        s, n, a = net.loss()
        out["loss%d" % it] = [s, float(n), a]
        if it == 0:
            out["output_last"] = net.outputs(len(wl.layers) - 1)
        net.update_parameter()
        out["param%d" % it] = net.get(capi.BUF_PARAMETERS)
    kind = wl.opt.type_optimizer_function
    if kind == capi.OPT_IRPROP_PLUS:     # previous derivatives (they share the first-moment slot); steps and delta weights ride along
        out["m"] = net.get(capi.BUF_PREVIOUS_DERIVATIVES)
        out["rprop_steps"] = net.get(capi.BUF_PREVIOUS_STEPS)
        out["rprop_delta"] = net.get(capi.BUF_PREVIOUS_DELTA)
    else:
        out["m"] = net.get(capi.BUF_FIRST_MOMENT) if kind != capi.OPT_GD else out["param0"] * 0
    if net.sizes()[3]:
        out["norm_mean_avg"] = net.get(capi.BUF_NORM_MEAN_AVERAGE)
        out["norm_sigma_avg"] = net.get(capi.BUF_NORM_VARIANCE_AVERAGE)
    out["index_map"] = [list(net.layer_index(l).as_tuple()) for l in range(len(wl.layers))]
    out["sizes"] = list(net.sizes())
    return out


def _lstm_case(name, opt, T=5, B=6, n_in=7, H=8, layers=2, zoneout=None, delays=None, out=None):
    out = out or H
    ls = [capi.fc(n_in)]
    for _ in range(layers):
        ls.append(capi.lstm(H, dropout=capi.DROP_ZONEOUT if zoneout else capi.DROP_NONE, p=(zoneout or 0.0, zoneout or 0.0, 0.0)))
    ls.append(capi.fc(out, capi.AF_LINEAR))
    wl = workloads.Workload(name, capi.net(ls, B, T=T, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE,
                                           time_delays=(T - 1 if delays is None else delays)), opt, n_in, out, False, ls)
    return wl


CASES.update({
    "c3_small": lambda: workloads.c3_lstm(scale=1.0 / 32, batch=10, T=6),
    "lstm1_all_steps_adam": lambda: _lstm_case("lstm1", capi.opt(capi.OPT_ADAM), layers=1, delays=0, H=12, out=16),
    "lstm2_zoneout_clip": lambda: _lstm_case("lstm2z", capi.opt(capi.OPT_ADAM, clip=1.0), zoneout=0.3, delays=2),
})


# Larger shapes that reach the kernels only big layers use (256 x 256 tensor-core tiles, column-read operand panels,
# 8-cells-per-thread and persistent LSTM steps).  Compared with the compiled reference on the GPU box, without a
# committed fixture (the parameter vectors would be megabytes).  Momentum descent, an update that is linear in the
# derivatives, so that the 1e-4 bound holds for every updated parameter.  Under Adam-type updates it does not, and the
# numbers are (one step at the stated widths, tests/test_full_width_parity_gpu.py): derivatives agree to 1.3e-6 (C1),
# 1.1e-5 (C2), 4.0e-6 (C3), 5.5e-6 (C4) of each tensor's largest, yet 1.5e-5 to 1.9e-4 of the UPDATED weights differ by
# more than 1e-4 - all of them elements whose float64 derivative is below 1e-4 of the tensor's largest, where the first
# Adam step lr * sign(g) is decided by rounding noise; that test arbitrates them with the reference's float64 build.
CASES_ORACLE_ONLY = {
    "lstm_wide_nesterov": lambda: _lstm_case("lstm_wide", capi.opt(capi.OPT_GD, gd_lr=0.001, momentum=0.9, nesterov=True), T=4, B=16, n_in=136,
                                             H=192, layers=1, out=192),
    "lstm2_wide_zoneout": lambda: _lstm_case("lstm2_wide", capi.opt(capi.OPT_GD, gd_lr=0.001, momentum=0.9), T=3, B=136, n_in=64, H=192, layers=2,
                                             out=192, zoneout=0.2, delays=0),
    "residual_wide_brn_shakedrop": lambda: _res_wide(),
}




# every activation function of the reference besides the ones the cases above already use (hidden layers of a small
# network, one of them normalized so that the derivative sees the normalized summation; momentum descent)
AF_NAMES = {capi.AF_COSINE: "cosine", capi.AF_COSINE_SYMMETRIC: "cosine_symmetric", capi.AF_ELLIOT: "elliot",
            capi.AF_ELLIOT_SYMMETRIC: "elliot_symmetric", capi.AF_GAUSSIAN: "gaussian", capi.AF_GAUSSIAN_SYMMETRIC: "gaussian_symmetric",
            capi.AF_ISRU: "isru", capi.AF_ISRLU: "isrlu", capi.AF_LINEAR_PIECE: "linear_piece",
            capi.AF_LINEAR_PIECE_SYMMETRIC: "linear_piece_symmetric", capi.AF_PARAMETRIC_RELU: "parametric_relu", capi.AF_SINE: "sine",
            capi.AF_SIGMOID_STEPWISE: "sigmoid_stepwise", capi.AF_SINE_SYMMETRIC: "sine_symmetric", capi.AF_TANH_STEPWISE: "tanh_stepwise",
            capi.AF_LEAKY_RELU: "leaky_relu"}
for _af, _n in AF_NAMES.items():
    CASES["mlp_af_" + _n] = (lambda af=_af, n=_n: _mlp_variant("af_" + n, [16, 12], af, capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9), B=9, n_in=10,
                                                            n_out=4, norm=capi.NORM_BN if af in (capi.AF_GAUSSIAN, capi.AF_ISRU, capi.AF_SINE) else capi.NORM_NONE))


def _pooling_case(name, kind, pars, norm=capi.NORM_NONE, af=capi.AF_TANH, recurrent=False):
    """a pooling layer (kernel, stride, padding, dilation) over a hidden layer's units, followed by more layers"""
    opt = capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9)
    if recurrent == "fc":
        ls = [capi.fc(10), capi.fc(12, af), capi.pooling(kind, *pars), capi.fc(7, capi.AF_RELU), capi.fc(5, capi.AF_LINEAR)]
        return workloads.Workload(name, capi.net(ls, 6, T=3, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE, time_delays=0), opt, 10, 5, False, ls)
    if recurrent:
        # (the output layer has at least as many biases as the LSTM layer has cells: its shifted bias base reaches that far)
        ls = [capi.fc(7), capi.lstm(8), capi.pooling(kind, *pars), capi.fc(10, capi.AF_LINEAR)]
        return workloads.Workload(name, capi.net(ls, 5, T=4, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE, time_delays=1), opt, 7, 10, False, ls)
    ls = [capi.fc(10), capi.fc(12, af, norm=norm), capi.pooling(kind, *pars), capi.fc(7, capi.AF_RELU), capi.fc(5, capi.AF_LINEAR)]
    return workloads.Workload(name, capi.net(ls, 6, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE), opt, 10, 5, False, ls)


CASES.update({
    "mlp_average_pooling_padded": lambda: _pooling_case("avgpool", capi.LAYER_AVERAGE_POOLING, (3, 2, 1, 1)),
    "mlp_average_pooling_dilated": lambda: _pooling_case("avgpool_d", capi.LAYER_AVERAGE_POOLING, (2, 1, 0, 2)),
    "mlp_max_pooling_bn_relu": lambda: _pooling_case("maxpool", capi.LAYER_MAX_POOLING, (3, 2, 1, 1), norm=capi.NORM_BN, af=capi.AF_RELU),
    "recurrent_fc_max_pooling": lambda: _pooling_case("rec_maxpool", capi.LAYER_MAX_POOLING, (3, 2, 1, 1), recurrent="fc"),
    "lstm_max_pooling": lambda: _pooling_case("lstm_maxpool", capi.LAYER_MAX_POOLING, (2, 2, 0, 1), recurrent=True),
    "lstm_average_pooling": lambda: _pooling_case("lstm_avgpool", capi.LAYER_AVERAGE_POOLING, (2, 2, 0, 1), recurrent=True),
})


def autoencoder_case(dropout=capi.DROP_NONE):
    """a five-layer autoencoder 10-7-4-7-10 for the pre-training passes (levels 1 and 2), optional dropout on the first
    hidden layer (the one that feeds the coded layer at level 2)"""
    ls = [capi.fc(10), capi.fc(7, capi.AF_TANH, dropout=dropout, p=(0.8, 0.0, 0.0)), capi.fc(4, capi.AF_TANH), capi.fc(7, capi.AF_ELU),
          capi.fc(10, capi.AF_LINEAR)]
    d = capi.net(ls, 8, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE)
    d.type_network = capi.NET_AUTOENCODER
    return workloads.Workload("autoencoder", d, capi.opt(capi.OPT_GD, gd_lr=0.05, momentum=0.9), 10, 10, False, ls)


def run_pre_training(net, wl, levels=(1, 2, 0), steps=2):
    """the training sequence at every pre-training level in turn (targets = inputs): derivatives, loss, the answering
    layer's outputs and the updated parameters of every step"""
    X, _ = wl.batch()
    wl.materialize(net)
    n = len(wl.layers)
    out = {}
    for level in levels:
        net.set_pre_training_level(level)
        for it in range(steps):
            net.reset_loss()
            net.forward(X); net.compute_error(X); net.backward(); net.update_derivative_weight()
            key = "level%d_step%d_" % (level, it)
            out[key + "grad"] = net.get(capi.BUF_DERIVATIVES)
            s_, n_, a_ = net.loss()
            out[key + "loss"] = [s_, float(n_), a_]
            out[key + "output"] = net.outputs(n - level if level else n - 1)
            net.update_parameter()
            out[key + "param"] = net.get(capi.BUF_PARAMETERS)
    net.set_pre_training_level(0)
    return out


def _ind_rnn_case(name, af, norm=capi.NORM_NONE, dropout=capi.DROP_NONE, T=4, stacked=False, lr=0.01):
    """independently recurrent fully connected layers (Ind-RNN): y_t = f(W x_t + b + u * y_{t-1})"""
    ls = [capi.fc(7), capi.fc_ind_rnn(9, af, norm=norm, dropout=dropout, p=(0.8, 0.0, 0.0))]
    if stacked:
        ls.append(capi.fc_ind_rnn(8, af))
    ls += [capi.fc(6, capi.AF_TANH), capi.fc(5, capi.AF_LINEAR)]
    return workloads.Workload(name, capi.net(ls, 6, T=T, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE, time_delays=1, **({"momentum": 0.9} if norm else {})),
                              capi.opt(capi.OPT_GD, gd_lr=lr, momentum=0.9), 7, 5, False, ls)


CASES.update({
    "ind_rnn_relu": lambda: _ind_rnn_case("indrnn", capi.AF_RELU),
    "ind_rnn_tanh_stacked_dropout": lambda: _ind_rnn_case("indrnn2", capi.AF_TANH, dropout=capi.DROP_BERNOULLI_INVERTED, stacked=True),
    "ind_rnn_batch_norm": lambda: _ind_rnn_case("indrnn_bn", capi.AF_TANH, norm=capi.NORM_BN),
    # a large step pushes recurrent weights against their bound +-2^(1/T) (the layer's weight constraint)
    "ind_rnn_relu_weights_at_bound": lambda: _ind_rnn_case("indrnn_clip", capi.AF_RELU, T=3, lr=1.5),
})


def _lstm_blocks_case(name, opt, cpb, T=4, B=5, n_in=7, blocks=(4, 3), out=12, zoneout=0.3, delays=1):
    """LSTM blocks of `cpb` cells each (the cells of a block share its gates); the output layer is at least as wide as
    the last LSTM layer has cells, as the reference's shifted bias base requires"""
    ls = [capi.fc(n_in)]
    for i, k in enumerate(blocks):
        z = zoneout if i == 0 else None
        ls.append(capi.lstm(k, cells_per_block=cpb, dropout=capi.DROP_ZONEOUT if z else capi.DROP_NONE, p=(z or 0.0, z or 0.0, 0.0)))
    ls.append(capi.fc(out, capi.AF_LINEAR))
    return workloads.Workload(name, capi.net(ls, B, T=T, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE, time_delays=delays), opt, n_in, out, False, ls)


def _recurrent_fc_norm_case(norm):
    """(the reference refuses a network that mixes the two kinds of normalization when it has more than one time step)"""
    ls = [capi.fc(7), capi.fc(10, capi.AF_TANH, norm=norm), capi.fc(8, capi.AF_RELU, norm=norm, dropout=capi.DROP_BERNOULLI, p=(0.8, 0.0, 0.0)),
          capi.fc(5, capi.AF_LINEAR)]
    return workloads.Workload("rec_fc_bn", capi.net(ls, 6, T=3, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE, time_delays=0, r_max=3.0, d_max=5.0, momentum=0.9),
                              capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9), 7, 5, False, ls)


def _lstm_fc_case(name, opt, T=4, B=6, n_in=7, below=10, H=8, above=6, out=5, drop_below=capi.DROP_BERNOULLI, drop_above=capi.DROP_BERNOULLI_INVERTED,
                  delays=1, cells_per_block=1, norm_below=capi.NORM_NONE, norm_above=capi.NORM_NONE):
    """fully connected hidden layers on both sides of an LSTM layer, each with its own per-time-step dropout mask"""
    ls = [capi.fc(n_in), capi.fc(below, capi.AF_TANH, norm=norm_below, dropout=drop_below, p=(0.7, 0.0, 0.0)), capi.lstm(H, cells_per_block=cells_per_block),
          capi.fc(above, capi.AF_RELU, norm=norm_above, dropout=drop_above, p=(0.8, 0.0, 0.0)), capi.fc(out, capi.AF_LINEAR)]
    kw = dict(r_max=3.0, d_max=5.0, momentum=0.9) if capi.NORM_BRN in (norm_below, norm_above) else {}
    return workloads.Workload(name, capi.net(ls, B, T=T, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE, time_delays=delays, **kw), opt, n_in, out, False, ls)


def _res_wide():
    return _res_case("res_wide", capi.opt(capi.OPT_GD, gd_lr=0.001, momentum=0.9), B=136, n_in=40, H=144, out=7, blocks=2)


CASES.update({
    # blocks of several cells, and a layer width that is no multiple of 4
    "lstm_two_cells_per_block": lambda: _lstm_blocks_case("lstm_cpb2", capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9), 2),
    "lstm_three_cells_per_block_adam": lambda: _lstm_blocks_case("lstm_cpb3", capi.opt(capi.OPT_ADAM), 3, blocks=(3, 2), delays=0),
    "lstm_width_7": lambda: _lstm_case("lstm_w7", capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9), H=7, out=9, delays=1),
    # max-norm constraint on LSTM weight runs (the run that starts at parameter 0 is passed over, as in the reference)
    "lstm_max_norm": lambda: _lstm_case("lstm_mn", capi.opt(capi.OPT_GD, gd_lr=0.05, momentum=0.9, max_norm=0.6), layers=1, H=8, out=8, delays=0),
    "lstm_two_cells_max_norm": lambda: _lstm_blocks_case("lstm_cpb2_mn", capi.opt(capi.OPT_GD, gd_lr=0.05, momentum=0.9, max_norm=0.5), 2),
    # L1 / L2 penalties: accepted and without effect (the reference's call hands its arguments over in the wrong order)
    "mlp_l1_l2_without_effect": lambda: _mlp_variant("l1l2", [14], capi.AF_TANH, capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9, l1=0.05, l2=0.05), B=8),
    # batch (re)normalization of fully connected layers in a recurrent network: every time step has its own statistics
    "recurrent_fc_batch_norm": lambda: _recurrent_fc_norm_case(capi.NORM_BN),
    "recurrent_fc_batch_renorm": lambda: _recurrent_fc_norm_case(capi.NORM_BRN),
    # recurrent networks with fully connected hidden layers around the LSTM layer and Bernoulli dropout drawn per time step
    "lstm_between_fc_bernoulli": lambda: _lstm_fc_case("lstm_fc", capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9)),
    # zero-padded identity: the block narrower / wider than its shortcut, and the residual layer's own normalization
    "res_zero_pad_narrow_block": lambda: _res_case("res_np", capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9), H=14, block_width=9, blocks=1),
    "res_zero_pad_wide_block": lambda: _res_case("res_wp", capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9), H=10, block_width=15, blocks=1),
    "res_block_level_norm": lambda: _res_case("res_bn", capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9), norm=capi.NORM_NONE, af=capi.AF_TANH,
                                              block_norm=capi.NORM_BN, blocks=2),
})


def _bilstm_case(name, opt, T=5, B=6, n_in=7, H=8, out=5, zoneout=None):
    ls = [capi.fc(n_in), capi.lstm(H, bidirectional=True, dropout=capi.DROP_ZONEOUT if zoneout else capi.DROP_NONE,
                                   p=(zoneout or 0.0, zoneout or 0.0, 0.0)), capi.fc(out, capi.AF_LINEAR)]
    return workloads.Workload(name, capi.net(ls, B, T=T, loss=capi.LOSS_MSE, accuracy=capi.ACC_DISTANCE), opt, n_in, out, False, ls)


# The reference's own bidirectional LSTM is unusable as an oracle (its two directions share overlapping buffers and the
# next layer gets a one-direction fan-in); these cases are checked against the numpy restatement only.
# A normalized layer in a network that also has LSTM layers: the reference itself crashes while it is being built
# (Set__Layer_Normalization -> Allocate__Parameter__Normalization -> Reallocate__Parameter ->
# Reset__Parameter__Normalized_Unit writes through the LSTM units' normalized-unit pointers, which are not set up),
# whatever the order of the calls, so there is no reference run to compare with.
CASES_WITHOUT_REFERENCE = {
    "lstm_between_fc_batch_norm": lambda: _lstm_fc_case("lstm_fc_bn", capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9), drop_below=capi.DROP_NONE,
                                                        norm_below=capi.NORM_BN, norm_above=capi.NORM_BRN),
    "c5_small": lambda: workloads.c5_bilstm(scale=1.0 / 128, batch=6, T=5, out=12),
    "bilstm_no_zoneout_amsgrad": lambda: _bilstm_case("bilstm", capi.opt(capi.OPT_AMSGRAD)),
}


def _res_case(name, opt, B=10, n_in=9, H=12, out=5, blocks=2, p=0.5, norm=capi.NORM_BRN, af=capi.AF_ELU, shake=True, inner_drop=capi.DROP_NONE,
              block_width=None, block_norm=capi.NORM_NONE):
    """block_width: width of the block's layers when it differs from the shortcut's H (zero-padded identity);
    block_norm: normalization on the residual layer itself (the block's output before ShakeDrop and the skip add)"""
    ls = [capi.fc(n_in), capi.fc(H, af)]
    W = block_width or H
    for _ in range(blocks):
        ls += [capi.residual(2, capi.DROP_SHAKEDROP if shake else capi.DROP_NONE, (p, 0, 0), block_norm), capi.fc(W, af), capi.fc(W, af, norm, inner_drop, (0.7, 0, 0))]
    ls.append(capi.fc(out, capi.AF_SOFTMAX))
    return workloads.Workload(name, capi.net(ls, B, loss=capi.LOSS_CE, accuracy=capi.ACC_CE, r_max=3.0, d_max=5.0), opt, n_in, out, True, ls)


CASES.update({
    "c4_small": lambda: workloads.c4_residual(scale=1.0 / 64, batch=24, blocks=2),
    "res_bn_tanh_adam_noshake": lambda: _res_case("res1", capi.opt(capi.OPT_GD, gd_lr=0.01, momentum=0.9), norm=capi.NORM_BN, af=capi.AF_TANH, shake=False, blocks=1),
    "res_plain_relu_shake_drop": lambda: _res_case("res2", capi.opt(capi.OPT_AMSGRAD), norm=capi.NORM_NONE, af=capi.AF_RELU, inner_drop=capi.DROP_BERNOULLI_INVERTED),
})


def shake_from_golden(gold, steps=STEPS):
    """per-step ShakeDrop draws stored in a golden fixture, in the form run_steps(shake=...) takes"""
    out = [dict() for _ in range(steps)]
    for key in gold.files:
        if key.startswith("shake_") and key.endswith("_mask"):
            _, it, layer, _ = key.split("_")
            it, layer = int(it), int(layer)
            out[it][layer] = (gold[key].astype(np.uint8), gold["shake_%d_%d_alpha" % (it, layer)], gold["shake_%d_%d_beta" % (it, layer)])
    return out
