"""Test infrastructure, not product code.

numpy restatement of the reference's residual blocks of fully connected layers with ShakeDrop (pre-activation order),
used through oracle.myea_oracle.OracleNet.  Follows (paths relative to
Neural_Network_Library_Windows/Source_Files/Neural_Network/):

  forward   Forward_Pass__Residual__Loop / __Residual__Layer / __Residual__FC   Neural_Network__Forward_Pass__Loop.cpp:3955-4536
            Forward_Pass__Dropout__ShakeDrop__Loop :5016-5045, Forward_Pass__Zero_Padded_Identity__Loop :5138-5211
  backward  Backward_Pass__Residual__Block / __Residual__FC                     Neural_Network__Backward_Pass__Loop.cpp:403-589
            Backward_Pass__Gradient__Residual__FC :867-1002, Backward_Pass__Dropout__ShakeDrop__Loop :1050-1077

The reference draws ShakeDrop's row mask and its forward (alpha ~ U(-1,1)) and backward (beta ~ U(0,1)) coefficients
while it runs; here they are inputs (OracleNet.set_shakedrop), obtained for a parity test by replaying the reference's
generators (oracle/ref_harness.cpp: ref_shakedrop_replay).  A block narrower or wider than its shortcut: the result
has max(A, W) columns and the narrower addend sits ((|A - W|) + 1) // 2 columns in (zero-padded identity).  A
normalization on the residual layer itself normalizes the block's last summations before they are added
(Forward_Pass__Residual :3861-3998 of the OpenMP twin, Backward_Pass__Residual__Block :351-452).
"""
import numpy as np

from myea_b200 import capi
from oracle.myea_oracle import af_derive, af_fire


def forward(net, r):
    R = net.layers[r]
    dt = net.dt
    x = net.layers[R.input_layer].values
    s = x
    for k in range(1, R.depth + 1):
        L = net.layers[r + k]
        norm = int(L.d.type_normalization) != capi.NORM_NONE
        v = s
        if k > 1:
            L.z_in = s
            pre = net._norm_forward(L, s) if norm else s
            L.pre_in = pre
            v = af_fire(int(L.d.type_activation_function), pre)
            drop = int(L.d.type_dropout)
            if drop in (capi.DROP_BERNOULLI, capi.DROP_BERNOULLI_INVERTED):
                p = dt(L.d.dropout_values[0])
                if net.training:
                    v = np.where(np.asarray(net.masks[r + k][0])[:v.shape[1]], v * (dt(1) / p) if drop == capi.DROP_BERNOULLI_INVERTED else v, dt(0))
                elif drop == capi.DROP_BERNOULLI:
                    v = v * p
        L.dw_input = v
        L.values = v
        s = v @ net._fc_weights(L).T
        if not norm:
            s = s + net._p()[L.idx["first_bias_connection_index"]:L.idx["first_bias_connection_index"] + L.n_out]
        L.summations = s
    last = net.layers[r + R.depth]
    A, W = x.shape[1], last.n_out
    if int(R.d.type_normalization) != capi.NORM_NONE:
        R.z_block = s
        s = net._norm_forward(R, s)
    if int(R.d.type_dropout) == capi.DROP_SHAKEDROP:
        if net.training:
            mask, alpha, _ = net.shake[r]
            s = np.where(mask[:, None], s * np.asarray(alpha)[:, :W], s)
        else:
            s = s * (dt(1) - dt(R.d.dropout_values[0]))
    out = np.zeros((x.shape[0], R.n_out), dt)
    pad = (abs(A - W) + 1) // 2
    oa, os_ = (pad if A < W else 0), (pad if W < A else 0)
    out[:, os_:os_ + W] = s
    out[:, oa:oa + A] = x + out[:, oa:oa + A]
    R.values = out.astype(dt)


def backward(net, r):
    """R.errors holds the error on the block output; returns the index of the layer feeding the block, whose errors
    are final afterwards."""
    R = net.layers[r]
    d_r = R.errors
    last = net.layers[r + R.depth]
    A, W = net.layers[r + 1].n_in, last.n_out
    pad = (abs(A - W) + 1) // 2
    oa, os_ = (pad if A < W else 0), (pad if W < A else 0)
    d = d_r[:, os_:os_ + W]
    if int(R.d.type_dropout) == capi.DROP_SHAKEDROP:
        mask, _, beta = net.shake[r]
        d = np.where(mask[:, None], d * np.asarray(beta)[:, :W], d)
    if int(R.d.type_normalization) != capi.NORM_NONE:
        d = net._norm_backward(R, R.z_block, d)
    for k in range(R.depth, 1, -1):
        L = net.layers[r + k]
        L.errors = d
        D = d @ net._fc_weights(L)
        da = D * af_derive(int(L.d.type_activation_function), L.pre_in, L.values)
        d = net._norm_backward(L, L.z_in, da) if int(L.d.type_normalization) != capi.NORM_NONE else da
    first = net.layers[r + 1]
    first.errors = d
    f = R.input_layer
    if f < 1:
        return 0
    F = net.layers[f]
    D = d_r[:, oa:oa + A] + d @ net._fc_weights(first)
    if F.type == capi.LAYER_FC:
        da = D * af_derive(int(F.d.type_activation_function), F.pre, F.values)
        F.errors = net._norm_backward(F, F.z, da) if int(F.d.type_normalization) != capi.NORM_NONE else da
    else:
        F.errors = D
    return f
