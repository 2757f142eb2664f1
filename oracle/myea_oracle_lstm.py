"""Test infrastructure, not product code.

numpy restatement of the reference's LSTM-with-peephole layer (one cell per block), used through
oracle.myea_oracle.OracleNet.  Follows, routine by routine (paths relative to
Neural_Network_Library_Windows/Source_Files/Neural_Network/):

  forward   Forward_Pass__LSTM__Gates_CIFO__Loop            Neural_Network__Recurrent_Forward_Pass__Loop.cpp:862-1039
            Forward_Pass__LSTM__Gates_CIF_AF_State[__Zoneout] :1041-1340
            Forward_Pass__LSTM__States_AF__Loop              :1531-1563
            Forward_Pass__LSTM__Output[__Zoneout]__Loop      :1342-1529
  backward  Backward_Pass__LSTM_Derivative__Output__Loop     Neural_Network__Recurrent_Backward_Pass__Loop.cpp:1115-1254
            Backward_Pass__LSTM_Derivative__Cell_State_AF    :1256-1305
            Backward_Pass__LSTM_Derivative__Gates_CIF_AF_State :1307-1577
            Backward_Pass__LSTM__Loop (error to the input)   :1011-1113
  weights   Recurrent__Update_Derivative_Weight__LSTM + Bias Neural_Network__Recurrent_Update_Derivative_Weight__Loop.cpp:485-757

Unidirectional layers are pinned against the compiled reference through tests/golden.  The bidirectional layer is NOT
(the reference overlaps the two directions' buffers and gives the following layer a one-direction fan-in): here it is
two independent one-direction layers over the same input, run forward and backward in time with exactly the routines
above, whose outputs sit side by side [forward | backward]; its bias block is the layer's true (unshifted) block with
one [bz|bi|bf|bo] run per direction.  For that layer parity is unpinned against the reference binary.
"""
import numpy as np


def _tanh(x):
    dt = x.dtype.type
    return dt(2) / (dt(1) + np.exp(dt(-2) * x)) - dt(1)


def _sig(x):
    dt = x.dtype.type
    return dt(1) / (dt(1) + np.exp(-x))


def _views(net, L, d):
    """weight views of direction d in the reference's per-block layout
    [Wz_in (in) | Wz_rec (C) | Wi_in Wf_in Wo_in | Wi_rec Wf_rec Wo_rec | p_i p_f p_o]"""
    dirs = 2 if L.d.use_bidirectional else 1
    C, I, S = L.n_out // dirs, L.n_in, L.idx["block_stride"]
    base = L.idx["first_connection_index"] + d * C * S

    def blk(buf):
        return buf[base:base + C * S].reshape(C, S)

    o = dict(z_in=(0, I), z_rec=(I, I + C), i_in=(I + C, 2 * I + C), f_in=(2 * I + C, 3 * I + C), o_in=(3 * I + C, 4 * I + C),
             i_rec=(4 * I + C, 4 * I + 2 * C), f_rec=(4 * I + 2 * C, 4 * I + 3 * C), o_rec=(4 * I + 3 * C, 4 * I + 4 * C),
             p_i=(4 * I + 4 * C, 4 * I + 4 * C + 1), p_f=(4 * I + 4 * C + 1, 4 * I + 4 * C + 2), p_o=(4 * I + 4 * C + 2, 4 * I + 4 * C + 3))
    fb = L.idx["first_bias_connection_index"]
    bias = fb if dirs == 1 else (fb - 2 * C) + d * 4 * C   # unidirectional: the reference's shifted base (bo aliases the next layer)
    return C, I, blk, o, bias


def forward(net, l, x):
    L = net.layers[l]
    dt = net.dt
    T, B = net.T, net.B
    dirs = 2 if L.d.use_bidirectional else 1
    C = L.n_out // dirs
    x = x.reshape(T, B, -1)
    H = np.zeros((T, B, dirs * C), dt)
    L.st = []
    zone = net.zone.get(l) if net.training else None
    for d in range(dirs):
        C, I, blk, o, bias = _views(net, L, d)
        W = blk(net._p())
        b = net._p()[bias:bias + 4 * C]
        Wg = {k: W[:, o[k][0]:o[k][1]] for k in o}
        z, ig, fg, og = (np.zeros((T, B, C), dt) for _ in range(4))
        cs, ca = np.zeros((T, B, C), dt), np.zeros((T, B, C), dt)
        steps = range(T) if d == 0 else range(T - 1, -1, -1)
        prev = None
        for t in steps:
            xt = x[t]
            sz = xt @ Wg["z_in"].T + b[0:C]
            si = xt @ Wg["i_in"].T + b[C:2 * C]
            so = xt @ Wg["o_in"].T + b[3 * C:4 * C]
            if prev is not None:
                hp, cp = H[prev, :, d * C:(d + 1) * C], cs[prev]
                sz = sz + hp @ Wg["z_rec"].T
                si = si + hp @ Wg["i_rec"].T + cp * Wg["p_i"][:, 0]
                sf = xt @ Wg["f_in"].T + b[2 * C:3 * C] + hp @ Wg["f_rec"].T + cp * Wg["p_f"][:, 0]
                so = so + hp @ Wg["o_rec"].T
                fg[t] = _sig(sf)
            z[t], ig[t] = _tanh(sz), _sig(si)
            c_new = z[t] * ig[t] + (fg[t] * cs[prev] if prev is not None else 0)
            if zone is not None:
                keep = zone[0][t, d * C:(d + 1) * C]
                c_new = np.where(keep, c_new, cs[prev] if prev is not None else dt(0))
            cs[t] = c_new
            ca[t] = _tanh(cs[t])
            og[t] = _sig(so + cs[t] * Wg["p_o"][:, 0])
            h_new = ca[t] * og[t]
            if zone is not None:
                keep = zone[1][t, d * C:(d + 1) * C]
                h_new = np.where(keep, h_new, H[prev, :, d * C:(d + 1) * C] if prev is not None else dt(0))
            H[t, :, d * C:(d + 1) * C] = h_new
            prev = t
        L.st.append(dict(z=z, i=ig, f=fg, o=og, c=cs, a=ca))
    L.values = H.reshape(T * B, dirs * C)
    L.x = x
    return L.values


def backward(net, l):
    """BPTT; L.dh [T*B, dirs*C] holds the error arriving from the consumers and receives the recurrent part in place.
    The zoneout masks are ignored, as in the reference."""
    L = net.layers[l]
    dt = net.dt
    T, B = net.T, net.B
    dirs = 2 if L.d.use_bidirectional else 1
    dh_all = np.array(L.dh, dt).reshape(T, B, -1)
    L.dg = []
    for d in range(dirs):
        C, I, blk, o, bias = _views(net, L, d)
        W = blk(net._p())
        Wg = {k: W[:, o[k][0]:o[k][1]] for k in o}
        st = L.st[d]
        dz, di, df, do, dc = (np.zeros((T, B, C), dt) for _ in range(5))
        order = range(T - 1, -1, -1) if d == 0 else range(T)
        nxt = None
        for t in order:
            prev = (t - 1 if d == 0 else t + 1)
            prev = prev if 0 <= prev < T else None
            dh = dh_all[t, :, d * C:(d + 1) * C]
            if nxt is not None:
                dh = dh + dz[nxt] @ Wg["z_rec"] + di[nxt] @ Wg["i_rec"] + df[nxt] @ Wg["f_rec"] + do[nxt] @ Wg["o_rec"]
                dh_all[t, :, d * C:(d + 1) * C] = dh
            og, a = st["o"][t], st["a"][t]
            do[t] = og * (1 - og) * (dh * a)
            c_err = dh * og * (1 - a * a)
            c_err = c_err + Wg["p_o"][:, 0] * do[t]
            if nxt is not None:
                c_err = c_err + Wg["p_i"][:, 0] * di[nxt] + Wg["p_f"][:, 0] * df[nxt] + dc[nxt] * st["f"][nxt]
            dc[t] = c_err
            zt, ig = st["z"][t], st["i"][t]
            dz[t] = c_err * ig * (1 - zt * zt)
            di[t] = (c_err * zt) * (ig * (1 - ig))
            if prev is not None:
                fg = st["f"][t]
                df[t] = (c_err * st["c"][prev]) * (fg * (1 - fg))
            nxt = t
        L.dg.append(dict(z=dz, i=di, f=df, o=do))
    L.dh = dh_all.reshape(T * B, -1)


def error_to_input(net, l):
    """error arriving on the outputs of the layer feeding LSTM layer l: sum over gates and directions of dg W_in"""
    L = net.layers[l]
    T, B = net.T, net.B
    dirs = 2 if L.d.use_bidirectional else 1
    out = 0
    for d in range(dirs):
        C, I, blk, o, bias = _views(net, L, d)
        W = blk(net._p())
        g = L.dg[d]
        out = out + (g["z"].reshape(T * B, C) @ W[:, o["z_in"][0]:o["z_in"][1]] + g["i"].reshape(T * B, C) @ W[:, o["i_in"][0]:o["i_in"][1]]
                     + g["f"].reshape(T * B, C) @ W[:, o["f_in"][0]:o["f_in"][1]] + g["o"].reshape(T * B, C) @ W[:, o["o_in"][0]:o["o_in"][1]])
    return out


def update_derivative_weight(net, l):
    L = net.layers[l]
    dt = net.dt
    T, B = net.T, net.B
    dirs = 2 if L.d.use_bidirectional else 1
    x = L.x.reshape(T * B, -1)
    H = L.values.reshape(T, B, -1)
    for d in range(dirs):
        C, I, blk, o, bias = _views(net, L, d)
        G = blk(net._g())
        g, st = L.dg[d], L.st[d]
        hd = H[:, :, d * C:(d + 1) * C]
        for name in ("z", "i", "f", "o"):
            dg = g[name]
            a, b = o[name + "_in"]
            G[:, a:b] += dg.reshape(T * B, C).T @ x
            if T > 1:
                a, b = o[name + "_rec"]
                if d == 0:   # gate error of step t+1 with the output of step t
                    G[:, a:b] += dg[1:].reshape(-1, C).T @ hd[:-1].reshape(-1, C)
                else:        # backward direction: gate error of step t-1 with the output of step t
                    G[:, a:b] += dg[:-1].reshape(-1, C).T @ hd[1:].reshape(-1, C)
        cs = st["c"]
        if T > 1:
            if d == 0:
                G[:, o["p_i"][0]] += (g["i"][1:] * cs[:-1]).sum((0, 1), dtype=dt)
                G[:, o["p_f"][0]] += (g["f"][1:] * cs[:-1]).sum((0, 1), dtype=dt)
            else:
                G[:, o["p_i"][0]] += (g["i"][:-1] * cs[1:]).sum((0, 1), dtype=dt)
                G[:, o["p_f"][0]] += (g["f"][:-1] * cs[1:]).sum((0, 1), dtype=dt)
        G[:, o["p_o"][0]] += (g["o"] * cs).sum((0, 1), dtype=dt)
        gb = net._g()
        for k, name in enumerate(("z", "i", "f", "o")):
            gb[bias + k * C: bias + (k + 1) * C] += g[name].sum((0, 1), dtype=dt)
