"""Test infrastructure, not product code.

numpy restatement of the reference's LSTM-with-peephole layer (blocks of one or more cells: the cells of a block
share its input, forget and output gate, and every gate sees the states of all the block's cells through its
peepholes), used through
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


class _Views:
    """index arrays into the flat parameter buffer for direction d, in the reference's per-block layout
    (Prepare__Connections__LSTM, Neural_Network__Prepare_Connections.cpp): per block, per cell [Wz_in (in) | Wz_rec (cells)],
    then Wi_in Wf_in Wo_in (in each), Wi_rec Wf_rec Wo_rec (cells each), then the peepholes p_i p_f p_o (one per cell of
    the block each).  Biases: [bz (cells) | bi | bf | bo (blocks each)]."""

    def __init__(self, L, d):
        dirs = 2 if L.d.use_bidirectional else 1
        cpb = max(1, int(L.d.unit_parameters[1]))
        K = int(L.d.unit_parameters[0])            # blocks of one direction
        C, I, S = K * cpb, L.n_in, L.idx["block_stride"]
        self.C, self.K, self.cpb, self.I = C, K, cpb, I
        base = L.idx["first_connection_index"] + d * K * S
        blk = base + np.arange(K)[:, None] * S     # [K, 1]
        cell = (blk + np.arange(cpb)[None, :] * (I + C)).reshape(C, 1)
        self.z_in = cell + np.arange(I)[None, :]
        self.z_rec = cell + I + np.arange(C)[None, :]
        g0 = blk + cpb * (I + C)
        self.g_in = [g0 + g * I + np.arange(I)[None, :] for g in range(3)]          # input, forget, output gate: [K, I]
        self.g_rec = [g0 + 3 * I + g * C + np.arange(C)[None, :] for g in range(3)]  # [K, C]
        self.peep = [g0 + 3 * I + 3 * C + g * cpb + np.arange(cpb)[None, :] for g in range(3)]  # [K, cpb]
        fb = L.idx["first_bias_connection_index"]
        # unidirectional: the reference's base, already shifted by the number of cells (the tail aliases the next layer's
        # biases); bidirectional (no usable reference): the layer's true block, one run per direction
        b0 = fb if dirs == 1 else (fb - dirs * C) + d * (C + 3 * K)
        self.b_z = b0 + np.arange(C)
        self.b_g = [b0 + C + g * K + np.arange(K) for g in range(3)]

    def cells(self, per_block):
        """[.., K] -> [.., C]: a block value seen by each of its cells"""
        return np.repeat(per_block, self.cpb, axis=-1)

    def blocks(self, per_cell):
        """[.., C] -> [.., K]: sum over the cells of a block"""
        return per_cell.reshape(per_cell.shape[:-1] + (self.K, self.cpb)).sum(-1, dtype=per_cell.dtype)

    def peep_term(self, p, g, c):
        """sum over the block's cells of peephole weight x cell state: [B, C] -> [B, K]"""
        return self.blocks(c * p[self.peep[g]].reshape(-1))


def forward(net, l, x):
    L = net.layers[l]
    dt = net.dt
    T, B = net.T, net.B
    dirs = 2 if L.d.use_bidirectional else 1
    x = x.reshape(T, B, -1)
    L.st, L.views = [], []
    zone = net.zone.get(l) if net.training else None
    p = net._p()
    outs = []
    for d in range(dirs):
        V = _Views(L, d)
        C, K = V.C, V.K
        z, cs, ca, H = (np.zeros((T, B, C), dt) for _ in range(4))
        ig, fg, og = (np.zeros((T, B, K), dt) for _ in range(3))
        steps = range(T) if d == 0 else range(T - 1, -1, -1)
        prev = None
        for t in steps:
            xt = x[t]
            sz = xt @ p[V.z_in].T + p[V.b_z]
            si = xt @ p[V.g_in[0]].T + p[V.b_g[0]]
            so = xt @ p[V.g_in[2]].T + p[V.b_g[2]]
            if prev is not None:
                hp, cp = H[prev], cs[prev]
                sz = sz + hp @ p[V.z_rec].T
                si = si + hp @ p[V.g_rec[0]].T + V.peep_term(p, 0, cp)
                sf = xt @ p[V.g_in[1]].T + p[V.b_g[1]] + hp @ p[V.g_rec[1]].T + V.peep_term(p, 1, cp)
                so = so + hp @ p[V.g_rec[2]].T
                fg[t] = _sig(sf)
            z[t], ig[t] = _tanh(sz), _sig(si)
            c_new = z[t] * V.cells(ig[t]) + (V.cells(fg[t]) * cs[prev] if prev is not None else 0)
            if zone is not None:
                keep = zone[0][t, d * C:(d + 1) * C]
                c_new = np.where(keep, c_new, cs[prev] if prev is not None else dt(0))
            cs[t] = c_new
            ca[t] = _tanh(cs[t])
            og[t] = _sig(so + V.peep_term(p, 2, cs[t]))
            h_new = ca[t] * V.cells(og[t])
            if zone is not None:
                keep = zone[1][t, d * C:(d + 1) * C]
                h_new = np.where(keep, h_new, H[prev] if prev is not None else dt(0))
            H[t] = h_new
            prev = t
        L.st.append(dict(z=z, i=ig, f=fg, o=og, c=cs, a=ca, h=H))
        L.views.append(V)
        outs.append(H)
    L.values = np.concatenate(outs, axis=2).reshape(T * B, -1)
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
    p = net._p()
    for d in range(dirs):
        V = L.views[d]
        C, K = V.C, V.K
        st = L.st[d]
        dz, dc = np.zeros((T, B, C), dt), np.zeros((T, B, C), dt)
        di, df, do = (np.zeros((T, B, K), dt) for _ in range(3))
        order = range(T - 1, -1, -1) if d == 0 else range(T)
        nxt = None
        for t in order:
            prev = (t - 1 if d == 0 else t + 1)
            prev = prev if 0 <= prev < T else None
            dh = dh_all[t, :, d * C:(d + 1) * C]
            if nxt is not None:
                dh = dh + dz[nxt] @ p[V.z_rec] + di[nxt] @ p[V.g_rec[0]] + df[nxt] @ p[V.g_rec[1]] + do[nxt] @ p[V.g_rec[2]]
                dh_all[t, :, d * C:(d + 1) * C] = dh
            og, a = st["o"][t], st["a"][t]
            do[t] = og * (1 - og) * V.blocks(dh * a)
            c_err = dh * V.cells(og) * (1 - a * a)
            c_err = c_err + p[V.peep[2]].reshape(-1) * V.cells(do[t])
            if nxt is not None:
                c_err = (c_err + p[V.peep[0]].reshape(-1) * V.cells(di[nxt]) + p[V.peep[1]].reshape(-1) * V.cells(df[nxt])
                         + dc[nxt] * V.cells(st["f"][nxt]))
            dc[t] = c_err
            zt, ig = st["z"][t], st["i"][t]
            dz[t] = c_err * V.cells(ig) * (1 - zt * zt)
            di[t] = V.blocks(c_err * zt) * (ig * (1 - ig))
            if prev is not None:
                fg = st["f"][t]
                df[t] = V.blocks(c_err * st["c"][prev]) * (fg * (1 - fg))
            nxt = t
        L.dg.append(dict(z=dz, i=di, f=df, o=do))
    L.dh = dh_all.reshape(T * B, -1)


def error_to_input(net, l):
    """error arriving on the outputs of the layer feeding LSTM layer l: sum over gates and directions of dg W_in"""
    L = net.layers[l]
    T, B = net.T, net.B
    dirs = 2 if L.d.use_bidirectional else 1
    p = net._p()
    out = 0
    for d in range(dirs):
        V, g = L.views[d], L.dg[d]
        out = out + g["z"].reshape(T * B, -1) @ p[V.z_in]
        for k, name in enumerate(("i", "f", "o")):
            out = out + g[name].reshape(T * B, -1) @ p[V.g_in[k]]
    return out


def update_derivative_weight(net, l):
    L = net.layers[l]
    dt = net.dt
    T, B = net.T, net.B
    dirs = 2 if L.d.use_bidirectional else 1
    x = L.x.reshape(T * B, -1)
    G = net._g()
    for d in range(dirs):
        V, g, st = L.views[d], L.dg[d], L.st[d]
        C, K, cpb = V.C, V.K, V.cpb
        hd, cs = st["h"], st["c"]
        # gate error of the step after t (in the layer's direction) meets the output / state of step t
        later = (lambda a: a[1:]) if d == 0 else (lambda a: a[:-1])
        earlier = (lambda a: a[:-1]) if d == 0 else (lambda a: a[1:])
        G[V.z_in] += g["z"].reshape(T * B, C).T @ x
        if T > 1:
            G[V.z_rec] += later(g["z"]).reshape(-1, C).T @ earlier(hd).reshape(-1, C)
        for k, name in enumerate(("i", "f", "o")):
            dg = g[name]
            G[V.g_in[k]] += dg.reshape(T * B, K).T @ x
            if T > 1:
                G[V.g_rec[k]] += later(dg).reshape(-1, K).T @ earlier(hd).reshape(-1, C)
        if T > 1:
            G[V.peep[0]] += (V.cells(later(g["i"])) * earlier(cs)).sum((0, 1), dtype=dt).reshape(K, cpb)
            G[V.peep[1]] += (V.cells(later(g["f"])) * earlier(cs)).sum((0, 1), dtype=dt).reshape(K, cpb)
        G[V.peep[2]] += (V.cells(g["o"]) * cs).sum((0, 1), dtype=dt).reshape(K, cpb)
        # np.add.at: with the reference's shifted bias base the ranges of neighbouring layers overlap
        np.add.at(G, V.b_z, g["z"].sum((0, 1), dtype=dt))
        for k, name in enumerate(("i", "f", "o")):
            np.add.at(G, V.b_g[k], g[name].sum((0, 1), dtype=dt))
