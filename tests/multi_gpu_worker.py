"""Worker of tests/test_multi_gpu.py (one process per GPU, launched by torch.distributed.run): every rank builds the same
network on its own GPU for its shard of the batch, the handles are joined by an NCCL communicator, two training steps run,
and rank 0 compares the resulting parameters and first moments with the single-process oracle on the whole batch."""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases  # noqa: E402
from myea_b200 import capi  # noqa: E402
from myea_b200.net import Net  # noqa: E402
from oracle import myea_oracle, ref  # noqa: E402


def main():
    name = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    wl = cases.CASES[name]()
    B = wl.B // world
    Xg, Yg = wl.batch()
    shard = cases.CASES[name]()
    shard.desc.batch_size = B
    net = Net(shard.desc, shard.opt, device=local)
    uid = [bytes(128)]
    if rank == 0:
        buf = (C.c_uint8 * 128)()
        assert net.lib.myea_b200_comm_unique_id(buf) == 0
        uid = [bytes(buf)]
    dist.broadcast_object_list(uid, 0)
    idb = (C.c_uint8 * 128).from_buffer_copy(uid[0])
    net._ck(net.lib.myea_b200_comm_init(net.h, world, rank, idb), "comm_init")
    wl.materialize(net)
    X = np.ascontiguousarray(Xg[:, rank * B:(rank + 1) * B])
    Y = np.ascontiguousarray(Yg[:, rank * B:(rank + 1) * B])
    losses = []
    for _ in range(2):
        net.reset_loss()
        net.forward(X); net.compute_error(Y); net.backward(); net.update_derivative_weight()
        losses.append(net.loss())
        net._ck(net.lib.myea_b200_update_parameter(net.h, wl.B, wl.B, C.byref(wl.opt)), "update_parameter")
    net.synchronize()
    got_p, got_m = net.get(capi.BUF_PARAMETERS), net.get(capi.BUF_FIRST_MOMENT)
    ok = True
    if rank == 0:
        single = ref.RefNet(wl.desc, wl.opt) if ref.available() else myea_oracle.OracleNet(wl.desc, wl.opt)
        wl.materialize(single)
        want_loss = []
        for _ in range(2):
            single.reset_loss()
            single.forward(Xg); single.compute_error(Yg); single.backward(); single.update_derivative_weight()
            want_loss.append(single.loss())
            single.update_parameter(training_size=wl.B)
        want_p, want_m = single.get(capi.BUF_PARAMETERS), single.get(capi.BUF_FIRST_MOMENT)
        ep = float(np.abs(got_p - want_p).max() / np.abs(want_p).max())
        em = float(np.abs(got_m - want_m).max() / max(np.abs(want_m).max(), 1e-30))
        el = abs(losses[1][0] - want_loss[1][0]) / abs(want_loss[1][0])
        print("multi-gpu %s world %d: params %.2e moments %.2e loss %.2e counts %s vs %s" % (name, world, ep, em, el, losses[1][1:], want_loss[1][1:]))
        ok = ep < 1e-4 and em < 1e-4 and el < 1e-4 and losses[1][1] == want_loss[1][1] and losses[1][2] == want_loss[1][2]
    net.close()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
