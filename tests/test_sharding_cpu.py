"""CPU test (gloo, world size 2) of the data-parallel algorithm the GPU library implements: each rank runs the step on
its half of the batch; batch-normalization column sums (forward: sum z, sum z^2; backward: d_mean, d_sigma) and the
derivative buffer are summed over ranks; scale / shift derivatives are accumulated from LOCAL sums so that the final
all-reduce counts them once.  The result must equal the one-process step on the whole batch, which is itself pinned
against the reference.  Uses the numpy restatement with an all-reduce hook; no GPU involved."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from conftest import rel_err
from myea_b200 import capi
from oracle import myea_oracle


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, name, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    wl = cases.CASES[name]()
    B = wl.B // world
    Xg, Yg = wl.batch()
    shard = cases.CASES[name]()
    shard.desc.batch_size = B
    net = myea_oracle.OracleNet(shard.desc, shard.opt)

    def allreduce(a):
        t = torch.from_numpy(np.ascontiguousarray(a, np.float64))
        dist.all_reduce(t)
        return t.numpy().astype(a.dtype)

    net.allreduce, net.world = allreduce, world
    wl.materialize(net)     # identical parameters and masks on every rank
    X, Y = Xg[:, rank * B:(rank + 1) * B], Yg[:, rank * B:(rank + 1) * B]
    for _ in range(2):
        net.forward(X); net.compute_error(Y); net.backward(); net.update_derivative_weight()
        net.update_parameter(training_size=wl.B)
    if rank == 0:
        np.save(out, net.get(capi.BUF_PARAMETERS))
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["c2_small", "c1_small", "mlp_bernoulli_amsbound_clip", "lstm2_zoneout_clip"])
def test_two_ranks_equal_one_process(name, tmp_path):
    wl = cases.CASES[name]()
    if wl.B % 2:
        pytest.skip("odd batch")
    out = str(tmp_path / "params.npy")
    mp.spawn(_worker, args=(2, _free_port(), name, out), nprocs=2, join=True)
    single = myea_oracle.OracleNet(wl.desc, wl.opt)
    X, Y = wl.batch()
    wl.materialize(single)
    for _ in range(2):
        single.forward(X); single.compute_error(Y); single.backward(); single.update_derivative_weight()
        single.update_parameter(training_size=wl.B)
    assert rel_err(np.load(out), single.get(capi.BUF_PARAMETERS)) < 2e-5
