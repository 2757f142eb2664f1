"""GPU test of the sharded step (skipped on a one-GPU box): 2 ranks, one per GPU, NCCL gradient sum overlapped per layer,
synchronised batch-normalization statistics; the result must equal the one-process oracle on the whole batch within the
1e-4 parity tolerance.  NVLS is switched off (plain ring / tree): the test ends by tearing the communicator down."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("name", ["c2_small", "c3_small", "c1_small", "lstm2_zoneout_clip", "mlp_bernoulli_amsbound_clip"])
def test_two_gpus_equal_one_process(name):
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "multi_gpu_worker.py"), name]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
