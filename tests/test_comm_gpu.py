"""The gradient exchange of the C ABI (he_comm_create / he_allreduce_grads / he_comm_poll) on two GPUs,
each rank a child process.  Failure scenarios follow the host-side form: a rank that leaves does so before it
has anything in flight, the survivor learns of it through a short deadline, NVLS is off and the library's
kernels never touch peer memory."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _gpu_count():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("scenario", ["allreduce", "layout_mismatch", "never_joins"])
def test_two_rank_gradient_exchange(scenario):
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    env.pop("HE_NCCL_LIBRARY", None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(HERE, "comm_worker.py"), scenario]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
