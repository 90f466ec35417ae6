"""The peer-memory all-reduce kernel and the MLP stack's peer_all_reduce mode, on two GPUs (skipped with fewer): two processes
under torch.distributed.run, each on its own GPU, compared with NCCL. The cross-GPU protocol cannot be exercised on one GPU:
kernels that wait for each other must not be separate launches on the same device."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def test_peer_allreduce_two_gpus():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29533",
           os.path.join(HERE, "workers", "peer_allreduce_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=400, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
