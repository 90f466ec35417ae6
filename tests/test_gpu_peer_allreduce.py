"""The peer-memory exchange kernels and the tensor-parallel MLP stack on 2, 4 and 8 GPUs (as many as the machine has; skipped with fewer
than two): one process per GPU under torch.distributed.run, compared with the CPU oracle of the tensor-parallel computation
(tests/workers/peer_allreduce_worker.py says what is compared with what). The cross-GPU protocol cannot be exercised on one GPU: kernels
that wait for each other must not be separate launches on the same device."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_exchange_kernels_and_tp_stack_against_the_oracle(world):
    import torch

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1", "--master-port",
           str(29533 + world), os.path.join(HERE, "workers", "peer_allreduce_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-3000:]
    for rank in range(world):
        assert f"rank {rank} ok" in r.stdout
    print("\n".join(ln for ln in r.stdout.splitlines() if ln.startswith("PARITY")))
