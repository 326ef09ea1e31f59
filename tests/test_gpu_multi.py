"""Multi-process (one process per GPU) parity of the peer-memory all-reduce and of the
tensor-parallel gated-MLP layer. Needs at least two GPUs; skipped otherwise."""
import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu

WORKER = os.path.join(ROOT, "tests", "multi_gpu_worker.py")


def _gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_allreduce_and_tp_layer(world):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), WORKER]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, (proc.stdout[-3000:], proc.stderr[-3000:])
    assert "MULTI_GPU_OK" in proc.stdout


@pytest.mark.parametrize("world", [2, 8])
def test_multicast_allreduce(world):
    """The in-switch form of the reduction (multimem.ld_reduce / multimem.st over an NVLink
    multicast mapping) against the fp32 sum and the oracle's fused residual + RMSNorm."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29520 + world),
           os.path.join(ROOT, "tests", "multicast_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, (proc.stdout[-3000:], proc.stderr[-3000:])
    assert "MULTICAST_OK" in proc.stdout
