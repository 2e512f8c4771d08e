"""Real multi-GPU parity (one process per GPU over CUDA IPC peer mappings).  Needs at least
two GPUs in the box; on a single-GPU box the emulated-rank tests of test_gpu_forward.py cover
the same kernels."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("route", ["direct", "comm"])
def test_forward_operators_across_real_peers(route):
    n = _gpus()
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29517",
           os.path.join(ROOT, "tests", "multirank_worker.py"), route]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    result = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-3000:]
    assert result.stdout.count("MULTIRANK PASS") == world
