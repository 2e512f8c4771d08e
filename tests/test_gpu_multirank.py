"""Real multi-GPU parity (one process per GPU over CUDA IPC peer mappings).  Needs at least
two GPUs in the box; on a single-GPU box the emulated-rank tests of test_gpu_forward.py cover
the same kernels."""
import os
import signal
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus():
    import torch
    return torch.cuda.device_count()


def _free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _run_group(cmd, env, timeout):
    """Runs the launcher in a process group of its own; on a time-out the whole group goes, so
    no worker outlives the test holding a port or a GPU."""
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env,
                            start_new_session=True)
    try:
        out, err = proc.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)
        out, err = proc.communicate()
        raise AssertionError("multi-rank run timed out\n" + out[-3000:] + err[-3000:])
    return proc.returncode, out, err


@pytest.mark.parametrize("route", ["direct", "comm"])
def test_forward_operators_across_real_peers(route):
    n = _gpus()
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "multirank_worker.py"), route]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    code, out, err = _run_group(cmd, env, 600)
    assert code == 0, out[-3000:] + err[-3000:]
    assert out.count("MULTIRANK PASS") == world
