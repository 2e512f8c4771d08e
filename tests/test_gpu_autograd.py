"""Conformance of the autograd wrappers (fuse_b200/autograd.py) with native torch: F.linear forward,
torch.autograd.grad backward, routes built with torch indexing (tests/autograd_reference.py) -- the
check benchmarks/sm90/backward/backward_torch_autograd.py of the reference makes for its fused
backward.  One GPU runs the context-parallel size 1 case in-process; with two or more GPUs the ranks
run as one process each (tests/autograd_worker.py)."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


@pytest.mark.parametrize("seq,hidden,q_heads,kv_heads", [(512, 512, 8, 2), (384, 256, 4, 4)])
def test_single_rank_block_matches_native_autograd(seq, hidden, q_heads, kv_heads):
    from fuse_b200.autograd import UlyssesProjections
    from fuse_b200.world import World
    from fuse_b200 import api
    from tests.autograd_reference import reference_world, toy_attention, close

    head_dim = 128
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(20260906)
    bf = torch.bfloat16
    width, a = (q_heads + 2 * kv_heads) * head_dim, q_heads * head_dim
    x = torch.randn((seq, hidden), generator=gen, device=dev).to(bf)
    w_qkv = (0.02 * torch.randn((width, hidden), generator=gen, device=dev)).to(bf)
    w_o = (0.02 * torch.randn((hidden, a), generator=gen, device=dev)).to(bf)
    dy = (0.01 * torch.randn((seq, hidden), generator=gen, device=dev)).to(bf)

    proj = UlyssesProjections(World(0, 1, 0), batch=1, seq_local=seq, hidden=hidden, q_heads=q_heads,
                              kv_heads=kv_heads, head_dim=head_dim, tag=f"t{seq}")
    for step in range(2):  # twice: epochs advance, buffers are reused
        xg, wq, wo = (t.clone().requires_grad_(True) for t in (x, w_qkv, w_o))
        q, k, v = proj.qkv(xg, wq)
        att = toy_attention(q, k, v, q_heads, kv_heads, head_dim)
        y = proj.oproj(att.contiguous(), wo)
        y.backward(dy)
        torch.cuda.synchronize()
        assert api.read_status()[0] == 0
        want = reference_world([x], w_qkv, w_o, [dy], cp=1, seq_local=seq, q_heads=q_heads, kv_heads=kv_heads,
                               head_dim=head_dim)[0]
        for name, got, ref in (("q", q, want["q"]), ("k", k, want["k"]), ("v", v, want["v"]), ("y", y, want["y"]),
                               ("dx", xg.grad, want["dx"]), ("dw_qkv", wq.grad, want["dw_qkv"]),
                               ("dw_o", wo.grad, want["dw_o"])):
            bad, worst = close(got, ref)
            assert bad == 0, (step, name, bad, worst)


def test_block_across_real_peers():
    from tests.test_gpu_multirank import _gpus, _free_port, _run_group
    n = _gpus()
    if n < 2:
        pytest.skip("needs >= 2 GPUs")
    world = 4 if n >= 4 else 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "autograd_worker.py")]
    code, out, err = _run_group(cmd, dict(os.environ, NCCL_NVLS_ENABLE="0"), 600)
    assert code == 0, out[-3000:] + err[-3000:]
    assert out.count("AUTOGRAD PASS") == world
