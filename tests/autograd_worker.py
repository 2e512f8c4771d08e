"""One rank of the multi-GPU autograd conformance run (launched by tests/test_gpu_autograd.py through
torch.distributed.run): the block x -> QKV -> toy attention -> output projection, forward and
backward through fuse_b200.autograd, against the native-torch model of ALL ranks computed locally
from the same seeds."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from fuse_b200 import api  # noqa: E402
from fuse_b200.autograd import UlyssesProjections  # noqa: E402
from fuse_b200.world import World  # noqa: E402
from tests.autograd_reference import close, reference_world, toy_attention  # noqa: E402


def main():
    rank, cp = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    seq, hidden, q_heads, kv_heads, head_dim = 512, 512, 8, 4, 128
    bf = torch.bfloat16
    width, a = (q_heads + 2 * kv_heads) * head_dim, q_heads * head_dim
    cpu = torch.Generator().manual_seed(20260906)
    xs = [torch.randn((seq, hidden), generator=cpu).to(bf).to(dev) for _ in range(cp)]
    dys = [(0.01 * torch.randn((seq, hidden), generator=cpu)).to(bf).to(dev) for _ in range(cp)]
    w_qkv = (0.02 * torch.randn((width, hidden), generator=cpu)).to(bf).to(dev)
    w_o = (0.02 * torch.randn((hidden, a), generator=cpu)).to(bf).to(dev)
    proj = UlyssesProjections(World(rank, cp, local_rank), batch=1, seq_local=seq, hidden=hidden, q_heads=q_heads,
                              kv_heads=kv_heads, head_dim=head_dim)
    want = reference_world(xs, w_qkv, w_o, dys, cp=cp, seq_local=seq, q_heads=q_heads, kv_heads=kv_heads,
                           head_dim=head_dim)[rank]
    torch.cuda.synchronize()
    dist.barrier()
    for step in range(3):
        xg, wq, wo = (t.clone().requires_grad_(True) for t in (xs[rank], w_qkv, w_o))
        q, k, v = proj.qkv(xg, wq)
        att = toy_attention(q, k, v, q_heads // cp, kv_heads // cp, head_dim)
        y = proj.oproj(att.contiguous(), wo)
        y.backward(dys[rank])
        torch.cuda.synchronize()
        status = api.read_status()
        assert status[0] == 0, status[:8]
        for name, got, ref in (("q", q, want["q"]), ("k", k, want["k"]), ("v", v, want["v"]), ("y", y, want["y"]),
                               ("dx", xg.grad, want["dx"]), ("dw_qkv", wq.grad, want["dw_qkv"]),
                               ("dw_o", wo.grad, want["dw_o"])):
            bad, worst = close(got, ref)
            assert bad == 0, (rank, step, name, bad, worst)
    # the caller-side reduction of the weight gradients, started behind each weight GEMM
    proj.reduce_weight_grads = True
    everyone = reference_world(xs, w_qkv, w_o, dys, cp=cp, seq_local=seq, q_heads=q_heads, kv_heads=kv_heads,
                               head_dim=head_dim)
    xg, wq, wo = (t.clone().requires_grad_(True) for t in (xs[rank], w_qkv, w_o))
    q, k, v = proj.qkv(xg, wq)
    y = proj.oproj(toy_attention(q, k, v, q_heads // cp, kv_heads // cp, head_dim).contiguous(), wo)
    y.backward(dys[rank])
    proj.finish_weight_grads()
    torch.cuda.synchronize()
    for name, got in (("dw_qkv", wq.grad), ("dw_o", wo.grad)):
        ref = sum(e[name].float() for e in everyone)
        bad, worst = close(got, ref, atol=0.03, rtol=0.03)  # BF16 all-reduce of BF16 partial sums
        assert bad == 0, (rank, "reduced " + name, bad, worst)
    dist.barrier()
    proj.world.close()
    dist.destroy_process_group()
    print(f"AUTOGRAD PASS rank {rank}/{cp}", flush=True)


if __name__ == "__main__":
    main()
