"""Host-side multi-rank logic on CPU: the handle exchange used by the symmetric-buffer world
and the shard plan, run as two gloo ranks."""
import os
import subprocess
import sys
import textwrap

from fuse_b200.world import shard_plan

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent('''
    import os, sys
    sys.path.insert(0, %r)
    import torch.distributed as dist
    from fuse_b200.world import exchange, shard_plan
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    mine = {"buffer": bytes([rank]) * 64, "rank": rank}
    everyone = exchange(mine)
    assert [e["rank"] for e in everyone] == list(range(world))
    assert all(e["buffer"] == bytes([i]) * 64 for i, e in enumerate(everyone))
    plan = shard_plan(world, rank, 4096, 8, 8)
    spans = exchange((plan["row_begin"], plan["row_end"]))
    assert spans[0][0] == 0 and spans[-1][1] == 4096
    assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
    dist.barrier()
    dist.destroy_process_group()
    print("GLOO PASS", rank)
''') % ROOT


def test_exchange_and_shard_plan_with_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    result = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert result.returncode == 0, result.stdout[-2000:] + result.stderr[-2000:]
    assert result.stdout.count("GLOO PASS") == 2


def test_shard_plan_arithmetic():
    plan = shard_plan(8, 3, 131072, 32, 8)
    assert plan["seq_local"] == 16384 and plan["row_begin"] == 3 * 16384
    assert plan["q_heads"] == (12, 16) and plan["kv_heads"] == (3, 4)
    try:
        shard_plan(3, 0, 4096, 8, 8)
    except ValueError:
        pass
    else:
        raise AssertionError("uneven shards must be rejected")
