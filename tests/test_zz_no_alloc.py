"""The allocation-free MXFP8 QKV entry point (fuse_b200_launch_gemm_a2a_mxfp8_static).

It exists for callers that cannot hand over scratch memory -- code inside a stream capture or
a latency-critical loop, plug-ins whose host owns the allocator -- and keeps the quantised
weight in a fixed array inside the library.  This file is collected last on purpose: a run that
stops at the first failure has then already exercised every other test.  The checks: called
twice in a row through the C ABI it gives the same result as the ordinary entry point with
caller scratch (the array keeps the first call's contents, the second call must not care), and
a weight too large for the array is refused."""
import numpy as np
import pytest

from fuse_b200 import _native as N
from fuse_b200 import api, synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _params(H, torch, m, n, k, q, kv, d, data, scales, w, local, planar, done, ready, workspace=None, epoch=1):
    problem = N.GemmProblem(m, n, k, max_swizzle_size=4)
    route = N.UlyssesRoute(world_size=1, rank=0, batch=1, global_seq=m, seq_local=m, q_heads=q, kv_heads=kv,
                           head_dim=d, kind=N.ROUTE_QKV_GQA_PACK)
    proj = N.GemmA2AParams(rhs_nt=w.data_ptr(), local_output=local.data_ptr(), ready=ready.data_ptr(), gemm=problem,
                           route=route, num_comm_ctas=4, epoch=epoch)
    proj.peer_output[0] = planar.data_ptr()
    proj.peer_route_done_epoch[0] = done.data_ptr()
    mp = N.Mxfp8GemmA2AParams(projection=proj, activation=N.Mxfp8Activation(
        data=data.data_ptr(), scales=scales.data_ptr(), data_bytes=data.numel(), scale_bytes=scales.numel()))
    if workspace is not None:
        mp.workspace, mp.workspace_bytes = workspace
    return mp


def test_static_scratch_entry_matches_caller_scratch_entry_twice():
    import torch
    from tests import harness as H
    m, q, kv, d, k = 384, 4, 2, 128, 512
    n = (q + 2 * kv) * d
    weights = [synthetic.normal_bf16((n, k), synthetic.BASE_SEED + 11 + i, 0.02) for i in range(2)]
    act = O.mxfp8_quantize(synthetic.normal_bf16((m, k), synthetic.rank_seed(0) + 1000, 1.0))
    data, scales = H.to_device_u8(act[0]), H.to_device_u8(act[1])
    done = torch.zeros(N.READY_FLAG_STRIDE, dtype=torch.int32, device=H.DEV)
    ready = torch.zeros(api.qkv_ready_elements(N.GemmProblem(m, n, k)), dtype=torch.int32, device=H.DEV)
    rc, ws_bytes = api.gemm_a2a_mxfp8_workspace_size(N.GemmProblem(m, n, k))
    assert rc == 0 and ws_bytes <= N.STATIC_SCRATCH_BYTES
    scratch = torch.zeros(ws_bytes + 256, dtype=torch.uint8, device=H.DEV)
    base = (scratch.data_ptr() + 255) // 256 * 256
    epoch = 0
    # two calls in a row with DIFFERENT weights: the array still holds the first weight's bytes
    # when the second call starts
    for w_bits in weights:
        w = H.to_device(w_bits)
        want_local, want_planar = H.poisoned(m, n), H.poisoned(m * n)
        epoch += 1
        mp = _params(H, torch, m, n, k, q, kv, d, data, scales, w, want_local, want_planar, done, ready,
                     workspace=(base, ws_bytes), epoch=epoch)
        assert api.launch_gemm_a2a_mxfp8_cutlass(mp, 0) == 0
        H.check_status()
        got_local, got_planar = H.poisoned(m, n), H.poisoned(m * n)
        epoch += 1
        mp = _params(H, torch, m, n, k, q, kv, d, data, scales, w, got_local, got_planar, done, ready, epoch=epoch)
        assert api.launch_gemm_a2a_mxfp8_static(mp, 0) == 0
        H.check_status()
        for got, want, what in ((got_local, want_local, "local output"), (got_planar, want_planar, "routed output")):
            ok, worst, bad = O.within_tolerance(H.to_bits(got), H.to_bits(want))
            assert ok, f"{what}: {bad} elements outside 0.01+0.01|b| (max abs err {worst})"
        wq, wsf = O.mxfp8_quantize(w_bits)
        ok, worst, bad = O.within_tolerance(H.to_bits(got_local), O.gemm_mxfp8(act[0], act[1], wq, wsf))
        assert ok, f"against the oracle: {bad} elements out of tolerance (max abs err {worst})"


def test_static_scratch_entry_rejects_oversized_weights():
    import torch
    from tests import harness as H
    m, q, kv, d, k = 128, 32, 8, 128, 4096          # weight 6144 x 4096 = 24 MiB of E4M3
    n = (q + 2 * kv) * d
    tiny = torch.zeros(1024, dtype=torch.uint8, device=H.DEV)
    flags = torch.zeros(4096, dtype=torch.int32, device=H.DEV)
    buf = torch.zeros(16, dtype=torch.bfloat16, device=H.DEV)
    mp = _params(H, torch, m, n, k, q, kv, d, tiny, tiny, buf, buf, buf, flags, flags)
    assert api.launch_gemm_a2a_mxfp8_static(mp, 0) == N.CUDA_ERROR_INVALID_VALUE
    torch.cuda.synchronize()
    assert api.read_status()[0] == 0
