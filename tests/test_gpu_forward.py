"""Parity of the CUDA forward operators with the CPU oracle, through the C ABI.

Routing is compared bit for bit; GEMM outputs with the reference's element test
|a-b| <= 0.01 + 0.01*|b| (benchmarks/sm103/fused_validation.cuh:71-77) against the oracle's
FP32-accumulated result on the same BF16 operands."""
import ctypes as C

import numpy as np
import pytest

from fuse_b200 import _native as N
from fuse_b200 import api, synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _inputs(world, m, k, n, generation=0, act_offset=1000, weight_offset=11, normal=True):
    gen = synthetic.normal_bf16 if normal else synthetic.uniform_bf16
    lhs = [gen((m, k), synthetic.rank_seed(r, generation) + act_offset, 1.0 if normal else 0.125)
           for r in range(world)]
    w = gen((n, k), synthetic.BASE_SEED + weight_offset, 0.02)
    return lhs, w


def _assert_close(actual, expected, what):
    ok, worst, bad = O.within_tolerance(actual, expected)
    assert ok, f"{what}: {bad} elements outside 0.01+0.01|b| (max abs err {worst})"


# (world, batch, seq_local, q_heads, kv_heads, head_dim, k, comm)
QKV_CASES = [
    (1, 1, 256, 4, 4, 128, 128, 2),        # one rank: route is a local repack
    (2, 1, 2048, 8, 8, 128, 1024, 8),      # the tiny 2-rank configuration (global seq 4096)
    (2, 2, 200, 8, 4, 64, 328, 3),         # batch 2, ragged M (not a tile multiple), K % 64 != 0
    (4, 1, 136, 16, 4, 80, 192, 5),        # head_dim 80: heads straddle 16-byte-aligned chunks only
    (8, 1, 128, 32, 8, 128, 256, 16),      # GQA 32/8 over 8 ranks
]


@pytest.mark.parametrize("route", ["comm", "direct"])
@pytest.mark.parametrize("case", QKV_CASES)
def test_qkv_forward_matches_oracle(case, route):
    from tests import harness as H
    world, batch, s, q, kv, d, k, comm = case
    m, n = batch * s, (q + 2 * kv) * d
    lhs, w = _inputs(world, m, k, n)
    local, peers = H.qkv_forward(world, batch, s, q, kv, d, lhs, w, comm=comm, route=route)
    want_local, want_peers = O.qkv_forward(world, batch, s, q, kv, d, lhs, w)
    for r in range(world):
        _assert_close(local[r], want_local[r], f"local_output[{r}]")
    # Routing: re-route the GPU's own local outputs with the oracle's sender-side map (pinned
    # against the reference's receiver-side validation map); the destination buffers must hold
    # exactly those bytes.
    rerouted = [np.full(peers[0].size, 0xFFFF, dtype=np.uint16) for _ in range(world)]
    table = O.ptr_array(rerouted)
    for r in range(world):
        O.lib().fo_qkv_forward_route(world, r, batch, s, q, kv, d, O.ptr(np.ascontiguousarray(local[r])), n, table)
    for dest in range(world):
        assert np.array_equal(peers[dest], rerouted[dest]), f"routed bytes differ at destination {dest}"
        _assert_close(peers[dest], want_peers[dest], f"peer_output[{dest}]")


@pytest.mark.parametrize("route,vector,block_n", [("direct", False, 0), ("direct", False, 128), ("direct", True, 0),
                                                  ("comm", False, 0)])
@pytest.mark.parametrize("case", [(1, 1, 256, 4, 2, 128, 256), (2, 1, 384, 8, 4, 128, 512), (4, 2, 128, 16, 4, 64, 320),
                                  (2, 1, 200, 8, 8, 40, 192)])
def test_qkv_forward_with_the_all_to_all_of_v_deferred(case, route, vector, block_n):
    # UlyssesRoute::defer_v_a2a (csrc/operators/sm103/detail/gemm_a2a.cuh:199-215,408,505-533): V stays in
    # the local output, Q and K of a destination's heads land in ONE [B*S_global, q_local + kv_local]
    # tensor there, and completion_epoch is published once the local output is complete.
    from tests import harness as H
    world, batch, s, q, kv, d, k = case
    m, n = batch * s, (q + 2 * kv) * d
    lhs, w = _inputs(world, m, k, n)
    local, peers = H.qkv_forward(world, batch, s, q, kv, d, lhs, w, comm=4, route=route, vector_epilogue=vector,
                                 block_n=block_n, defer_v=True, epochs=2)
    want_local, _ = O.qkv_forward(world, batch, s, q, kv, d, lhs, w, defer_v=True)
    for r in range(world):
        _assert_close(local[r], want_local[r], f"local_output[{r}]")
    # the GPU's own local outputs re-routed by the oracle; what nobody routes (the V share of the
    # buffer) keeps the caller's poison
    expected = [np.full(peers[0].size, 0xFFFF, dtype=np.uint16) for _ in range(world)]
    table = O.ptr_array(expected)
    for r in range(world):
        O.lib().fo_qkv_forward_route_defer_v(world, r, batch, s, q, kv, d, O.ptr(np.ascontiguousarray(local[r])), n, table)
    for dest in range(world):
        assert np.array_equal(peers[dest], expected[dest]), f"routed bytes differ at destination {dest}"


@pytest.mark.parametrize("defer_v", [False, True])
@pytest.mark.parametrize("route,vector,block_n", [("direct", False, 0), ("direct", False, 128), ("direct", True, 0),
                                                  ("comm", False, 0)])
@pytest.mark.parametrize("case", [(2, 1, 384, 8, 4, 128, 512), (4, 2, 128, 16, 4, 64, 320), (2, 1, 200, 8, 8, 40, 192)])
def test_qkv_forward_with_offline_interleaved_weights(case, route, vector, block_n, defer_v):
    # UlyssesRoute::qkv_peer_interleaved (include/fuse/layout/ulysses.h:35-39,
    # csrc/operators/sm103/detail/gemm_a2a.cuh:404-415): with the weight prepacked so that physical head p
    # of Q and of K belongs to owner p % world, the routed Q | K | V is what the standard weight gives.
    from tests import harness as H
    from tests.test_oracle_golden import _prepack_interleaved
    world, batch, s, q, kv, d, k = case
    m, n = batch * s, (q + 2 * kv) * d
    lhs, w = _inputs(world, m, k, n)
    local, peers = H.qkv_forward(world, batch, s, q, kv, d, lhs, _prepack_interleaved(w, world, q, kv, d), comm=4,
                                 route=route, vector_epilogue=vector, block_n=block_n, defer_v=defer_v, interleaved=True,
                                 raster=N.RASTER_ALONG_M)
    _, want_peers = O.qkv_forward(world, batch, s, q, kv, d, lhs, w, defer_v=defer_v)   # standard weight, standard route
    expected = [np.full(peers[0].size, 0xFFFF, dtype=np.uint16) for _ in range(world)]
    table = O.ptr_array(expected)
    for r in range(world):
        O.lib().fo_qkv_forward_route_variant(world, r, batch, s, q, kv, d, int(defer_v), 1,
                                             O.ptr(np.ascontiguousarray(local[r])), n, table)
    for dest in range(world):
        assert np.array_equal(peers[dest], expected[dest]), f"routed bytes differ at destination {dest}"
        routed = want_peers[dest] != 0xFFFF
        assert (peers[dest][~routed] == 0xFFFF).all()
        _assert_close(peers[dest][routed], want_peers[dest][routed], f"peer_output[{dest}]")


def test_qkv_forward_interleaved_weights_are_refused_with_the_n_raster():
    # csrc/operators/sm103/detail/gemm_a2a.cuh:258-259
    import torch
    from tests import harness as H
    x = torch.zeros((256, 128), dtype=torch.bfloat16, device=H.DEV)
    w = torch.zeros((1024, 128), dtype=torch.bfloat16, device=H.DEV)
    out = torch.zeros((256, 1024), dtype=torch.bfloat16, device=H.DEV)
    flags = torch.zeros(4096, dtype=torch.int32, device=H.DEV)
    route = N.UlyssesRoute(world_size=1, rank=0, batch=1, global_seq=256, seq_local=256, q_heads=4, kv_heads=2,
                           head_dim=128, kind=N.ROUTE_QKV_GQA_PACK, qkv_peer_interleaved=1)
    p = N.GemmA2AParams(lhs=x.data_ptr(), rhs_nt=w.data_ptr(), local_output=out.data_ptr(), ready=flags.data_ptr(),
                        gemm=N.GemmProblem(256, 1024, 128, raster=N.RASTER_ALONG_N), route=route, num_comm_ctas=2, epoch=1)
    p.peer_output[0] = out.data_ptr()
    p.peer_route_done_epoch[0] = flags.data_ptr()
    assert api.launch_gemm_a2a_cutlass(p, 0) == 801


def test_qkv_forward_two_payloads_and_epochs():
    # Stale data cannot pass: a second payload through the same buffers and flags with the next
    # epoch (benchmarks/sm103/fused_bf16.cu: two generations, poisoned outputs).
    from tests import harness as H
    world, batch, s, q, kv, d, k = 2, 1, 384, 8, 8, 64, 256
    m, n = batch * s, (q + 2 * kv) * d
    for generation in (0, 1):
        lhs, w = _inputs(world, m, k, n, generation=generation, normal=False)
        local, peers = H.qkv_forward(world, batch, s, q, kv, d, lhs, w, comm=6, epochs=2, alpha=0.5)
        want_local, want_peers = O.qkv_forward(world, batch, s, q, kv, d, lhs, w, alpha=0.5)
        for r in range(world):
            _assert_close(local[r], want_local[r], f"gen {generation} local[{r}]")
            _assert_close(peers[r], want_peers[r], f"gen {generation} peer[{r}]")


@pytest.mark.parametrize("raster,swizzle,block_n", [(N.RASTER_ALONG_M, 1, 128), (N.RASTER_ALONG_N, 2, 256),
                                                    (N.RASTER_ALONG_N, 8, 128), (N.RASTER_ALONG_M, 8, 256)])
def test_qkv_forward_knobs_do_not_change_results(raster, swizzle, block_n):
    from tests import harness as H
    world, batch, s, q, kv, d, k = 2, 1, 640, 8, 4, 128, 192
    m, n = batch * s, (q + 2 * kv) * d
    lhs, w = _inputs(world, m, k, n)
    base_local, base_peers = H.qkv_forward(world, batch, s, q, kv, d, lhs, w, comm=4)
    for route, vector in (("comm", False), ("direct", False), ("direct", True)):
        local, peers = H.qkv_forward(world, batch, s, q, kv, d, lhs, w, comm=7, raster=raster, swizzle=swizzle,
                                     block_n=block_n, route=route, vector_epilogue=vector)
        for r in range(world):  # same K order per element => identical bits whatever the schedule
            assert np.array_equal(local[r], base_local[r]) and np.array_equal(peers[r], base_peers[r])


# (world, batch, seq_local, heads, head_dim, n, comm, causal, cyclic)
OPROJ_CASES = [
    (1, 1, 256, 4, 128, 512, 2, False, False),
    (2, 1, 1024, 8, 128, 1024, 6, False, False),
    (4, 2, 200, 16, 64, 520, 5, True, False),     # causal two-chunk rows, ragged M and N
    (8, 1, 128, 32, 128, 4096, 16, False, True),  # cyclic K-shard order
    (4, 1, 96, 8, 40, 256, 3, True, True),        # K shard (80) not a multiple of the K block
    (1, 1, 130, 80, 128, 128, 2, False, False),   # one 20 KiB row per shard: rows cut into pieces
]


@pytest.mark.parametrize("pull", ["bulk", "vector"])
@pytest.mark.parametrize("case", OPROJ_CASES)
def test_oproj_forward_matches_oracle(case, pull):
    from tests import harness as H
    world, batch, s, heads, d, n, comm, causal, cyclic = case
    k = heads * d
    peer_in = [synthetic.normal_bf16((batch * s * world, k // world), synthetic.rank_seed(r) + 2000, 1.0)
               for r in range(world)]
    w = synthetic.normal_bf16((n, k), synthetic.BASE_SEED + 17, 0.02)
    for rank in sorted({0, world - 1, world // 2}):
        staging, out = H.oproj_forward(world, rank, batch, s, peer_in, w, comm=comm, causal=causal,
                                       cyclic=cyclic, pull=pull, vector_epilogue=(pull == "vector"))
        want_staging, want_out = O.oproj_forward(world, rank, batch, s, peer_in, w, causal=causal, cyclic=cyclic)
        assert np.array_equal(staging, want_staging), f"gathered lhs differs on rank {rank}"
        _assert_close(out, want_out, f"output[{rank}]")


@pytest.mark.parametrize("pair,embedded", [("0", "0"), ("1", "0"), ("1", "1")])
def test_oproj_forward_tile_and_pull_variants(monkeypatch, pair, embedded):
    # one-CTA tiles, CTA pairs with communication CTAs, CTA pairs with the embedded copy warps:
    # the switches are read on every launch
    from tests import harness as H
    monkeypatch.setenv("FUSE_B200_PAIR", pair)
    monkeypatch.setenv("FUSE_B200_EMBEDDED_PULL", embedded)
    world, batch, s, heads, d, n, comm = 4, 1, 512, 8, 128, 512, 4
    k = heads * d
    peer_in = [synthetic.normal_bf16((batch * s * world, k // world), synthetic.rank_seed(r) + 2000, 1.0)
               for r in range(world)]
    w = synthetic.normal_bf16((n, k), synthetic.BASE_SEED + 17, 0.02)
    for rank in (0, 3):
        staging, out = H.oproj_forward(world, rank, batch, s, peer_in, w, comm=comm)
        want_staging, want_out = O.oproj_forward(world, rank, batch, s, peer_in, w)
        assert np.array_equal(staging, want_staging), f"gathered lhs differs on rank {rank}"
        _assert_close(out, want_out, f"output[{rank}]")


def test_plain_gemm_entry_points_match_fused_outputs():
    import torch
    from tests import harness as H
    m, n, k = 520, 768, 328
    lhs, w = _inputs(1, m, k, n)
    a, b, d = H.to_device(lhs[0]), H.to_device(w), H.poisoned(m, n)
    p = N.GemmA2AParams(lhs=a.data_ptr(), rhs_nt=b.data_ptr(), local_output=d.data_ptr(),
                        gemm=N.GemmProblem(m, n, k), num_comm_ctas=1, epoch=1, alpha=2.0)
    assert api.launch_batched_cutlass_reference(p, 0, 20) == 0
    H.check_status()
    _assert_close(H.to_bits(d), O.gemm_bf16(0, lhs[0], w, m, n, k, alpha=2.0), "pure GEMM")
    torch.cuda.synchronize()


def test_device_generator_matches_host_generator():
    import torch
    from tests import harness as H
    count = 300001
    out = torch.zeros(count, dtype=torch.bfloat16, device=H.DEV)
    assert api.generate_bf16(out.data_ptr(), count, 777, 0.125, normal=False) == 0
    torch.cuda.synchronize()
    assert np.array_equal(H.to_bits(out), synthetic.uniform_bf16((count,), 777, 0.125))
    assert api.generate_bf16(out.data_ptr(), count, 778, 0.02, normal=True) == 0
    z = out.float()
    assert abs(float(z.mean())) < 2e-4 and abs(float(z.std()) - 0.02) < 2e-4


def test_rejections_on_device():
    # detail/gemm_a2a.cuh:237-299: geometry the route cannot express is cudaErrorNotSupported;
    # a communication budget that leaves no compute SM is cudaErrorInvalidValue.
    import torch
    from tests import harness as H
    buf = torch.zeros(1 << 20, dtype=torch.bfloat16, device=H.DEV)
    flags = torch.zeros(4096, dtype=torch.int32, device=H.DEV)

    def params(**route_kw):
        route = dict(world_size=2, rank=0, batch=1, global_seq=512, seq_local=256, q_heads=4, kv_heads=2,
                     head_dim=64, kind=N.ROUTE_QKV_GQA_PACK)
        route.update(route_kw)
        p = N.GemmA2AParams(lhs=buf.data_ptr(), rhs_nt=buf.data_ptr(), local_output=buf.data_ptr(),
                            ready=flags.data_ptr(), gemm=N.GemmProblem(256, 512, 64),
                            route=N.UlyssesRoute(**route), num_comm_ctas=4, epoch=1)
        for r in range(2):
            p.peer_output[r] = buf.data_ptr()
            p.peer_route_done_epoch[r] = flags.data_ptr()
        return p

    assert api.launch_gemm_a2a_cutlass(params(q_heads=3), 0) == N.CUDA_ERROR_NOT_SUPPORTED
    assert api.launch_gemm_a2a_cutlass(params(global_seq=500), 0) == N.CUDA_ERROR_NOT_SUPPORTED
    assert api.launch_gemm_a2a_cutlass(params(kind=N.ROUTE_HEAD_TO_SEQUENCE), 0) == N.CUDA_ERROR_NOT_SUPPORTED
    assert api.launch_gemm_a2a_cutlass(params(head_dim=60), 0) == N.CUDA_ERROR_NOT_SUPPORTED
    p = params()
    p.num_comm_ctas = 4096
    assert api.launch_gemm_a2a_cutlass(p, 0) == N.CUDA_ERROR_INVALID_VALUE
    p = params()
    p.peer_output[1] = buf.data_ptr() + 2  # misaligned peer buffer
    assert api.launch_gemm_a2a_cutlass(p, 0) == N.CUDA_ERROR_NOT_SUPPORTED
    torch.cuda.synchronize()
    assert api.read_status()[0] == 0


def test_bounded_wait_reports_instead_of_hanging():
    # An upstream flag that nothing publishes: the wait runs out after its budget, the kernel
    # returns, the status record says where, and the next launch works.
    import torch
    from tests import harness as H
    world, s, heads, d, n = 2, 256, 4, 64, 256
    k = heads * d
    peer_in = [H.to_device(synthetic.normal_bf16((s * world, k // world), 5 + r, 1.0)) for r in range(world)]
    w = H.to_device(synthetic.normal_bf16((n, k), 9, 0.02))
    staging, out = H.poisoned(s, k), H.poisoned(s, n)
    never = torch.zeros(N.READY_FLAG_STRIDE, dtype=torch.int32, device=H.DEV)
    problem = N.GemmProblem(s, n, k)
    route = N.UlyssesRoute(world_size=world, rank=0, batch=1, global_seq=s * world, seq_local=s,
                           kind=N.ROUTE_HEAD_TO_SEQUENCE, direction=N.ROUTE_INVERSE)
    ready = torch.zeros(api.a2a_lhs_gemm_ready_elements(problem, route), dtype=torch.int32, device=H.DEV)
    p = N.A2AGemmParams(input_staging=staging.data_ptr(), rhs_nt=w.data_ptr(), output=out.data_ptr(),
                        ready=ready.data_ptr(), gemm=problem, route=route, num_comm_ctas=2, epoch=1,
                        input_epoch=1)
    for q in range(world):
        p.peer_input[q] = peer_in[q].data_ptr()
        p.peer_input_ready[q] = never.data_ptr()
    assert api.launch_a2a_gemm_cutlass(p, 0, H.options(wait_ms=30.0)) == 0
    torch.cuda.synchronize()
    status = api.read_status(clear=True)
    assert status[0] != 0 and status[1] in (1, 2, 3) and status[7] == 1
    # the same launch with the flag published completes and is correct
    never.fill_(1)
    p.epoch = 2
    assert api.launch_a2a_gemm_cutlass(p, 0, H.options()) == 0
    H.check_status()
    want_staging, want_out = O.oproj_forward(world, 0, 1, s, [H.to_bits(x) for x in peer_in], H.to_bits(w))
    assert np.array_equal(H.to_bits(staging), want_staging)
    _assert_close(H.to_bits(out), want_out, "output after recovery")


def test_launch_from_a_second_host_thread():
    """A host thread that has never made a CUDA call of its own (a framework's backward thread)
    launches an operator: the library binds the device's context to the thread itself."""
    import threading
    import torch
    from tests import harness as H
    m, n, k = 256, 512, 256
    a = torch.randn((m, k), device=H.DEV).bfloat16()
    b = torch.randn((n, k), device=H.DEV).bfloat16()
    d = torch.zeros((m, n), dtype=torch.bfloat16, device=H.DEV)
    torch.cuda.synchronize()
    p = N.GemmA2AParams(lhs=a.data_ptr(), rhs_nt=b.data_ptr(), local_output=d.data_ptr(),
                        gemm=N.GemmProblem(m, n, k, max_swizzle_size=1), num_comm_ctas=1, epoch=1)
    result = {}

    def run():
        result["rc"] = api.launch_batched_cutlass_reference(p, 0, 0)

    thread = threading.Thread(target=run)
    thread.start()
    thread.join()
    torch.cuda.synchronize()
    assert result["rc"] == 0, result
    want = a.float() @ b.float().t()
    assert torch.allclose(d.float(), want, atol=0.5, rtol=0.02)
