"""MXFP8 on the GPU against the CPU oracle: quantised bytes and scale bytes bit for bit
(csrc/operators/sm103/detail/quantization.cuh:91-141 arithmetic, native scale layout), block-scaled
GEMM outputs within 0.01 + 0.01*|b| of the oracle's GEMM on the represented operands
(benchmarks/sm103/fused_mxfp8.cuh:54-73), routing bit-exact."""
import numpy as np
import pytest

from fuse_b200 import synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _wide_range(shape, seed):
    """BF16 values spanning many binades, with zero blocks and exact powers of two."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(shape) * np.exp(rng.uniform(-8, 8, (shape[0], 1)))
    x = x.astype(np.float32)
    x[0, :32] = 0.0
    if shape[0] > 2:
        x[1, :32] = 448.0
        x[2, :32] = 2.0 ** -130  # BF16 subnormal range
    return O.f32_to_bf16(x)


@pytest.mark.parametrize("shape", [(128, 128), (160, 256), (300, 1024), (1, 32)])
def test_row_quantiser_is_bit_exact(shape):
    from tests import harness as H
    src = _wide_range(shape, 3)
    data, scales = H.quantize_mxfp8(src)
    want_data, want_scales = O.mxfp8_quantize(src)
    assert np.array_equal(data, want_data)
    assert np.array_equal(scales, want_scales)


# (128, 256), (384, 192), (256, 64), (1024, 320): the tiled kernel (128-row x 64-column tiles; 192 and 320
# columns leave half a row atom to be filled with neutral scales); the others: the general kernel
@pytest.mark.parametrize("shape", [(128, 256), (96, 130), (512, 1000), (32, 2), (384, 192), (256, 64), (1024, 320)])
def test_transposed_quantiser_is_bit_exact(shape):
    from tests import harness as H
    src = _wide_range(shape, 5)
    data, scales = H.quantize_mxfp8(src, transposed=True)
    want_data, want_scales = O.mxfp8_quantize_transposed(src)
    assert np.array_equal(data, want_data)
    assert np.array_equal(scales, want_scales)


def _mx_inputs(world, m, k, n):
    acts = [synthetic.normal_bf16((m, k), synthetic.rank_seed(r) + 1000, 1.0) for r in range(world)]
    w = synthetic.normal_bf16((n, k), synthetic.BASE_SEED + 11, 0.02)
    quant = [O.mxfp8_quantize(a) for a in acts]
    return acts, w, [q[0] for q in quant], [q[1] for q in quant]


def _close(actual, expected, what):
    ok, worst, bad = O.within_tolerance(actual, expected)
    assert ok, f"{what}: {bad} elements outside 0.01+0.01|b| (max abs err {worst})"


@pytest.mark.parametrize("shape", [(128, 256, 128), (256, 512, 512), (384, 384, 256), (1000, 776, 640)])
def test_block_scaled_gemm_matches_oracle(shape):
    from tests import harness as H
    m, n, k = shape
    _, w, data, scales = _mx_inputs(1, m, k, n)
    heads = n // 128 if n % 384 == 0 else None
    # geometry only matters for routing; compute mode ignores the route
    local, _, (wq, wsf) = H.qkv_forward_mxfp8(1, 1, m, 1, 1, 8, data, scales, w, mode="compute")
    want_wq, want_wsf = O.mxfp8_quantize(w)
    assert np.array_equal(wq, want_wq) and np.array_equal(wsf, want_wsf)
    _close(local[0], O.gemm_mxfp8(data[0], scales[0], want_wq, want_wsf), "block-scaled GEMM")
    del heads


# (world, batch, seq_local, q_heads, kv_heads, head_dim, k, comm)
MX_QKV_CASES = [
    (1, 1, 256, 4, 4, 128, 256, 2),
    (2, 1, 512, 8, 8, 128, 512, 4),
    (2, 2, 200, 8, 4, 64, 384, 3),       # ragged M: vector push
    (4, 1, 128, 16, 4, 128, 1024, 6),
]


@pytest.mark.parametrize("route", ["direct", "comm"])
@pytest.mark.parametrize("case", MX_QKV_CASES)
def test_qkv_forward_mxfp8_matches_oracle(case, route):
    from tests import harness as H
    world, batch, s, q, kv, d, k, comm = case
    m, n = batch * s, (q + 2 * kv) * d
    _, w, data, scales = _mx_inputs(world, m, k, n)
    local, peers, (wq, wsf) = H.qkv_forward_mxfp8(world, batch, s, q, kv, d, data, scales, w, comm=comm, route=route)
    want_wq, want_wsf = O.mxfp8_quantize(w)
    assert np.array_equal(wq, want_wq) and np.array_equal(wsf, want_wsf), "in-kernel weight quantisation"
    for r in range(world):
        _close(local[r], O.gemm_mxfp8(data[r], scales[r], want_wq, want_wsf), f"local[{r}]")
    rerouted = [np.full(peers[0].size, 0xFFFF, dtype=np.uint16) for _ in range(world)]
    table = O.ptr_array(rerouted)
    for r in range(world):
        O.lib().fo_qkv_forward_route(world, r, batch, s, q, kv, d, O.ptr(np.ascontiguousarray(local[r])), n, table)
    for dest in range(world):
        assert np.array_equal(peers[dest], rerouted[dest]), f"routed bytes differ at destination {dest}"


def test_prepared_and_in_kernel_weight_paths_agree():
    from tests import harness as H
    world, batch, s, q, kv, d, k = 1, 1, 384, 4, 2, 128, 512
    m, n = batch * s, (q + 2 * kv) * d
    _, w, data, scales = _mx_inputs(world, m, k, n)
    full, peers_full, _ = H.qkv_forward_mxfp8(world, batch, s, q, kv, d, data, scales, w, mode="full", alpha=0.5)
    prep, peers_prep, _ = H.qkv_forward_mxfp8(world, batch, s, q, kv, d, data, scales, w, mode="prepared", alpha=0.5)
    assert np.array_equal(full[0], prep[0]) and np.array_equal(peers_full[0], peers_prep[0])


def test_oproj_forward_mxfp8_refuses_scheduler_windows_the_reference_refuses():
    # csrc/operators/sm103/detail/persistent_gemm.cuh:55-59: both window sizes powers of two when either is set
    from tests import harness as H
    world, batch, s, heads, d, n = 1, 1, 256, 4, 128, 512
    src = synthetic.normal_bf16((batch * s, heads * d), 5, 1.0)
    data, scales = O.mxfp8_quantize(src)
    w = synthetic.normal_bf16((n, heads * d), 6, 0.02)
    for window in ((3, 4), (64, 0), (0, 4), (-2, 2)):
        H.oproj_forward_mxfp8(world, 0, batch, s, [data], [scales], w, comm=2, window=window, expect_rc=801)


# (world, batch, seq_local, heads, head_dim, n, comm, causal, cyclic)
MX_OPROJ_CASES = [
    (1, 1, 256, 4, 128, 512, 2, False, False),
    (2, 1, 512, 8, 128, 1024, 4, False, False),
    (4, 2, 256, 16, 64, 520, 5, True, False),     # causal halves of 128 rows, batch 2, ragged N
    (8, 1, 128, 32, 128, 2048, 8, False, True),   # cyclic K-shard order
    (1, 1, 128, 80, 128, 128, 2, False, False),   # 80 scale atoms per row group: two scale chunks
]


@pytest.mark.parametrize("case", MX_OPROJ_CASES)
def test_oproj_forward_mxfp8_matches_oracle(case):
    from tests import harness as H
    world, batch, s, heads, d, n, comm, causal, cyclic = case
    k = heads * d
    shard = k // world
    rows = batch * s * world
    # every source rank quantises its own head shard [B*S_global, K/world] along its own K
    sources = [synthetic.normal_bf16((rows, shard), synthetic.rank_seed(r) + 2000, 1.0) for r in range(world)]
    quant = [O.mxfp8_quantize(x) for x in sources]
    w = synthetic.normal_bf16((n, k), synthetic.BASE_SEED + 17, 0.02)
    want_wq, want_wsf = O.mxfp8_quantize(w)
    for rank in sorted({0, world - 1}):
        # (the scheduler windows of the reference's published rows, H64 / P4, are accepted as hints)
        staged, staged_scales, out = H.oproj_forward_mxfp8(world, rank, batch, s, [q[0] for q in quant],
                                                           [q[1] for q in quant], w, comm=comm, causal=causal,
                                                           cyclic=cyclic, window=(64, 4) if rank else (0, 0))
        # byte + scale-byte transport oracle (benchmarks/sm103/fused_mxfp8.cuh:25-47)
        m = batch * s
        want_data = np.empty((m, k), dtype=np.uint8)
        want_scales = np.zeros(O.lib().fo_mxfp8_scale_bytes(m, k), dtype=np.uint8)
        for row in range(m):
            src_row = O.lib().fo_global_row(world, rank, s, int(causal), row)
            for j in range(world):
                peer = (rank + j) % world if cyclic else j
                want_data[row, j * shard:(j + 1) * shard] = quant[peer][0][src_row]
                for kk in range(0, shard, 32):
                    want_scales[O.lib().fo_mxfp8_scale_offset(row, j * shard + kk, k)] = \
                        quant[peer][1][O.lib().fo_mxfp8_scale_offset(src_row, kk, shard)]
        assert np.array_equal(staged, want_data), f"gathered bytes differ on rank {rank}"
        assert np.array_equal(staged_scales, want_scales), f"gathered scales differ on rank {rank}"
        _close(out, O.gemm_mxfp8(want_data, want_scales, want_wq, want_wsf), f"output[{rank}]")
