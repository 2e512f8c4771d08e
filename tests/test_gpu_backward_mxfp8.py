"""MXFP8 backward against the CPU oracle: routed bytes / scales / BF16 masters bit for bit, GEMM
outputs within 0.01 + 0.01*|e| of the oracle's GEMM on the represented operands (the reference's
CPU check, benchmarks/sm103/backward/mxfp8_smoke.cu:87-134)."""
import numpy as np
import pytest

from fuse_b200 import synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _close(actual, expected, what):
    ok, worst, bad = O.within_tolerance(actual, expected)
    assert ok, f"{what}: {bad} elements outside 0.01+0.01|b| (max abs err {worst})"


def _weight_gradient_oracle(a_bits, b_bits, alpha, beta=0.0, init=None):
    """dW = alpha * A^T B + beta * dW with both operands re-quantised along the token axis."""
    qa, sa = O.mxfp8_quantize_transposed(a_bits)
    qb, sb = O.mxfp8_quantize_transposed(b_bits)
    prod = O.mxfp8_dequantize(qa, sa).astype(np.float64) @ O.mxfp8_dequantize(qb, sb).astype(np.float64).T
    if beta:
        prod = alpha * prod + beta * O.bf16_to_f32(init).astype(np.float64)
    else:
        prod = alpha * prod
    return O.f32_to_bf16(prod.astype(np.float32))


# (world, batch, seq_local, q_heads, kv_heads, hidden, comm, causal)
CASES = [
    (1, 1, 256, 2, 2, 256, 2, False),
    (2, 1, 256, 4, 2, 384, 4, True),       # causal halves of 128 rows
    (4, 2, 128, 8, 4, 512, 6, False),
]


@pytest.mark.parametrize("vector", [False, True])
@pytest.mark.parametrize("case", CASES)
def test_qkv_backward_mxfp8_matches_oracle(case, vector):
    from tests import harness as H
    world, batch, s, q, kv, hidden, comm, causal = case
    d = 128
    m, width, rows = batch * s, (q + 2 * kv) * d, batch * s * world
    planes = [tuple(synthetic.normal_bf16((rows, heads // world * d), synthetic.rank_seed(r) + 100 * seg + 101, 0.01)
                    for seg, heads in enumerate((q, kv, kv))) for r in range(world)]
    planes_q = [tuple(O.mxfp8_quantize(pl) for pl in planes[r]) for r in range(world)]
    w = synthetic.normal_bf16((width, hidden), synthetic.BASE_SEED + 11, 0.02)
    wt_q, wt_s = O.mxfp8_quantize_transposed(w)           # [H, QKV], quantised along QKV
    for rank in sorted({0, world - 1}):
        x = synthetic.normal_bf16((m, hidden), synthetic.rank_seed(rank) + 1000, 1.0)
        dw0 = synthetic.normal_bf16((width, hidden), synthetic.rank_seed(rank) + 7, 0.05)
        staging, dx, dw = H.qkv_backward_mxfp8(world, rank, batch, s, q, kv, planes, planes_q, w, x, comm=comm,
                                               causal=causal, alpha=0.5, beta=1.0, dw_init_bits=dw0, vector=vector)
        want_staging, _, _ = O.qkv_backward(world, rank, batch, s, q, kv, d, planes, w, x, causal=causal)
        assert np.array_equal(staging, want_staging), "BF16 masters routed for the weight gradient differ"
        # packed lhs of the data GEMM: owners' bytes and scale atoms, element by element
        lhs = np.empty((m, width), dtype=np.uint8)
        lhs_s = np.zeros(O.lib().fo_mxfp8_scale_bytes(m, width), dtype=np.uint8)
        import ctypes as C
        owner, seg, off = C.c_int32(), C.c_int32(), C.c_int64()
        for row in range(m):
            for head in range(q + 2 * kv):
                O.lib().fo_qkv_backward_source(world, rank, s, q, kv, d, int(causal), row, head * d,
                                               C.byref(owner), C.byref(seg), C.byref(off))
                data, scales = planes_q[owner.value][seg.value]
                pw = data.shape[1]
                src_row, src_col = off.value // pw, off.value % pw
                lhs[row, head * d:(head + 1) * d] = data[src_row, src_col:src_col + d]
                for kk in range(0, d, 32):
                    lhs_s[O.lib().fo_mxfp8_scale_offset(row, head * d + kk, width)] = \
                        scales[O.lib().fo_mxfp8_scale_offset(src_row, src_col + kk, pw)]
        _close(dx, O.gemm_mxfp8(lhs, lhs_s, wt_q, wt_s, alpha=0.5), f"dX[{rank}]")
        _close(dw, _weight_gradient_oracle(want_staging, x, 0.5, 1.0, dw0), f"dW[{rank}]")


@pytest.mark.parametrize("case", [(1, 1, 256, 2, 256, False), (2, 1, 256, 4, 384, True), (4, 2, 128, 8, 512, False)])
def test_oproj_backward_mxfp8_matches_oracle(case):
    from tests import harness as H
    world, batch, s, q, hidden, causal = case
    d = 128
    m, a = batch * s, q * d
    dys = [synthetic.normal_bf16((m, hidden), synthetic.rank_seed(r) + 301, 0.01) for r in range(world)]
    dy_q = [O.mxfp8_quantize(x) for x in dys]
    wo = synthetic.normal_bf16((hidden, a), synthetic.BASE_SEED + 17, 0.02)
    wot_q, wot_s = O.mxfp8_quantize_transposed(wo)        # [A, H], quantised along H
    attn = [synthetic.normal_bf16((m, a), synthetic.rank_seed(r) + 2000, 1.0) for r in range(world)]
    da, routed, dwo = H.oproj_backward_mxfp8(world, batch, s, q, dys, dy_q, wo, attn, causal=causal)
    for r in range(world):
        _close(da[r], O.gemm_mxfp8(dy_q[r][0], dy_q[r][1], wot_q, wot_s), f"dA[{r}]")
        _close(dwo[r], _weight_gradient_oracle(dys[r], attn[r], 1.0), f"dWo[{r}]")
    stacked = np.stack([x.reshape(-1) for x in da])
    shard, rows = a // world, batch * s * world
    for dest in range(world):
        idx = np.arange(rows * shard, dtype=np.int64)
        row, col = idx // shard, idx % shard
        b, seq = row // (s * world), row % (s * world)
        if causal:
            half = s // 2
            chunk = seq // half
            src = np.where(chunk < world, chunk, 2 * world - chunk - 1)
            local_row = np.where(chunk < world, 0, half) + seq % half
        else:
            src, local_row = seq // s, seq % s
        assert np.array_equal(routed[dest], stacked[src, (b * s + local_row) * a + dest * shard + col]), \
            f"routed bytes differ at destination {dest}"
