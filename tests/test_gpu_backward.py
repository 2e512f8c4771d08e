"""Parity of the CUDA backward operators (data gradient through the reverse all-to-all, local
weight gradient) with the CPU oracle, through the C ABI.  Routing bit-exact; GEMM outputs
within the reference's backward tolerance 0.02 + 0.02*|b|
(benchmarks/sm103/backward/validation.cuh:60-73)."""
import numpy as np
import pytest

from fuse_b200 import synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _close(actual, expected, what):
    ok, worst, bad = O.within_tolerance(actual, expected, 0.02, 0.02)
    assert ok, f"{what}: {bad} elements outside 0.02+0.02|b| (max abs err {worst})"


# (world, batch, seq_local, q_heads, kv_heads, head_dim, hidden, comm, causal)
QKV_BWD_CASES = [
    (1, 1, 256, 4, 2, 64, 256, 2, False),
    (2, 1, 384, 8, 4, 128, 320, 4, False),
    (2, 2, 136, 4, 4, 64, 192, 3, True),      # batch 2, ragged M, causal two-chunk rows
    (4, 1, 128, 16, 4, 128, 512, 6, True),
]


@pytest.mark.parametrize("vector", [False, True])
@pytest.mark.parametrize("case", QKV_BWD_CASES)
def test_qkv_backward_matches_oracle(case, vector):
    from tests import harness as H
    world, batch, s, q, kv, d, hidden, comm, causal = case
    m, width, rows = batch * s, (q + 2 * kv) * d, batch * s * world
    # upstream gradients ~ N(0, 1e-2), activations ~ N(0, 1), weights ~ N(0, 0.02)
    planes = [tuple(synthetic.normal_bf16((rows, heads // world * d), synthetic.rank_seed(r) + 100 * seg + 101, 0.01)
                    for seg, heads in enumerate((q, kv, kv))) for r in range(world)]
    w = synthetic.normal_bf16((width, hidden), synthetic.BASE_SEED + 11, 0.02)
    xs = [synthetic.normal_bf16((m, hidden), synthetic.rank_seed(r) + 1000, 1.0) for r in range(world)]
    dw0 = [synthetic.normal_bf16((width, hidden), synthetic.rank_seed(r) + 7, 0.05) for r in range(world)]
    got = H.qkv_backward(world, batch, s, q, kv, d, planes, w, xs, comm=comm, causal=causal, alpha=0.5,
                         beta=1.0, dw_init_bits=dw0, vector=vector)
    for r in range(world):
        staging, dx, dw = O.qkv_backward(world, r, batch, s, q, kv, d, planes, w, xs[r], causal=causal,
                                         alpha=0.5, beta=1.0, grad_weight=dw0[r])
        assert np.array_equal(got[r][0], staging), f"routed gradient differs on rank {r}"
        _close(got[r][1], dx, f"dX[{r}]")
        _close(got[r][2], dw, f"dW[{r}]")


def test_timed_out_launch_publishes_no_completion_and_the_next_launch_is_correct():
    # Head gates that nobody releases (no rank has pushed yet): the GEMM's bounded wait runs out,
    # the status record says so, and the rank must NOT release its completion epoch to the peers --
    # they would read half-written rows behind it.  After a clear, the full run is correct.
    from tests import harness as H
    world, batch, s, q, kv, d, hidden, comm = 2, 1, 256, 4, 2, 128, 256, 4
    m, width, rows = batch * s, (q + 2 * kv) * d, batch * s * world
    planes = [tuple(synthetic.normal_bf16((rows, heads // world * d), synthetic.rank_seed(r) + 100 * seg + 31, 0.01)
                    for seg, heads in enumerate((q, kv, kv))) for r in range(world)]
    w = synthetic.normal_bf16((width, hidden), synthetic.BASE_SEED + 11, 0.02)
    xs = [synthetic.normal_bf16((m, hidden), synthetic.rank_seed(r) + 1000, 1.0) for r in range(world)]
    got = H.qkv_backward(world, batch, s, q, kv, d, planes, w, xs, comm=comm, starved_first=True)
    for r in range(world):
        staging, dx, dw = O.qkv_backward(world, r, batch, s, q, kv, d, planes, w, xs[r])
        assert np.array_equal(got[r][0], staging), f"routed gradient differs on rank {r}"
        _close(got[r][1], dx, f"dX[{r}]")
        _close(got[r][2], dw, f"dW[{r}]")


def test_qkv_backward_weight_overwrites_when_beta_is_zero():
    from tests import harness as H
    world, batch, s, q, kv, d, hidden = 1, 1, 200, 2, 2, 64, 136
    rows, width = batch * s * world, (q + 2 * kv) * d
    planes = [tuple(synthetic.normal_bf16((rows, heads * d), 50 + seg, 0.01) for seg, heads in enumerate((q, kv, kv)))]
    w = synthetic.normal_bf16((width, hidden), 3, 0.02)
    xs = [synthetic.normal_bf16((batch * s, hidden), 4, 1.0)]
    got = H.qkv_backward(world, batch, s, q, kv, d, planes, w, xs, comm=2)  # dW starts poisoned (NaN)
    staging, dx, dw = O.qkv_backward(world, 0, batch, s, q, kv, d, planes, w, xs[0])
    assert np.array_equal(got[0][0], staging)
    _close(got[0][1], dx, "dX")
    _close(got[0][2], dw, "dW")


# (world, batch, seq_local, q_heads, head_dim, hidden, comm, causal)
OPROJ_BWD_CASES = [
    (1, 1, 256, 4, 64, 256, 2, False),
    (2, 1, 512, 8, 128, 384, 4, True),        # causal, half = 256 rows: tensor-store push
    (2, 2, 200, 4, 64, 192, 3, True),         # ragged: vector push
    (4, 1, 128, 16, 128, 512, 6, False),
]


@pytest.mark.parametrize("route", ["direct", "comm"])
@pytest.mark.parametrize("case", OPROJ_BWD_CASES)
def test_oproj_backward_matches_oracle(case, route):
    from tests import harness as H
    world, batch, s, q, d, hidden, comm, causal = case
    m, a = batch * s, q * d
    dys = [synthetic.normal_bf16((m, hidden), synthetic.rank_seed(r) + 301, 0.01) for r in range(world)]
    wo = synthetic.normal_bf16((hidden, a), synthetic.BASE_SEED + 17, 0.02)
    attn = [synthetic.normal_bf16((m, a), synthetic.rank_seed(r) + 2000, 1.0) for r in range(world)]
    da, routed, dwo = H.oproj_backward(world, batch, s, q, d, dys, wo, attn, comm=comm, causal=causal, route=route)
    want_da, want_routed, want_dwo = O.oproj_backward(world, batch, s, q, d, dys, wo, attn, causal=causal)
    # route: the destination buffers hold exactly the bytes of the GPU's own dA at the mapped places
    for r in range(world):
        _close(da[r], want_da[r], f"dA[{r}]")
        _close(dwo[r], want_dwo[r], f"dWo[{r}]")
        _close(routed[r], want_routed[r], f"routed[{r}]")
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
        expect = stacked[src, (b * s + local_row) * a + dest * shard + col]
        assert np.array_equal(routed[dest], expect), f"routed bytes differ at destination {dest}"
