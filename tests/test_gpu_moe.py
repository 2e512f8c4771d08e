"""MoE dispatch -> expert FC1 grouped GEMM against the CPU oracle: gathered rows bit for bit,
GEMM within the reference's grouped tolerance 0.002 + 0.008*|b|
(benchmarks/sm103/grouped_validation.cuh:119-123), untouched capacity still holding the poison."""
import numpy as np
import pytest

from fuse_b200 import synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu
POISON = 0x7F7F


def _routes(world, tokens, experts, topk, seed, zipf=1.1):
    """Router scores ~ N(0,1) + per-expert Zipf(s) bias under a seeded permutation; top-k distinct
    experts per token (ties to the lower id); rows of an expert ordered by (rank, token, slot)."""
    rng = np.random.default_rng(seed)
    ranks = rng.permutation(experts) + 1
    bias = np.log(1.0 / ranks.astype(np.float64) ** zipf)
    bias -= bias.mean()
    chosen = []
    for r in range(world):
        scores = (synthetic.normal_f32((tokens, experts), seed + 17 * r + 1, 1.0) + bias).astype(np.float32)
        c = np.empty((tokens, topk), dtype=np.int32)
        O.lib().fo_moe_topk(O.ptr(np.ascontiguousarray(scores)), tokens, experts, topk, O.ptr(c))
        chosen.append(c)
    return chosen


def _rows_for(world, dest, experts_local, tokens, topk, chosen):
    offs = np.empty(experts_local + 1, dtype=np.int32)
    total = O.lib().fo_moe_build_rows(world, dest, experts_local, tokens, topk, O.ptr_array(chosen), O.ptr(offs), None)
    src = np.empty((max(total, 1), 3), dtype=np.int32)
    O.lib().fo_moe_build_rows(world, dest, experts_local, tokens, topk, O.ptr_array(chosen), O.ptr(offs), O.ptr(src))
    return offs.astype(np.int64), src[:total]


def _check(world, rank, experts_local, toks, weights, offs, src, capacity, lhs, out):
    e, n, k = weights.shape
    want_lhs = np.full((e, capacity, k), POISON, dtype=np.uint16)
    want_out = np.full((e, capacity, n), POISON, dtype=np.uint16)
    rc = O.lib().fo_moe_dispatch_fc1(e, O.ptr(offs.astype(np.int32)), O.ptr(np.ascontiguousarray(src, dtype=np.int32)),
                                     O.ptr_array(toks), O.ptr(np.ascontiguousarray(weights)), n, k, capacity,
                                     O.ptr(want_lhs), O.ptr(want_out))
    assert rc == 0
    assert np.array_equal(lhs.reshape(e, capacity, k), want_lhs), "gathered rows (or untouched capacity) differ"
    got = out.reshape(e, capacity, n)
    for ex in range(e):
        rows = int(offs[ex + 1] - offs[ex])
        ok, worst, bad = O.within_tolerance(got[ex, :rows], want_out[ex, :rows], 0.002, 0.008)
        assert ok, f"expert {ex}: {bad} elements outside 0.002+0.008|b| (max abs err {worst})"
        assert (got[ex, rows:] == POISON).all(), f"expert {ex}: rows past M_e were written"


# (world, tokens/rank, experts, topk, K, N, comm, tile_n)
MOE_CASES = [
    (1, 96, 4, 2, 256, 512, 2, 256),
    (2, 160, 8, 2, 512, 768, 4, 256),
    (4, 128, 16, 4, 1024, 384, 5, 128),     # K row = 2 KiB, N not a tile multiple
    (2, 64, 4, 2, 9216, 256, 3, 256),       # 18 KiB rows: a row is cut into two pieces
]


@pytest.mark.parametrize("case", MOE_CASES)
def test_moe_dispatch_fc1_matches_oracle(case):
    from tests import harness as H
    world, tokens, experts, topk, k, n, comm, tile_n = case
    experts_local = experts // world
    chosen = _routes(world, tokens, experts, topk, synthetic.GROUPED_SEED)
    toks = [synthetic.normal_bf16((tokens, k), synthetic.GROUPED_SEED + 31 * r + 5, 1.0) for r in range(world)]
    for rank in sorted({0, world - 1}):
        weights = synthetic.normal_bf16((experts_local, n, k), synthetic.GROUPED_SEED + 1000 + rank, 0.02)
        offs, src = _rows_for(world, rank, experts_local, tokens, topk, chosen)
        capacity = max(256, int(-(-int(np.diff(offs).max()) // 256) * 256))
        lhs, out = H.moe_dispatch_fc1(world, rank, experts_local, toks, weights, offs, src, capacity, comm=comm,
                                      tile_n=tile_n)
        _check(world, rank, experts_local, toks, weights, offs, src, capacity, lhs, out)


@pytest.mark.parametrize("auto", [False, True])
@pytest.mark.parametrize("case", [c for c in MOE_CASES if c[7] == 256])
def test_moe_dispatch_fc1_on_cta_pairs_matches_oracle(case, auto):
    # policy.mma_sm_count = 2: 256 x 256 tiles on CTA pairs, whole pairs of communication CTAs; with
    # policy.num_comm_ctas = 0 (Auto) no communication CTA at all: one thread of every compute CTA pulls
    from tests import harness as H
    world, tokens, experts, topk, k, n, comm, tile_n = case
    comm = 0 if auto else comm + comm % 2
    experts_local = experts // world
    chosen = _routes(world, tokens, experts, topk, synthetic.GROUPED_SEED)
    toks = [synthetic.normal_bf16((tokens, k), synthetic.GROUPED_SEED + 31 * r + 5, 1.0) for r in range(world)]
    for rank in sorted({0, world - 1}):
        weights = synthetic.normal_bf16((experts_local, n, k), synthetic.GROUPED_SEED + 1000 + rank, 0.02)
        offs, src = _rows_for(world, rank, experts_local, tokens, topk, chosen)
        capacity = max(256, int(-(-int(np.diff(offs).max()) // 256) * 256))
        lhs, out = H.moe_dispatch_fc1(world, rank, experts_local, toks, weights, offs, src, capacity, comm=comm,
                                      tile_n=tile_n, mma_sm_count=2)
        _check(world, rank, experts_local, toks, weights, offs, src, capacity, lhs, out)


@pytest.mark.parametrize("comm,mma_sm_count", [(4, 1), (4, 2), (0, 2)])
def test_moe_dispatch_gives_up_when_a_peer_never_enters_and_runs_clean_afterwards(comm, mma_sm_count):
    # bounded wait of the pull (communication CTAs, and the copy thread embedded in every compute CTA):
    # a peer's started epoch that nothing publishes
    from tests import harness as H
    world, tokens, experts, topk, k, n = 2, 96, 4, 2, 512, 512
    experts_local = experts // world
    chosen = _routes(world, tokens, experts, topk, synthetic.GROUPED_SEED)
    toks = [synthetic.normal_bf16((tokens, k), synthetic.GROUPED_SEED + 31 * r + 5, 1.0) for r in range(world)]
    weights = synthetic.normal_bf16((experts_local, n, k), synthetic.GROUPED_SEED + 1000, 0.02)
    offs, src = _rows_for(world, 0, experts_local, tokens, topk, chosen)
    capacity = max(256, int(-(-int(np.diff(offs).max()) // 256) * 256))
    lhs, out = H.moe_dispatch_fc1(world, 0, experts_local, toks, weights, offs, src, capacity, comm=comm,
                                  mma_sm_count=mma_sm_count, starved_first=True)
    _check(world, 0, experts_local, toks, weights, offs, src, capacity, lhs, out)


@pytest.mark.parametrize("mma_sm_count", [1, 2])
def test_moe_every_boundary_row_count_of_the_reference_list(mma_sm_count):
    # the reference's boundary list (benchmarks/sm103/grouped_validation.cuh:33), one expert each
    from tests import harness as H
    counts = [1, 7, 8, 9, 15, 16, 17, 63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256, 257, 0]
    world, tokens, k, n = 2, 400, 256, 256
    e = len(counts)
    toks = [synthetic.normal_bf16((tokens, k), 177 + r, 1.0) for r in range(world)]
    weights = synthetic.normal_bf16((e, n, k), 199, 0.02)
    rng = np.random.default_rng(15)
    offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    total = int(offs[-1])
    src = np.stack([rng.integers(0, world, total), rng.integers(0, tokens, total), rng.integers(0, 2, total)], 1).astype(np.int32)
    capacity = 512
    lhs, out = H.moe_dispatch_fc1(world, 1, e, toks, weights, offs, src, capacity, comm=4, mma_sm_count=mma_sm_count)
    _check(world, 1, e, toks, weights, offs, src, capacity, lhs, out)


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("mma_sm_count", [1, 2])
def test_moe_boundary_row_counts_empty_experts_and_replay_with_new_routes(mma_sm_count, graph):
    # Row counts at tile boundaries and empty experts (benchmarks/sm103/grouped_validation.cuh:20-50);
    # then the same plan replayed with different device routes -- eagerly, and as replays of ONE
    # captured CUDA graph (the launch allocates nothing and reads row counts and routes on the device).
    from tests import harness as H
    world, tokens, k, n = 2, 600, 256, 512
    counts_a = [1, 0, 127, 128, 129, 257, 0, 63]
    counts_b = [0, 255, 256, 7, 0, 193, 65, 9]
    e = len(counts_a)
    toks = [synthetic.normal_bf16((tokens, k), 77 + r, 1.0) for r in range(world)]
    weights = synthetic.normal_bf16((e, n, k), 99, 0.02)
    rng = np.random.default_rng(5)

    def make(counts):
        offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
        total = int(offs[-1])
        src = np.stack([rng.integers(0, world, total), rng.integers(0, tokens, total), rng.integers(0, 2, total)], 1)
        return offs, src.astype(np.int32)

    first, second = make(counts_a), make(counts_b)
    capacity = 512
    comm = 3 if mma_sm_count == 1 else 0  # pairs: Auto, the embedded pull
    lhs, out = H.moe_dispatch_fc1(world, 0, e, toks, weights, first[0], first[1], capacity, comm=comm, launches=2,
                                  mma_sm_count=mma_sm_count, graph=graph)
    _check(world, 0, e, toks, weights, first[0], first[1], capacity, lhs, out)
    lhs, out = H.moe_dispatch_fc1(world, 0, e, toks, weights, first[0], first[1], capacity, comm=comm,
                                  second_route=second, mma_sm_count=mma_sm_count, graph=graph)
    _check(world, 0, e, toks, weights, second[0], second[1], capacity, lhs, out)


# ---------------------------------------------------------------------------------------------
# combine: expert FC2 grouped GEMM -> rows scattered to the token owners
# (world, tokens/rank, experts, topk, K, N, tile_n, mma_sm_count)
COMBINE_CASES = [
    (1, 96, 4, 2, 256, 512, 256, 1),
    (2, 160, 8, 2, 512, 768, 256, 1),
    (4, 128, 16, 4, 256, 392, 128, 1),      # N neither a tile nor a 64-column multiple
    (2, 160, 8, 2, 512, 768, 256, 2),       # CTA pairs
    (4, 200, 8, 3, 320, 1024, 256, 2),
]


@pytest.mark.parametrize("starved_first", [False, True])
@pytest.mark.parametrize("case", COMBINE_CASES)
def test_moe_fc2_combine_matches_oracle(case, starved_first):
    # The reference's checks for this direction (benchmarks/sm103/grouped_validation.cuh:119-157): the
    # expert's output slab within 0.002 + 0.008|b| with untouched capacity still poisoned, and every
    # received branch row BIT-EXACT equal to the row its owner's slab holds; rows no expert routes keep
    # the poison.
    # starved_first: rank 0 first launches while no destination has entered the invocation; the
    # bounded wait before its first remote write runs out and the launch publishes no done epoch.
    from tests import harness as H
    world, tokens, experts, topk, k, n, tile_n, mma = case
    if starved_first and (world == 1 or tile_n != 256):
        pytest.skip("needs a peer; one case per tile family is enough")
    e_local = experts // world
    chosen = _routes(world, tokens, experts, topk, seed=23)
    routes = [_rows_for(world, r, e_local, tokens, topk, chosen) for r in range(world)]
    capacity = int(-(-max(int(np.diff(o).max()) for o, _ in routes) // 256) * 256)
    lhs = [synthetic.normal_bf16((e_local, capacity, k), synthetic.GROUPED_SEED + 7 * r, 1.0) for r in range(world)]
    weights = [synthetic.normal_bf16((e_local, n, k), synthetic.GROUPED_SEED + 500 + r, 0.02) for r in range(world)]
    outputs, received = H.moe_fc2_combine(world, e_local, lhs, weights, [o for o, _ in routes], [s for _, s in routes],
                                          capacity, tokens, topk, tile_n=tile_n, mma_sm_count=mma, launches=2,
                                          starved_first=starved_first)
    want_received = [np.full((tokens * topk, n), POISON, dtype=np.uint16) for _ in range(world)]
    table = O.ptr_array(want_received)
    for r in range(world):
        offs, src = routes[r]
        want_out = np.full((e_local, capacity, n), POISON, dtype=np.uint16)
        assert O.lib().fo_moe_fc2_combine(e_local, O.ptr(offs.astype(np.int32)), O.ptr(np.ascontiguousarray(src, dtype=np.int32)),
                                          O.ptr(lhs[r]), O.ptr(weights[r]), n, k, capacity, topk, O.ptr(want_out), table) == 0
        got = outputs[r].reshape(e_local, capacity, n)
        for ex in range(e_local):
            rows = int(offs[ex + 1] - offs[ex])
            ok, worst, bad = O.within_tolerance(got[ex, :rows], want_out[ex, :rows], 0.002, 0.008)
            assert ok, f"rank {r} expert {ex}: {bad} elements outside 0.002+0.008|b| (max abs err {worst})"
            assert (got[ex, rows:] == POISON).all(), f"rank {r} expert {ex}: rows past M_e were written"
            # the scattered rows are the slab's rows, bit for bit
            for row in range(rows):
                rank, token, slot = (int(v) for v in src[int(offs[ex]) + row])
                assert np.array_equal(received[rank].reshape(tokens * topk, n)[token * topk + slot], got[ex, row]), \
                    f"branch row of rank {rank} token {token} slot {slot} differs from its owner's slab"
    for r in range(world):
        got = received[r].reshape(tokens * topk, n)
        routed = (want_received[r] != POISON).any(axis=1)
        assert (got[~routed] == POISON).all(), "a branch row nobody routes was written"
        ok, worst, bad = O.within_tolerance(got[routed], want_received[r][routed], 0.002, 0.008)
        assert ok, f"received rows of rank {r}: {bad} elements outside tolerance (max abs err {worst})"
        assert routed.all(), "top-k routing covers every (token, slot)"
