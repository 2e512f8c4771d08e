"""Pins the CPU oracle (oracle/fuse_oracle.c) against golden vectors recorded from the
reference's own host code (tests/golden/make_golden.py), against that code directly where the
reference tree is mounted, and against the known answers the reference's tests hold."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))
L = O.lib()


def test_gqa_feature_map_matches_reference_vectors():
    # include/fuse/layout/ulysses.h:77-137 answers for every feature of eight geometries,
    # including out-of-range features and the uneven-head rejections.
    rows = GOLDEN["gqa_map"]
    for w, q, kv, d, f, valid, owner, local, seg, head, off, inv in rows[::3]:
        a = (C.c_int32 * 5)()
        got = L.fo_map_qkv_gqa_feature(int(w), int(q), int(kv), int(d), int(f), a)
        assert got == valid
        assert list(a) == [owner, local, seg, head, off]
        if valid:
            assert L.fo_qkv_gqa_global_feature(int(w), int(q), int(kv), int(d), a[0], a[1]) == inv == f


def test_gqa_map_is_invertible_and_rejects_uneven_heads():
    # benchmarks/sm90/QKVproj+a2a/fuse_smoke.cu:228-270.
    for (w, q, kv, d) in [(2, 8, 8, 64), (2, 8, 4, 96), (4, 16, 4, 80), (4, 32, 4, 128)]:
        seen = set()
        for f in range((q + 2 * kv) * d):
            a = (C.c_int32 * 5)()
            assert L.fo_map_qkv_gqa_feature(w, q, kv, d, f, a) == 1
            assert L.fo_qkv_gqa_global_feature(w, q, kv, d, a[0], a[1]) == f
            seen.add((a[0], a[1]))
        assert len(seen) == (q + 2 * kv) * d
    a = (C.c_int32 * 5)()
    assert L.fo_map_qkv_gqa_feature(3, 8, 8, 64, 0, a) == 0
    assert L.fo_qkv_gqa_global_feature(3, 8, 8, 64, 0, 0) == -1


def test_qkv_receiver_view_matches_reference_vectors():
    for w, s, q, kv, d, dest, index, rank, off in GOLDEN["qkv_oracle"]:
        r, o = C.c_int32(), C.c_uint64()
        L.fo_qkv_oracle_source(int(w), int(dest), int(s), int(q * d), int(kv * d), int(index),
                               C.byref(r), C.byref(o))
        assert (r.value, o.value) == (rank, off)


def test_qkv_sender_and_receiver_views_agree():
    # The sender-side map (what the kernel computes) must be the inverse of the reference's
    # receiver-side validation oracle, element by element.
    for (w, s, q, kv, d) in [(2, 6, 4, 2, 8), (4, 5, 8, 4, 16), (8, 3, 16, 8, 8)]:
        n = (q + 2 * kv) * d
        for rank in range(w):
            for row in range(s):
                for f in range(n):
                    dest, off = C.c_int32(), C.c_int64()
                    assert L.fo_qkv_forward_destination(w, rank, 1, s, q, kv, d, row, f,
                                                        C.byref(dest), C.byref(off))
                    r, o = C.c_int32(), C.c_uint64()
                    L.fo_qkv_oracle_source(w, dest.value, s, q * d, kv * d, off.value,
                                           C.byref(r), C.byref(o))
                    assert (r.value, o.value) == (rank, row * n + f)


def test_oproj_gather_matches_reference_vectors():
    for w, s, width, causal, dest, index, rank, off in GOLDEN["oproj_gather"]:
        r, o = C.c_int32(), C.c_uint64()
        L.fo_oproj_gather_source(int(w), int(dest), int(s), int(width), int(causal), 0, int(index),
                                 C.byref(r), C.byref(o))
        assert (r.value, o.value) == (rank, off)


def test_route_formulas_of_the_reference_python_tests():
    # scripts/test_sm103_fusion_routes.py:70-86: qkv_sequence_row / oproj_sequence_row.
    def sequence_row(world, rank, seq_local, row, causal):
        if not causal:
            return rank * seq_local + row
        half = seq_local // 2
        chunk = rank if row < half else 2 * world - rank - 1
        return chunk * half + row % half
    for world in (2, 4, 8):
        for seq_local in (4, 10):
            for rank in range(world):
                for row in range(seq_local):
                    for causal in (0, 1):
                        assert L.fo_global_row(world, rank, seq_local, causal, row) == \
                            sequence_row(world, rank, seq_local, row, causal)
    # causal assignment is a permutation of the global sequence
    for world in (2, 4):
        rows = sorted(L.fo_global_row(world, r, 8, 1, i) for r in range(world) for i in range(8))
        assert rows == list(range(8 * world))


def test_backward_routes_are_inverses_of_forward_routes():
    # OProj backward (seq->head) receiver view inverts the forward gather; QKV backward
    # receiver view inverts the forward QKV push (benchmarks/sm103/backward/validation.cuh:27-57).
    w, s, heads, d = 4, 6, 8, 8
    width = heads * d
    for causal in (0, 1):
        for rank in range(w):
            for index in range(s * w * (width // w)):
                src, off = C.c_int32(), C.c_uint64()
                L.fo_oproj_backward_source(w, rank, 1, s, width, causal, index, C.byref(src), C.byref(off))
                # forward gather of element `off` at rank `src` must read (rank, index)
                r2, o2 = C.c_int32(), C.c_uint64()
                L.fo_oproj_gather_source(w, src.value, s, width, causal, 0, off.value, C.byref(r2), C.byref(o2))
                assert (r2.value, o2.value) == (rank, index)
    q, kv = 8, 4
    n = (q + 2 * kv) * d
    for rank in range(w):
        for row in range(s):
            for f in range(n):
                owner, seg, off = C.c_int32(), C.c_int32(), C.c_int64()
                L.fo_qkv_backward_source(w, rank, s, q, kv, d, 0, row, f, C.byref(owner), C.byref(seg), C.byref(off))
                dest, doff = C.c_int32(), C.c_int64()
                L.fo_qkv_forward_destination(w, rank, 1, s, q, kv, d, row, f, C.byref(dest), C.byref(doff))
                rows = s * w
                base = 0 if seg.value == 0 else rows * (q // w * d) + (rows * (kv // w * d) if seg.value == 2 else 0)
                assert dest.value == owner.value and doff.value == base + off.value


def test_swizzle_rule():
    # benchmarks/sm103/fused_bf16.cu:196-206.
    assert L.fo_swizzle_size(8, 6, 100) == 8
    assert L.fo_swizzle_size(8, 5, 100) == 4
    assert L.fo_swizzle_size(4, 3, 3) == 4
    assert L.fo_swizzle_size(4, 2, 9) == 2
    assert L.fo_swizzle_size(2, 2, 2) == 2
    assert L.fo_swizzle_size(8, 1, 50) == 1
    assert L.fo_swizzle_size(1, 50, 50) == 1


def test_scalar_formats_match_reference_vectors():
    dec = GOLDEN["e4m3_decode"]
    for v in range(256):
        got = L.fo_e4m3_to_f32(v)
        assert (got == dec[v]) or (np.isnan(got) and np.isnan(dec[v]))
    xs, e4, bf = GOLDEN["e4m3_encode_in"], GOLDEN["e4m3_encode_out"], GOLDEN["bf16_encode_out"]
    for x, a, b in zip(xs[::5], e4[::5], bf[::5]):
        assert L.fo_f32_to_e4m3(float(x)) == a
        assert L.fo_f32_to_bf16(float(x)) == b
    assert np.array_equal(O.f32_to_bf16(xs), bf)
    for w, v in zip(GOLDEN["uniform_words"], GOLDEN["uniform_out"]):
        assert L.fo_uniform_value(int(w), 0.125) == v


def test_mxfp8_exponent_formulations_agree():
    # csrc/operators/sm103/detail/quantization.cuh:91-105 (integer form) must agree with the
    # validators' frexp form (benchmarks/sm103/fused_mxfp8.cuh:64-71) on every BF16 magnitude.
    for bits in range(0, 0x7F80):
        amax = float(O.bf16_to_f32(np.array([bits], dtype=np.uint16))[0])
        assert L.fo_mxfp8_scale_exponent(amax) == L.fo_mxfp8_scale_exponent_frexp(amax), hex(bits)
    assert L.fo_mxfp8_scale_exponent(0.0) == 0
    assert L.fo_mxfp8_scale_exponent(448.0) == 0
    assert L.fo_mxfp8_scale_exponent(449.0) == 1
    assert L.fo_mxfp8_scale_exponent(1.0) == -8


def test_mxfp8_quantise_roundtrip_and_layout():
    rng = np.random.default_rng(3)
    rows, k = 160, 256  # rows not a multiple of 128: scale storage is padded to 128 rows
    src = O.f32_to_bf16((rng.standard_normal((rows, k)) * np.exp(rng.uniform(-6, 6, (rows, 1)))).astype(np.float32))
    src[5, 32:64] = 0  # an all-zero K block keeps scale 2^0 and zero data
    data, scales = O.mxfp8_quantize(src)
    assert scales.size == 2 * 2 * 512
    assert scales[L.fo_mxfp8_scale_offset(5, 32, k)] == 127 and not data[5, 32:64].any()
    deq = O.mxfp8_dequantize(data, scales)
    rep = np.empty((rows, k), dtype=np.float32)
    L.fo_mxfp8_represented(O.ptr(src), rows * k, O.ptr(rep))
    assert np.array_equal(deq, rep)  # the two independent formulations give the same operand
    ref = O.bf16_to_f32(src)
    amax = np.abs(ref.reshape(rows, k // 32, 32)).max(-1, keepdims=True)
    err = np.abs(deq.reshape(rows, k // 32, 32) - ref.reshape(rows, k // 32, 32))
    assert (err <= amax / 8 + 1e-30).all()  # E4M3 has 3 mantissa bits below the block maximum
    # scale offsets: every (row, k-block) of a padded operand maps to a distinct byte
    offs = {L.fo_mxfp8_scale_offset(r, kk, k) for r in range(256) for kk in range(0, k, 32)}
    assert len(offs) == 256 * (k // 32) and max(offs) < 2 * 2 * 512
    # transposed quantiser == quantiser of the transpose
    t_data, t_scales = O.mxfp8_quantize_transposed(src)
    d2, s2 = O.mxfp8_quantize(np.ascontiguousarray(src.T))
    assert np.array_equal(t_data, d2) and np.array_equal(t_scales, s2)


def test_gemm_orientations_agree_with_numpy():
    rng = np.random.default_rng(5)
    m, n, k = 70, 56, 96
    a = O.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    b = O.f32_to_bf16(rng.standard_normal((n, k)).astype(np.float32) * 0.1)
    want = O.bf16_to_f32(a).astype(np.float64) @ O.bf16_to_f32(b).astype(np.float64).T
    nt = O.gemm_bf16(0, a, b, m, n, k)
    nn = O.gemm_bf16(1, a, np.ascontiguousarray(b.T), m, n, k)
    tn = O.gemm_bf16(2, np.ascontiguousarray(a.T), np.ascontiguousarray(b.T), m, n, k)
    for got in (nt, nn, tn):
        assert np.array_equal(got, nt)
        assert np.abs(O.bf16_to_f32(got) - want).max() <= 0.01 + 0.01 * np.abs(want).max()
    acc = O.gemm_bf16(0, a, b, m, n, k, alpha=0.5, beta=1.0, d=nt.copy())
    assert np.allclose(O.bf16_to_f32(acc), 1.5 * want, rtol=0.02, atol=0.02)


def test_multi_rank_simulators_roundtrip():
    # config "tiny BF16 QKV, 2 simulated ranks" in miniature: route, then invert with the
    # reference's receiver-side map, and gather for the output projection.
    rng = np.random.default_rng(7)
    world, batch, s, q, kv, d, k = 2, 1, 16, 4, 2, 8, 32
    n = (q + 2 * kv) * d
    lhs = [O.f32_to_bf16(rng.standard_normal((batch * s, k)).astype(np.float32)) for _ in range(world)]
    w = O.f32_to_bf16(rng.standard_normal((n, k)).astype(np.float32) * 0.05)
    local, peers = O.qkv_forward(world, batch, s, q, kv, d, lhs, w)
    for dest in range(world):
        assert not (peers[dest] == 0xFFFF).all()
        for index in range(peers[dest].size):
            r, o = C.c_int32(), C.c_uint64()
            L.fo_qkv_oracle_source(world, dest, s, q * d, kv * d, index, C.byref(r), C.byref(o))
            assert peers[dest][index] == local[r.value].reshape(-1)[o.value]
    heads_in = [O.f32_to_bf16(rng.standard_normal((batch * s * world, q * d // world)).astype(np.float32))
                for _ in range(world)]
    wo = O.f32_to_bf16(rng.standard_normal((24, q * d)).astype(np.float32) * 0.05)
    staging, out = O.oproj_forward(world, 1, batch, s, heads_in, wo)
    assert np.array_equal(staging[:, :q * d // world], heads_in[0][s:2 * s])
    assert out.shape == (batch * s, 24)


def test_moe_route_builder():
    rng = np.random.default_rng(11)
    world, tokens, experts, topk = 2, 12, 8, 3
    scores = [rng.standard_normal((tokens, experts)).astype(np.float32) for _ in range(world)]
    scores[0][0, :] = 1.0  # all ties: lowest expert ids win
    chosen = []
    for sc in scores:
        c = np.empty((tokens, topk), dtype=np.int32)
        L.fo_moe_topk(O.ptr(sc), tokens, experts, topk, O.ptr(c))
        chosen.append(c)
    assert list(chosen[0][0]) == [0, 1, 2]
    for c, sc in zip(chosen, scores):
        for t in range(tokens):
            assert len(set(c[t])) == topk
            assert set(c[t]) == set(np.argsort(-sc[t], kind="stable")[:topk])
    total = 0
    for dest in range(world):
        offs = np.empty(experts // world + 1, dtype=np.int32)
        n = L.fo_moe_build_rows(world, dest, experts // world, tokens, topk, O.ptr_array(chosen), O.ptr(offs), None)
        src = np.empty((n, 3), dtype=np.int32)
        L.fo_moe_build_rows(world, dest, experts // world, tokens, topk, O.ptr_array(chosen), O.ptr(offs), O.ptr(src))
        total += n
        for e in range(experts // world):
            seg = src[offs[e]:offs[e + 1]]
            assert all(chosen[r][t, sl] == dest * (experts // world) + e for r, t, sl in seg)
            assert [tuple(x) for x in seg] == sorted(tuple(x) for x in seg)
    assert total == world * tokens * topk


@pytest.mark.skipif(O.ref() is None, reason="reference tree not mounted")
def test_oracle_against_reference_headers_directly():
    R = O.ref()
    rng = np.random.default_rng(13)
    for _ in range(300):
        w = int(rng.choice([1, 2, 4, 8]))
        q = w * int(rng.integers(1, 5)) * 2
        kv = w * int(rng.integers(1, 3))
        d = int(rng.choice([8, 64, 80, 128]))
        f = int(rng.integers(0, (q + 2 * kv) * d))
        a, b = (C.c_int32 * 5)(), (C.c_int32 * 5)()
        assert L.fo_map_qkv_gqa_feature(w, q, kv, d, f, a) == R.ref_map_qkv_gqa_feature(w, q, kv, d, f, b)
        assert list(a) == list(b)
        s = int(rng.integers(1, 40)) * 2
        width = w * 8 * int(rng.integers(1, 9))
        dest = int(rng.integers(0, w))
        index = int(rng.integers(0, s * width))
        causal = int(rng.integers(0, 2))
        r1, o1, r2, o2 = C.c_int32(), C.c_uint64(), C.c_int32(), C.c_uint64()
        L.fo_oproj_gather_source(w, dest, s, width, causal, 0, index, C.byref(r1), C.byref(o1))
        R.ref_oproj_gather_source(w, dest, s, width, causal, index, C.byref(r2), C.byref(o2))
        assert (r1.value, o1.value) == (r2.value, o2.value)
        qidx = int(rng.integers(0, s * w * (q + 2 * kv) * d // w))
        L.fo_qkv_oracle_source(w, dest, s, q * d, kv * d, qidx, C.byref(r1), C.byref(o1))
        R.ref_qkv_oracle_source(w, dest, s, q * d, kv * d, qidx, C.byref(r2), C.byref(o2))
        assert (r1.value, o1.value) == (r2.value, o2.value)
    xs = (rng.standard_normal(5000) * np.exp(rng.uniform(-12, 7, 5000))).astype(np.float32)
    for x in xs:
        assert L.fo_f32_to_e4m3(float(x)) == R.ref_f32_to_e4m3(float(x))
        assert L.fo_f32_to_bf16(float(x)) == R.ref_f32_to_bf16(float(x))


def test_qkv_route_with_v_deferred_keeps_q_and_k_per_row_and_v_local():
    # UlyssesRoute::defer_v_a2a (csrc/operators/sm103/detail/gemm_a2a.cuh:199-215,408,505-533): one
    # [B*S_global, q_local + kv_local] tensor per destination, Q columns then K columns; V is not routed
    from fuse_b200 import synthetic
    world, s, q, kv, d, k = 4, 8, 8, 4, 8, 16
    lhs = [synthetic.normal_bf16((s, k), 40 + r, 1.0) for r in range(world)]
    w = synthetic.normal_bf16(((q + 2 * kv) * d, k), 9, 0.02)
    local, peers = O.qkv_forward(world, 1, s, q, kv, d, lhs, w, defer_v=True)
    plain_local, plain_peers = O.qkv_forward(world, 1, s, q, kv, d, lhs, w)
    ql, kvl = q // world * d, kv // world * d
    rows = s * world
    for dest in range(world):
        got = peers[dest][:rows * (ql + kvl)].reshape(rows, ql + kvl)
        assert (peers[dest][rows * (ql + kvl):] == 0xFFFF).all()          # the V share is never written
        planar_q = plain_peers[dest][:rows * ql].reshape(rows, ql)
        planar_k = plain_peers[dest][rows * ql:rows * (ql + kvl)].reshape(rows, kvl)
        assert np.array_equal(got[:, :ql], planar_q) and np.array_equal(got[:, ql:], planar_k)
    for r in range(world):
        assert np.array_equal(local[r], plain_local[r])                    # V stays where the GEMM wrote it


def _prepack_interleaved(w, world, q, kv, d):
    """The offline prepack UlyssesRoute::qkv_peer_interleaved expects: inside Q and inside K, physical
    head p = local_head * world + owner holds logical head owner * local_heads + local_head."""
    out = w.copy()
    for base, heads in ((0, q), (q * d, kv)):
        local_heads = heads // world
        for p in range(heads):
            owner, local_head = p % world, p // world
            logical = owner * local_heads + local_head
            out[base + p * d:base + (p + 1) * d] = w[base + logical * d:base + (logical + 1) * d]
    return out


def test_qkv_route_with_interleaved_weights_leaves_the_routed_layout_unchanged():
    # include/fuse/layout/ulysses.h:35-39: "The final routed Q/K/V layout is unchanged."
    from fuse_b200 import synthetic
    world, s, q, kv, d, k = 4, 8, 8, 4, 8, 16
    lhs = [synthetic.normal_bf16((s, k), 60 + r, 1.0) for r in range(world)]
    w = synthetic.normal_bf16(((q + 2 * kv) * d, k), 11, 0.02)
    _, plain = O.qkv_forward(world, 1, s, q, kv, d, lhs, w)
    _, packed = O.qkv_forward(world, 1, s, q, kv, d, lhs, _prepack_interleaved(w, world, q, kv, d), interleaved=True)
    for dest in range(world):
        assert np.array_equal(plain[dest], packed[dest])
    _, plain_d = O.qkv_forward(world, 1, s, q, kv, d, lhs, w, defer_v=True)
    _, packed_d = O.qkv_forward(world, 1, s, q, kv, d, lhs, _prepack_interleaved(w, world, q, kv, d), defer_v=True,
                                interleaved=True)
    for dest in range(world):
        assert np.array_equal(plain_d[dest], packed_d[dest])
