"""ctypes/numpy front end of the CPU oracle (test infrastructure only).

Only tests/, the smoke entry and the CPU-baseline leg of bench.py import this
module.  The product package never does: it drives the CUDA library and fails
when that library is missing.

`lib()` loads oracle/_build/libfuse_oracle.so (built by `make -C oracle`, built on
demand when absent).  `ref()` loads oracle/_ref/libfuse_ref.so, the reference's own
host headers compiled in place; it exists only where the reference tree is
mounted and returns None elsewhere.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

i32, i64, u8, u16, u32, u64, f32 = (C.c_int32, C.c_int64, C.c_uint8, C.c_uint16, C.c_uint32,
                                    C.c_uint64, C.c_float)
P = C.c_void_p


def _make(target: str) -> None:
    cmd = ["make", "-C", _HERE, target]
    if target == "ref":
        cmd.append("REF_ROOT=" + reference_root())
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)


def _sig(lib, name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    path = os.path.join(_HERE, "_build", "libfuse_oracle.so")
    src = os.path.join(_HERE, "fuse_oracle.c")
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
        _make("all")
    L = C.CDLL(path)
    _sig(L, "fo_bf16_to_f32", f32, u16)
    _sig(L, "fo_f32_to_bf16", u16, f32)
    _sig(L, "fo_f32_to_e4m3", u8, f32)
    _sig(L, "fo_e4m3_to_f32", f32, u8)
    _sig(L, "fo_uniform_value", f32, u32, f32)
    _sig(L, "fo_backward_random_value", u16, i64, C.c_int)
    _sig(L, "fo_map_qkv_gqa_feature", C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, P)
    _sig(L, "fo_qkv_gqa_global_feature", C.c_int, *([C.c_int] * 6))
    _sig(L, "fo_global_row", i64, C.c_int, C.c_int, C.c_int, C.c_int, i64)
    _sig(L, "fo_qkv_forward_destination", C.c_int, *([C.c_int] * 7), i64, C.c_int, P, P)
    _sig(L, "fo_qkv_oracle_source", None, C.c_int, C.c_int, u64, u64, u64, u64, P, P)
    _sig(L, "fo_oproj_gather_source", None, C.c_int, C.c_int, C.c_int, i64, C.c_int, C.c_int, u64,
         P, P)
    _sig(L, "fo_qkv_backward_source", None, *([C.c_int] * 7), i64, C.c_int, P, P, P)
    _sig(L, "fo_oproj_backward_source", None, C.c_int, C.c_int, C.c_int, C.c_int, i64, C.c_int,
         u64, P, P)
    _sig(L, "fo_swizzle_size", C.c_int, C.c_int, C.c_int, C.c_int)
    _sig(L, "fo_mxfp8_scale_exponent", C.c_int, f32)
    _sig(L, "fo_mxfp8_scale_exponent_frexp", C.c_int, f32)
    _sig(L, "fo_mxfp8_scaled_value", f32, f32, C.c_int)
    _sig(L, "fo_mxfp8_scale_offset", i64, i64, i64, i64)
    _sig(L, "fo_mxfp8_scale_bytes", i64, i64, i64)
    _sig(L, "fo_mxfp8_quantize", None, P, i64, i64, i64, P, P)
    _sig(L, "fo_mxfp8_quantize_transposed", None, P, i64, i64, i64, P, P)
    _sig(L, "fo_mxfp8_dequantize", None, P, P, i64, i64, P)
    _sig(L, "fo_mxfp8_represented", None, P, i64, P)
    _sig(L, "fo_gemm_f32_nt", None, P, P, P, i64, i64, i64, i64, f32, f32)
    _sig(L, "fo_gemm_bf16", C.c_int, C.c_int, P, i64, P, i64, P, i64, i64, i64, i64, f32, f32)
    _sig(L, "fo_gemm_mxfp8_nt", C.c_int, P, P, P, P, P, i64, i64, i64, i64, f32)
    _sig(L, "fo_qkv_forward_route", None, *([C.c_int] * 7), P, i64, P)
    _sig(L, "fo_qkv_forward_route_defer_v", None, *([C.c_int] * 7), P, i64, P)
    _sig(L, "fo_qkv_forward_route_variant", None, *([C.c_int] * 9), P, i64, P)
    _sig(L, "fo_qkv_forward_destination_defer_v", C.c_int, *([C.c_int] * 7), i64, C.c_int, P, P)
    _sig(L, "fo_oproj_forward_gather", None, C.c_int, C.c_int, C.c_int, C.c_int, i64, C.c_int,
         C.c_int, P, P)
    _sig(L, "fo_qkv_backward_gather", None, *([C.c_int] * 8), P, P)
    _sig(L, "fo_moe_topk", None, P, i64, C.c_int, C.c_int, P)
    _sig(L, "fo_moe_build_rows", i64, C.c_int, C.c_int, C.c_int, i64, C.c_int, P, P, P)
    _sig(L, "fo_moe_dispatch_fc1", C.c_int, C.c_int, P, P, P, P, i64, i64, i64, P, P)
    _sig(L, "fo_moe_fc2_combine", C.c_int, C.c_int, P, P, P, P, i64, i64, i64, C.c_int, P, P)
    _sig(L, "fo_num_threads", C.c_int)
    _sig(L, "fo_set_num_threads", None, C.c_int)
    _sig(L, "fo_qkv_oracle_source_batch", None, C.c_int, C.c_int, u64, u64, u64, P, i64, P, P)
    _sig(L, "fo_oproj_gather_source_batch", None, C.c_int, C.c_int, C.c_int, i64, C.c_int, C.c_int, P, i64, P, P)
    _sig(L, "fo_qkv_backward_source_batch", None, *([C.c_int] * 7), P, P, i64, P, P, P)
    _sig(L, "fo_oproj_backward_source_batch", None, C.c_int, C.c_int, C.c_int, C.c_int, i64, C.c_int, P, i64, P, P)
    _sig(L, "fo_global_row_batch", None, C.c_int, C.c_int, C.c_int, C.c_int, P, i64, P)
    _sig(L, "fo_mxfp8_scale_offset_batch", None, P, P, i64, i64, P)
    _LIB = L
    return L


def reference_root() -> str:
    """Where the reference project is mounted: $FUSE_REF_ROOT, else a directory named
    `reference` beside this repository (absent on the GPU box: callers then skip)."""
    return os.environ.get("FUSE_REF_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def ref(build: bool = True):
    """The reference's own host headers behind a C interface, or None."""
    global _REF
    if _REF is not None:
        return _REF
    path = os.path.join(_HERE, "_ref", "libfuse_ref.so")
    if not os.path.exists(path):
        if not build or not os.path.isdir(reference_root()):
            return None
        try:
            _make("ref")
        except subprocess.CalledProcessError:
            return None
    R = C.CDLL(path)
    _sig(R, "ref_map_qkv_gqa_feature", C.c_int, *([C.c_int] * 5), P)
    _sig(R, "ref_qkv_gqa_global_feature", C.c_int, *([C.c_int] * 6))
    _sig(R, "ref_qkv_oracle_source", None, C.c_int, C.c_int, u64, u64, u64, u64, P, P)
    _sig(R, "ref_oproj_gather_source", None, C.c_int, C.c_int, u64, u64, C.c_int, u64, P, P)
    _sig(R, "ref_uniform_value", f32, u32, f32)
    _sig(R, "ref_bf16_to_f32", f32, u16)
    _sig(R, "ref_f32_to_bf16", u16, f32)
    _sig(R, "ref_f32_to_e4m3", u8, f32)
    _sig(R, "ref_e4m3_to_f32", f32, u8)
    _REF = R
    return R


# ---------------------------------------------------------------------------------------------
# numpy helpers
# ---------------------------------------------------------------------------------------------

def ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(P)


def ptr_array(arrays):
    """A C array of pointers to the given numpy arrays (keeps them alive via the return)."""
    table = (P * len(arrays))(*[a.ctypes.data for a in arrays])
    return table


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even FP32 -> BF16 bit patterns (uint16)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, ((bits >> 16) | 0x40).astype(np.uint16), rounded)


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(x, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def gemm_bf16(mode: int, a: np.ndarray, b: np.ndarray, m: int, n: int, k: int, alpha=1.0,
              beta=0.0, d: np.ndarray | None = None) -> np.ndarray:
    """D = alpha * op(A) op(B) (+ beta * D) with BF16 bit-pattern operands; see fo_gemm_bf16."""
    out = np.zeros((m, n), dtype=np.uint16) if d is None else d
    rc = lib().fo_gemm_bf16(mode, ptr(a), a.shape[1], ptr(b), b.shape[1], ptr(out), out.shape[1],
                            m, n, k, alpha, beta)
    assert rc == 0
    return out


def qkv_forward(world, batch, seq_local, q_heads, kv_heads, head_dim, lhs, rhs_nt, alpha=1.0, defer_v=False,
                interleaved=False):
    """Simulate every rank of the fused QKV projection + sequence->head all-to-all.

    lhs: list of [M, K] uint16 (BF16 bits) per rank; rhs_nt: [N, K].  Returns
    (local_outputs, peer_outputs): per rank [M, N] and the planar Q|K|V buffer (flat uint16).
    defer_v: V stays local; the destination buffer is [B*S_global, q_local + kv_local] (Q | K per
    row), still sized like the planar buffer, elements nobody routes keep 0xFFFF.
    interleaved: rhs_nt is the offline-prepacked weight (inside Q and K physical head p = local_head *
    world + owner); the routed layout is the standard one."""
    L = lib()
    m = batch * seq_local
    n = (q_heads + 2 * kv_heads) * head_dim
    k = rhs_nt.shape[1]
    rows = batch * seq_local * world
    local = [gemm_bf16(0, lhs[r], rhs_nt, m, n, k, alpha) for r in range(world)]
    peers = [np.full(rows * n // world, 0xFFFF, dtype=np.uint16) for _ in range(world)]
    table = ptr_array(peers)
    for r in range(world):
        if interleaved:
            L.fo_qkv_forward_route_variant(world, r, batch, seq_local, q_heads, kv_heads, head_dim, int(defer_v), 1,
                                           ptr(local[r]), n, table)
        elif defer_v:
            L.fo_qkv_forward_route_defer_v(world, r, batch, seq_local, q_heads, kv_heads, head_dim, ptr(local[r]), n, table)
        else:
            L.fo_qkv_forward_route(world, r, batch, seq_local, q_heads, kv_heads, head_dim, ptr(local[r]), n, table)
    return local, peers


def oproj_forward(world, rank, batch, seq_local, peer_input, rhs_nt, causal=False, cyclic=False,
                  alpha=1.0):
    """One rank of head->sequence all-to-all + output projection.  Returns (staging, output)."""
    L = lib()
    m = batch * seq_local
    n, k = rhs_nt.shape
    staging = np.empty((m, k), dtype=np.uint16)
    L.fo_oproj_forward_gather(world, rank, batch, seq_local, k, int(causal), int(cyclic),
                              ptr_array(peer_input), ptr(staging))
    return staging, gemm_bf16(0, staging, rhs_nt, m, n, k, alpha)


def mxfp8_quantize(source: np.ndarray):
    """[rows, k] BF16 bits -> (E4M3 bytes [rows, k], native scale bytes)."""
    rows, k = source.shape
    data = np.empty((rows, k), dtype=np.uint8)
    scales = np.zeros(lib().fo_mxfp8_scale_bytes(rows, k), dtype=np.uint8)
    lib().fo_mxfp8_quantize(ptr(source), rows, k, k, ptr(data), ptr(scales))
    return data, scales


def mxfp8_quantize_transposed(source: np.ndarray):
    """[rows, cols] BF16 bits -> (E4M3 [cols, rows] quantised along rows, native scales)."""
    rows, cols = source.shape
    data = np.empty((cols, rows), dtype=np.uint8)
    scales = np.zeros(lib().fo_mxfp8_scale_bytes(cols, rows), dtype=np.uint8)
    lib().fo_mxfp8_quantize_transposed(ptr(source), rows, cols, cols, ptr(data), ptr(scales))
    return data, scales


def mxfp8_dequantize(data: np.ndarray, scales: np.ndarray) -> np.ndarray:
    rows, k = data.shape
    out = np.empty((rows, k), dtype=np.float32)
    lib().fo_mxfp8_dequantize(ptr(data), ptr(scales), rows, k, ptr(out))
    return out


def gemm_mxfp8(a, a_scales, b, b_scales, alpha=1.0) -> np.ndarray:
    m, k = a.shape
    n = b.shape[0]
    out = np.zeros((m, n), dtype=np.uint16)
    rc = lib().fo_gemm_mxfp8_nt(ptr(a), ptr(a_scales), ptr(b), ptr(b_scales), ptr(out), n, m, n, k,
                                alpha)
    assert rc == 0
    return out


def within_tolerance(actual_bits, expected_bits, absolute=0.01, relative=0.01):
    """The reference's element test |a-b| <= abs + rel*|b|
    (benchmarks/sm103/fused_validation.cuh:71-77).  Returns (ok, worst_excess, count_bad)."""
    a = bf16_to_f32(np.asarray(actual_bits)).astype(np.float64)
    b = bf16_to_f32(np.asarray(expected_bits)).astype(np.float64)
    err = np.abs(a - b)
    bad = ~(err <= absolute + relative * np.abs(b))
    return (not bad.any()), float(err.max() if err.size else 0.0), int(bad.sum())


def qkv_backward(world, rank, batch, seq_local, q_heads, kv_heads, head_dim, planes, weight, saved_input,
                 causal=False, alpha=1.0, beta=0.0, grad_weight=None):
    """One rank of the QKV projection backward.  planes[r] = (dQ, dK, dV) of rank r, each
    [B*S_global, local_heads*head_dim]; weight [QKV, H]; saved_input [M, H].
    Returns (staging [M, QKV], dX [M, H], dW [QKV, H])."""
    m = batch * seq_local
    width = (q_heads + 2 * kv_heads) * head_dim
    hidden = weight.shape[1]
    flat = [np.ascontiguousarray(pl) for r in range(world) for pl in planes[r]]
    staging = np.empty((m, width), dtype=np.uint16)
    lib().fo_qkv_backward_gather(world, rank, batch, seq_local, q_heads, kv_heads, head_dim, int(causal),
                                 ptr_array(flat), ptr(staging))
    dx = gemm_bf16(1, staging, weight, m, hidden, width, alpha)
    dw = gemm_bf16(2, staging, saved_input, width, hidden, m, alpha, beta,
                   None if grad_weight is None else grad_weight.copy())
    return staging, dx, dw


def oproj_backward(world, batch, seq_local, q_heads, head_dim, grad_outputs, weight, saved_attention,
                   causal=False, alpha=1.0):
    """Every rank of the output projection backward.  grad_outputs[r] = dY of rank r [M, H];
    weight Wo [H, A]; saved_attention[r] = forward lhs of rank r [M, A].
    Returns (dA per rank [M, A], routed per rank [B*S_global, A/world] flat, dWo per rank [H, A])."""
    m = batch * seq_local
    hidden, a = weight.shape
    da = [gemm_bf16(1, grad_outputs[r], weight, m, a, hidden, alpha) for r in range(world)]
    shard = a // world
    rows = batch * seq_local * world
    routed = []
    rank_out, offset_out = C.c_int32(), C.c_uint64()
    for dest in range(world):
        idx = np.arange(rows * shard, dtype=np.uint64)
        # vectorised restatement of fo_oproj_backward_source (checked against it below)
        row, col = idx // shard, idx % shard
        b, seq = row // (seq_local * world), row % (seq_local * world)
        if causal:
            half = seq_local // 2
            chunk = seq // half
            src = np.where(chunk < world, chunk, 2 * world - chunk - 1)
            local_row = np.where(chunk < world, 0, half) + seq % half
        else:
            src, local_row = seq // seq_local, seq % seq_local
        off = (b * seq_local + local_row) * a + dest * shard + col
        for probe in (0, int(idx[-1]) // 2, int(idx[-1])):
            lib().fo_oproj_backward_source(world, dest, batch, seq_local, a, int(causal), probe,
                                           C.byref(rank_out), C.byref(offset_out))
            assert (rank_out.value, offset_out.value) == (int(src[probe]), int(off[probe]))
        stacked = np.stack([x.reshape(-1) for x in da])
        routed.append(stacked[src.astype(np.int64), off.astype(np.int64)])
    dwo = [gemm_bf16(2, grad_outputs[r], saved_attention[r], hidden, a, m, alpha) for r in range(world)]
    return da, routed, dwo
