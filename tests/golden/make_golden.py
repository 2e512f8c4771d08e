"""Regenerates tests/golden/reference_vectors.npz from the REFERENCE'S OWN code.

Runs only where the reference tree is mounted: it loads oracle/_ref/libfuse_ref.so (the
reference's include/fuse/layout/ulysses.h, benchmarks/sm103/fused_validation.cuh and
fused_inputs.cuh plus CUTLASS host numerics, compiled in place by `make -C oracle ref`) and
records its answers on fixed inputs.  The committed .npz lets the CPU oracle be pinned on
machines where the reference is absent.

    python tests/golden/make_golden.py
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

# (world, q_heads, kv_heads, head_dim): the invertibility cases of
# benchmarks/sm90/QKVproj+a2a/fuse_smoke.cu:228-270 plus the benchmark geometries.
GQA_CASES = [(2, 8, 8, 64), (2, 8, 4, 96), (4, 16, 4, 80), (4, 32, 4, 128), (8, 32, 8, 128),
             (8, 64, 8, 128), (3, 8, 8, 64), (4, 6, 4, 64)]
# (world, seq_local, q_heads, kv_heads, head_dim)
QKV_ORACLE_CASES = [(2, 6, 4, 2, 8), (4, 5, 8, 4, 16), (8, 3, 16, 8, 8)]
# (world, seq_local, width, causal)
OPROJ_CASES = [(2, 6, 16, 0), (2, 6, 16, 1), (4, 8, 32, 0), (4, 8, 32, 1), (8, 4, 64, 1)]


def main():
    R = O.ref()
    if R is None:
        raise SystemExit("reference tree not available: cannot regenerate golden vectors")
    out = {}
    rows = []
    for (w, q, kv, d) in GQA_CASES:
        n = (q + 2 * kv) * d
        for f in list(range(-1, n + 1)):
            a = (C.c_int32 * 5)()
            valid = R.ref_map_qkv_gqa_feature(w, q, kv, d, f, a)
            inv = R.ref_qkv_gqa_global_feature(w, q, kv, d, a[0], a[1]) if valid else -1
            rows.append([w, q, kv, d, f, valid, a[0], a[1], a[2], a[3], a[4], inv])
    out["gqa_map"] = np.array(rows, dtype=np.int64)

    rows = []
    for (w, s, q, kv, d) in QKV_ORACLE_CASES:
        qw, kvw = q * d, kv * d
        per_dest = s * w * (qw + 2 * kvw) // w
        for dest in range(w):
            for index in range(per_dest):
                rank, off = C.c_int32(), C.c_uint64()
                R.ref_qkv_oracle_source(w, dest, s, qw, kvw, index, C.byref(rank), C.byref(off))
                rows.append([w, s, q, kv, d, dest, index, rank.value, off.value])
    out["qkv_oracle"] = np.array(rows, dtype=np.int64)

    rows = []
    for (w, s, width, causal) in OPROJ_CASES:
        for dest in range(w):
            for index in range(s * width):
                rank, off = C.c_int32(), C.c_uint64()
                R.ref_oproj_gather_source(w, dest, s, width, causal, index, C.byref(rank), C.byref(off))
                rows.append([w, s, width, causal, dest, index, rank.value, off.value])
    out["oproj_gather"] = np.array(rows, dtype=np.int64)

    # E4M3: decode of all 256 codes; encode of a fixed float sample (CUTLASS host numerics).
    out["e4m3_decode"] = np.array([R.ref_e4m3_to_f32(v) for v in range(256)], dtype=np.float32)
    rng = np.random.default_rng(20260906)
    sample = np.concatenate([
        rng.standard_normal(4096).astype(np.float32) * s for s in (2.0 ** -12, 0.02, 1.0, 60.0, 500.0)
    ] + [np.array([0.0, -0.0, 448.0, 449.0, 464.0, 465.0, 1e9, np.inf, -np.inf, 2.0 ** -9,
                   2.0 ** -10, 1.5 * 2.0 ** -10, 2.0 ** -6, 0.0146, 0.0155, 17.0, 18.0, 19.0, 20.0,
                   21.0, 22.0, 23.0, 25.0, 27.0, 29.0, 31.0], dtype=np.float32)])
    out["e4m3_encode_in"] = sample
    out["e4m3_encode_out"] = np.array([R.ref_f32_to_e4m3(float(x)) for x in sample], dtype=np.uint8)
    out["bf16_encode_out"] = np.array([R.ref_f32_to_bf16(float(x)) for x in sample], dtype=np.uint16)
    words = rng.integers(0, 2 ** 32, size=2048, dtype=np.uint64).astype(np.uint32)
    out["uniform_words"] = words
    out["uniform_out"] = np.array([R.ref_uniform_value(int(w), 0.125) for w in words], dtype=np.float32)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print(path, {k: v.shape for k, v in out.items()}, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
