"""Seeded synthetic inputs (numpy, host side) for the tests and the benchmark.

Counter-based Philox4x32-10, so that a tensor's values depend only on (seed, element index) and
are identical on every machine and for every rank that asks for the same seed.  The element
mapping follows the reference harness's generator (benchmarks/sm103/fused_inputs.cuh:122-141:
65536 generator threads, thread t is Philox subsequence t, its r-th draw of four words fills
elements 4*(r*65536+t) .. +3), and `uniform_bf16` applies its word -> value map
(fused_inputs.cuh:22-29).  `normal_bf16` (Box-Muller on the same words) provides the N(0, sigma)
payloads the benchmark configurations name.

Seeds follow benchmarks/sm103/fused_bf16.cu:100,1482-1505: base seed 20260906, per rank and
generation `seed + generation*100003 + rank*101`, activations +1000 (QKV) / +2000 (OProj),
weights seed+11 / seed+17."""
from __future__ import annotations

import numpy as np

BASE_SEED = 20260906
GROUPED_SEED = 20260916
_THREADS = 65536

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = np.uint32(0x9E3779B9)
_W1 = np.uint32(0xBB67AE85)


def philox4x32_10(counter: np.ndarray, key: np.ndarray) -> np.ndarray:
    """counter [n, 4] uint32, key [2] or [n, 2] uint32 -> [n, 4] uint32 (ten rounds)."""
    c = [counter[:, i].astype(np.uint32) for i in range(4)]
    key = np.broadcast_to(np.asarray(key, dtype=np.uint32), (counter.shape[0], 2))
    k0, k1 = key[:, 0].copy(), key[:, 1].copy()
    with np.errstate(over="ignore"):
        for _ in range(10):
            p0 = _M0 * c[0].astype(np.uint64)
            p1 = _M1 * c[2].astype(np.uint64)
            hi0, lo0 = (p0 >> np.uint64(32)).astype(np.uint32), p0.astype(np.uint32)
            hi1, lo1 = (p1 >> np.uint64(32)).astype(np.uint32), p1.astype(np.uint32)
            c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
            k0 = k0 + _W0
            k1 = k1 + _W1
    return np.stack(c, axis=1)


def random_words(count: int, seed: int) -> np.ndarray:
    """`count` uint32 words in the reference generator's element order."""
    rounds = -(-count // (4 * _THREADS))
    out = np.empty(rounds * _THREADS * 4, dtype=np.uint32)
    key = np.array([seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF], dtype=np.uint32)
    chunk = 32  # rounds per vectorised Philox call
    for r0 in range(0, rounds, chunk):
        r1 = min(rounds, r0 + chunk)
        n = (r1 - r0) * _THREADS
        counter = np.zeros((n, 4), dtype=np.uint32)
        counter[:, 0] = np.repeat(np.arange(r0, r1, dtype=np.uint32), _THREADS)
        counter[:, 2] = np.tile(np.arange(_THREADS, dtype=np.uint32), r1 - r0)
        out[r0 * _THREADS * 4:r1 * _THREADS * 4] = philox4x32_10(counter, key).reshape(-1)
    return out[:count]


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((bits + np.uint64(0x7FFF) + ((bits >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)).astype(np.uint16)


def bf16_bits_to_f32(x: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(x, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def uniform_bf16(shape, seed: int, magnitude: float) -> np.ndarray:
    """BF16 bit patterns, uniform in [-magnitude, magnitude) (fused_inputs.cuh:22-29)."""
    count = int(np.prod(shape))
    words = random_words(count, seed)
    unit = (words >> np.uint32(8)).astype(np.float32) / np.float32(16777216.0)
    value = (unit - np.float32(0.5)) * np.float32(2 * magnitude)
    return f32_to_bf16_bits(value).reshape(shape)


def normal_f32(shape, seed: int, sigma: float = 1.0) -> np.ndarray:
    count = int(np.prod(shape))
    words = random_words(2 * ((count + 1) // 2), seed).astype(np.float64)
    u1 = (words[0::2] + 1.0) / 4294967296.0   # (0, 1]
    u2 = words[1::2] / 4294967296.0           # [0, 1)
    radius = np.sqrt(-2.0 * np.log(u1))
    z = np.empty(2 * u1.size, dtype=np.float64)
    z[0::2] = radius * np.cos(2.0 * np.pi * u2)
    z[1::2] = radius * np.sin(2.0 * np.pi * u2)
    return (z[:count] * sigma).astype(np.float32).reshape(shape)


def normal_bf16(shape, seed: int, sigma: float = 1.0) -> np.ndarray:
    """BF16 bit patterns of N(0, sigma^2) samples."""
    return f32_to_bf16_bits(normal_f32(shape, seed, sigma)).reshape(shape)


def rank_seed(rank: int, generation: int = 0, base: int = BASE_SEED) -> int:
    return base + generation * 100003 + rank * 101
