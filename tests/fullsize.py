"""Checker for benchmark-size runs: samples rows of the operators' outputs on the device and
compares them with the CPU oracle (test infrastructure: this module is imported by bench.py and
bench_suite.py after their timed regions, never by the product package).

Protocol, after the reference's own benchmark validation (benchmarks/sm103/fused_bf16.cu:2507-2585,
fused_validation.cuh:71-77,104-138): outputs are poisoned, one more launch runs, then
  * GEMM outputs of a stated row sample are recomputed by the oracle (FP32 accumulate, BF16 out)
    and must lie within the reference's tolerance;
  * routed / gathered elements of those rows are traced back through the oracle's receiver-view
    address maps to the element the source rank produced and must be BIT-EXACT -- including what
    peers wrote into this rank (the sampled source rows travel between ranks over
    torch.distributed, which is only the checker's transport).
Everything here works on CPU tensors as well, so the multi-rank logic is tested with gloo."""
from __future__ import annotations

import os

import numpy as np
import torch
import torch.distributed as dist

from oracle import oracle as O

POISON16 = -1  # int16 view of the BF16 NaN pattern 0xFFFF


def world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def use_host_threads(ranks_on_host: int) -> int:
    """Gives the oracle this rank's share of the host cores (torchrun sets OMP_NUM_THREADS=1)."""
    threads = max(1, (os.cpu_count() or 1) // max(1, ranks_on_host))
    O.lib().fo_set_num_threads(threads)
    return threads


def sample_rows(m: int, count: int = 256, edge: int = 32, seed: int = 1234) -> np.ndarray:
    """Sorted local rows: the first and last `edge` rows (first / last tile) plus a seeded spread."""
    count = min(count, m)
    edge = min(edge, count // 2)
    picked = set(range(edge)) | set(range(m - edge, m))
    rng = np.random.default_rng(seed)
    while len(picked) < count:
        picked.update(int(v) for v in rng.integers(0, m, count - len(picked)))
    return np.array(sorted(picked), dtype=np.int64)


def bits(t: torch.Tensor) -> np.ndarray:
    """BF16 tensor -> numpy uint16 bit patterns (host)."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def index_tensor(a: np.ndarray, like: torch.Tensor) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int64)).to(like.device)


def poison(*tensors: torch.Tensor) -> None:
    """BF16 tensors get the NaN pattern 0xFFFF, byte tensors 0xA5."""
    for t in tensors:
        if t.element_size() == 2:
            t.view(torch.int16).fill_(POISON16)
        else:
            t.fill_(0xA5)


def unwritten(t: torch.Tensor) -> int:
    """Elements of a BF16 tensor that still hold the poison pattern (full size, on the device)."""
    return int((t.view(torch.int16) == POISON16).sum())


def compare(actual: np.ndarray, expected: np.ndarray, absolute: float, relative: float) -> dict:
    ok, worst, bad = O.within_tolerance(actual, expected, absolute, relative)
    return {"ok": bool(ok), "max_abs_err": float(worst), "bad": int(bad), "elements": int(actual.size),
            "tolerance": f"{absolute}+{relative}*|b|"}


def all_gather_rows(t: torch.Tensor) -> torch.Tensor:
    """[R, C] on every rank -> [world, R, C]."""
    if world_size() == 1:
        return t.unsqueeze(0).contiguous()
    out = torch.empty((world_size(),) + tuple(t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out.view(-1).view(torch.uint8), t.contiguous().view(-1).view(torch.uint8))  # as bytes
    return out


def exchange_rows(send: torch.Tensor) -> torch.Tensor:
    """send[d] goes to rank d; returns recv with recv[s] = what rank s sent here."""
    if world_size() == 1:
        return send.clone()
    send = send.contiguous()
    recv = torch.empty_like(send)
    try:
        dist.all_to_all_single(recv.view(-1).view(torch.uint8), send.view(-1).view(torch.uint8))  # as bytes
    except RuntimeError:  # a backend without all-to-all: everyone gathers everything
        everything = all_gather_rows(send)
        recv = everything[:, dist.get_rank()].contiguous()
    return recv


def global_rows(world: int, rank: int, seq_local: int, causal: bool, rows: np.ndarray) -> np.ndarray:
    out = np.empty(len(rows), dtype=np.int64)
    local = np.ascontiguousarray(rows, dtype=np.int64)
    O.lib().fo_global_row_batch(world, rank, seq_local, int(causal), O.ptr(local), len(local), O.ptr(out))
    return out


def _row_positions(m: int, rows: np.ndarray) -> np.ndarray:
    pos = np.full(m, -1, dtype=np.int64)
    pos[rows] = np.arange(len(rows))
    return pos


# ---------------------------------------------------------------------------------------------
# forward
# ---------------------------------------------------------------------------------------------

def check_qkv_forward(world, rank, seq_local, q_heads, kv_heads, head_dim, x, w, local, planar, rows,
                      alpha=1.0, tolerance=(0.01, 0.01), expected_local=None) -> dict:
    """x [M,K], w [N,K], local [M,N], planar = this rank's flat Q|K|V buffer (batch 1).
    expected_local: the oracle's rows of `local` when the caller computed them (block-scaled operands)."""
    m, n = seq_local, (q_heads + 2 * kv_heads) * head_dim
    rt = index_tensor(rows, local)
    mine = local[rt].contiguous()
    want = expected_local if expected_local is not None else \
        O.gemm_bf16(0, bits(x[rt]), bits(w), len(rows), n, x.shape[1], alpha=alpha)
    gemm = compare(bits(mine), want, *tolerance)
    gathered = bits(all_gather_rows(mine))                                # [world, R, N]
    # every element the sampled source rows contribute to THIS rank's planar buffer
    q_local, kv_local = q_heads // world * head_dim, kv_heads // world * head_dim
    rows_total = seq_local * world
    parts = []
    for base, width in ((0, q_local), (rows_total * q_local, kv_local),
                        (rows_total * (q_local + kv_local), kv_local)):
        g = (np.arange(world, dtype=np.int64)[:, None] * seq_local + rows[None, :]).reshape(-1)
        parts.append((base + g[:, None] * width + np.arange(width, dtype=np.int64)[None, :]).reshape(-1))
    index = np.ascontiguousarray(np.concatenate(parts).astype(np.uint64))
    source_rank = np.empty(len(index), dtype=np.int32)
    source_offset = np.empty(len(index), dtype=np.uint64)
    O.lib().fo_qkv_oracle_source_batch(world, rank, seq_local, q_heads * head_dim, kv_heads * head_dim, O.ptr(index),
                                       len(index), O.ptr(source_rank), O.ptr(source_offset))
    source_offset = source_offset.astype(np.int64)
    pos = _row_positions(m, rows)[source_offset // n]
    assert (pos >= 0).all(), "the oracle traced a sampled planar element to a row outside the sample"
    expected = gathered[source_rank, pos, source_offset % n]
    got = bits(planar.view(-1)[index_tensor(index.astype(np.int64), planar)])
    mismatches = int((got != expected).sum())
    return {"gemm": gemm, "route_bitexact": mismatches == 0, "route_mismatches": mismatches,
            "route_elements": int(len(index)), "rows": int(len(rows)),
            "unwritten_local": unwritten(local), "unwritten_routed": unwritten(planar)}


def check_qkv_forward_mxfp8(world, rank, seq_local, q_heads, kv_heads, head_dim, data, scales, w, wq, wq_scales, local,
                            planar, rows, alpha=1.0, tolerance=(0.01, 0.01)) -> dict:
    """data [M, K] E4M3 + native `scales` (the pre-quantised activation); w [N, K] BF16 master, wq /
    wq_scales its in-kernel quantisation; local [M, N]; planar = this rank's flat Q|K|V buffer."""
    k = data.shape[1]
    rt = index_tensor(rows, data)
    want_wq, want_ws = O.mxfp8_quantize(bits(w))
    weight_mismatches = _bytes_equal(wq, want_wq) + _bytes_equal(wq_scales, want_ws)
    got_s = scale_rows(scales, rows, k).cpu().numpy()
    want = O.gemm_mxfp8(np.ascontiguousarray(data[rt].cpu().numpy()), compact_scales(got_s, k), want_wq, want_ws, alpha=alpha)
    route = check_qkv_forward(world, rank, seq_local, q_heads, kv_heads, head_dim, None, None, local, planar, rows,
                              expected_local=want, tolerance=tolerance)
    route["route_mismatches"] += weight_mismatches
    route["route_bitexact"] = route["route_mismatches"] == 0
    route["route_elements"] += int(want_wq.size + want_ws.size)
    return route


def check_oproj_forward(world, rank, seq_local, k, attn, staging, w, out, rows, causal=False, cyclic=False,
                        alpha=1.0, tolerance=(0.01, 0.01)) -> dict:
    """attn = this rank's head shard [B*S_global, K/world]; staging [M,K]; w [N,K]; out [M,N]."""
    shard, n = k // world, w.shape[0]
    rt = index_tensor(rows, staging)
    attn2d = attn.view(-1, shard)
    send = torch.stack([attn2d[index_tensor(global_rows(world, dest, seq_local, causal, rows), attn2d)]
                        for dest in range(world)])                     # [dest, R, shard]
    recv = bits(exchange_rows(send))                                   # [source, R, shard]
    index = np.ascontiguousarray((rows[:, None] * k + np.arange(k, dtype=np.int64)[None, :]).reshape(-1).astype(np.uint64))
    source_rank = np.empty(len(index), dtype=np.int32)
    source_offset = np.empty(len(index), dtype=np.uint64)
    O.lib().fo_oproj_gather_source_batch(world, rank, seq_local, k, int(causal), int(cyclic), O.ptr(index), len(index),
                                         O.ptr(source_rank), O.ptr(source_offset))
    source_offset = source_offset.astype(np.int64)
    mine = global_rows(world, rank, seq_local, causal, rows)
    assert np.array_equal(source_offset // shard, np.repeat(mine, k)), "oracle row map and sample disagree"
    expected = recv[source_rank, np.repeat(np.arange(len(rows)), k), source_offset % shard].reshape(len(rows), k)
    got = bits(staging[rt])
    mismatches = int((got != expected).sum())
    want = O.gemm_bf16(0, got, bits(w), len(rows), n, k, alpha=alpha)
    gemm = compare(bits(out[rt]), want, *tolerance)
    return {"gemm": gemm, "route_bitexact": mismatches == 0, "route_mismatches": mismatches,
            "route_elements": int(got.size), "rows": int(len(rows)),
            "unwritten_local": unwritten(out), "unwritten_routed": unwritten(staging)}


def merge(*checks: dict) -> dict:
    """One verdict over several operators' checks (and, with a process group, over all ranks)."""
    ok = all(c["gemm"]["ok"] and c["route_bitexact"] and c["unwritten_local"] == 0 and c["unwritten_routed"] == 0
             for c in checks)
    summary = {
        "ok": ok,
        "rows": int(sum(c["rows"] for c in checks)),
        "max_abs_err": max(c["gemm"]["max_abs_err"] for c in checks),
        "gemm_elements": int(sum(c["gemm"]["elements"] for c in checks)),
        "gemm_out_of_tolerance": int(sum(c["gemm"]["bad"] for c in checks)),
        "route_bitexact": all(c["route_bitexact"] for c in checks),
        "route_elements": int(sum(c["route_elements"] for c in checks)),
        "route_mismatches": int(sum(c["route_mismatches"] for c in checks)),
        "unwritten_elements": int(sum(c["unwritten_local"] + c["unwritten_routed"] for c in checks)),
    }
    if world_size() > 1:
        everyone = [None] * world_size()
        dist.all_gather_object(everyone, summary)
        summary = {
            "ok": all(s["ok"] for s in everyone),
            "rows": sum(s["rows"] for s in everyone),
            "max_abs_err": max(s["max_abs_err"] for s in everyone),
            "gemm_elements": sum(s["gemm_elements"] for s in everyone),
            "gemm_out_of_tolerance": sum(s["gemm_out_of_tolerance"] for s in everyone),
            "route_bitexact": all(s["route_bitexact"] for s in everyone),
            "route_elements": sum(s["route_elements"] for s in everyone),
            "route_mismatches": sum(s["route_mismatches"] for s in everyone),
            "unwritten_elements": sum(s["unwritten_elements"] for s in everyone),
            "ranks": len(everyone),
        }
    return summary


# ---------------------------------------------------------------------------------------------
# BF16 backward
# ---------------------------------------------------------------------------------------------

def _traced_backward_rows(world, rank, seq_local, q_heads, kv_heads, head_dim, causal, planes, rows, step=1):
    """Expected rows of the packed [M, (q+2kv)*d] gradient (or, with step 32, of its per-K32-group
    scale bytes when `planes` hold one value per 32 features): every sampled element traced through
    the oracle's receiver-view map to the owner's plane; the owners' rows travel between ranks."""
    width = (q_heads + 2 * kv_heads) * head_dim
    received = []
    for plane in planes:  # [B*S_global, plane_width / step]
        send = torch.stack([plane[index_tensor(global_rows(world, dest, seq_local, causal, rows), plane)]
                            for dest in range(world)])
        received.append(exchange_rows(send).cpu().numpy())              # [owner, R, plane_width / step]
    features = np.arange(0, width, step, dtype=np.int32)
    row = np.ascontiguousarray(np.repeat(rows, len(features)))
    feature = np.ascontiguousarray(np.tile(features, len(rows)))
    owner = np.empty(len(row), dtype=np.int32)
    segment = np.empty(len(row), dtype=np.int32)
    offset = np.empty(len(row), dtype=np.int64)
    O.lib().fo_qkv_backward_source_batch(world, rank, seq_local, q_heads, kv_heads, head_dim, int(causal), O.ptr(row),
                                         O.ptr(feature), len(row), O.ptr(owner), O.ptr(segment), O.ptr(offset))
    mine = np.repeat(global_rows(world, rank, seq_local, causal, rows), len(features))
    position = np.repeat(np.arange(len(rows)), len(features))
    expected = np.empty(len(row), dtype=received[0].dtype)
    for s, heads in enumerate((q_heads, kv_heads, kv_heads)):
        plane_width = heads // world * head_dim
        pick = segment == s
        assert np.array_equal(offset[pick] // plane_width, mine[pick]), "oracle row map and sample disagree"
        expected[pick] = received[s][owner[pick], position[pick], (offset[pick] % plane_width) // step]
    return expected.reshape(len(rows), len(features))


def check_qkv_backward_data(world, rank, seq_local, q_heads, kv_heads, head_dim, planes, w, staging, dx, rows,
                            causal=False, alpha=1.0, tolerance=(0.02, 0.02)) -> dict:
    """planes = this rank's (dQ, dK, dV) [B*S_global, local_heads*d]; w [QKV, H]; staging [M, QKV]; dx [M, H]."""
    width, hidden = (q_heads + 2 * kv_heads) * head_dim, w.shape[1]
    rt = index_tensor(rows, staging)
    expected = _traced_backward_rows(world, rank, seq_local, q_heads, kv_heads, head_dim, causal,
                                     [p.view(torch.int16) for p in planes], rows).view(np.uint16)
    got = bits(staging.view(-1, width)[rt])
    mismatches = int((got != expected).sum())
    want = O.gemm_bf16(1, got, bits(w), len(rows), hidden, width, alpha=alpha)
    gemm = compare(bits(dx[rt]), want, *tolerance)
    return {"gemm": gemm, "route_bitexact": mismatches == 0, "route_mismatches": mismatches,
            "route_elements": int(got.size), "rows": int(len(rows)),
            "unwritten_local": unwritten(dx), "unwritten_routed": unwritten(staging)}


def check_weight_gradient(a_km, b_kn, dw, picked, alpha=1.0, tolerance=(0.02, 0.02)) -> dict:
    """dW[m_out, n_out] = alpha * A^T B with A stored [tokens, m_out], B stored [tokens, n_out]:
    the `picked` rows of dW, every column."""
    ct = index_tensor(picked, dw)
    tokens, n_out = b_kn.shape
    a_sub = bits(a_km[:, ct])                                            # [tokens, C]
    want = O.gemm_bf16(2, a_sub, bits(b_kn), len(picked), n_out, tokens, alpha=alpha)
    gemm = compare(bits(dw[ct]), want, *tolerance)
    return {"gemm": gemm, "route_bitexact": True, "route_mismatches": 0, "route_elements": 0, "rows": int(len(picked)),
            "unwritten_local": unwritten(dw), "unwritten_routed": 0}


def check_oproj_backward_data(world, rank, seq_local, a_width, dy, wo, da, routed, rows, causal=False, alpha=1.0,
                              tolerance=(0.02, 0.02), expected_local=None) -> dict:
    """dy [M, H]; wo [H, A]; da [M, A]; routed = this rank's head shard [B*S_global, A/world] of every rank's dA.
    expected_local: the oracle's rows of `da` when the caller computed them (block-scaled operands)."""
    shard = a_width // world
    rt = index_tensor(rows, da)
    mine = da[rt].contiguous()
    want = expected_local if expected_local is not None else \
        O.gemm_bf16(1, bits(dy[rt]), bits(wo), len(rows), a_width, dy.shape[1], alpha=alpha)
    gemm = compare(bits(mine), want, *tolerance)
    gathered = bits(all_gather_rows(mine))                                # [world, R, A]
    g = np.concatenate([global_rows(world, source, seq_local, causal, rows) for source in range(world)])
    index = np.ascontiguousarray((g[:, None] * shard + np.arange(shard, dtype=np.int64)[None, :]).reshape(-1).astype(np.uint64))
    source_rank = np.empty(len(index), dtype=np.int32)
    source_offset = np.empty(len(index), dtype=np.uint64)
    O.lib().fo_oproj_backward_source_batch(world, rank, 1, seq_local, a_width, int(causal), O.ptr(index), len(index),
                                           O.ptr(source_rank), O.ptr(source_offset))
    source_offset = source_offset.astype(np.int64)
    pos = _row_positions(seq_local, rows)[source_offset // a_width]
    assert (pos >= 0).all(), "the oracle traced a sampled element to a row outside the sample"
    expected = gathered[source_rank, pos, source_offset % a_width]
    got = bits(routed.view(-1)[index_tensor(index.astype(np.int64), routed)])
    mismatches = int((got != expected).sum())
    return {"gemm": gemm, "route_bitexact": mismatches == 0, "route_mismatches": mismatches,
            "route_elements": int(len(index)), "rows": int(len(rows)),
            "unwritten_local": unwritten(da), "unwritten_routed": unwritten(routed)}


# ---------------------------------------------------------------------------------------------
# MXFP8
# ---------------------------------------------------------------------------------------------

def scale_rows(scales: torch.Tensor, rows: np.ndarray, width: int) -> torch.Tensor:
    """The UE8M0 bytes of `rows` of a [*, width] operand from its native scale storage: [R, width/32]."""
    groups = width // 32
    row = np.ascontiguousarray(np.repeat(rows, groups).astype(np.int64))
    k = np.ascontiguousarray(np.tile(np.arange(groups, dtype=np.int64) * 32, len(rows)))
    offset = np.empty(len(row), dtype=np.int64)
    O.lib().fo_mxfp8_scale_offset_batch(O.ptr(row), O.ptr(k), width, len(row), O.ptr(offset))
    return scales.view(-1)[index_tensor(offset, scales)].view(len(rows), groups)


def compact_scales(values: np.ndarray, width: int) -> np.ndarray:
    """[R, width/32] scale bytes -> native scale storage of a compact [R, width] operand."""
    r, groups = values.shape
    out = np.full(O.lib().fo_mxfp8_scale_bytes(r, width), 127, dtype=np.uint8)
    row = np.ascontiguousarray(np.repeat(np.arange(r, dtype=np.int64), groups))
    k = np.ascontiguousarray(np.tile(np.arange(groups, dtype=np.int64) * 32, r))
    offset = np.empty(len(row), dtype=np.int64)
    O.lib().fo_mxfp8_scale_offset_batch(O.ptr(row), O.ptr(k), width, len(row), O.ptr(offset))
    out[offset] = values.reshape(-1)
    return out


def _bytes_equal(device_tensor: torch.Tensor, expected: np.ndarray) -> int:
    """Mismatching bytes between a device byte tensor and a host array of the same size."""
    want = torch.from_numpy(np.ascontiguousarray(expected).reshape(-1)).to(device_tensor.device)
    return int((device_tensor.reshape(-1)[:want.numel()] != want).sum())


def check_oproj_forward_mxfp8(world, rank, seq_local, k, data, scales, staged, staged_scales, w, wq, wq_scales, out,
                              rows, causal=False, alpha=1.0, tolerance=(0.01, 0.01)) -> dict:
    """data [B*S_global, K/world] E4M3 + native `scales` of this rank's shard; staged [M, K] bytes +
    native staged_scales (the operator's gathered lhs); w [N, K] BF16 master, wq / wq_scales its
    in-kernel quantisation; out [M, N]."""
    shard, n = k // world, w.shape[0]
    rt = index_tensor(rows, staged)
    send = torch.stack([data[index_tensor(global_rows(world, dest, seq_local, causal, rows), data)] for dest in range(world)])
    recv = exchange_rows(send).cpu().numpy()                              # [source, R, shard] bytes
    send_s = torch.stack([scale_rows(scales, global_rows(world, dest, seq_local, causal, rows), shard) for dest in range(world)])
    recv_s = exchange_rows(send_s).cpu().numpy()                          # [source, R, shard/32]
    index = np.ascontiguousarray((rows[:, None] * k + np.arange(k, dtype=np.int64)[None, :]).reshape(-1).astype(np.uint64))
    source_rank = np.empty(len(index), dtype=np.int32)
    source_offset = np.empty(len(index), dtype=np.uint64)
    O.lib().fo_oproj_gather_source_batch(world, rank, seq_local, k, int(causal), 0, O.ptr(index), len(index),
                                         O.ptr(source_rank), O.ptr(source_offset))
    source_offset = source_offset.astype(np.int64)
    position = np.repeat(np.arange(len(rows)), k)
    expected = recv[source_rank, position, source_offset % shard].reshape(len(rows), k)
    got = staged[rt].cpu().numpy()
    mismatches = int((got != expected).sum())
    first = slice(0, None, 32)                                           # first element of every K32 group
    expected_s = recv_s[source_rank[first], position[first], (source_offset[first] % shard) // 32].reshape(len(rows), k // 32)
    got_s = scale_rows(staged_scales, rows, k).cpu().numpy()
    mismatches += int((got_s != expected_s).sum())
    want_wq, want_ws = O.mxfp8_quantize(bits(w))
    weight_mismatches = _bytes_equal(wq, want_wq) + _bytes_equal(wq_scales, want_ws)
    want = O.gemm_mxfp8(np.ascontiguousarray(got), compact_scales(got_s, k), want_wq, want_ws, alpha=alpha)
    gemm = compare(bits(out[rt]), want, *tolerance)
    return {"gemm": gemm, "route_bitexact": mismatches == 0 and weight_mismatches == 0,
            "route_mismatches": mismatches + weight_mismatches,
            "route_elements": int(got.size + got_s.size + want_wq.size + want_ws.size), "rows": int(len(rows)),
            "unwritten_local": unwritten(out), "unwritten_routed": 0}


def check_qkv_backward_data_mxfp8(world, rank, seq_local, q_heads, kv_heads, masters, planes_q, planes_s, w, staging,
                                  packed, packed_scales, wq, wq_scales, dx, rows, causal=False, alpha=1.0,
                                  tolerance=(0.01, 0.01)) -> dict:
    """masters / planes_q / planes_s = this rank's BF16, E4M3 and native-scale planes (dQ, dK, dV);
    staging [M, QKV] BF16 masters as routed; packed [M, QKV] bytes + native packed_scales (the GEMM's
    lhs); w [QKV, H] master, wq [H, QKV] / wq_scales its in-kernel transposed quantisation; dx [M, H]."""
    d = 128
    width, hidden = (q_heads + 2 * kv_heads) * d, w.shape[1]
    rt = index_tensor(rows, staging)
    want_master = _traced_backward_rows(world, rank, seq_local, q_heads, kv_heads, d, causal,
                                        [p.view(torch.int16) for p in masters], rows).view(np.uint16)
    mismatches = int((bits(staging.view(-1, width)[rt]) != want_master).sum())
    want_bytes = _traced_backward_rows(world, rank, seq_local, q_heads, kv_heads, d, causal, planes_q, rows)
    got = packed[rt].cpu().numpy()
    mismatches += int((got != want_bytes).sum())
    heads = (q_heads, kv_heads, kv_heads)
    rows_global = seq_local * world
    scale_planes = [scale_rows(s, np.arange(rows_global), h // world * d) for s, h in zip(planes_s, heads)]
    want_s = _traced_backward_rows(world, rank, seq_local, q_heads, kv_heads, d, causal, scale_planes, rows, step=32)
    got_s = scale_rows(packed_scales, rows, width).cpu().numpy()
    mismatches += int((got_s != want_s).sum())
    want_wq, want_ws = O.mxfp8_quantize_transposed(bits(w))
    weight_mismatches = _bytes_equal(wq, want_wq) + _bytes_equal(wq_scales, want_ws)
    want = O.gemm_mxfp8(np.ascontiguousarray(got), compact_scales(got_s, width), want_wq, want_ws, alpha=alpha)
    gemm = compare(bits(dx[rt]), want, *tolerance)
    return {"gemm": gemm, "route_bitexact": mismatches == 0 and weight_mismatches == 0,
            "route_mismatches": mismatches + weight_mismatches,
            "route_elements": int(want_master.size + got.size + got_s.size + want_wq.size + want_ws.size),
            "rows": int(len(rows)), "unwritten_local": unwritten(dx), "unwritten_routed": unwritten(staging)}


def check_oproj_backward_data_mxfp8(world, rank, seq_local, a_width, dy_q, dy_s, wo, da, routed, rows, causal=False,
                                    alpha=1.0, tolerance=(0.01, 0.01)) -> dict:
    """dy_q [M, H] E4M3 + native dy_s (the upstream-quantised output gradient); wo [H, A] BF16 master,
    re-quantised along H inside the operator; da [M, A]; routed as in check_oproj_backward_data."""
    hidden = dy_q.shape[1]
    rt = index_tensor(rows, dy_q)
    w_q, w_s = O.mxfp8_quantize_transposed(bits(wo))                      # [A, H] along H
    got_s = scale_rows(dy_s, rows, hidden).cpu().numpy()
    want = O.gemm_mxfp8(np.ascontiguousarray(dy_q[rt].cpu().numpy()), compact_scales(got_s, hidden), w_q, w_s, alpha=alpha)
    return check_oproj_backward_data(world, rank, seq_local, a_width, None, None, da, routed, rows, causal=causal,
                                     tolerance=tolerance, expected_local=want)


def check_weight_gradient_mxfp8(a_km, b_kn, dw, picked, columns, alpha=1.0, tolerance=(0.01, 0.01)) -> dict:
    """Block-scaled dW = alpha * q(A^T) q(B^T)^T (both operands re-quantised along the token axis):
    the `picked` rows x `columns` columns of dW, recomputed from the BF16 masters."""
    ct, ht = index_tensor(picked, dw), index_tensor(columns, dw)
    a_q, a_s = O.mxfp8_quantize_transposed(bits(a_km[:, ct]))
    b_q, b_s = O.mxfp8_quantize_transposed(bits(b_kn[:, ht]))
    want = O.gemm_mxfp8(a_q, a_s, b_q, b_s, alpha=alpha)
    gemm = compare(bits(dw[ct][:, ht]), want, *tolerance)
    return {"gemm": gemm, "route_bitexact": True, "route_mismatches": 0, "route_elements": 0, "rows": int(len(picked)),
            "unwritten_local": unwritten(dw), "unwritten_routed": 0}


# ---------------------------------------------------------------------------------------------
# MoE dispatch + FC1
# ---------------------------------------------------------------------------------------------

def check_moe_dispatch_fc1(world, tokens, lhs, out, weights, row_offsets, sources, per_expert=8,
                           tolerance=(0.002, 0.008)) -> dict:
    """tokens [T, K] of this rank; lhs [E, capacity, K] / out [E, capacity, N] as the operator left them
    (poisoned with 0xFFFF before the launch); weights [E, N, K]; row_offsets [E+1], sources [rows, 3].
    EVERY dispatched row is compared, bit for bit, on the device with the token its source names
    (all ranks' tokens are gathered); FC1 is recomputed by the oracle for a few rows per expert."""
    experts = weights.shape[0]
    everyone = all_gather_rows(tokens)                                    # [world, T, K]
    src = torch.from_numpy(np.ascontiguousarray(sources[:, :2], dtype=np.int64)).to(tokens.device)
    mismatches = elements = unwritten_rows = 0
    checks = []
    rng = np.random.default_rng(99)
    for e in range(experts):
        begin, end = int(row_offsets[e]), int(row_offsets[e + 1])
        count = end - begin
        if count == 0:
            continue
        expected = everyone[src[begin:end, 0], src[begin:end, 1]]
        got = lhs[e, :count]
        mismatches += int((got.view(torch.int16) != expected.view(torch.int16)).sum())
        elements += int(got.numel())
        unwritten_rows += unwritten(out[e, :count])
        picked = sorted({0, count - 1} | {int(v) for v in rng.integers(0, count, per_expert)})
        pt = index_tensor(np.array(picked), lhs)
        n, k = weights.shape[1], weights.shape[2]
        want = O.gemm_bf16(0, bits(got[pt]), bits(weights[e]), len(picked), n, k)
        checks.append(compare(bits(out[e][pt]), want, *tolerance))
    gemm = {"ok": all(c["ok"] for c in checks), "max_abs_err": max((c["max_abs_err"] for c in checks), default=0.0),
            "bad": sum(c["bad"] for c in checks), "elements": sum(c["elements"] for c in checks),
            "tolerance": checks[0]["tolerance"] if checks else ""}
    return {"gemm": gemm, "route_bitexact": mismatches == 0, "route_mismatches": mismatches, "route_elements": elements,
            "rows": int(sum(c["elements"] for c in checks) // max(1, weights.shape[1])),
            "unwritten_local": unwritten_rows, "unwritten_routed": 0}


def check_moe_fc2_combine(world, rank, lhs, weights, out, received, row_offsets, sources, chosen, experts_local, topk,
                          sample=1024, per_expert=8, tolerance=(0.002, 0.008)) -> dict:
    """lhs [E, capacity, K], weights [E, N, K], out [E, capacity, N] of this rank; received =
    this rank's [tokens * topk, N] branch rows as the owners wrote them; row_offsets / sources =
    this rank's routes, chosen[r] = rank r's [tokens, topk] expert table (every rank holds all).
    A seeded sample of (token, slot) branches per rank is compared BIT-EXACT with the row the
    owner's slab holds (the owners send those rows); FC2 is recomputed by the oracle for a few rows
    per expert; no branch row may still hold the poison."""
    experts, n, k = weights.shape
    tokens = chosen[0].shape[0]
    rng = np.random.default_rng(4321)
    picks = np.unique(np.concatenate([[0, tokens * topk - 1], rng.integers(0, tokens * topk, sample)]))
    picks = np.resize(picks, sample).astype(np.int64)            # the same branches on every rank, fixed count
    token, slot = picks // topk, picks % topk
    # as an owner: where each routed branch sits in this rank's slabs
    row_of = np.full((world, tokens, topk), -1, dtype=np.int64)
    if len(sources):
        row_of[sources[:, 0], sources[:, 1], sources[:, 2]] = np.arange(len(sources))
    offsets = np.asarray(row_offsets, dtype=np.int64)
    send = torch.zeros((world, sample, n), dtype=out.dtype, device=out.device)
    for dest in range(world):
        rows = row_of[dest, token, slot]
        mine = rows >= 0
        if mine.any():
            expert = np.searchsorted(offsets, rows[mine], side="right") - 1
            local = rows[mine] - offsets[expert]
            send[dest, index_tensor(np.nonzero(mine)[0], out)] = out[index_tensor(expert, out), index_tensor(local, out)]
    recv = exchange_rows(send)                                           # [owner, sample, N]
    owner = (chosen[rank][token, slot] // experts_local).astype(np.int64)
    expected = recv[index_tensor(owner, out), index_tensor(np.arange(sample), out)]
    got = received.view(-1, n)[index_tensor(picks, received)]
    mismatches = int((got.view(torch.int16) != expected.view(torch.int16)).sum())
    checks = []
    for e in range(experts):
        count = int(offsets[e + 1] - offsets[e])
        if count == 0:
            continue
        picked = sorted({0, count - 1} | {int(v) for v in rng.integers(0, count, per_expert)})
        pt = index_tensor(np.array(picked), lhs)
        want = O.gemm_bf16(0, bits(lhs[e][pt]), bits(weights[e]), len(picked), n, k)
        checks.append(compare(bits(out[e][pt]), want, *tolerance))
    gemm = {"ok": all(c["ok"] for c in checks), "max_abs_err": max((c["max_abs_err"] for c in checks), default=0.0),
            "bad": sum(c["bad"] for c in checks), "elements": sum(c["elements"] for c in checks),
            "tolerance": checks[0]["tolerance"] if checks else ""}
    return {"gemm": gemm, "route_bitexact": mismatches == 0, "route_mismatches": mismatches,
            "route_elements": int(got.numel()), "rows": int(sample), "unwritten_local": 0,
            "unwritten_routed": unwritten(received)}
