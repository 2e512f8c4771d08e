"""Offline calibration of the host planner on one B200.

    python -m fuse_b200.calibrate [--write]

Measures what the planner's model needs -- the GEMM rate of one SM inside the persistent kernels
(CTA pairs and one-CTA tiles, BF16 and MXFP8), the copy rate of one communication CTA and of one
embedded copy warp for every transfer kind (copy-only launches: FUSE_B200_COMM_ONLY), and the
start-up time of a transfer -- and, with --write, rewrites fuse_b200/csrc/calibration_b200.h and
fuse_b200/calibration/b200.json.  Copies are local (one GPU) so that the copy pipelines, not a link,
are measured; rebuild the library afterwards."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from fuse_b200 import _native as N  # noqa: E402
from fuse_b200 import api  # noqa: E402

BF16, U8, I32 = torch.bfloat16, torch.uint8, torch.int32
SMS = 148


def median_ms(fn, warmup=2, samples=7):
    def once():
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = fn()
        assert not (isinstance(rc, int) and rc), f"cudaError {rc}"
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)
    for _ in range(warmup):
        once()
    return statistics.median(once() for _ in range(samples))


def gen(shape, seed, scale):
    t = torch.empty(shape, dtype=BF16, device="cuda")
    assert api.generate_bf16(t.data_ptr(), t.numel(), seed, scale, normal=True) == 0
    return t


def options(flags):
    o = N.Options()
    o.flags = flags
    return o


def with_env(name, value, fn):
    old = os.environ.get(name)
    os.environ[name] = value
    try:
        return fn()
    finally:
        if old is None:
            os.environ.pop(name, None)
        else:
            os.environ[name] = old


def gemm_rates(out):
    m, n, k = 16384, 6144, 4096
    a, b, d = gen((m, k), 1, 1.0), gen((n, k), 2, 0.02), torch.empty((m, n), dtype=BF16, device="cuda")
    p = N.GemmA2AParams(lhs=a.data_ptr(), rhs_nt=b.data_ptr(), local_output=d.data_ptr(),
                        gemm=N.GemmProblem(m, n, k, raster=N.RASTER_ALONG_M, max_swizzle_size=8), num_comm_ctas=1, epoch=1)
    flops = 2.0 * m * n * k
    pair = median_ms(lambda: api.launch_batched_cutlass_reference(p, 0, 0))
    cta = with_env("FUSE_B200_PAIR", "0", lambda: median_ms(lambda: api.launch_batched_cutlass_reference(p, 0, 0)))
    out["bf16_pair"] = {"shape": [m, n, k], "ms": pair, "tflops_per_sm": flops / pair / 1e9 / SMS}
    out["bf16_cta"] = {"shape": [m, n, k], "ms": cta, "tflops_per_sm": flops / cta / 1e9 / SMS}
    del a, b, d
    m, n, k = 16384, 8192, 8192
    act = gen((m, k), 3, 1.0)
    qd = torch.empty((m, k), dtype=U8, device="cuda")
    qs = torch.empty(api.mxfp8_scale_bytes(m, k), dtype=U8, device="cuda")
    assert api.quantize_mxfp8(act.data_ptr(), k, m, k, qd.data_ptr(), qs.data_ptr(), 0) == 0
    w = gen((n, k), 4, 0.02)
    d = torch.empty((m, n), dtype=BF16, device="cuda")
    prob = N.GemmProblem(m, n, k, max_swizzle_size=8)
    rc, ws = api.gemm_a2a_mxfp8_workspace_size(prob)
    buf = torch.empty(ws + 256, dtype=U8, device="cuda")
    base = (buf.data_ptr() + 255) // 256 * 256
    pq = N.GemmA2AParams(rhs_nt=w.data_ptr(), local_output=d.data_ptr(), gemm=prob, num_comm_ctas=0, epoch=1)
    mp = N.Mxfp8GemmA2AParams(projection=pq, workspace=base, workspace_bytes=ws,
                              activation=N.Mxfp8Activation(data=qd.data_ptr(), scales=qs.data_ptr(), data_bytes=qd.numel(),
                                                           scale_bytes=qs.numel()))
    assert api.prepare_gemm_a2a_mxfp8(mp, 0) == 0
    flops = 2.0 * m * n * k
    pair = median_ms(lambda: api.launch_gemm_a2a_mxfp8_compute_reference(mp, 0))
    cta = with_env("FUSE_B200_PAIR", "0", lambda: median_ms(lambda: api.launch_gemm_a2a_mxfp8_compute_reference(mp, 0)))
    out["mx_pair"] = {"shape": [m, n, k], "ms": pair, "tflops_per_sm": flops / pair / 1e9 / SMS}
    out["mx_cta"] = {"shape": [m, n, k], "ms": cta, "tflops_per_sm": flops / cta / 1e9 / SMS}


def pull_rates(out):
    """a2a -> OProj lhs pull, BF16, C2 shape, local copies."""
    m, n, k = 16384, 4096, 4096
    attn, w = gen((m, k), 5, 1.0), gen((n, k), 6, 0.02)
    staging, d = torch.empty((m, k), dtype=BF16, device="cuda"), torch.empty((m, n), dtype=BF16, device="cuda")
    prob = N.GemmProblem(m, n, k, raster=N.RASTER_ALONG_N, max_swizzle_size=8)
    route = N.UlyssesRoute(world_size=1, rank=0, batch=1, global_seq=m, seq_local=m, q_heads=32, head_dim=128,
                           kind=N.ROUTE_HEAD_TO_SEQUENCE, direction=N.ROUTE_INVERSE)
    ready = torch.zeros(api.a2a_lhs_gemm_ready_elements(prob, route), dtype=I32, device="cuda")
    p = N.A2AGemmParams(input_staging=staging.data_ptr(), rhs_nt=w.data_ptr(), output=d.data_ptr(), ready=ready.data_ptr(),
                        gemm=prob, route=route, num_comm_ctas=16, epoch=0)
    p.peer_input[0] = attn.data_ptr()
    bytes_ = m * k * 2.0
    epoch = [0]

    def launch(flags):
        epoch[0] += 1
        p.epoch = epoch[0]
        return api.launch_a2a_gemm_cutlass(p, 0, options(flags))

    rows = {}
    for comm in (8, 16, 32):
        p.num_comm_ctas = comm
        ms = with_env("FUSE_B200_EMBEDDED_PULL", "0", lambda: median_ms(lambda: launch(N.COMM_ONLY)))
        rows[comm] = {"ms": ms, "gbs_per_cta": bytes_ / ms / 1e6 / comm}
    p.num_comm_ctas = 16
    emb = with_env("FUSE_B200_EMBEDDED_PULL", "1", lambda: median_ms(lambda: launch(N.COMM_ONLY)))
    # the whole operator both ways, and the GEMM alone: what the two candidates really cost against the model
    full = with_env("FUSE_B200_EMBEDDED_PULL", "1", lambda: median_ms(lambda: launch(0)))
    fused_comm = {}
    for comm in (8, 16, 32):
        p.num_comm_ctas = comm
        fused_comm[comm] = with_env("FUSE_B200_EMBEDDED_PULL", "0", lambda: median_ms(lambda: launch(0)))
    pure = median_ms(lambda: api.launch_a2a_gemm_cutlass_reference(p, 0, 0))
    out["pull"] = {"shape": [m, n, k], "bytes": bytes_, "comm_ctas": rows,
                   "embedded": {"ms": emb, "gbs_per_cta": bytes_ / emb / 1e6 / SMS},
                   "fused_embedded_ms": full, "fused_comm_ms": fused_comm, "pure_ms": pure}
    api.read_status()


def push_rates(out):
    """QKV backward data, BF16, C2 shape: sender push of the planar gradients, local copies."""
    m, hid, q, kv, d = 16384, 4096, 32, 8, 128
    n = (q + 2 * kv) * d
    planes = [gen((m, h * d), 10 + i, 0.01) for i, h in enumerate((q, kv, kv))]
    w = gen((n, hid), 7, 0.02)
    staging, dx = torch.empty((m, n), dtype=BF16, device="cuda"), torch.empty((m, hid), dtype=BF16, device="cuda")
    done = torch.zeros(N.READY_FLAG_STRIDE, dtype=I32, device="cuda")
    bp = N.QkvBackwardDataParams(local_tokens=m, hidden=hid, batch=1, q_heads=q, kv_heads=kv, head_dim=d, world_size=1,
                                 rank=0, num_comm_ctas=16, epoch=0)
    bp.gemm_tuning.max_swizzle_size = 8
    ready = torch.zeros(api.qkv_backward_ready_elements(bp), dtype=I32, device="cuda")
    bp.grad_q, bp.grad_k, bp.grad_v = (t.data_ptr() for t in planes)
    bp.weight, bp.grad_input = w.data_ptr(), dx.data_ptr()
    bp.peer_dqkv_staging[0], bp.peer_ready[0], bp.peer_done_epoch[0] = staging.data_ptr(), ready.data_ptr(), done.data_ptr()
    bytes_ = m * n * 2.0
    epoch = [0]

    def launch(flags):
        epoch[0] += 1
        bp.epoch = epoch[0]
        return api.launch_qkv_backward_data(bp, 0, options(flags))

    rows = {}
    for comm in (8, 16, 32):
        bp.num_comm_ctas = comm
        ms = with_env("FUSE_B200_EMBEDDED_PULL", "0", lambda: median_ms(lambda: launch(N.COMM_ONLY)))
        rows[comm] = {"ms": ms, "gbs_per_cta": bytes_ / ms / 1e6 / comm}
    bp.num_comm_ctas = 16
    emb = with_env("FUSE_B200_EMBEDDED_PULL", "1", lambda: median_ms(lambda: launch(N.COMM_ONLY)))
    out["push"] = {"shape": [m, hid, n], "bytes": bytes_, "comm_ctas": rows,
                   "embedded": {"ms": emb, "gbs_per_cta": bytes_ / emb / 1e6 / SMS}}
    api.read_status()


def gradpull_rates(out):
    """QKV backward data, MXFP8, a quarter of the C4 rows: receiver pull of bytes, scales and masters."""
    m, hid, q, kv, d = 16384, 5120, 64, 8, 128
    width = (q + 2 * kv) * d
    masters = [gen((m, h * d), 20 + i, 0.01) for i, h in enumerate((q, kv, kv))]
    quant = []
    for t in masters:
        qd = torch.empty(t.shape, dtype=U8, device="cuda")
        qs = torch.empty(api.mxfp8_scale_bytes(*t.shape), dtype=U8, device="cuda")
        assert api.quantize_mxfp8(t.data_ptr(), t.shape[1], t.shape[0], t.shape[1], qd.data_ptr(), qs.data_ptr(), 0) == 0
        quant.append((qd, qs))
    w = gen((width, hid), 8, 0.02)
    staging, dx = torch.empty((m, width), dtype=BF16, device="cuda"), torch.empty((m, hid), dtype=BF16, device="cuda")
    done = torch.zeros(N.READY_FLAG_STRIDE, dtype=I32, device="cuda")
    proj = N.QkvBackwardDataParams(weight=w.data_ptr(), grad_input=dx.data_ptr(), local_tokens=m, hidden=hid, batch=1,
                                   q_heads=q, kv_heads=kv, head_dim=d, world_size=1, rank=0, num_comm_ctas=16, epoch=0)
    proj.gemm_tuning.max_swizzle_size = 8
    ready = torch.zeros(api.qkv_backward_ready_elements(proj), dtype=I32, device="cuda")
    proj.peer_dqkv_staging[0], proj.peer_ready[0], proj.peer_done_epoch[0] = staging.data_ptr(), ready.data_ptr(), done.data_ptr()
    rc, ws = api.qkv_backward_mxfp8_data_workspace_size(proj)
    buf = torch.empty(ws + 256, dtype=U8, device="cuda")
    mp = N.Mxfp8QkvBackwardDataParams(projection=proj, workspace=(buf.data_ptr() + 255) // 256 * 256, workspace_bytes=ws)
    act = lambda i: N.Mxfp8Activation(data=quant[i][0].data_ptr(), scales=quant[i][1].data_ptr(),
                                      data_bytes=quant[i][0].numel(), scale_bytes=quant[i][1].numel())
    mp.peer_input[0] = N.Mxfp8QkvBackwardInput(grad_q=act(0), grad_k=act(1), grad_v=act(2), master_q=masters[0].data_ptr(),
                                               master_k=masters[1].data_ptr(), master_v=masters[2].data_ptr())
    bytes_ = m * width * (3.0 + 1.0 / 32)
    epoch = [0]

    def launch(flags):
        epoch[0] += 1
        mp.projection.epoch = epoch[0]
        return api.launch_qkv_backward_mxfp8_data(mp, 0, options(flags))

    rows = {}
    for comm in (8, 16, 32):
        mp.projection.num_comm_ctas = comm
        ms = with_env("FUSE_B200_EMBEDDED_PULL", "0", lambda: median_ms(lambda: launch(N.COMM_ONLY)))
        rows[comm] = {"ms": ms, "gbs_per_cta": bytes_ / ms / 1e6 / comm}
    mp.projection.num_comm_ctas = 16
    emb = with_env("FUSE_B200_EMBEDDED_PULL", "1", lambda: median_ms(lambda: launch(N.COMM_ONLY)))
    out["gradpull"] = {"shape": [m, hid, width], "bytes": bytes_, "comm_ctas": rows,
                       "embedded": {"ms": emb, "gbs_per_cta": bytes_ / emb / 1e6 / SMS},
                       "note": "COMM_ONLY launches still run the W^T quantisation kernel (52 MB written)"}
    api.read_status()


def dispatch_rates(out):
    """MoE dispatch with a GEMM too small to matter (N 256): the row pull alone."""
    tokens, hid, experts, n = 16384, 7168, 32, 256
    toks = gen((tokens, hid), 30, 1.0)
    cap = tokens // experts * 2
    rows_per = tokens * 2 // experts
    import numpy as np
    src = np.stack([np.zeros(tokens * 2, np.int32), np.arange(tokens * 2, dtype=np.int32) % tokens,
                    np.arange(tokens * 2, dtype=np.int32) // tokens], 1)
    offs = (np.arange(experts + 1) * rows_per).astype(np.int64)
    w = gen((experts, n, hid), 31, 0.02)
    lhs = torch.empty((experts, cap, hid), dtype=BF16, device="cuda")
    eo = torch.empty((experts, cap, n), dtype=BF16, device="cuda")
    ptrs = lambda t: torch.tensor([t[i].data_ptr() for i in range(experts)], dtype=torch.int64, device="cuda")
    lp, wp, op = ptrs(lhs), ptrs(w), ptrs(eo)
    offs_d, src_d = torch.from_numpy(offs).cuda(), torch.from_numpy(src).cuda()
    started = torch.zeros(N.READY_FLAG_STRIDE, dtype=I32, device="cuda")
    done = torch.zeros(N.READY_FLAG_STRIDE, dtype=I32, device="cuda")
    gp = N.Bf16GroupedGemmParams(lhs=lp.data_ptr(), weight_nt=wp.data_ptr(), output=op.data_ptr(), row_offsets=offs_d.data_ptr(),
                                 source=src_d.data_ptr(), experts=experts, n=n, k=hid, expert_row_capacity=cap, rank=0,
                                 world_size=1, topk=2)
    gp.peer_input[0], gp.peer_started[0], gp.peer_done[0] = toks.data_ptr(), started.data_ptr(), done.data_ptr()
    bytes_ = tokens * 2 * hid * 2.0
    rows = {}
    for comm in (8, 16, 32):
        gp.policy = N.GroupedGemmPolicy(num_comm_ctas=comm, num_compute_ctas=148 - comm, tile_n=256, mma_sm_count=2)
        rc, plan = api.create_bf16_a2a_grouped_gemm(gp)
        assert rc == 0, rc
        ms = median_ms(lambda: api.launch_bf16_grouped_gemm(plan, 0))
        api.destroy_bf16_grouped_gemm(plan)
        rows[comm] = {"ms": ms, "gbs_per_cta": bytes_ / ms / 1e6 / comm}
    out["dispatch"] = {"shape": [tokens * 2, n, hid], "bytes": bytes_, "comm_ctas": rows,
                       "note": "whole operator with N = 256: the FC1 GEMM is 3 % of the C5 one"}
    api.read_status()


# One GPU cannot measure a link.  The lhs pull alone (bench.py: nvlink.copy_only, 32 communication
# CTAs) moved 492 GB/s on 2 GPUs (half of the bytes remote) and 534 GB/s on 4 (three quarters remote)
# against 1180 GB/s locally: 10-14 GB/s per CTA over NVLink against 37, i.e. 0.26-0.38; the MoE
# dispatch on 2 GPUs was transfer-bound with 16 CTAs at 16.6 GB/s per CTA (0.25 for its remote half)
# and on 8 GPUs ran at >= 14.4 GB/s per CTA with 20 (>= 0.32).  Too few CTAs costs far more than
# too many (16 against 20 on 2 GPUs: -11 %; 28 against 20: -4 %), so the low side of the range.
REMOTE_CTA_FACTOR = 0.30
# The gradient PUSH (BF16 QKV backward data, C2 shape) is the one transfer whose embedded variant loses
# over NVLink: 0.570 ms on one GPU, 0.598-0.606 on 2 (16 communication CTAs: 0.612-0.617), 0.638-0.645
# on 4 (12 CTAs 0.630, 16 CTAs 0.611-0.614, 20 CTAs 0.619, 24 CTAs 0.673).  Communication CTAs are
# flat in the remote share, the embedded push grows with it; the crossover lies between 1/2 and 3/4.
PUSH_EMBEDDED_MAX_REMOTE_SHARE = 0.6
PUSH_REMOTE_MIN_CTAS = 16


def model_comm_us(flops, nbytes, tiles, comm, tflops_per_sm, cta_gbs, startup_us=25.0, sms=SMS, group=2):
    """The planner's makespan of a communication budget (planner.cuh: score_comm), for the fit below."""
    units, comm_units = sms // group, comm // group
    compute = min(tiles, units - comm_units)
    tau = flops / tiles / (group * tflops_per_sm * 1e6)
    t_c = startup_us + nbytes / (comm * cta_gbs * 1e3)
    best = max(-(-tiles // compute) * tau, t_c + tau)
    w1 = 0
    while w1 * compute < tiles:
        rest = tiles - w1 * compute
        w2 = -(-rest // (compute + comm_units))
        best = min(best, max((w1 + w2) * tau, t_c + w2 * tau))
        w1 += 1
    return best


HEADER = '''// Calibration of the host planner, measured on one B200 by `python -m fuse_b200.calibrate`
// (which rewrites this file and fuse_b200/calibration/b200.json; the measurements behind every
// number are in the JSON).  Rates are what ONE SM / ONE communication CTA / ONE embedded copy warp
// sustains inside the persistent kernels, copies local (HBM to HBM) so that the pipeline, not a
// link, is measured.
#pragma once

namespace fuse_b200 {
namespace planner {

struct Calibration {
  double bf16_pair_tflops_per_sm, mx_pair_tflops_per_sm, bf16_cta_tflops_per_sm, mx_cta_tflops_per_sm,
      grouped_pair_tflops_per_sm;
  double pull_cta_gbs, pull_embedded_gbs, push_cta_gbs, push_embedded_gbs, gradpull_cta_gbs, gradpull_embedded_gbs,
      qkv_push_cta_gbs, dispatch_cta_gbs;
  // measured / modelled: the GEMM beside its embedded copy warp against the pure GEMM, and the
  // operator with communication CTAs against the wave model (contention the model leaves out)
  double embedded_compute_factor, comm_model_factor, startup_us;
  // rate of a communication CTA whose bytes cross NVLink, relative to the local rate above
  double remote_cta_factor;
  // gradient push: the embedded copy warps are used up to this share of remote bytes, beyond it
  // communication CTAs, at least this many (measured on 2 and 4 GPUs)
  double push_embedded_max_remote_share, push_remote_min_ctas;
};

constexpr Calibration kCalibrationB200 = {
%s
};

}  // namespace planner
}  // namespace fuse_b200
'''


def derive(raw):
    """The planner's constants from the raw measurements (also from a stored b200.json: --from-json)."""
    cta = lambda kind: statistics.median(v["gbs_per_cta"] for v in raw[kind]["comm_ctas"].values())
    c2 = dict(flops=2.0 * 16384 * 4096 * 4096, tiles=64 * 16)
    pair = raw["bf16_pair"]["tflops_per_sm"]
    # the planner's own time of the C2 GEMM on all pairs: whole waves of 74 tiles
    tau = c2["flops"] / c2["tiles"] / (2 * pair * 1e6)
    waves = -(-c2["tiles"] // (SMS // 2))
    return [
        ("bf16_pair_tflops_per_sm", pair),
        ("mx_pair_tflops_per_sm", raw["mx_pair"]["tflops_per_sm"]),
        ("bf16_cta_tflops_per_sm", raw["bf16_cta"]["tflops_per_sm"]),
        ("mx_cta_tflops_per_sm", raw["mx_cta"]["tflops_per_sm"]),
        ("grouped_pair_tflops_per_sm", pair * 0.96),
        ("pull_cta_gbs", cta("pull")), ("pull_embedded_gbs", raw["pull"]["embedded"]["gbs_per_cta"]),
        ("push_cta_gbs", cta("push")), ("push_embedded_gbs", raw["push"]["embedded"]["gbs_per_cta"]),
        ("gradpull_cta_gbs", cta("gradpull")), ("gradpull_embedded_gbs", raw["gradpull"]["embedded"]["gbs_per_cta"]),
        ("qkv_push_cta_gbs", cta("pull")),
        ("dispatch_cta_gbs", cta("dispatch")),
        # both candidates are anchored on what the whole operator measured at the C2 shape: the
        # planner's time of the embedded variant there IS the measured one, and the communication
        # budgets carry the median of measured / modelled over the budgets measured
        ("embedded_compute_factor", min(1.0, waves * tau / (raw["pull"]["fused_embedded_ms"] * 1e3))),
        ("comm_model_factor", statistics.median(
            ms * 1e3 / model_comm_us(c2["flops"], raw["pull"]["bytes"], c2["tiles"], int(comm), pair, cta("pull"))
            for comm, ms in raw["pull"]["fused_comm_ms"].items())),
        ("startup_us", 25.0),
        ("remote_cta_factor", REMOTE_CTA_FACTOR),
        ("push_embedded_max_remote_share", PUSH_EMBEDDED_MAX_REMOTE_SHARE),
        ("push_remote_min_ctas", float(PUSH_REMOTE_MIN_CTAS)),
    ]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--write", action="store_true")
    ap.add_argument("--out", default="", help="write b200.json and calibration_b200.h into this directory instead")
    ap.add_argument("--from-json", default="", help="derive the constants again from stored measurements (no GPU)")
    args = ap.parse_args()
    if args.from_json:
        with open(args.from_json) as f:
            raw = json.load(f)
    else:
        torch.cuda.set_device(0)
        N.lib()
        raw = {"gpu": torch.cuda.get_device_name(0)}
        gemm_rates(raw)
        pull_rates(raw)
        push_rates(raw)
        gradpull_rates(raw)
        dispatch_rates(raw)
    values = derive(raw)
    raw["constants"] = dict(values)
    print(json.dumps(raw, indent=1))
    if args.write or args.out:
        json_dir = args.out or os.path.join(HERE, "calibration")
        header_dir = args.out or os.path.join(HERE, "csrc")
        os.makedirs(json_dir, exist_ok=True)
        with open(os.path.join(json_dir, "b200.json"), "w") as f:
            json.dump(raw, f, indent=1)
        body = "\n".join(f"    /* {name:30s} */ {value:.4g}," for name, value in values)
        with open(os.path.join(header_dir, "calibration_b200.h"), "w") as f:
            f.write(HEADER % body)


if __name__ == "__main__":
    main()
