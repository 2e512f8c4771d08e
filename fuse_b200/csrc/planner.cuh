// Host-side plans: how many communication CTAs a fused operator gets when the caller asks for
// Auto (`num_comm_ctas == 0`), from an offline calibration of compute and copy rates on B200.
//
// The reference resolves Auto from tables of independently measured services -- GEMM time at each
// SM split, copy time per communication budget -- and picks the budget whose slower side,
// compute or transfer, finishes first (csrc/operators/sm103/detail/autotune.cuh:25-75,109-203:
// "minimize max(C, P)"; an explicit budget is used exactly, never silently changed).  This planner
// keeps those rules with this library's own services (calibration_b200.h, written by
// `python -m fuse_b200.calibrate` on a B200):
//   * compute: TFLOP/s one SM sustains inside the persistent kernels, per tile family;
//   * transfer: GB/s one communication CTA moves through its copy pipeline, and GB/s the single
//     copy warp embedded in a compute CTA moves (it costs the GEMM one of its six stages);
//   * a fixed start-up time before the first tile can run.
// Candidates: the embedded copy warps (no SM given up), and communication budgets 4 ... 48 whose
// CTAs join the GEMM when their transfers are done (the wave model of launch.cuh: plan_join).
// The makespan of a candidate is max(compute side, transfer side); the smallest wins, ties go to
// fewer communication CTAs.
#pragma once

#include <cstdint>

#include "calibration_b200.h"

namespace fuse_b200 {
namespace planner {

enum Kind : int32_t {
  kLhsPullBf16 = 0,   // a2a -> OProj, BF16
  kLhsPullMx = 1,     // a2a -> OProj, MXFP8 (bytes + scale atoms)
  kGradPushBf16 = 2,  // QKV backward data, BF16 (sender push)
  kGradPullMx = 3,    // QKV backward data, MXFP8 (receiver pull: E4M3 + scales + BF16 masters)
  kQkvPushBf16 = 4,   // QKVProj -> a2a from communication CTAs (the epilogue push needs none)
  kQkvPushMx = 5,
  kDispatchBf16 = 6,  // MoE dispatch -> FC1
  kKinds = 7,
};

struct Choice {
  int32_t comm_ctas;   // communication CTAs of the launch (0 with embedded copy warps)
  int32_t embedded;    // 1: one warp of every compute CTA runs the copy pipeline
  double makespan_us, compute_us, transfer_us;
};

struct Services {
  double tflops_per_sm;        // GEMM rate of one SM inside the kernel
  double cta_gbs;              // copy rate of one communication CTA
  double embedded_gbs;         // copy rate of one embedded copy warp (0: the mode has none)
  double embedded_compute;     // GEMM rate factor with the copy ring in place of the sixth stage
  double comm_model;           // measured / modelled time of the operator with communication CTAs
  double startup_us;
  double remote_cta;           // copy rate of a communication CTA over NVLink / its local rate
};

inline Services services(Kind kind) {
  const Calibration& c = kCalibrationB200;
  switch (kind) {
    case kLhsPullBf16: return {c.bf16_pair_tflops_per_sm, c.pull_cta_gbs, c.pull_embedded_gbs, c.embedded_compute_factor, c.comm_model_factor, c.startup_us, c.remote_cta_factor};
    case kLhsPullMx: return {c.mx_pair_tflops_per_sm, c.pull_cta_gbs, c.pull_embedded_gbs, c.embedded_compute_factor, c.comm_model_factor, c.startup_us, c.remote_cta_factor};
    case kGradPushBf16: return {c.bf16_pair_tflops_per_sm, c.push_cta_gbs, c.push_embedded_gbs, c.embedded_compute_factor, c.comm_model_factor, c.startup_us, 1.0};
    case kGradPullMx: return {c.mx_pair_tflops_per_sm, c.gradpull_cta_gbs, c.gradpull_embedded_gbs, c.embedded_compute_factor, c.comm_model_factor, c.startup_us, c.remote_cta_factor};
    case kQkvPushBf16: return {c.bf16_cta_tflops_per_sm, c.qkv_push_cta_gbs, 0.0, 1.0, c.comm_model_factor, c.startup_us, c.remote_cta_factor};
    case kQkvPushMx: return {c.mx_cta_tflops_per_sm, c.qkv_push_cta_gbs, 0.0, 1.0, c.comm_model_factor, c.startup_us, c.remote_cta_factor};
    default: return {c.grouped_pair_tflops_per_sm, c.dispatch_cta_gbs, 0.0, 1.0, c.comm_model_factor, c.startup_us, c.remote_cta_factor};
  }
}

// Makespan with `comm` communication CTAs (in units of `group` SMs: 2 for CTA pairs) that join the
// GEMM after their transfers: the same wave model the launch uses to place the join.
inline Choice score_comm(const Services& s, double flops, double bytes, int64_t tiles, int sm_count, int group,
                         int comm, double remote_share = 0.0) {
  const int64_t units = sm_count / group, comm_units = comm / group;
  const int64_t compute = tiles < units - comm_units ? tiles : units - comm_units;
  Choice out{comm, 0, 0.0, 0.0, 0.0};
  if (compute <= 0 || tiles <= 0) {
    out.makespan_us = 1.0e30;
    return out;
  }
  const double tau = flops / double(tiles) / (double(group) * s.tflops_per_sm * 1.0e6);  // us per tile and unit
  // bytes that cross NVLink move at the (lower) remote rate of a communication CTA (pulls: loads
  // wait for the round trip; pushes are posted stores and measured flat in the remote share)
  const double weighted = bytes * ((1.0 - remote_share) + remote_share / s.remote_cta);
  const double t_c = s.startup_us + weighted / (double(comm) * s.cta_gbs * 1.0e3);
  const int64_t all = compute + comm_units;
  double best = double((tiles + compute - 1) / compute) * tau;
  best = best > t_c + tau ? best : t_c + tau;  // the last tile cannot start before its rows are there
  for (int64_t w1 = 0; w1 * compute < tiles; ++w1) {
    const int64_t rest = tiles - w1 * compute, w2 = (rest + all - 1) / all;
    const double compute_side = double(w1 + w2) * tau, comm_side = t_c + double(w2) * tau;
    const double makespan = compute_side > comm_side ? compute_side : comm_side;
    if (makespan < best) best = makespan;
  }
  out.makespan_us = best * s.comm_model;
  out.compute_us = double((tiles + compute - 1) / compute) * tau;
  out.transfer_us = t_c;
  return out;
}

inline Choice score_embedded(const Services& s, double flops, double bytes, int64_t tiles, int sm_count, int group) {
  const int64_t units = sm_count / group;
  const double tau = flops / double(tiles) / (double(group) * s.tflops_per_sm * s.embedded_compute * 1.0e6);
  Choice out{0, 1, 0.0, 0.0, 0.0};
  out.compute_us = double((tiles + units - 1) / units) * tau;
  out.transfer_us = s.startup_us + bytes / (double(sm_count) * s.embedded_gbs * 1.0e3);
  out.makespan_us = out.compute_us > out.transfer_us + tau ? out.compute_us : out.transfer_us + tau;
  return out;
}

// explicit_comm > 0: that many communication CTAs, exactly (the plan only reports their score).
// explicit_comm == 0: Auto.  embedded_allowed: the launch can run embedded copy warps (geometry and
// kernel family permitting).  remote_share: fraction of the bytes that cross NVLink, (world - 1) /
// world for the all-to-all routes.
inline Choice choose(Kind kind, double flops, double bytes, int64_t tiles, int sm_count, int group, int explicit_comm,
                     bool embedded_allowed, double remote_share = 0.0) {
  const Services s = services(kind);
  if (explicit_comm > 0) return score_comm(s, flops, bytes, tiles, sm_count, group, explicit_comm, remote_share);
  Choice best{0, 0, 1.0e30, 0.0, 0.0};
  static const int kBudgets[] = {4, 8, 12, 16, 20, 24, 32, 40, 48};
  for (int comm : kBudgets) {
    if (comm % group != 0 || comm >= sm_count) continue;
    const Choice c = score_comm(s, flops, bytes, tiles, sm_count, group, comm, remote_share);
    if (c.makespan_us < best.makespan_us * (1.0 - 1.0e-9)) best = c;  // ties: the earlier (smaller) budget
  }
  if (embedded_allowed && s.embedded_gbs > 0.0) {
    // A communication budget has to be predicted clearly faster (10 %) than the embedded copy warps
    // to be taken.  That is the model's error: it reproduces its own BF16 calibration points to
    // -9 ... +2 %, and for the block-scaled output projection it put 8 communication CTAs 6.5 % ahead
    // of the embedded warps where they measured 3.4 % behind.  Wherever both were measured (BF16 and
    // MXFP8 pulls and pushes, 1 to 8 GPUs) the embedded warps won when the GEMM was the longer side,
    // and over NVLink communication CTAs lose more than the embedded warps do; a budget is taken
    // where the transfer is the longer side (narrow GEMMs), which the embedded warps cannot shorten.
    const Choice e = score_embedded(s, flops, bytes, tiles, sm_count, group);
    // The gradient push is the one transfer whose embedded variant loses over NVLink (measured: ahead
    // of 16 communication CTAs by 2 % on 2 GPUs, behind by 4.5 % on 4): beyond the calibrated share
    // of remote bytes it runs on communication CTAs, at least the calibrated number of them.
    const Calibration& c = kCalibrationB200;
    if (kind == kGradPushBf16 && remote_share > c.push_embedded_max_remote_share) {
      const int floor_ctas = int(c.push_remote_min_ctas);
      if (best.comm_ctas < floor_ctas && floor_ctas % group == 0 && floor_ctas < sm_count)
        best = score_comm(s, flops, bytes, tiles, sm_count, group, floor_ctas, remote_share);
      return best;
    }
    if (e.makespan_us * 0.90 <= best.makespan_us) best = e;
  }
  return best;
}

}  // namespace planner
}  // namespace fuse_b200
