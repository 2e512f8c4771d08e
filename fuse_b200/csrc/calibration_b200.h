// Calibration of the host planner, measured on one B200 by `python -m fuse_b200.calibrate`
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
};

constexpr Calibration kCalibrationB200 = {
    /* bf16_pair_tflops_per_sm    */ 10.75,
    /* mx_pair_tflops_per_sm      */ 18.48,
    /* bf16_cta_tflops_per_sm     */ 10.04,
    /* mx_cta_tflops_per_sm       */ 17.17,
    /* grouped_pair_tflops_per_sm */ 10.32,
    /* pull_cta_gbs               */ 40.71,
    /* pull_embedded_gbs          */ 7.58,
    /* push_cta_gbs               */ 41.4,
    /* push_embedded_gbs          */ 5.561,
    /* gradpull_cta_gbs           */ 41.29,
    /* gradpull_embedded_gbs      */ 10.23,
    /* qkv_push_cta_gbs           */ 40.71,
    /* dispatch_cta_gbs           */ 41.27,
    /* embedded_compute_factor    */ 0.8796,
    /* comm_model_factor          */ 1.049,
    /* startup_us                 */ 25,
};

}  // namespace planner
}  // namespace fuse_b200
