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
  // rate of a communication CTA whose bytes cross NVLink, relative to the local rate above
  double remote_cta_factor;
  // gradient push: the embedded copy warps are used up to this share of remote bytes, beyond it
  // communication CTAs, at least this many (measured on 2 and 4 GPUs)
  double push_embedded_max_remote_share, push_remote_min_ctas;
};

constexpr Calibration kCalibrationB200 = {
    /* bf16_pair_tflops_per_sm        */ 10.87,
    /* mx_pair_tflops_per_sm          */ 18.66,
    /* bf16_cta_tflops_per_sm         */ 10.07,
    /* mx_cta_tflops_per_sm           */ 17.24,
    /* grouped_pair_tflops_per_sm     */ 10.43,
    /* pull_cta_gbs                   */ 36.82,
    /* pull_embedded_gbs              */ 7.312,
    /* push_cta_gbs                   */ 40.5,
    /* push_embedded_gbs              */ 5.47,
    /* gradpull_cta_gbs               */ 42.77,
    /* gradpull_embedded_gbs          */ 10.23,
    /* qkv_push_cta_gbs               */ 36.82,
    /* dispatch_cta_gbs               */ 41.44,
    /* embedded_compute_factor        */ 0.9308,
    /* comm_model_factor              */ 0.9741,
    /* startup_us                     */ 25,
    /* remote_cta_factor              */ 0.3,
    /* push_embedded_max_remote_share */ 0.6,
    /* push_remote_min_ctas           */ 16,
};

}  // namespace planner
}  // namespace fuse_b200
