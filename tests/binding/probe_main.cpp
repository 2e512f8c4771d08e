// A caller written purely against the reference's C++ interface (its own headers and records,
// value-initialised), linked with the binding of sm100_entry.cpp and libfuse_b200.so.
// The calls below are refused during host-side validation, before any device is touched, so the
// program runs without a GPU: it proves that the reference's records reach the library intact.
#include <cstdio>

#include "fuse/operators/primitives/a2a_gemm.h"
#include "fuse/operators/primitives/gemm_a2a.h"
#include "fuse/operators/primitives/grouped_gemm.h"

int main() {
  fuse::GemmA2AParams qkv{};             // epoch == 0: invalid by the reference's own rule
  qkv.gemm.m = 256;
  qkv.gemm.n = 1024;
  qkv.gemm.k = 128;
  qkv.num_comm_ctas = 4;
  const int a = static_cast<int>(fuse::launch_gemm_a2a_cutlass(qkv, nullptr));
  fuse::A2AGemmParams oproj{};
  oproj.gemm.m = 256;
  oproj.gemm.n = 512;
  oproj.gemm.k = 512;
  oproj.epoch = 1;
  oproj.num_comm_ctas = -3;              // a negative budget
  const int b = static_cast<int>(fuse::launch_a2a_gemm_cutlass(oproj, nullptr));
  const fuse::KernelTraits traits = fuse::cutlass_kernel_traits();
  fuse::Bf16GroupedGemmPlan* plan = nullptr;
  fuse::Bf16GroupedGemmParams moe{};     // no experts: invalid
  const int c = static_cast<int>(fuse::create_bf16_a2a_grouped_gemm(moe, &plan));
  std::printf("%d %d %d %d %d\n", a, b, c, traits.block_m, traits.threads);
  return 0;
}
