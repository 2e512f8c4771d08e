// The backend translation unit a maintainer of the reference would add next to
// csrc/operators/sm103/entry.cu to run the hot path on libfuse_b200.so: every public free function
// of namespace fuse on that path, defined by forwarding to the C ABI.  The parameter records are
// layout-identical (tests/test_abi_layout.py), so they are passed through reinterpret_cast.
// tests/test_binding_compiles.py compiles this file against the reference's own headers: a
// signature that drifted from the reference's declaration fails to compile there.
#include <cstddef>
#include <cstdint>

#include "fuse/operators/primitives/a2a_gemm.h"
#include "fuse/operators/primitives/a2a_gemm_mxfp8.h"
#include "fuse/operators/primitives/gemm_a2a.h"
#include "fuse/operators/primitives/gemm_a2a_mxfp8.h"
#include "fuse/operators/primitives/grouped_gemm.h"
#include "fuse/operators/ulysses/oproj_backward.h"
#include "fuse/operators/ulysses/qkv_backward.h"
#include "fuse_b200.h"

namespace fuse {
namespace {
template <class To, class From>
const To* as(const From& record) {
  static_assert(sizeof(To) == sizeof(From), "record sizes differ");
  return reinterpret_cast<const To*>(&record);
}
inline cudaError_t status(int code) { return static_cast<cudaError_t>(code); }
inline fuse_stream stream_of(cudaStream_t stream) { return reinterpret_cast<fuse_stream>(stream); }
inline KernelTraits traits_of(const fuse_kernel_traits& t) {
  KernelTraits out{};
  out.block_m = t.block_m;
  out.block_n = t.block_n;
  out.block_k = t.block_k;
  out.threads = t.threads;
  out.dynamic_smem_bytes = t.dynamic_smem_bytes;
  return out;
}
}  // namespace

// ---- BF16 forward (primitives/gemm_a2a.h, primitives/a2a_gemm.h)
cudaError_t launch_gemm_a2a_cutlass(const GemmA2AParams& p, cudaStream_t s) {
  return status(fuse_launch_gemm_a2a_cutlass(as<fuse_gemm_a2a_params>(p), stream_of(s)));
}
cudaError_t launch_a2a_gemm_cutlass(const A2AGemmParams& p, cudaStream_t s) {
  return status(fuse_launch_a2a_gemm_cutlass(as<fuse_a2a_gemm_params>(p), stream_of(s)));
}
cudaError_t launch_batched_cutlass_reference(const GemmA2AParams& p, cudaStream_t s, int32_t reserved_comm_ctas) {
  return status(fuse_launch_batched_cutlass_reference(as<fuse_gemm_a2a_params>(p), stream_of(s), reserved_comm_ctas));
}
cudaError_t launch_a2a_gemm_cutlass_reference(const A2AGemmParams& p, cudaStream_t s, int32_t reserved_comm_ctas) {
  return status(fuse_launch_a2a_gemm_cutlass_reference(as<fuse_a2a_gemm_params>(p), stream_of(s), reserved_comm_ctas));
}
KernelTraits qkv_cutlass_kernel_traits(const GemmProblem& g) {
  fuse_kernel_traits t{};
  fuse_qkv_cutlass_kernel_traits(as<fuse_gemm_problem>(g), &t);
  return traits_of(t);
}
KernelTraits cutlass_kernel_traits() {
  fuse_kernel_traits t{};
  fuse_cutlass_kernel_traits(&t);
  return traits_of(t);
}
int64_t a2a_lhs_gemm_ready_elements(const GemmProblem& g, const UlyssesRoute& r) {
  return fuse_a2a_lhs_gemm_ready_elements(as<fuse_gemm_problem>(g), as<fuse_ulysses_route>(r));
}
int32_t recommended_gemm_a2a_comm_ctas(const GemmProblem& g, const UlyssesRoute& r) {
  return fuse_recommended_gemm_a2a_comm_ctas(as<fuse_gemm_problem>(g), as<fuse_ulysses_route>(r));
}
int32_t recommended_a2a_lhs_gemm_comm_ctas(const GemmProblem& g, const UlyssesRoute& r) {
  return fuse_recommended_a2a_lhs_gemm_comm_ctas(as<fuse_gemm_problem>(g), as<fuse_ulysses_route>(r));
}

// ---- BF16 backward (ulysses/qkv_backward.h, ulysses/oproj_backward.h)
cudaError_t launch_qkv_backward_data(const QkvBackwardDataParams& p, cudaStream_t s) {
  return status(fuse_launch_qkv_backward_data(as<fuse_qkv_backward_data_params>(p), stream_of(s)));
}
cudaError_t launch_qkv_backward_weight(const QkvBackwardWeightParams& p, cudaStream_t s) {
  return status(fuse_launch_qkv_backward_weight(as<fuse_qkv_backward_weight_params>(p), stream_of(s)));
}
cudaError_t launch_qkv_backward(const QkvBackwardParams& p, cudaStream_t s) {
  return status(fuse_launch_qkv_backward(as<fuse_qkv_backward_params>(p), stream_of(s)));
}
cudaError_t launch_oproj_backward_data(const OprojBackwardDataParams& p, cudaStream_t s) {
  return status(fuse_launch_oproj_backward_data(as<fuse_oproj_backward_data_params>(p), stream_of(s)));
}
cudaError_t launch_oproj_backward_weight(const OprojBackwardWeightParams& p, cudaStream_t s) {
  return status(fuse_launch_oproj_backward_weight(as<fuse_oproj_backward_weight_params>(p), stream_of(s)));
}
cudaError_t launch_oproj_backward(const OprojBackwardParams& p, cudaStream_t s) {
  return status(fuse_launch_oproj_backward(as<fuse_oproj_backward_params>(p), stream_of(s)));
}
int64_t qkv_backward_ready_elements(const QkvBackwardDataParams& p) {
  return fuse_qkv_backward_ready_elements(as<fuse_qkv_backward_data_params>(p));
}
int64_t oproj_backward_ready_elements(const OprojBackwardDataParams& p) {
  return fuse_oproj_backward_ready_elements(as<fuse_oproj_backward_data_params>(p));
}
int32_t recommended_qkv_backward_comm_ctas(const QkvBackwardDataParams& p) {
  return fuse_recommended_qkv_backward_comm_ctas(as<fuse_qkv_backward_data_params>(p));
}
int32_t recommended_oproj_backward_comm_ctas(const OprojBackwardDataParams& p) {
  return fuse_recommended_oproj_backward_comm_ctas(as<fuse_oproj_backward_data_params>(p));
}

// ---- MXFP8 forward (primitives/gemm_a2a_mxfp8.h, primitives/a2a_gemm_mxfp8.h)
KernelTraits mxfp8_qkv_cutlass_kernel_traits(int32_t epilogue_n) {
  fuse_kernel_traits t{};
  fuse_mxfp8_qkv_cutlass_kernel_traits(epilogue_n, &t);
  return traits_of(t);
}
KernelTraits mxfp8_oproj_cutlass_kernel_traits(int32_t epilogue_n, bool overlap_postnorm) {
  fuse_kernel_traits t{};
  fuse_mxfp8_oproj_cutlass_kernel_traits(epilogue_n, overlap_postnorm ? 1 : 0, &t);
  return traits_of(t);
}
cudaError_t gemm_a2a_mxfp8_activation_size(const GemmProblem& g, size_t* data_bytes, size_t* scale_bytes) {
  return status(fuse_gemm_a2a_mxfp8_activation_size(as<fuse_gemm_problem>(g), data_bytes, scale_bytes));
}
cudaError_t quantize_gemm_a2a_mxfp8_activation(const GemmProblem& g, const Bf16* source, const Mxfp8Activation& out,
                                               cudaStream_t s) {
  return status(fuse_quantize_gemm_a2a_mxfp8_activation(as<fuse_gemm_problem>(g), reinterpret_cast<const fuse_bf16*>(source),
                                                        as<fuse_mxfp8_activation>(out), stream_of(s)));
}
cudaError_t gemm_a2a_mxfp8_workspace_size(const GemmProblem& g, size_t* bytes) {
  return status(fuse_gemm_a2a_mxfp8_workspace_size(as<fuse_gemm_problem>(g), bytes));
}
cudaError_t launch_gemm_a2a_mxfp8_cutlass(const Mxfp8GemmA2AParams& p, cudaStream_t s) {
  return status(fuse_launch_gemm_a2a_mxfp8_cutlass(as<fuse_mxfp8_gemm_a2a_params>(p), stream_of(s)));
}
cudaError_t a2a_gemm_mxfp8_activation_size(const GemmProblem& g, const UlyssesRoute& r, size_t* data_bytes,
                                           size_t* scale_bytes) {
  return status(fuse_a2a_gemm_mxfp8_activation_size(as<fuse_gemm_problem>(g), as<fuse_ulysses_route>(r), data_bytes,
                                                    scale_bytes));
}
cudaError_t a2a_gemm_mxfp8_workspace_size(const GemmProblem& g, size_t* bytes) {
  return status(fuse_a2a_gemm_mxfp8_workspace_size(as<fuse_gemm_problem>(g), bytes));
}
cudaError_t a2a_gemm_mxfp8_workspace_size(const Mxfp8A2AGemmParams& p, size_t* bytes) {
  return status(fuse_a2a_gemm_mxfp8_workspace_size_for_params(as<fuse_mxfp8_a2a_gemm_params>(p), bytes));
}
cudaError_t a2a_gemm_mxfp8_staging_view(const Mxfp8A2AGemmParams& p, Mxfp8Activation* activation) {
  return status(fuse_a2a_gemm_mxfp8_staging_view(as<fuse_mxfp8_a2a_gemm_params>(p),
                                                 reinterpret_cast<fuse_mxfp8_activation*>(activation)));
}
cudaError_t launch_a2a_gemm_mxfp8_cutlass(const Mxfp8A2AGemmParams& p, cudaStream_t s) {
  return status(fuse_launch_a2a_gemm_mxfp8_cutlass(as<fuse_mxfp8_a2a_gemm_params>(p), stream_of(s)));
}

// ---- MXFP8 backward (ulysses/qkv_backward.h:252-283, ulysses/oproj_backward.h:222-237)
cudaError_t qkv_backward_mxfp8_data_workspace_size(const QkvBackwardDataParams& p, size_t* bytes) {
  return status(fuse_qkv_backward_mxfp8_data_workspace_size(as<fuse_qkv_backward_data_params>(p), bytes));
}
cudaError_t qkv_backward_mxfp8_weight_workspace_size(const QkvBackwardWeightParams& p, size_t* bytes) {
  return status(fuse_qkv_backward_mxfp8_weight_workspace_size(as<fuse_qkv_backward_weight_params>(p), bytes));
}
cudaError_t launch_qkv_backward_mxfp8_data(const Mxfp8QkvBackwardDataParams& p, cudaStream_t s) {
  return status(fuse_launch_qkv_backward_mxfp8_data(as<fuse_mxfp8_qkv_backward_data_params>(p), stream_of(s)));
}
cudaError_t launch_qkv_backward_mxfp8_weight(const Mxfp8QkvBackwardWeightParams& p, cudaStream_t s) {
  return status(fuse_launch_qkv_backward_mxfp8_weight(as<fuse_mxfp8_qkv_backward_weight_params>(p), stream_of(s)));
}
cudaError_t launch_qkv_backward_mxfp8(const Mxfp8QkvBackwardParams& p, cudaStream_t s) {
  return status(fuse_launch_qkv_backward_mxfp8(as<fuse_mxfp8_qkv_backward_params>(p), stream_of(s)));
}
cudaError_t oproj_backward_mxfp8_data_workspace_size(const OprojBackwardDataParams& p, size_t* bytes) {
  return status(fuse_oproj_backward_mxfp8_data_workspace_size(as<fuse_oproj_backward_data_params>(p), bytes));
}
cudaError_t oproj_backward_mxfp8_weight_workspace_size(const OprojBackwardWeightParams& p, size_t* bytes) {
  return status(fuse_oproj_backward_mxfp8_weight_workspace_size(as<fuse_oproj_backward_weight_params>(p), bytes));
}
cudaError_t launch_oproj_backward_mxfp8_data(const Mxfp8OprojBackwardDataParams& p, cudaStream_t s) {
  return status(fuse_launch_oproj_backward_mxfp8_data(as<fuse_mxfp8_oproj_backward_data_params>(p), stream_of(s)));
}
cudaError_t launch_oproj_backward_mxfp8_weight(const Mxfp8OprojBackwardWeightParams& p, cudaStream_t s) {
  return status(fuse_launch_oproj_backward_mxfp8_weight(as<fuse_mxfp8_oproj_backward_weight_params>(p), stream_of(s)));
}
cudaError_t launch_oproj_backward_mxfp8(const Mxfp8OprojBackwardParams& p, cudaStream_t s) {
  return status(fuse_launch_oproj_backward_mxfp8(as<fuse_mxfp8_oproj_backward_params>(p), stream_of(s)));
}

// ---- MoE (primitives/grouped_gemm.h:86-98); the plan is an opaque pointer on both sides
cudaError_t create_bf16_a2a_grouped_gemm(const Bf16GroupedGemmParams& p, Bf16GroupedGemmPlan** plan) {
  return status(fuse_create_bf16_a2a_grouped_gemm(as<fuse_bf16_grouped_gemm_params>(p),
                                                  reinterpret_cast<fuse_bf16_grouped_gemm_plan**>(plan)));
}
cudaError_t create_bf16_grouped_gemm_a2a(const Bf16GroupedGemmParams& p, Bf16GroupedGemmPlan** plan) {
  return status(fuse_create_bf16_grouped_gemm_a2a(as<fuse_bf16_grouped_gemm_params>(p),
                                                  reinterpret_cast<fuse_bf16_grouped_gemm_plan**>(plan)));
}
cudaError_t launch_bf16_grouped_gemm(Bf16GroupedGemmPlan* plan, cudaStream_t s) {
  return status(fuse_launch_bf16_grouped_gemm(reinterpret_cast<fuse_bf16_grouped_gemm_plan*>(plan), stream_of(s)));
}
cudaError_t destroy_bf16_grouped_gemm(Bf16GroupedGemmPlan* plan) {
  return status(fuse_destroy_bf16_grouped_gemm(reinterpret_cast<fuse_bf16_grouped_gemm_plan*>(plan)));
}
}  // namespace fuse
