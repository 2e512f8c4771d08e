// MoE grouped GEMMs (dispatch -> expert FC1; expert FC2 -> combine): plan object and entry points.
// Interface: include/fuse/operators/primitives/grouped_gemm.h:10-100 of the reference;
// plan lifetime and validation follow csrc/operators/sm103/api/grouped.cuh:58-428.
#include <new>
#include <vector>

#include "grouped.cuh"
#include "launch.cuh"

struct fuse_bf16_grouped_gemm_plan {
  fuse_b200::GroupedParams params{};
  void* metadata = nullptr;  // one private device allocation: tensor maps, flags, epoch, prefix
  int block_n = 256;
  bool pair = false;  // CTA pairs (policy.mma_sm_count == 2)
  bool combine = false;  // GEMM -> scatter to the token owners (no communication CTAs)
  int grid = 0;
  int device = -1;
};

namespace fuse_b200 {
namespace {

using namespace launch;

size_t align256(size_t n) { return (n + 255) & ~size_t{255}; }

// combine: the plan of the FC2 -> scatter direction (peer_output instead of peer_input; every CTA
// computes, so policy.num_comm_ctas only has to be a valid count)
cudaError_t create_plan(const fuse_bf16_grouped_gemm_params& p, bool combine, fuse_bf16_grouped_gemm_plan** out) {
  if (out == nullptr) return cudaErrorInvalidValue;
  *out = nullptr;
  if (p.lhs == nullptr || p.weight_nt == nullptr || p.output == nullptr || p.row_offsets == nullptr ||
      p.source == nullptr || p.experts <= 0 || p.n <= 0 || p.k <= 0 || p.expert_row_capacity <= 0 ||
      p.world_size <= 0 || p.world_size > FUSE_MAX_WORLD_SIZE || p.rank < 0 || p.rank >= p.world_size ||
      p.topk <= 0 || p.policy.num_comm_ctas < 0 || p.policy.num_compute_ctas <= 0)
    return cudaErrorInvalidValue;
  for (int r = 0; r < p.world_size; ++r)
    if (!host::aligned16(combine ? static_cast<const void*>(p.peer_output[r]) : static_cast<const void*>(p.peer_input[r])) ||
        (combine && p.peer_output[r] == nullptr) || !host::aligned4(p.peer_started[r]) || !host::aligned4(p.peer_done[r]))
      return cudaErrorInvalidValue;
  // geometry outside this implementation's domain
  if (p.n % 8 != 0 || p.k % 8 != 0 || (p.policy.tile_n != 128 && p.policy.tile_n != 256) ||
      (p.policy.mma_sm_count != 1 && p.policy.mma_sm_count != 2) || p.policy.swap_ab ||
      (p.dispatch_buffer_rows != 0 && p.dispatch_buffer_rows != p.expert_row_capacity))
    return cudaErrorNotSupported;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  if (p.policy.num_comm_ctas >= info.sm_count) return cudaErrorInvalidValue;
  // policy.num_comm_ctas == 0: Auto.  Row counts live on the device, so the plan is made for slabs
  // half full (its budget stays fixed over replays, as a captured launch needs).
  int dispatch_ctas = p.policy.num_comm_ctas;
  // Auto on CTA pairs: no communication CTA at all -- one thread of every compute CTA pulls (its ring
  // is the epilogue staging the dispatch kernel does not use, so the GEMM keeps all six stages).  A
  // pull over NVLink is bounded by what ONE SM may have in flight, so 148 SMs pulling a little each
  // move far more than 20 CTAs pulling flat out.  FUSE_B200_EMBEDDED_PULL=0 keeps communication CTAs.
  const bool embedded_possible = !combine && p.policy.mma_sm_count == 2 && p.policy.tile_n == 256 && info.sm_count % 2 == 0;
  bool embedded = dispatch_ctas == 0 && embedded_possible;
  if (const char* text = std::getenv("FUSE_B200_EMBEDDED_PULL")) {  // 1 / 0: force / forbid, whatever the budget says
    embedded = std::atoi(text) != 0 && embedded_possible;
    if (embedded) dispatch_ctas = 0;
  }
  if (dispatch_ctas == 0 && !combine && !embedded) {
    const double rows = 0.5 * double(p.experts) * p.expert_row_capacity;
    const int group = p.policy.mma_sm_count == 2 ? 2 : 1;
    const int64_t tiles = int64_t(rows / (128 * group) + 1) * host::ceil_div(p.n, p.policy.tile_n);
    dispatch_ctas = planner::choose(planner::kDispatchBf16, 2.0 * rows * p.n * p.k, rows * p.k * 2.0, tiles, info.sm_count,
                                    group, 0, false, double(p.world_size - 1) / double(p.world_size))
                        .comm_ctas;
  }

  std::vector<void*> lhs(p.experts), weights(p.experts);
  if ((status = cudaMemcpy(lhs.data(), p.lhs, sizeof(void*) * p.experts, cudaMemcpyDeviceToHost)) != cudaSuccess)
    return status;
  if ((status = cudaMemcpy(weights.data(), p.weight_nt, sizeof(void*) * p.experts, cudaMemcpyDeviceToHost)) !=
      cudaSuccess)
    return status;

  auto* plan = new (std::nothrow) fuse_bf16_grouped_gemm_plan;
  if (plan == nullptr) return cudaErrorMemoryAllocation;
  plan->device = info.device;
  plan->block_n = p.policy.tile_n;
  // mma_sm_count 2: CTA pairs (256 x 256 tiles); needs the 256-wide tile, whole pairs of
  // communication and compute CTAs, and is otherwise outside this implementation's domain.
  plan->pair = p.policy.mma_sm_count == 2;
  plan->combine = combine;
  if (plan->pair && (p.policy.tile_n != 256 || (!combine && dispatch_ctas % 2 != 0) || info.sm_count % 2 != 0)) {
    delete plan;
    return cudaErrorNotSupported;
  }
  const int cap_tiles = host::ceil_div(p.expert_row_capacity, kBlockM);
  const size_t maps_bytes = align256(sizeof(CUtensorMap) * size_t(p.experts));
  const size_t ready_bytes = align256(size_t(p.experts) * cap_tiles * FUSE_READY_FLAG_STRIDE * sizeof(uint32_t));
  const size_t prefix_bytes = align256(sizeof(int32_t) * size_t(p.experts + 1));
  const size_t total = 2 * maps_bytes + ready_bytes + 256 + prefix_bytes;
  if ((status = cudaMalloc(&plan->metadata, total)) != cudaSuccess) {
    delete plan;
    return status;
  }
  auto fail = [&](cudaError_t error) {
    cudaFree(plan->metadata);
    delete plan;
    return error;
  };
  if ((status = cudaMemset(plan->metadata, 0, total)) != cudaSuccess) return fail(status);
  std::vector<CUtensorMap> maps_a(p.experts), maps_b(p.experts);
  for (int e = 0; e < p.experts; ++e) {
    if (!host::aligned16(lhs[e]) || !host::aligned16(weights[e])) return fail(cudaErrorInvalidValue);
    if ((status = encode_operand(&maps_a[e], lhs[e], p.expert_row_capacity, p.k, p.k, false, kBlockM)) != cudaSuccess)
      return fail(status);
    if ((status = encode_operand(&maps_b[e], weights[e], p.n, p.k, p.k, false, plan->pair ? 128 : plan->block_n)) !=
        cudaSuccess)
      return fail(status);
  }
  uint8_t* base = static_cast<uint8_t*>(plan->metadata);
  if ((status = cudaMemcpy(base, maps_a.data(), sizeof(CUtensorMap) * p.experts, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (status = cudaMemcpy(base + maps_bytes, maps_b.data(), sizeof(CUtensorMap) * p.experts,
                           cudaMemcpyHostToDevice)) != cudaSuccess)
    return fail(status);

  GroupedParams& g = plan->params;
  g.experts = p.experts;
  g.n = p.n;
  g.k = p.k;
  g.capacity = p.expert_row_capacity;
  g.lhs_rows = p.expert_row_capacity;
  g.rank = p.rank;
  g.world = p.world_size;
  g.n_tiles = host::ceil_div(p.n, plan->block_n);
  g.cap_tiles = cap_tiles;
  g.tile_m = plan->pair ? 2 * kBlockM : kBlockM;
  g.num_comm_ctas = combine ? 0 : dispatch_ctas;
  g.embedded = embedded ? 1 : 0;
  g.topk = p.topk;
  g.maps_a = reinterpret_cast<const CUtensorMap*>(base);
  g.maps_b = reinterpret_cast<const CUtensorMap*>(base + maps_bytes);
  g.lhs = reinterpret_cast<uint16_t* const*>(p.lhs);
  g.output = reinterpret_cast<uint16_t* const*>(p.output);
  g.row_offsets = p.row_offsets;
  g.source = reinterpret_cast<const GroupedTokenSource*>(p.source);
  g.ready = reinterpret_cast<uint32_t*>(base + 2 * maps_bytes);
  g.epoch_word = reinterpret_cast<uint32_t*>(base + 2 * maps_bytes + ready_bytes);
  g.tile_prefix = reinterpret_cast<int32_t*>(base + 2 * maps_bytes + ready_bytes + 256);
  for (int r = 0; r < p.world_size; ++r) {
    g.peer_input[r] = p.peer_input[r];
    g.peer_output[r] = reinterpret_cast<uint16_t*>(p.peer_output[r]);
    g.peer_started[r] = p.peer_started[r];
    g.peer_done[r] = p.peer_done[r];
  }
  const int compute = combine ? info.sm_count
                              : (p.policy.num_compute_ctas < info.sm_count - dispatch_ctas && p.policy.num_comm_ctas != 0
                                     ? p.policy.num_compute_ctas
                                     : info.sm_count - dispatch_ctas);
  plan->grid = g.num_comm_ctas + (plan->pair ? compute / 2 * 2 : compute);
  g.wait.status = info.status;
  if ((status = cudaDeviceSynchronize()) != cudaSuccess) return fail(status);
  *out = plan;
  return cudaSuccess;
}

cudaError_t launch_plan(fuse_bf16_grouped_gemm_plan* plan, const fuse_b200_options* options, cudaStream_t stream) {
  if (plan == nullptr) return cudaErrorInvalidValue;
  GroupedParams g = plan->params;
  g.flags = options ? options->flags : 0u;
  g.wait.launch_id = host::next_launch_id();
  g.wait.epoch = 0;  // read from the device epoch word
  g.wait.budget_ns = options && options->wait_budget_ns ? options->wait_budget_ns : host::default_wait_budget_ns();
  grouped_prepare_kernel<<<1, 256, 0, stream>>>(g);
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess) return status;
  host::count_launch();
  if (plan->pair)
    return plan->combine ? host::launch_kernel(grouped_pair_kernel<true>, plan->grid, kThreads,
                                               PairLayoutT<false>::kDynamicBytes, true, stream, g)
                         : host::launch_kernel(grouped_pair_kernel<false>, plan->grid, kThreads,
                                               PairLayoutT<false>::kDynamicBytes, true, stream, g);
  if (plan->block_n == 256) {
    using Layout = SmemLayout<256, 4, false>;
    return plan->combine ? host::launch_kernel(grouped_gemm_kernel<256, 4, true>, plan->grid, kThreads,
                                               Layout::kDynamicBytes, true, stream, g)
                         : host::launch_kernel(grouped_gemm_kernel<256, 4, false>, plan->grid, kThreads,
                                               Layout::kDynamicBytes, true, stream, g);
  }
  using Layout = SmemLayout<128, 6, false>;
  return plan->combine ? host::launch_kernel(grouped_gemm_kernel<128, 6, true>, plan->grid, kThreads, Layout::kDynamicBytes,
                                             true, stream, g)
                       : host::launch_kernel(grouped_gemm_kernel<128, 6, false>, plan->grid, kThreads, Layout::kDynamicBytes,
                                             true, stream, g);
}

}  // namespace
}  // namespace fuse_b200

extern "C" {

int fuse_create_bf16_a2a_grouped_gemm(const fuse_bf16_grouped_gemm_params* params,
                                      fuse_bf16_grouped_gemm_plan** plan) {
  if (params == nullptr) return int(cudaErrorInvalidValue);
  return int(fuse_b200::create_plan(*params, false, plan));
}
int fuse_create_bf16_grouped_gemm_a2a(const fuse_bf16_grouped_gemm_params* params,
                                      fuse_bf16_grouped_gemm_plan** plan) {
  if (params == nullptr) return int(cudaErrorInvalidValue);
  return int(fuse_b200::create_plan(*params, true, plan));
}
int fuse_launch_bf16_grouped_gemm(fuse_bf16_grouped_gemm_plan* plan, fuse_stream stream) {
  return int(fuse_b200::launch_plan(plan, nullptr, reinterpret_cast<cudaStream_t>(stream)));
}
int fuse_launch_bf16_grouped_gemm_ex(fuse_bf16_grouped_gemm_plan* plan, const fuse_b200_options* options,
                                     fuse_stream stream) {
  return int(fuse_b200::launch_plan(plan, options, reinterpret_cast<cudaStream_t>(stream)));
}
int fuse_destroy_bf16_grouped_gemm(fuse_bf16_grouped_gemm_plan* plan) {
  if (plan == nullptr) return int(cudaErrorInvalidValue);
  const cudaError_t status = cudaFree(plan->metadata);
  delete plan;
  return int(status);
}

}  // extern "C"
