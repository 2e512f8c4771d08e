// BF16 backward entry points.
//
//   QKV backward, data:   planar dQ,dK,dV --(head -> sequence all-to-all)--> dQKV[M,QKV];
//                         dX[M,H] = alpha * dQKV * Wqkv[QKV,H]        (NN: W is read as stored)
//   QKV backward, weight: dWqkv[QKV,H] = alpha * dQKV^T X + beta * dWqkv  (TN, local, no reduce)
//   OProj backward, data: dA[M,A] = alpha * dY[M,H] * Wo[H,A]          (NN), then
//                         dA --(sequence -> head all-to-all)--> peers' head-sharded gradients
//   OProj backward, weight: dWo[H,A] = alpha * dY^T A_saved + beta * dWo
//
// Interface and validation follow include/fuse/operators/ulysses/{qkv,oproj}_backward.h and
// csrc/operators/sm103/api/backward.cuh:67-93,121-329 of the reference.
#include "launch.cuh"

namespace fuse_b200 {
namespace {

using namespace launch;

// api/backward.cuh:67-76 (backward_shape_supported) + the tuning domain of :40-65.
template <class P>
bool shape_supported(const P& p) {
  return p.world_size > 0 && p.world_size <= FUSE_MAX_WORLD_SIZE && p.rank >= 0 &&
         p.rank < p.world_size && p.batch > 0 && p.local_tokens > 0 && p.local_tokens % p.batch == 0 &&
         p.hidden > 0 && p.hidden % 8 == 0 && p.q_heads > 0 && p.q_heads % p.world_size == 0 &&
         p.head_dim > 0 && p.head_dim % 64 == 0 &&
         int64_t(p.local_tokens) * p.world_size <= INT32_MAX &&
         int64_t(p.q_heads) * p.head_dim <= INT32_MAX &&
         (!p.causal_load_balanced || (p.local_tokens / p.batch) % 2 == 0) && std::isfinite(p.alpha) &&
         p.epoch > 0 &&
         (p.gemm_tuning.max_swizzle_size == 0 || p.gemm_tuning.max_swizzle_size == 1 ||
          p.gemm_tuning.max_swizzle_size == 2 || p.gemm_tuning.max_swizzle_size == 4 ||
          p.gemm_tuning.max_swizzle_size == 8) &&
         p.gemm_policy >= 0 && p.gemm_policy <= 6;
}

int block_n_of(int32_t policy, int n, const fuse_b200_options* options) {
  if (options && (options->block_n == 128 || options->block_n == 256)) return options->block_n;
  if (policy == 5) return 256;                 // kM128N256
  if (policy >= 1 && policy <= 4) return 128;  // finer reference tiles map to the 128-wide tile
  return launch::choose_block_n(n, nullptr);
}

cudaError_t qkv_backward_data(const fuse_qkv_backward_data_params& p, const fuse_b200_options* options,
                              cudaStream_t stream) {
  if (!shape_supported(p) || p.kv_heads <= 0 || p.q_heads % p.kv_heads != 0 ||
      p.kv_heads % p.world_size != 0 ||
      (int64_t(p.q_heads) + 2LL * p.kv_heads) * p.head_dim > INT32_MAX)
    return cudaErrorInvalidValue;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  const int m = p.local_tokens, n = p.hidden, k = (p.q_heads + 2 * p.kv_heads) * p.head_dim;
  // Auto: the planner's choice (embedded copy warps, or a communication budget); explicit: exactly that
  const planner::Choice plan =
      launch::plan_transfer(planner::kGradPushBf16, m, n, k, double(m) * k * 2.0, info.sm_count, p.num_comm_ctas < 0 ? 0 : p.num_comm_ctas,
                            true, p.world_size);
  const int comm = p.num_comm_ctas ? p.num_comm_ctas : (plan.comm_ctas ? plan.comm_ctas : fuse_recommended_qkv_backward_comm_ctas(&p));
  if (comm <= 0 || comm >= info.sm_count) return cudaErrorInvalidValue;
  if (!host::aligned16(p.grad_q) || !host::aligned16(p.grad_k) || !host::aligned16(p.grad_v) ||
      !host::aligned16(p.weight) || !host::aligned16(p.grad_input))
    return cudaErrorNotSupported;
  for (int peer = 0; peer < p.world_size; ++peer)
    if (!host::aligned16(p.peer_dqkv_staging[peer]) || !host::aligned4(p.peer_ready[peer]) ||
        !host::aligned4(p.peer_done_epoch[peer]))
      return cudaErrorNotSupported;

  const int block_n = block_n_of(p.gemm_policy, n, options);
  Operands maps;
  if ((status = encode_operand(&maps.a, p.peer_dqkv_staging[p.rank], m, k, k, false, kBlockM)) != cudaSuccess)
    return status;
  if ((status = encode_operand(&maps.b, p.weight, n, k, n, true, block_n)) != cudaSuccess) return status;

  FusedParams f{};
  launch::fill_core(&f, m, n, k, block_n, comm, p.alpha, 0.0f, p.grad_input, n,
                    p.gemm_tuning.along_m ? FUSE_RASTER_ALONG_M : FUSE_RASTER_ALONG_N,
                    p.gemm_tuning.max_swizzle_size ? p.gemm_tuning.max_swizzle_size : 1);
  f.ready = p.peer_ready[p.rank];
  f.flags = options ? options->flags : 0u;
  f.wait = host::make_wait(info, p.epoch, options ? options->wait_budget_ns : 0);
  copy_trace(&f, options);
  const int seq_local = p.local_tokens / p.batch;
  f.grad.world = p.world_size;
  f.grad.rank = p.rank;
  f.grad.seq_local = seq_local;
  f.grad.global_seq = seq_local * p.world_size;
  f.grad.m = m;
  f.grad.q_heads = p.q_heads;
  f.grad.kv_heads = p.kv_heads;
  f.grad.head_dim = p.head_dim;
  f.grad.causal = p.causal_load_balanced ? 1 : 0;
  f.grad.m_group = wave_m_group(f, info.sm_count);
  f.grad.grad[0] = p.grad_q;
  f.grad.grad[1] = p.grad_k;
  f.grad.grad[2] = p.grad_v;
  f.qkv.world = p.world_size;  // completion handshake
  f.qkv.rank = p.rank;
  for (int peer = 0; peer < p.world_size; ++peer) {
    f.grad.peer_staging[peer] = p.peer_dqkv_staging[peer];
    f.grad.peer_ready[peer] = p.peer_ready[peer];
    f.qkv.peer_done[peer] = p.peer_done_epoch[peer];
  }
  plan_join(&f, block_n, info.sm_count, double(m) * k * 2.0, false);
  // Tensor-copy push when a head is one 128-column box and 64-row boxes never straddle a
  // sequence block; otherwise the register (16-byte) push.
  const int row_block = p.causal_load_balanced ? seq_local / 2 : seq_local;
  if (p.head_dim == 128 && row_block % 64 == 0 && !(options && (options->flags & FUSE_B200_VECTOR_PULL))) {
    GradPushMaps push{};
    bool encoded = true;
    const fuse_bf16* planes[3] = {p.grad_q, p.grad_k, p.grad_v};
    const int heads[3] = {p.q_heads, p.kv_heads, p.kv_heads};
    const uint64_t rows_global = uint64_t(p.batch) * uint64_t(seq_local) * uint64_t(p.world_size);
    for (int s = 0; s < 3 && encoded; ++s)
      encoded = encode_copy_map(&push.plane[s], planes[s], 2, rows_global, uint64_t(heads[s] / p.world_size) * 128, 64, 128) ==
                cudaSuccess;
    for (int peer = 0; peer < p.world_size && encoded; ++peer)
      encoded = encode_copy_map(&push.staging[peer], p.peer_dqkv_staging[peer], 2, uint64_t(m), uint64_t(k), 64, 128) ==
                cudaSuccess;
    if (encoded && block_n == 256 && comm % 2 == 0 && info.sm_count % 2 == 0 && !vector_epilogue_requested(options) &&
        launch::pair_tiles_requested()) {
      // CTA pairs: whole pairs of communication CTAs, 256-row tiles
      FusedParams pf = f;
      pf.grad.m_group = 2 * launch::wave_m_group_pairs(pf, info.sm_count);
      // no communication CTAs at all: one warp of every compute CTA pushes (FUSE_B200_EMBEDDED_PULL=0:
      // communication CTAs)
      if (launch::embedded_copy_selected(p.num_comm_ctas, plan))
        return launch::launch_pair_kernel<kModeHeadGate, GradPushMaps, false, false, true, true>(
            maps, maps.a, maps.a, push, pf, p.gemm_tuning.max_swizzle_size ? p.gemm_tuning.max_swizzle_size : 1, info, stream,
            0.0);
      return launch::launch_pair_kernel<kModeHeadGate, GradPushMaps, false, false, true>(
          maps, maps.a, maps.a, push, pf, p.gemm_tuning.max_swizzle_size ? p.gemm_tuning.max_swizzle_size : 1, info, stream,
          double(m) * k * 2.0);
    }
    if (encoded)
      return launch_mode<kModeHeadGate, false, true, false, GradPushMaps>(maps, push, f, block_n, info, stream,
                                                                          !vector_epilogue_requested(options));
  }
  StoreMaps stores{};
  return launch_mode<kModeHeadGate, false, true>(maps, stores, f, block_n, info, stream,
                                                 !vector_epilogue_requested(options));
}

cudaError_t oproj_backward_data(const fuse_oproj_backward_data_params& p,
                                const fuse_b200_options* options, cudaStream_t stream) {
  if (!shape_supported(p)) return cudaErrorInvalidValue;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  // (the default route is the epilogue push, which needs no communication CTA; the budget only
  // matters when the caller asks for the communication-CTA route)
  const int comm = p.num_comm_ctas ? p.num_comm_ctas : fuse_recommended_oproj_backward_comm_ctas(&p);
  if (comm <= 0 || comm >= info.sm_count) return cudaErrorInvalidValue;
  if (!host::aligned16(p.grad_output) || !host::aligned16(p.weight) ||
      !host::aligned16(p.local_grad_attention))
    return cudaErrorNotSupported;
  for (int peer = 0; peer < p.world_size; ++peer)
    if (!host::aligned16(p.peer_grad_attention[peer]) || !host::aligned4(p.peer_done_epoch[peer]))
      return cudaErrorNotSupported;

  const int m = p.local_tokens, n = p.q_heads * p.head_dim, k = p.hidden;
  const int block_n = block_n_of(p.gemm_policy, n, options);
  Operands maps;
  if ((status = encode_operand(&maps.a, p.grad_output, m, k, k, false, kBlockM)) != cudaSuccess) return status;
  if ((status = encode_operand(&maps.b, p.weight, n, k, n, true, block_n)) != cudaSuccess) return status;

  // Route from communication CTAs only when asked for (and a `ready` array exists); the default
  // is the epilogue push of every compute CTA.
  const bool comm_route =
      options != nullptr && (options->flags & FUSE_B200_QKV_ROUTE_COMM_CTAS) && host::aligned4(p.ready);
  FusedParams f{};
  launch::fill_core(&f, m, n, k, block_n, comm_route ? comm : 0, p.alpha, 0.0f, p.local_grad_attention, n,
                    p.gemm_tuning.along_m ? FUSE_RASTER_ALONG_M : FUSE_RASTER_ALONG_N,
                    p.gemm_tuning.max_swizzle_size ? p.gemm_tuning.max_swizzle_size : 1);
  f.ready = p.ready;
  f.flags = options ? options->flags : 0u;
  f.wait = host::make_wait(info, p.epoch, options ? options->wait_budget_ns : 0);
  copy_trace(&f, options);
  const int seq_local = p.local_tokens / p.batch;
  f.qkv.world = p.world_size;
  f.qkv.rank = p.rank;
  f.qkv.batch = p.batch;
  f.qkv.seq_local = seq_local;
  f.qkv.global_seq = seq_local * p.world_size;
  f.qkv.q_heads = p.q_heads;
  f.qkv.kv_heads = 0;  // head-only route: one planar tensor per destination
  f.qkv.head_dim = p.head_dim;
  f.qkv.causal = p.causal_load_balanced ? 1 : 0;
  for (int peer = 0; peer < p.world_size; ++peer) {
    f.qkv.peer_output[peer] = p.peer_grad_attention[peer];
    f.qkv.peer_done[peer] = p.peer_done_epoch[peer];
  }
  StoreMaps stores{};
  if (comm_route) return launch_mode<kModeQkvPush, false, true>(maps, stores, f, block_n, info, stream, false);
  // Tensor-store push: 128-row tiles must land on consecutive destination rows.
  const int row_block = p.causal_load_balanced ? seq_local / 2 : seq_local;
  bool tma = !vector_epilogue_requested(options) && row_block % kBlockM == 0;
  if (tma)
    tma = encode_peer_store_maps(&stores, p.peer_grad_attention, p.world_size,
                                 uint64_t(p.batch) * uint64_t(f.qkv.global_seq),
                                 int64_t(p.q_heads) / p.world_size * p.head_dim, 0);
  if (tma && block_n == 256 && info.sm_count % 2 == 0 && launch::pair_tiles_requested()) {
    Operands pair_maps = maps;
    if (encode_operand(&pair_maps.a, p.grad_output, m, k, k, false, kBlockM) == cudaSuccess)
      return launch::launch_pair_kernel<kModeQkvDirect, StoreMaps, false, false, true>(
          pair_maps, maps.a, maps.a, stores, f, p.gemm_tuning.max_swizzle_size ? p.gemm_tuning.max_swizzle_size : 1, info,
          stream, 0.0);
  }
  return launch_mode<kModeQkvDirect, false, true>(maps, stores, f, block_n, info, stream, tma);
}

// api/backward.cuh:252-268 (backward_weight_impl): D[m,n] = alpha * A^T B + beta * D with
// A stored [k, m] and B stored [k, n] (k = tokens), on the whole device.
cudaError_t weight_gradient(int m, int n, int k, const fuse_bf16* a, const fuse_bf16* b, fuse_bf16* d,
                            float alpha, float beta, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || k <= 0 || a == nullptr || b == nullptr || d == nullptr ||
      !std::isfinite(alpha) || !std::isfinite(beta))
    return cudaErrorInvalidValue;
  if (m % 8 != 0 || n % 8 != 0 || !host::aligned16(a) || !host::aligned16(b) || !host::aligned16(d))
    return cudaErrorNotSupported;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  const int block_n = launch::choose_block_n(n, nullptr);
  Operands maps;
  if ((status = encode_operand(&maps.a, a, m, k, m, true, kBlockM)) != cudaSuccess) return status;
  if ((status = encode_operand(&maps.b, b, n, k, n, true, block_n)) != cudaSuccess) return status;
  FusedParams f{};
  launch::fill_core(&f, m, n, k, block_n, 0, alpha, beta, d, n, FUSE_RASTER_ALONG_M, 8);
  f.wait = host::make_wait(info, 1, 0);
  StoreMaps stores{};
  if (block_n == 256 && beta == 0.0f && info.sm_count % 2 == 0 && launch::pair_tiles_requested())
    return launch::launch_pair_kernel<kModePlain, StoreMaps, false, true, true>(maps, maps.a, maps.a, stores, f, 8, info,
                                                                                stream, 0.0);
  return launch_mode<kModePlain, true, true>(maps, stores, f, block_n, info, stream, beta == 0.0f);
}

}  // namespace
}  // namespace fuse_b200

extern "C" {

using namespace fuse_b200;

int fuse_launch_qkv_backward_data_ex(const fuse_qkv_backward_data_params* p, const fuse_b200_options* o,
                                     fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  return int(qkv_backward_data(*p, o, reinterpret_cast<cudaStream_t>(s)));
}
int fuse_launch_qkv_backward_data(const fuse_qkv_backward_data_params* p, fuse_stream s) {
  return fuse_launch_qkv_backward_data_ex(p, nullptr, s);
}
int fuse_launch_qkv_backward_weight(const fuse_qkv_backward_weight_params* p, fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  const int64_t n = (p->q_heads + 2LL * p->kv_heads) * p->head_dim;
  if (n <= 0 || n > INT32_MAX) return int(cudaErrorInvalidValue);
  return int(weight_gradient(int(n), p->hidden, p->local_tokens, p->dqkv_staging, p->saved_input,
                             p->grad_weight, p->alpha, p->beta, reinterpret_cast<cudaStream_t>(s)));
}
int fuse_launch_qkv_backward(const fuse_qkv_backward_params* p, fuse_stream s) {
  if (p == nullptr || (p->weight_mode != 0 && p->weight_mode != 1)) return int(cudaErrorInvalidValue);
  const int status = fuse_launch_qkv_backward_data(&p->data, s);
  return status == 0 && p->weight_mode == 0 ? fuse_launch_qkv_backward_weight(&p->weight, s) : status;
}

int fuse_launch_oproj_backward_data_ex(const fuse_oproj_backward_data_params* p,
                                       const fuse_b200_options* o, fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  return int(oproj_backward_data(*p, o, reinterpret_cast<cudaStream_t>(s)));
}
int fuse_launch_oproj_backward_data(const fuse_oproj_backward_data_params* p, fuse_stream s) {
  return fuse_launch_oproj_backward_data_ex(p, nullptr, s);
}
int fuse_launch_oproj_backward_weight(const fuse_oproj_backward_weight_params* p, fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  const int64_t n = int64_t(p->q_heads) * p->head_dim;
  if (n <= 0 || n > INT32_MAX) return int(cudaErrorInvalidValue);
  return int(weight_gradient(p->hidden, int(n), p->local_tokens, p->grad_output, p->saved_attention,
                             p->grad_weight, p->alpha, p->beta, reinterpret_cast<cudaStream_t>(s)));
}
int fuse_launch_oproj_backward(const fuse_oproj_backward_params* p, fuse_stream s) {
  if (p == nullptr || (p->weight_mode != 0 && p->weight_mode != 1)) return int(cudaErrorInvalidValue);
  const int status = fuse_launch_oproj_backward_data(&p->data, s);
  return status == 0 && p->weight_mode == 0 ? fuse_launch_oproj_backward_weight(&p->weight, s) : status;
}

int64_t fuse_qkv_backward_ready_elements(const fuse_qkv_backward_data_params* p) {
  if (p == nullptr || p->local_tokens <= 0 || p->q_heads <= 0 || p->kv_heads <= 0) return 0;
  return int64_t(host::ceil_div(p->local_tokens, kBlockM)) * (p->q_heads + 2LL * p->kv_heads) *
         FUSE_READY_FLAG_STRIDE;
}
int64_t fuse_oproj_backward_ready_elements(const fuse_oproj_backward_data_params* p) {
  if (p == nullptr) return 0;
  const int64_t n = int64_t(p->q_heads) * p->head_dim;
  if (p->local_tokens <= 0 || n <= 0 || n > INT32_MAX) return 0;
  // sized for the finest publication tile (128 columns) so that every tile choice fits
  return int64_t(host::ceil_div(p->local_tokens, kBlockM)) * host::ceil_div(int(n), 128) *
         FUSE_READY_FLAG_STRIDE;
}
// The planner's best communication budget for the operator run with communication CTAs.
int32_t fuse_recommended_qkv_backward_comm_ctas(const fuse_qkv_backward_data_params* p) {
  if (p == nullptr || p->local_tokens <= 0 || p->hidden <= 0) return 0;
  const int64_t k = (int64_t(p->q_heads) + 2 * p->kv_heads) * p->head_dim;
  return launch::plan_transfer(planner::kGradPushBf16, p->local_tokens, p->hidden, k, double(p->local_tokens) * k * 2.0, 148, 0,
                               false)
      .comm_ctas;
}
int32_t fuse_recommended_oproj_backward_comm_ctas(const fuse_oproj_backward_data_params* p) {
  if (p == nullptr || p->local_tokens <= 0 || p->hidden <= 0) return 0;
  const int64_t n = int64_t(p->q_heads) * p->head_dim;
  const int64_t tiles = ((int64_t(p->local_tokens) + 127) / 128) * ((n + 255) / 256);
  return planner::choose(planner::kQkvPushBf16, 2.0 * double(p->local_tokens) * n * p->hidden,
                         double(p->local_tokens) * n * 2.0, tiles, 148, 1, 0, false)
      .comm_ctas;
}

}  // extern "C"
