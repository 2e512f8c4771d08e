// MXFP8 backward entry points (straight-through: every operand orientation is re-quantised along
// its own K axis from its BF16 master, FP8 bytes and scales are never transposed).
//
//   QKV data:    W[QKV,H] -> transpose+quantise -> [H,QKV];  owners' prequantised planar dQ,dK,dV
//                (+ BF16 masters) --pull--> packed lhs [M,QKV] (+ BF16 staging);  dX = lhs W
//   QKV weight:  staging[M,QKV] -> [QKV,M], X[M,H] -> [H,M] (both quantised along M);
//                dW = alpha lhs rhs^T + beta dW
//   OProj data:  Wo[H,A] -> [A,H];  dA = dY_q Wo  (block-scaled), routed sequence -> head
//   OProj weight: dY[M,H] -> [H,M], A[M,A] -> [A,M];  dWo = alpha ... + beta dWo
//
// Interface: include/fuse/operators/ulysses/{qkv,oproj}_backward.h:186-283 of the reference;
// kernel sequence: csrc/operators/sm103/api/backward_mxfp8.cuh:113-497.
#include "launch.cuh"

extern "C" int fuse_b200_quantize_mxfp8_transposed(const fuse_bf16* source, int64_t row_stride, int32_t rows,
                                                   int32_t cols, uint8_t* data, uint8_t* scales, fuse_stream stream);

namespace fuse_b200 {
namespace {

using namespace launch;

size_t align256(size_t n) { return (n + 255) & ~size_t{255}; }
size_t scale_bytes(int64_t rows, int64_t k) { return size_t((rows + 127) / 128) * size_t((k + 127) / 128) * 512; }

struct Quantised {
  uint8_t* data;
  uint8_t* scales;
};
// Carves one [rows, k] E4M3 operand + scales out of `cursor` (NULL cursor: size only).
Quantised carve(uint8_t*& cursor, size_t& total, int64_t rows, int64_t k) {
  Quantised q{cursor, nullptr};
  const size_t data = align256(size_t(rows) * size_t(k)), scales = align256(scale_bytes(rows, k));
  if (cursor != nullptr) {
    q.scales = cursor + data;
    cursor += data + scales;
  }
  total += data + scales;
  return q;
}

bool workspace_ok(const void* workspace, size_t have, size_t need) {
  return workspace != nullptr && reinterpret_cast<uintptr_t>(workspace) % 256 == 0 && have >= need;
}

cudaError_t transpose_quantise(const fuse_bf16* source, int64_t stride, int rows, int cols, const Quantised& out,
                               cudaStream_t stream) {
  return cudaError_t(fuse_b200_quantize_mxfp8_transposed(source, stride, rows, cols, out.data, out.scales,
                                                         reinterpret_cast<fuse_stream>(stream)));
}

// D[m,n] = alpha * A_q[m,k] B_q[n,k]^T + beta * D on the whole device.
cudaError_t mx_gemm(const Quantised& a, const Quantised& b, fuse_bf16* d, int m, int n, int k, float alpha,
                    float beta, int max_swizzle, bool along_m, cudaStream_t stream) {
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  const int block_n = launch::choose_block_n(n, nullptr);
  Operands maps;
  if ((status = encode_operand_u8(&maps.a, a.data, m, k, k, kBlockM)) != cudaSuccess) return status;
  if ((status = encode_operand_u8(&maps.b, b.data, n, k, k, block_n)) != cudaSuccess) return status;
  FusedParams f{};
  launch::fill_core(&f, m, n, k, block_n, 0, alpha, beta, d, n, along_m ? FUSE_RASTER_ALONG_M : FUSE_RASTER_ALONG_N,
                    max_swizzle ? max_swizzle : 8);
  f.sfa = a.scales;
  f.sfb = b.scales;
  f.k_atoms = k / 128;
  f.wait = host::make_wait(info, 1, 0);
  StoreMaps stores{};
  if (block_n == 256 && beta == 0.0f && k % 128 == 0 && info.sm_count % 2 == 0 && launch::pair_tiles_requested()) {
    // CTA pairs: B boxed by half tiles, scale storage read through tensor maps
    Operands pair_maps = maps;
    CUtensorMap sfa_map, sfb_map;
    if (encode_operand_u8(&pair_maps.b, b.data, n, k, k, launch::kPairMxBRows) == cudaSuccess &&
        launch::encode_scale_atoms(&sfa_map, a.scales, m, k) == cudaSuccess &&
        launch::encode_scale_atoms(&sfb_map, b.scales, n, k) == cudaSuccess)
      return launch::launch_pair_kernel<kModePlain, StoreMaps, true>(pair_maps, sfa_map, sfb_map, stores, f,
                                                                     max_swizzle ? max_swizzle : 8, info, stream, 0.0);
  }
  return launch_mode<kModePlain, false, false, true>(maps, stores, f, block_n, info, stream, beta == 0.0f);
}

// dW[m_out, n_out] = alpha * A^T B + beta * dW with A stored [tokens, m_out], B stored [tokens, n_out].
cudaError_t mx_weight_gradient(const fuse_bf16* a, int m_out, const fuse_bf16* b, int n_out, int tokens,
                               fuse_bf16* d, float alpha, float beta, const fuse_backward_gemm_tuning& tuning,
                               void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (a == nullptr || b == nullptr || d == nullptr || m_out <= 0 || n_out <= 0 || tokens <= 0 ||
      !std::isfinite(alpha) || !std::isfinite(beta))
    return cudaErrorInvalidValue;
  if (tokens % 128 != 0 || m_out % 8 != 0 || n_out % 8 != 0) return cudaErrorNotSupported;
  uint8_t* cursor = static_cast<uint8_t*>(workspace);
  size_t need = 0;
  const Quantised qa = carve(cursor, need, m_out, tokens), qb = carve(cursor, need, n_out, tokens);
  if (!workspace_ok(workspace, workspace_bytes, need)) return cudaErrorInvalidValue;
  cudaError_t status = transpose_quantise(a, m_out, tokens, m_out, qa, stream);
  if (status != cudaSuccess) return status;
  if ((status = transpose_quantise(b, n_out, tokens, n_out, qb, stream)) != cudaSuccess) return status;
  return mx_gemm(qa, qb, d, m_out, n_out, tokens, alpha, beta, tuning.max_swizzle_size, tuning.along_m != 0, stream);
}

template <class P>
bool shape_supported(const P& p) {
  return p.world_size > 0 && p.world_size <= FUSE_MAX_WORLD_SIZE && p.rank >= 0 && p.rank < p.world_size &&
         p.batch > 0 && p.local_tokens > 0 && p.local_tokens % p.batch == 0 && p.hidden > 0 && p.q_heads > 0 &&
         p.q_heads % p.world_size == 0 && p.head_dim == 128 /* api/backward_mxfp8.cuh:52 */ &&
         (!p.causal_load_balanced || (p.local_tokens / p.batch) % 2 == 0) && std::isfinite(p.alpha) && p.epoch > 0;
}

cudaError_t qkv_data(const fuse_mxfp8_qkv_backward_data_params& mp, const fuse_b200_options* options,
                     cudaStream_t stream) {
  const fuse_qkv_backward_data_params& p = mp.projection;
  if (!shape_supported(p) || p.kv_heads <= 0 || p.q_heads % p.kv_heads != 0 || p.kv_heads % p.world_size != 0 ||
      p.num_comm_ctas < 0)
    return cudaErrorInvalidValue;
  const int seq_local = p.local_tokens / p.batch;
  const int row_block = p.causal_load_balanced ? seq_local / 2 : seq_local;
  const int m = p.local_tokens, n = p.hidden, k = (p.q_heads + 2 * p.kv_heads) * p.head_dim;
  if (row_block % 128 != 0 || n % 8 != 0) return cudaErrorNotSupported;  // whole scale atoms per row group
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  if (p.num_comm_ctas >= info.sm_count) return cudaErrorInvalidValue;
  // Auto: the planner's choice (embedded copy warps, or a communication budget); explicit: exactly that
  const planner::Choice plan = launch::plan_transfer(planner::kGradPullMx, m, n, k, double(m) * k * (3.0 + 1.0 / 32),
                                                     info.sm_count, p.num_comm_ctas, true, p.world_size);
  const int num_comm_ctas = p.num_comm_ctas ? p.num_comm_ctas : (plan.comm_ctas ? plan.comm_ctas : 16);
  uint8_t* cursor = static_cast<uint8_t*>(mp.workspace);
  size_t need = 0;
  const Quantised wq = carve(cursor, need, n, k), lhs = carve(cursor, need, m, k);
  if (!workspace_ok(mp.workspace, mp.workspace_bytes, need)) return cudaErrorInvalidValue;
  if (!host::aligned16(p.weight) || !host::aligned16(p.grad_input) || !host::aligned16(p.peer_dqkv_staging[p.rank]) ||
      !host::aligned4(p.peer_ready[p.rank]))
    return cudaErrorInvalidValue;
  for (int peer = 0; peer < p.world_size; ++peer) {
    const fuse_mxfp8_qkv_backward_input& in = mp.peer_input[peer];
    if (!host::aligned16(in.grad_q.data) || !host::aligned16(in.grad_k.data) || !host::aligned16(in.grad_v.data) ||
        !host::aligned16(in.grad_q.scales) || !host::aligned16(in.grad_k.scales) ||
        !host::aligned16(in.grad_v.scales) || !host::aligned16(in.master_q) || !host::aligned16(in.master_k) ||
        !host::aligned16(in.master_v) || !host::aligned4(p.peer_done_epoch[peer]))
      return cudaErrorInvalidValue;
  }
  // kernel 1: W[QKV,H] -> [H,QKV] quantised along QKV
  if ((status = transpose_quantise(p.weight, n, k, n, wq, stream)) != cudaSuccess) return status;
  // kernel 2: fused pull + block-scaled dX GEMM
  const int block_n = launch::choose_block_n(n, options);
  Operands maps;
  if ((status = encode_operand_u8(&maps.a, lhs.data, m, k, k, kBlockM)) != cudaSuccess) return status;
  if ((status = encode_operand_u8(&maps.b, wq.data, n, k, k, block_n)) != cudaSuccess) return status;
  FusedParams f{};
  launch::fill_core(&f, m, n, k, block_n, num_comm_ctas, p.alpha, 0.0f, p.grad_input, n,
                    p.gemm_tuning.along_m ? FUSE_RASTER_ALONG_M : FUSE_RASTER_ALONG_N,
                    p.gemm_tuning.max_swizzle_size ? p.gemm_tuning.max_swizzle_size : 1);
  f.sfa = lhs.scales;
  f.sfb = wq.scales;
  f.k_atoms = k / 128;
  f.ready = p.peer_ready[p.rank];
  f.flags = options ? options->flags : 0u;
  f.wait = host::make_wait(info, p.epoch, options ? options->wait_budget_ns : 0);
  copy_trace(&f, options);
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
  f.grad.lhs_bytes = lhs.data;
  f.grad.lhs_scales = lhs.scales;
  f.grad.master_staging = p.peer_dqkv_staging[p.rank];
  f.qkv.world = p.world_size;
  f.qkv.rank = p.rank;
  for (int peer = 0; peer < p.world_size; ++peer) {
    const fuse_mxfp8_qkv_backward_input& in = mp.peer_input[peer];
    const fuse_mxfp8_activation* planes[3] = {&in.grad_q, &in.grad_k, &in.grad_v};
    const fuse_bf16* masters[3] = {in.master_q, in.master_k, in.master_v};
    for (int s = 0; s < 3; ++s) {
      f.grad.peer_bytes[peer][s] = planes[s]->data;
      f.grad.peer_scales[peer][s] = planes[s]->scales;
      f.grad.peer_master[peer][s] = masters[s];
    }
    f.qkv.peer_done[peer] = p.peer_done_epoch[peer];
  }
  plan_join(&f, block_n, info.sm_count, double(m) * k * (3.0 + 1.0 / 32), true);
  if (!(options && (options->flags & FUSE_B200_VECTOR_PULL))) {
    GradPullMaps pull{};
    const uint64_t rows_global = uint64_t(p.batch) * uint64_t(seq_local) * uint64_t(p.world_size);
    const int heads[3] = {p.q_heads, p.kv_heads, p.kv_heads};
    bool encoded = encode_copy_map(&pull.lhs, lhs.data, 1, uint64_t(m), uint64_t(k), 128, 128) == cudaSuccess &&
                   encode_copy_map(&pull.master, p.peer_dqkv_staging[p.rank], 2, uint64_t(m), uint64_t(k), 64, 128) ==
                       cudaSuccess;
    for (int peer = 0; peer < p.world_size && encoded; ++peer)
      for (int s = 0; s < 3 && encoded; ++s) {
        const uint64_t plane_width = uint64_t(heads[s] / p.world_size) * 128;
        encoded = encode_copy_map(&pull.bytes[peer][s], f.grad.peer_bytes[peer][s], 1, rows_global, plane_width, 128, 128) ==
                      cudaSuccess &&
                  encode_copy_map(&pull.masters[peer][s], f.grad.peer_master[peer][s], 2, rows_global, plane_width, 64, 128) ==
                      cudaSuccess;
      }
    if (encoded && block_n == 256 && num_comm_ctas % 2 == 0 && info.sm_count % 2 == 0 &&
        !vector_epilogue_requested(options) && launch::pair_tiles_requested()) {
      // CTA pairs: whole pairs of communication CTAs, 256-row tiles
      Operands pair_maps = maps;
      CUtensorMap sfa_map, sfb_map;
      FusedParams pf = f;
      pf.grad.m_group = 2 * launch::wave_m_group_pairs(pf, info.sm_count, launch::kPairMxBlockN);
      if (encode_operand_u8(&pair_maps.b, wq.data, n, k, k, launch::kPairMxBRows) == cudaSuccess &&
          launch::encode_scale_atoms(&sfa_map, f.sfa, m, k) == cudaSuccess &&
          launch::encode_scale_atoms(&sfb_map, f.sfb, n, k) == cudaSuccess)
      {
        if (launch::embedded_copy_selected(p.num_comm_ctas, plan))  // one warp of every compute CTA pulls
          return launch::launch_pair_kernel<kModeGradPull, GradPullMaps, true, false, false, true>(
              pair_maps, sfa_map, sfb_map, pull, pf, p.gemm_tuning.max_swizzle_size ? p.gemm_tuning.max_swizzle_size : 1,
              info, stream, 0.0);
        return launch::launch_pair_kernel<kModeGradPull, GradPullMaps, true>(
            pair_maps, sfa_map, sfb_map, pull, pf, p.gemm_tuning.max_swizzle_size ? p.gemm_tuning.max_swizzle_size : 1, info,
            stream, double(m) * k * (3.0 + 1.0 / 32));
      }
    }
    if (encoded)
      return launch_mode<kModeGradPull, false, false, true, GradPullMaps>(maps, pull, f, block_n, info, stream,
                                                                          !vector_epilogue_requested(options));
  }
  StoreMaps stores{};
  return launch_mode<kModeGradPull, false, false, true>(maps, stores, f, block_n, info, stream,
                                                        !vector_epilogue_requested(options));
}

cudaError_t oproj_data(const fuse_mxfp8_oproj_backward_data_params& mp, const fuse_b200_options* options,
                       cudaStream_t stream) {
  const fuse_oproj_backward_data_params& p = mp.projection;
  // (the route is the epilogue push: no communication CTA runs, whatever the budget says)
  if (!shape_supported(p) || p.num_comm_ctas < 0) return cudaErrorInvalidValue;
  const int m = p.local_tokens, n = p.q_heads * p.head_dim, k = p.hidden;
  if (k % 128 != 0) return cudaErrorNotSupported;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  if (p.num_comm_ctas >= info.sm_count) return cudaErrorInvalidValue;
  uint8_t* cursor = static_cast<uint8_t*>(mp.workspace);
  size_t need = 0;
  const Quantised wq = carve(cursor, need, n, k);
  if (!workspace_ok(mp.workspace, mp.workspace_bytes, need)) return cudaErrorInvalidValue;
  if (!host::aligned16(mp.grad_output.data) || !host::aligned16(mp.grad_output.scales) ||
      mp.grad_output.data_bytes < size_t(m) * size_t(k) || mp.grad_output.scale_bytes < scale_bytes(m, k) ||
      !host::aligned16(p.weight) || !host::aligned16(p.local_grad_attention))
    return cudaErrorInvalidValue;
  for (int peer = 0; peer < p.world_size; ++peer)
    if (!host::aligned16(p.peer_grad_attention[peer]) || !host::aligned4(p.peer_done_epoch[peer]))
      return cudaErrorInvalidValue;
  // kernel 1: Wo[H,A] -> [A,H] quantised along H
  if ((status = transpose_quantise(p.weight, n, k, n, wq, stream)) != cudaSuccess) return status;
  // kernel 2: block-scaled dA GEMM whose epilogue pushes sequence -> head
  const int block_n = launch::choose_block_n(n, options);
  Operands maps;
  if ((status = encode_operand_u8(&maps.a, mp.grad_output.data, m, k, k, kBlockM)) != cudaSuccess) return status;
  if ((status = encode_operand_u8(&maps.b, wq.data, n, k, k, block_n)) != cudaSuccess) return status;
  const int seq_local = p.local_tokens / p.batch;
  FusedParams f{};
  launch::fill_core(&f, m, n, k, block_n, 0, p.alpha, 0.0f, p.local_grad_attention, n,
                    p.gemm_tuning.along_m ? FUSE_RASTER_ALONG_M : FUSE_RASTER_ALONG_N,
                    p.gemm_tuning.max_swizzle_size ? p.gemm_tuning.max_swizzle_size : 1);
  f.sfa = mp.grad_output.scales;
  f.sfb = wq.scales;
  f.k_atoms = k / 128;
  f.flags = options ? options->flags : 0u;
  f.wait = host::make_wait(info, p.epoch, options ? options->wait_budget_ns : 0);
  copy_trace(&f, options);
  f.qkv.world = p.world_size;
  f.qkv.rank = p.rank;
  f.qkv.batch = p.batch;
  f.qkv.seq_local = seq_local;
  f.qkv.global_seq = seq_local * p.world_size;
  f.qkv.q_heads = p.q_heads;
  f.qkv.kv_heads = 0;
  f.qkv.head_dim = p.head_dim;
  f.qkv.causal = p.causal_load_balanced ? 1 : 0;
  for (int peer = 0; peer < p.world_size; ++peer) {
    f.qkv.peer_output[peer] = p.peer_grad_attention[peer];
    f.qkv.peer_done[peer] = p.peer_done_epoch[peer];
  }
  StoreMaps stores{};
  const int row_block = p.causal_load_balanced ? seq_local / 2 : seq_local;
  bool tma = !vector_epilogue_requested(options) && row_block % kBlockM == 0;
  if (tma)
    tma = encode_peer_store_maps(&stores, p.peer_grad_attention, p.world_size,
                                 uint64_t(p.batch) * uint64_t(f.qkv.global_seq),
                                 int64_t(p.q_heads) / p.world_size * p.head_dim, 0);
  if (tma && block_n == 256 && k % 128 == 0 && info.sm_count % 2 == 0 && launch::pair_tiles_requested()) {
    Operands pair_maps = maps;
    CUtensorMap sfa_map, sfb_map;
    if (encode_operand_u8(&pair_maps.b, wq.data, n, k, k, launch::kPairMxBRows) == cudaSuccess &&
        launch::encode_scale_atoms(&sfa_map, f.sfa, m, k) == cudaSuccess &&
        launch::encode_scale_atoms(&sfb_map, f.sfb, n, k) == cudaSuccess)
      return launch::launch_pair_kernel<kModeQkvDirect, StoreMaps, true>(
          pair_maps, sfa_map, sfb_map, stores, f, p.gemm_tuning.max_swizzle_size ? p.gemm_tuning.max_swizzle_size : 1, info,
          stream, 0.0);
  }
  return launch_mode<kModeQkvDirect, false, false, true>(maps, stores, f, block_n, info, stream, tma);
}

size_t data_workspace(int64_t m, int64_t n, int64_t k, bool with_lhs) {
  uint8_t* none = nullptr;
  size_t need = 0;
  carve(none, need, n, k);
  if (with_lhs) carve(none, need, m, k);
  return need;
}

}  // namespace
}  // namespace fuse_b200

extern "C" {

using namespace fuse_b200;

int fuse_qkv_backward_mxfp8_data_workspace_size(const fuse_qkv_backward_data_params* p, size_t* bytes) {
  if (p == nullptr || bytes == nullptr || p->local_tokens <= 0 || p->hidden <= 0) return int(cudaErrorInvalidValue);
  *bytes = data_workspace(p->local_tokens, p->hidden, (p->q_heads + 2LL * p->kv_heads) * p->head_dim, true);
  return 0;
}
int fuse_qkv_backward_mxfp8_weight_workspace_size(const fuse_qkv_backward_weight_params* p, size_t* bytes) {
  if (p == nullptr || bytes == nullptr || p->local_tokens <= 0 || p->hidden <= 0) return int(cudaErrorInvalidValue);
  *bytes = data_workspace(p->hidden, (p->q_heads + 2LL * p->kv_heads) * p->head_dim, p->local_tokens, true);
  return 0;
}
int fuse_oproj_backward_mxfp8_data_workspace_size(const fuse_oproj_backward_data_params* p, size_t* bytes) {
  if (p == nullptr || bytes == nullptr || p->hidden <= 0) return int(cudaErrorInvalidValue);
  *bytes = data_workspace(0, int64_t(p->q_heads) * p->head_dim, p->hidden, false);
  return 0;
}
int fuse_oproj_backward_mxfp8_weight_workspace_size(const fuse_oproj_backward_weight_params* p, size_t* bytes) {
  if (p == nullptr || bytes == nullptr || p->local_tokens <= 0 || p->hidden <= 0) return int(cudaErrorInvalidValue);
  *bytes = data_workspace(int64_t(p->q_heads) * p->head_dim, p->hidden, p->local_tokens, true);
  return 0;
}

int fuse_launch_qkv_backward_mxfp8_data_ex(const fuse_mxfp8_qkv_backward_data_params* p, const fuse_b200_options* o,
                                           fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  return int(qkv_data(*p, o, reinterpret_cast<cudaStream_t>(s)));
}
int fuse_launch_qkv_backward_mxfp8_data(const fuse_mxfp8_qkv_backward_data_params* p, fuse_stream s) {
  return fuse_launch_qkv_backward_mxfp8_data_ex(p, nullptr, s);
}
int fuse_launch_qkv_backward_mxfp8_weight(const fuse_mxfp8_qkv_backward_weight_params* p, fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  const fuse_qkv_backward_weight_params& w = p->projection;
  const int64_t n = (w.q_heads + 2LL * w.kv_heads) * w.head_dim;
  if (n <= 0 || n > INT32_MAX) return int(cudaErrorInvalidValue);
  return int(mx_weight_gradient(w.dqkv_staging, int(n), w.saved_input, w.hidden, w.local_tokens, w.grad_weight,
                                w.alpha, w.beta, p->gemm_tuning, p->workspace, p->workspace_bytes,
                                reinterpret_cast<cudaStream_t>(s)));
}
int fuse_launch_qkv_backward_mxfp8(const fuse_mxfp8_qkv_backward_params* p, fuse_stream s) {
  if (p == nullptr || (p->weight_mode != 0 && p->weight_mode != 1)) return int(cudaErrorInvalidValue);
  const int status = fuse_launch_qkv_backward_mxfp8_data(&p->data, s);
  return status == 0 && p->weight_mode == 0 ? fuse_launch_qkv_backward_mxfp8_weight(&p->weight, s) : status;
}

int fuse_launch_oproj_backward_mxfp8_data_ex(const fuse_mxfp8_oproj_backward_data_params* p,
                                             const fuse_b200_options* o, fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  return int(oproj_data(*p, o, reinterpret_cast<cudaStream_t>(s)));
}
int fuse_launch_oproj_backward_mxfp8_data(const fuse_mxfp8_oproj_backward_data_params* p, fuse_stream s) {
  return fuse_launch_oproj_backward_mxfp8_data_ex(p, nullptr, s);
}
int fuse_launch_oproj_backward_mxfp8_weight(const fuse_mxfp8_oproj_backward_weight_params* p, fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  const fuse_oproj_backward_weight_params& w = p->projection;
  const int64_t n = int64_t(w.q_heads) * w.head_dim;
  if (n <= 0 || n > INT32_MAX) return int(cudaErrorInvalidValue);
  return int(mx_weight_gradient(w.grad_output, w.hidden, w.saved_attention, int(n), w.local_tokens, w.grad_weight,
                                w.alpha, w.beta, p->gemm_tuning, p->workspace, p->workspace_bytes,
                                reinterpret_cast<cudaStream_t>(s)));
}
int fuse_launch_oproj_backward_mxfp8(const fuse_mxfp8_oproj_backward_params* p, fuse_stream s) {
  if (p == nullptr || (p->weight_mode != 0 && p->weight_mode != 1)) return int(cudaErrorInvalidValue);
  const int status = fuse_launch_oproj_backward_mxfp8_data(&p->data, s);
  return status == 0 && p->weight_mode == 0 ? fuse_launch_oproj_backward_mxfp8_weight(&p->weight, s) : status;
}

}  // extern "C"
