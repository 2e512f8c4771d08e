// BF16 forward entry points: QKV projection -> sequence-to-head all-to-all, and
// head-to-sequence all-to-all -> output projection.  Validation follows the reference's
// launch path (csrc/operators/sm103/detail/launch.cuh:364-591, detail/gemm_a2a.cuh:237-299,
// detail/gemm.cuh:53-70): the same conditions produce the same error codes.
#include <cmath>
#include <cstring>

#include "launch.cuh"

namespace fuse_b200 {
namespace {

using namespace launch;

// detail/gemm.cuh:53-70 (supported_problem): row-major A[M,K], B[N,K], D[M,N], 16-byte rows.
bool supported_problem(const fuse_gemm_problem& g) {
  const int64_t lda = packed_or(g.stride_a.row, g.k), ldb = packed_or(g.stride_b.row, g.k),
                ldd = packed_or(g.stride_d.row, g.n);
  return g.m > 0 && g.n > 0 && g.k > 0 && g.l == 1 && !g.transpose_a && !g.transpose_b &&
         g.input_dtype == FUSE_DTYPE_BF16 && g.weight_dtype == FUSE_DTYPE_BF16 &&
         g.output_dtype == FUSE_DTYPE_BF16 && (g.stride_a.column < 0 || g.stride_a.column == 1) &&
         (g.stride_b.column < 0 || g.stride_b.column == 1) &&
         (g.stride_d.column < 0 || g.stride_d.column == 1) && lda >= g.k && lda % 8 == 0 &&
         ldb >= g.k && ldb % 8 == 0 && ldd >= g.n && ldd % 8 == 0 &&
         (g.max_swizzle_size == 1 || g.max_swizzle_size == 2 || g.max_swizzle_size == 4 ||
          g.max_swizzle_size == 8) &&
         (g.raster == FUSE_RASTER_HEURISTIC || g.raster == FUSE_RASTER_ALONG_M ||
          g.raster == FUSE_RASTER_ALONG_N);
}

cudaError_t encode_operands(Operands* maps, const void* a, int64_t lda, const void* b, int64_t ldb,
                            const fuse_gemm_problem& g, int block_n) {
  cudaError_t status = encode_operand(&maps->a, a, g.m, g.k, lda, false, kBlockM);
  if (status != cudaSuccess) return status;
  return encode_operand(&maps->b, b, g.n, g.k, ldb, false, block_n);
}

void fill_core(FusedParams* p, const fuse_gemm_problem& g, int block_n, int num_comm_ctas,
               float alpha, void* d, int default_raster) {
  launch::fill_core(p, g.m, g.n, g.k, block_n, num_comm_ctas, alpha, 0.0f, d, packed_or(g.stride_d.row, g.n),
                    g.raster == FUSE_RASTER_HEURISTIC ? default_raster : g.raster, g.max_swizzle_size);
}

int choose_block_n(const fuse_gemm_problem& g, const fuse_b200_options* options) {
  return launch::choose_block_n(g.n, options);
}

// How the routed output leaves the SM: from communication CTAs that copy published tiles
// (the reference's structure, `num_comm_ctas` of them), or straight from the GEMM epilogue of
// every compute CTA ("direct", all SMs compute).  Option flag first, then the environment
// variable FUSE_B200_QKV_ROUTE = comm | direct (read on every launch, like the reference's
// FUSE_QKV_GEMM_POLICY: csrc/operators/sm103/detail/launch.cuh:165-195).
bool qkv_direct_push(const fuse_b200_options* options) {
  if (options != nullptr && (options->flags & FUSE_B200_QKV_ROUTE_COMM_CTAS)) return false;
  if (options != nullptr && (options->flags & FUSE_B200_QKV_ROUTE_DIRECT)) return true;
  const char* text = std::getenv("FUSE_B200_QKV_ROUTE");
  if (text != nullptr && std::strcmp(text, "comm") == 0) return false;
  if (text != nullptr && std::strcmp(text, "direct") == 0) return true;
  return false;
}

// BF16 operands of the pair kernel: A boxes of 128 rows, B boxes of 128 rows (half a tile).
template <int kMode, class Maps>
cudaError_t launch_pair(const void* a, int64_t lda, const void* b, int64_t ldb, const fuse_gemm_problem& g,
                        Maps& stores, const FusedParams& k, const DeviceInfo& info, cudaStream_t stream,
                        double comm_bytes = 0.0) {
  Operands maps;
  cudaError_t status = encode_operand(&maps.a, a, g.m, g.k, lda, false, kBlockM);
  if (status != cudaSuccess) return status;
  if ((status = encode_operand(&maps.b, b, g.n, g.k, ldb, false, PairLayout::kBlockN / 2)) != cudaSuccess) return status;
  return launch::launch_pair_kernel<kMode, Maps, false>(maps, maps.a, maps.a, stores, k, g.max_swizzle_size, info, stream,
                                                        comm_bytes);
}

// detail/gemm_a2a.cuh:237-299 (can_implement) for the plain QKV GQA pack route.
cudaError_t check_qkv_route(const fuse_gemm_a2a_params& p) {
  const fuse_ulysses_route& r = p.route;
  if (r.world_size <= 0 || r.world_size > FUSE_MAX_WORLD_SIZE || r.rank < 0 ||
      r.rank >= r.world_size || r.batch <= 0 || r.seq_local <= 0 || r.global_seq <= 0 ||
      r.q_heads <= 0 || r.kv_heads <= 0 || r.head_dim <= 0 || r.kind != FUSE_ROUTE_QKV_GQA_PACK ||
      r.direction != FUSE_ROUTE_FORWARD || r.channel_count != 1 || r.cyclic_peer_order ||
      r.packed_source_row != nullptr || r.packed_row_granularity != 0 ||
      (p.completion_epoch != nullptr && !r.defer_v_a2a) || r.q_heads % r.kv_heads != 0 ||
      r.q_heads % r.world_size != 0 || r.kv_heads % r.world_size != 0 || r.head_dim % 8 != 0)
    return cudaErrorNotSupported;
  // Offline-interleaved weights: refused with the N raster, as the reference refuses it
  // (csrc/operators/sm103/detail/gemm_a2a.cuh:258-259).
  if (r.qkv_peer_interleaved && p.gemm.raster == FUSE_RASTER_ALONG_N) return cudaErrorNotSupported;
  if (p.completion_epoch != nullptr && !host::aligned4(p.completion_epoch)) return cudaErrorInvalidValue;
  if (int64_t(r.seq_local) * r.world_size != r.global_seq ||
      int64_t(r.batch) * r.seq_local != p.gemm.m ||
      int64_t(r.batch) * r.global_seq > INT32_MAX ||
      (int64_t(r.q_heads) + 2 * int64_t(r.kv_heads)) * r.head_dim != p.gemm.n)
    return cudaErrorNotSupported;
  if (!host::aligned16(p.lhs) || !host::aligned16(p.rhs_nt) || !host::aligned16(p.local_output) ||
      !host::aligned4(p.ready))
    return cudaErrorNotSupported;
  for (int peer = 0; peer < r.world_size; ++peer)
    if (!host::aligned16(p.peer_output[peer]) || !host::aligned4(p.peer_route_done_epoch[peer]))
      return cudaErrorNotSupported;
  return cudaSuccess;
}

cudaError_t qkv_forward(const fuse_gemm_a2a_params& p, const fuse_b200_options* options,
                        cudaStream_t stream) {
  // The reference's entry point rejects num_comm_ctas <= 0 (detail/launch.cuh:508-511) and so does the
  // entry point of the same name here; Auto (0) is accepted through the _ex entry point.
  if (!supported_problem(p.gemm) || !std::isfinite(p.alpha) || p.epoch == 0 || p.num_comm_ctas < 0 ||
      (p.num_comm_ctas == 0 && options == nullptr))
    return cudaErrorInvalidValue;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  if (p.num_comm_ctas >= info.sm_count) return cudaErrorInvalidValue;
  if ((status = check_qkv_route(p)) != cudaSuccess) return status;
  // Auto (num_comm_ctas == 0): the epilogue push, which needs no communication CTA at all, unless
  // the caller asked for the communication-CTA route; that route then gets the planned budget.
  const bool auto_plan = p.num_comm_ctas == 0;
  const bool direct = qkv_direct_push(options) ||
                      (auto_plan && !(options != nullptr && (options->flags & FUSE_B200_QKV_ROUTE_COMM_CTAS)));
  const int num_comm_ctas = auto_plan ? fuse_recommended_gemm_a2a_comm_ctas(&p.gemm, &p.route) : p.num_comm_ctas;

  const int block_n = choose_block_n(p.gemm, options);
  Operands maps;
  status = encode_operands(&maps, p.lhs, packed_or(p.gemm.stride_a.row, p.gemm.k), p.rhs_nt,
                           packed_or(p.gemm.stride_b.row, p.gemm.k), p.gemm, block_n);
  if (status != cudaSuccess) return status;

  FusedParams k{};
  fill_core(&k, p.gemm, block_n, direct ? 0 : num_comm_ctas, p.alpha, p.local_output,
            FUSE_RASTER_ALONG_M);
  k.ready = p.ready;
  k.flags = options ? options->flags : 0u;
  k.wait = host::make_wait(info, p.epoch, options ? options->wait_budget_ns : 0);
  // ranks start at different column tiles so that their pushes go to different owners
  k.order.n_shift = int32_t(int64_t(p.route.rank) * k.order.n_tiles / p.route.world_size);
  k.qkv.world = p.route.world_size;
  k.qkv.rank = p.route.rank;
  k.qkv.batch = p.route.batch;
  k.qkv.seq_local = p.route.seq_local;
  k.qkv.global_seq = p.route.global_seq;
  k.qkv.q_heads = p.route.q_heads;
  k.qkv.kv_heads = p.route.kv_heads;
  k.qkv.head_dim = p.route.head_dim;
  k.qkv.defer_v = p.route.defer_v_a2a ? 1 : 0;
  k.qkv.interleaved = p.route.qkv_peer_interleaved ? 1 : 0;
  k.qkv.completion_epoch = p.route.defer_v_a2a ? p.completion_epoch : nullptr;
  for (int peer = 0; peer < p.route.world_size; ++peer) {
    k.qkv.peer_output[peer] = p.peer_output[peer];
    k.qkv.peer_done[peer] = p.peer_route_done_epoch[peer];
  }
  StoreMaps stores{};
  if (!direct) return launch_mode<kModeQkvPush>(maps, stores, k, block_n, info, stream, false);
  // The tensor-store push needs every 64-column block inside one head and every 128-row tile
  // on consecutive destination rows; other shapes push with 16-byte stores from registers.
  const fuse_ulysses_route& r = p.route;
  bool tma = !vector_epilogue_requested(options) && r.head_dim % 64 == 0 && r.seq_local % kBlockM == 0;
  if (tma) {
    // (defer_v: one map per destination over its [rows, q_local + kv_local] tensor)
    const int64_t q_local = int64_t(r.q_heads) / r.world_size * r.head_dim;
    const int64_t kv_local = int64_t(r.kv_heads) / r.world_size * r.head_dim;
    tma = encode_peer_store_maps(&stores, p.peer_output, r.world_size, uint64_t(r.batch) * uint64_t(r.global_seq),
                                 r.defer_v_a2a ? q_local + kv_local : q_local, r.defer_v_a2a ? 0 : kv_local);
  }
  if (tma && block_n == 256 && pair_tiles_requested())
    return launch_pair<kModeQkvDirect>(p.lhs, packed_or(p.gemm.stride_a.row, p.gemm.k), p.rhs_nt,
                             packed_or(p.gemm.stride_b.row, p.gemm.k), p.gemm, stores, k, info, stream);
  return launch_mode<kModeQkvDirect>(maps, stores, k, block_n, info, stream, tma);
}

// detail/a2a_gemm.cuh (can_implement of the lhs pull) restated for the BF16 row layout.
cudaError_t check_lhs_route(const fuse_a2a_gemm_params& p) {
  const fuse_ulysses_route& r = p.route;
  if (r.world_size <= 0 || r.world_size > FUSE_MAX_WORLD_SIZE || r.rank < 0 ||
      r.rank >= r.world_size || r.batch <= 0 || r.seq_local <= 0 || r.global_seq <= 0 ||
      r.kind != FUSE_ROUTE_HEAD_TO_SEQUENCE || r.direction != FUSE_ROUTE_INVERSE ||
      r.channel_count != 1 || r.packed_source_row != nullptr || r.packed_row_granularity != 0 ||
      r.qkv_peer_interleaved || r.defer_v_a2a)
    return cudaErrorNotSupported;
  if (int64_t(r.seq_local) * r.world_size != r.global_seq ||
      int64_t(r.batch) * r.seq_local != p.gemm.m || p.gemm.k % r.world_size != 0 ||
      (p.gemm.k / r.world_size) % 8 != 0 || (r.causal_load_balanced && r.seq_local % 2 != 0))
    return cudaErrorNotSupported;
  if (r.q_heads > 0 && r.head_dim > 0 && int64_t(r.q_heads) * r.head_dim != p.gemm.k)
    return cudaErrorNotSupported;
  if (!host::aligned16(p.input_staging) || !host::aligned16(p.rhs_nt) || !host::aligned16(p.output) ||
      !host::aligned4(p.ready))
    return cudaErrorNotSupported;
  for (int peer = 0; peer < r.world_size; ++peer) {
    if (!host::aligned16(p.peer_input[peer])) return cudaErrorNotSupported;
    if (p.peer_input_ready[peer] != nullptr && !host::aligned4(p.peer_input_ready[peer]))
      return cudaErrorNotSupported;
  }
  return cudaSuccess;
}

cudaError_t oproj_forward(const fuse_a2a_gemm_params& p, const fuse_b200_options* options,
                          cudaStream_t stream) {
  if (!supported_problem(p.gemm) || !std::isfinite(p.alpha) || p.epoch == 0 || p.lhs_policy != 0)
    return cudaErrorInvalidValue;
  if (p.num_comm_ctas < 0) return cudaErrorInvalidValue;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  // Auto: the planner's choice (embedded copy warps, or a communication budget); explicit: exactly that
  const planner::Choice plan = plan_transfer(planner::kLhsPullBf16, p.gemm.m, p.gemm.n, p.gemm.k,
                                             double(p.gemm.m) * p.gemm.k * 2.0, info.sm_count, p.num_comm_ctas, true,
                                             p.route.world_size);
  const int num_comm_ctas = p.num_comm_ctas ? p.num_comm_ctas
                                            : (plan.comm_ctas ? plan.comm_ctas
                                                              : fuse_recommended_a2a_lhs_gemm_comm_ctas(&p.gemm, &p.route));
  if (num_comm_ctas >= info.sm_count) return cudaErrorInvalidValue;
  if ((status = check_lhs_route(p)) != cudaSuccess) return status;

  const int block_n = choose_block_n(p.gemm, options);
  const int64_t lda = packed_or(p.gemm.stride_a.row, p.gemm.k);
  Operands maps;
  status = encode_operands(&maps, p.input_staging, lda, p.rhs_nt,
                           packed_or(p.gemm.stride_b.row, p.gemm.k), p.gemm, block_n);
  if (status != cudaSuccess) return status;

  FusedParams k{};
  fill_core(&k, p.gemm, block_n, num_comm_ctas, p.alpha, p.output, FUSE_RASTER_ALONG_N);
  k.ready = p.ready;
  k.flags = options ? options->flags : 0u;
  if (options && (options->flags & FUSE_B200_VECTOR_PULL)) k.flags |= kFlagVectorPull;
  k.wait = host::make_wait(info, p.epoch, options ? options->wait_budget_ns : 0);
  copy_trace(&k, options);
  k.lhs.world = p.route.world_size;
  k.lhs.rank = p.route.rank;
  k.lhs.seq_local = p.route.seq_local;
  k.lhs.global_seq = p.route.global_seq;
  k.lhs.shard_width = p.gemm.k / p.route.world_size;
  k.lhs.causal = p.route.causal_load_balanced ? 1 : 0;
  k.lhs.cyclic = p.route.cyclic_peer_order ? 1 : 0;
  k.lhs.input_epoch = p.input_epoch;
  k.lhs.staging = p.input_staging;
  k.lhs.lda = lda;
  k.lhs.element_bytes = 2;
  for (int peer = 0; peer < p.route.world_size; ++peer) {
    k.lhs.peer_input[peer] = p.peer_input[peer];
    k.lhs.peer_input_ready[peer] = p.peer_input_ready[peer];
  }
  plan_lhs_slices(&k, info.sm_count);
  plan_join(&k, block_n, info.sm_count, double(p.gemm.m) * p.gemm.k * 2.0, false);
  if (!(k.flags & kFlagVectorPull)) {
    LhsPullMaps pull{};
    if (encode_lhs_pull_maps(&pull, k, uint64_t(p.route.batch) * uint64_t(p.route.global_seq))) {
      // CTA pairs: whole pairs of communication CTAs, 256-row tiles (the slices of the M tiles of
      // one wave are then delivered for twice as many 128-row tiles)
      if (block_n == 256 && num_comm_ctas % 2 == 0 && info.sm_count % 2 == 0 && pair_tiles_requested()) {
        FusedParams pk = k;
        pk.lhs.m_group = 2 * wave_m_group_pairs(pk, info.sm_count);
        if (launch::embedded_copy_selected(p.num_comm_ctas, plan)) {
          Operands pair_maps;
          if (encode_operand(&pair_maps.a, p.input_staging, p.gemm.m, p.gemm.k, lda, false, kBlockM) == cudaSuccess &&
              encode_operand(&pair_maps.b, p.rhs_nt, p.gemm.n, p.gemm.k, packed_or(p.gemm.stride_b.row, p.gemm.k), false,
                             PairLayout::kBlockN / 2) == cudaSuccess)
            return launch::launch_pair_kernel<kModeLhsPull, LhsPullMaps, false, false, false, true>(
                pair_maps, pair_maps.a, pair_maps.a, pull, pk, p.gemm.max_swizzle_size, info, stream, 0.0);
        }
        return launch_pair<kModeLhsPull>(p.input_staging, lda, p.rhs_nt, packed_or(p.gemm.stride_b.row, p.gemm.k), p.gemm,
                                         pull, pk, info, stream, double(p.gemm.m) * p.gemm.k * 2.0);
      }
    }
    if (encode_lhs_pull_maps(&pull, k, uint64_t(p.route.batch) * uint64_t(p.route.global_seq)))
      return launch_mode<kModeLhsPull, false, false, false, LhsPullMaps>(maps, pull, k, block_n, info, stream,
                                                                         !vector_epilogue_requested(options));
  }
  k.lhs.virt = 1;  // bulk-copy or vector pull: one gate per shard
  k.lhs.virt_width = k.lhs.shard_width;
  if (k.lhs.gate_start != 0) k.lhs.gate_start = k.lhs.rank;
  StoreMaps stores{};
  return launch_mode<kModeLhsPull>(maps, stores, k, block_n, info, stream,
                                   !vector_epilogue_requested(options));
}

cudaError_t plain_gemm(const fuse_gemm_problem& g, const void* a, const void* b, void* d, float alpha,
                       int reserved_comm_ctas, cudaStream_t stream) {
  if (!supported_problem(g) || !std::isfinite(alpha) || reserved_comm_ctas < 0)
    return cudaErrorInvalidValue;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  if (reserved_comm_ctas >= info.sm_count || !host::aligned16(a) || !host::aligned16(b) ||
      !host::aligned16(d))
    return cudaErrorInvalidValue;
  const int block_n = choose_block_n(g, nullptr);
  Operands maps;
  status = encode_operands(&maps, a, packed_or(g.stride_a.row, g.k), b,
                           packed_or(g.stride_b.row, g.k), g, block_n);
  if (status != cudaSuccess) return status;
  FusedParams k{};
  fill_core(&k, g, block_n, 0, alpha, d, FUSE_RASTER_ALONG_M);
  k.wait = host::make_wait(info, 1, 0);
  // The reserved CTAs are simply not launched: the GEMM runs on SMs - reserved.
  DeviceInfo reduced = info;
  reduced.sm_count = info.sm_count - reserved_comm_ctas;
  StoreMaps stores{};
  if (block_n == 256 && pair_tiles_requested())
    return launch_pair<kModePlain>(a, packed_or(g.stride_a.row, g.k), b, packed_or(g.stride_b.row, g.k), g, stores, k,
                              reduced, stream);
  return launch_mode<kModePlain>(maps, stores, k, block_n, reduced, stream, true);
}

}  // namespace
}  // namespace fuse_b200

extern "C" {

int fuse_launch_gemm_a2a_cutlass_ex(const fuse_gemm_a2a_params* params,
                                    const fuse_b200_options* options, fuse_stream stream) {
  if (params == nullptr) return int(cudaErrorInvalidValue);
  return int(fuse_b200::qkv_forward(*params, options, reinterpret_cast<cudaStream_t>(stream)));
}

int fuse_launch_gemm_a2a_cutlass(const fuse_gemm_a2a_params* params, fuse_stream stream) {
  return fuse_launch_gemm_a2a_cutlass_ex(params, nullptr, stream);
}

int fuse_launch_a2a_gemm_cutlass_ex(const fuse_a2a_gemm_params* params,
                                    const fuse_b200_options* options, fuse_stream stream) {
  if (params == nullptr) return int(cudaErrorInvalidValue);
  return int(fuse_b200::oproj_forward(*params, options, reinterpret_cast<cudaStream_t>(stream)));
}

int fuse_launch_a2a_gemm_cutlass(const fuse_a2a_gemm_params* params, fuse_stream stream) {
  return fuse_launch_a2a_gemm_cutlass_ex(params, nullptr, stream);
}

int fuse_launch_batched_cutlass_reference(const fuse_gemm_a2a_params* params, fuse_stream stream,
                                          int32_t reserved_comm_ctas) {
  if (params == nullptr) return int(cudaErrorInvalidValue);
  return int(fuse_b200::plain_gemm(params->gemm, params->lhs, params->rhs_nt, params->local_output,
                                   params->alpha, reserved_comm_ctas,
                                   reinterpret_cast<cudaStream_t>(stream)));
}

int fuse_launch_a2a_gemm_cutlass_reference(const fuse_a2a_gemm_params* params, fuse_stream stream,
                                           int32_t reserved_comm_ctas) {
  if (params == nullptr) return int(cudaErrorInvalidValue);
  return int(fuse_b200::plain_gemm(params->gemm, params->input_staging, params->rhs_nt,
                                   params->output, params->alpha, reserved_comm_ctas,
                                   reinterpret_cast<cudaStream_t>(stream)));
}

void fuse_qkv_cutlass_kernel_traits(const fuse_gemm_problem* problem, fuse_kernel_traits* out) {
  (void)problem;
  // Finest publication tile this library launches; `ready` sized for it fits every choice.
  using Layout = fuse_b200::SmemLayout<128, 6>;
  *out = {fuse_b200::kBlockM, 128, fuse_b200::kBlockK, fuse_b200::kThreads,
          int32_t(Layout::kDynamicBytes)};
}

void fuse_cutlass_kernel_traits(fuse_kernel_traits* out) {
  using Layout = fuse_b200::SmemLayout<256, 4>;
  *out = {fuse_b200::kBlockM, 256, fuse_b200::kBlockK, fuse_b200::kThreads,
          int32_t(Layout::kDynamicBytes)};
}

int64_t fuse_a2a_lhs_gemm_ready_elements(const fuse_gemm_problem* problem,
                                         const fuse_ulysses_route* route) {
  if (problem == nullptr || route == nullptr || problem->m <= 0 || route->world_size <= 0) return 0;
  return int64_t(fuse_b200::host::ceil_div(problem->m, fuse_b200::kBlockM)) * route->world_size *
         FUSE_READY_FLAG_STRIDE;
}

// The communication budgets Auto uses when an operator runs with communication CTAs (the planner's
// best budget with the embedded copy warps left out; 148 SMs assumed when no device is current).
int32_t fuse_recommended_gemm_a2a_comm_ctas(const fuse_gemm_problem* problem,
                                            const fuse_ulysses_route* route) {
  if (problem == nullptr || problem->m <= 0 || problem->n <= 0 || problem->k <= 0) return 0;
  (void)route;
  const int64_t tiles = ((int64_t(problem->m) + 127) / 128) * ((int64_t(problem->n) + 255) / 256);
  return fuse_b200::planner::choose(fuse_b200::planner::kQkvPushBf16,
                                    2.0 * double(problem->m) * double(problem->n) * double(problem->k),
                                    double(problem->m) * double(problem->n) * 2.0, tiles, 148, 1, 0, false)
      .comm_ctas;
}

int32_t fuse_recommended_a2a_lhs_gemm_comm_ctas(const fuse_gemm_problem* problem,
                                                const fuse_ulysses_route* route) {
  if (problem == nullptr || problem->m <= 0 || problem->n <= 0 || problem->k <= 0) return 0;
  (void)route;
  return fuse_b200::launch::plan_transfer(fuse_b200::planner::kLhsPullBf16, problem->m, problem->n, problem->k,
                                          double(problem->m) * double(problem->k) * 2.0, 148, 0, false)
      .comm_ctas;
}

// The planner itself, for callers and tests: kind as in planner.cuh (0 BF16 lhs pull, 1 MXFP8 lhs
// pull, 2 BF16 gradient push, 3 MXFP8 gradient pull, 4 / 5 QKV push from communication CTAs BF16 /
// MXFP8, 6 MoE dispatch).  out = {comm_ctas, embedded, makespan_us, compute_us, transfer_us}.
int fuse_b200_plan(int32_t kind, double flops, double bytes, int64_t tiles, int32_t sm_count, int32_t group,
                   int32_t explicit_comm_ctas, int32_t embedded_allowed, double out[5]) {
  return fuse_b200_plan_remote(kind, flops, bytes, tiles, sm_count, group, explicit_comm_ctas, embedded_allowed, 0.0, out);
}

int fuse_b200_plan_remote(int32_t kind, double flops, double bytes, int64_t tiles, int32_t sm_count, int32_t group,
                          int32_t explicit_comm_ctas, int32_t embedded_allowed, double remote_share, double out[5]) {
  if (!(remote_share >= 0.0 && remote_share < 1.0)) return int(cudaErrorInvalidValue);
  if (kind < 0 || kind >= fuse_b200::planner::kKinds || !(flops > 0.0) || !(bytes >= 0.0) || tiles <= 0 ||
      sm_count <= 0 || (group != 1 && group != 2) || explicit_comm_ctas < 0 || explicit_comm_ctas >= sm_count ||
      out == nullptr)
    return int(cudaErrorInvalidValue);
  const fuse_b200::planner::Choice c = fuse_b200::planner::choose(
      fuse_b200::planner::Kind(kind), flops, bytes, tiles, sm_count, group, explicit_comm_ctas, embedded_allowed != 0,
      remote_share);
  out[0] = c.comm_ctas;
  out[1] = c.embedded;
  out[2] = c.makespan_us;
  out[3] = c.compute_us;
  out[4] = c.transfer_us;
  return 0;
}

int fuse_b200_abi_sizeof(int record) {
  switch (record) {
    case 0: return int(sizeof(fuse_gemm_problem));
    case 1: return int(sizeof(fuse_ulysses_route));
    case 2: return int(sizeof(fuse_gemm_a2a_params));
    case 3: return int(sizeof(fuse_a2a_gemm_params));
    case 4: return int(sizeof(fuse_kernel_traits));
    case 5: return int(sizeof(fuse_b200_options));
    case 6: return int(sizeof(fuse_qkv_backward_data_params));
    case 7: return int(sizeof(fuse_qkv_backward_weight_params));
    case 8: return int(sizeof(fuse_qkv_backward_params));
    case 9: return int(sizeof(fuse_oproj_backward_data_params));
    case 10: return int(sizeof(fuse_oproj_backward_weight_params));
    case 11: return int(sizeof(fuse_oproj_backward_params));
    case 12: return int(sizeof(fuse_mxfp8_activation));
    case 13: return int(sizeof(fuse_mxfp8_gemm_a2a_params));
    case 14: return int(sizeof(fuse_mxfp8_a2a_gemm_params));
    case 15: return int(sizeof(fuse_grouped_gemm_policy));
    case 16: return int(sizeof(fuse_bf16_grouped_gemm_params));
    case 17: return int(sizeof(fuse_mxfp8_qkv_backward_data_params));
    case 18: return int(sizeof(fuse_mxfp8_qkv_backward_weight_params));
    case 19: return int(sizeof(fuse_mxfp8_qkv_backward_params));
    case 20: return int(sizeof(fuse_mxfp8_oproj_backward_data_params));
    case 21: return int(sizeof(fuse_mxfp8_oproj_backward_weight_params));
    case 22: return int(sizeof(fuse_mxfp8_oproj_backward_params));
    default: return -1;
  }
}

}  // extern "C"
