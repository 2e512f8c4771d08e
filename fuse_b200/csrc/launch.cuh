// Host-side launch helpers shared by the operator entry points: operand tensor maps for K-major
// and MN-major operands, the epilogue's store maps, grid sizing and the kernel launch itself.
#pragma once

#include <cmath>
#include <cstring>

#include "fuse_b200.h"
#include "fused_gemm.cuh"
#include "pair_gemm.cuh"
#include "host.cuh"
#include "planner.cuh"

namespace fuse_b200 {
namespace launch {

using host::DeviceInfo;

inline int64_t packed_or(int64_t stride, int64_t packed) { return stride < 0 ? packed : stride; }

struct Operands {
  CUtensorMap a, b;
};

// K-major operand: stored [rows, k] row-major (rows = M for A, N for B), boxed
// [block_rows x 64].  MN-major operand: stored [k, rows] row-major, boxed [64 x 64].
// One-byte (E4M3) K-major operand [rows, k]: boxes of block_rows x 128 bytes.
inline cudaError_t encode_operand_u8(CUtensorMap* map, const void* base, int64_t rows, int64_t k,
                                     int64_t pitch_bytes, int block_rows) {
  return host::encode_tensor_map_2d(map, base, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, uint64_t(rows), uint64_t(k),
                                    uint64_t(pitch_bytes), uint32_t(block_rows), 2 * kBlockK,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
}

inline cudaError_t encode_operand(CUtensorMap* map, const void* base, int64_t rows, int64_t k,
                                  int64_t pitch_elements, bool mn_major, int block_rows) {
  if (!mn_major)
    return host::encode_tensor_map_2d(map, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, uint64_t(rows),
                                      uint64_t(k), uint64_t(pitch_elements) * 2, uint32_t(block_rows),
                                      kBlockK, CU_TENSOR_MAP_SWIZZLE_128B);
  return host::encode_tensor_map_2d(map, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, uint64_t(k),
                                    uint64_t(rows), uint64_t(pitch_elements) * 2, kBlockK, 64,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
}

// Tensor map of a row-major BF16 [rows, cols] destination for the TMA-store epilogue.
inline cudaError_t encode_store_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                                    int64_t pitch_elements) {
  return host::encode_tensor_map_2d(map, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, cols,
                                    uint64_t(pitch_elements) * 2, kBlockM, 64,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
}

inline void fill_core(FusedParams* p, int m, int n, int k, int block_n, int num_comm_ctas, float alpha,
                      float beta, void* d, int64_t ldd, int raster, int max_swizzle) {
  p->m = m;
  p->n = n;
  p->k = k;
  p->order.m_tiles = host::ceil_div(m, kBlockM);
  p->order.n_tiles = host::ceil_div(n, block_n);
  p->order.swizzle = select_swizzle(max_swizzle, p->order.m_tiles, p->order.n_tiles);
  p->order.along_n = raster == FUSE_RASTER_ALONG_N ? 1 : 0;
  p->num_comm_ctas = num_comm_ctas;
  p->alpha = alpha;
  p->beta = beta;
  p->d = static_cast<uint16_t*>(d);
  p->ldd = ldd;
  p->join_tile = p->order.count();
}

// Host plan for the tail share of tiles that communication CTAs compute once their transfers are
// done (pull and gradient modes).  Calibration on B200: one SM sustains about 10.3 TFLOP/s of
// BF16 UMMA (17 TFLOP/s block-scaled E4M3) inside these kernels and one communication CTA moves
// about 35 GB/s through its copy pipeline.  With tau the time of one tile and t_c the time the
// transfers take, the plan tries every whole number of compute-only waves w1: the first
// w1 * compute_ctas tiles go to the compute CTAs alone, the rest is dealt to the whole grid, and
// the split with the smallest makespan max((w1 + w2) * tau, t_c + w2 * tau) wins, w2 being the
// waves of the shared part.  FUSE_B200_JOIN_WAVES=0 keeps the communication CTAs out of the GEMM.
// M tiles that one wave of compute CTAs works on at the same time under the launch's tile order:
// a band of `swizzle` M tiles with the N raster, compute_ctas / band width with the M raster.
inline int32_t wave_m_group(const FusedParams& p, int sm_count) {
  const int32_t compute = sm_count - p.num_comm_ctas;
  const int32_t swizzle = p.order.swizzle > 0 ? p.order.swizzle : 1;
  int32_t group = p.order.along_n ? swizzle : (compute + swizzle - 1) / swizzle;
  if (group > p.order.m_tiles) group = p.order.m_tiles;
  return group < 1 ? 1 : group;
}

// The same for CTA pairs (256-row tiles, `block_n` columns): result in 256-row tiles.
inline int32_t wave_m_group_pairs(const FusedParams& p, int sm_count, int block_n = 256) {
  const int32_t compute = (sm_count - p.num_comm_ctas) / 2;
  const int32_t m_tiles = (p.m + 2 * kBlockM - 1) / (2 * kBlockM);
  const int32_t n_tiles = (p.n + block_n - 1) / block_n;
  const int32_t smaller = m_tiles < n_tiles ? m_tiles : n_tiles;
  int32_t swizzle = p.order.swizzle > 0 ? p.order.swizzle : 1;
  while (swizzle > 1 && swizzle > smaller) swizzle /= 2;
  int32_t group = p.order.along_n ? swizzle : (compute + swizzle - 1) / swizzle;
  if (group > m_tiles) group = m_tiles;
  return group < 1 ? 1 : group;
}

// Column slices of the lhs pull: the largest power of two (at most 16, the pairs of words a flag
// line holds) that keeps a slice at least 1 KiB wide and a whole number of 128-byte K blocks.
inline void plan_lhs_slices(FusedParams* p, int sm_count) {
  const int64_t shard_bytes = int64_t(p->lhs.shard_width) * p->lhs.element_bytes;
  int virt = 1;
  while (virt < 16 && shard_bytes % (2 * virt * 128) == 0 && shard_bytes / (2 * virt) >= 1024) virt *= 2;
  p->lhs.virt = virt;
  p->lhs.virt_width = p->lhs.shard_width / virt;
  p->lhs.m_group = wave_m_group(*p, sm_count);
  // K rotation: start at this rank's own shard when shards are whole K blocks.
  const int block_elems = p->lhs.element_bytes == 1 ? 2 * kBlockK : kBlockK;
  const bool rotate = p->lhs.shard_width % block_elems == 0 && p->k == p->lhs.shard_width * p->lhs.world;
  const int shard_first = p->lhs.cyclic ? 0 : p->lhs.rank;  // cyclic order already puts the own shard first
  p->lhs.gate_start = rotate ? shard_first * virt : 0;
  p->lhs.k_block_start = rotate ? shard_first * (p->lhs.shard_width / block_elems) : 0;
}

// `group` = CTAs that work on one tile together (2 for CTA pairs: `order` then counts 256-row
// tiles and the waves are waves of pairs).
inline void plan_join(FusedParams* p, int block_n, int sm_count, double comm_bytes, bool block_scaled,
                      int group = 1) {
  const int64_t tiles = p->order.count();
  const int comm = p->num_comm_ctas / group;
  if (comm <= 0 || tiles <= 0) return;
  if (const char* text = std::getenv("FUSE_B200_JOIN_WAVES"))
    if (std::atoll(text) == 0) return;
  const int64_t units = sm_count / group;
  const int64_t compute = tiles < units - comm ? tiles : units - comm;
  const int64_t all = comm + compute;
  // one tile per unit: a pair does twice the rows on twice the SMs
  const double tau = 2.0 * kBlockM * block_n * double(p->k) / (block_scaled ? 17.0e12 : (group == 2 ? 11.0e12 : 10.3e12));
  const double t_c = 25.0e-6 + comm_bytes / (p->num_comm_ctas * 35.0e9);
  double best = double((tiles + compute - 1) / compute) * tau;  // no sharing
  int64_t best_join = tiles;
  for (int64_t w1 = 0; w1 * compute < tiles; ++w1) {
    const int64_t join = w1 * compute, rest = tiles - join;
    const int64_t w2 = (rest + all - 1) / all;
    const double compute_side = double(w1 + w2) * tau, comm_side = t_c + double(w2) * tau;
    const double makespan = compute_side > comm_side ? compute_side : comm_side;
    if (makespan < best - 1.0e-9) {
      best = makespan;
      best_join = join;
    }
  }
  p->join_tile = best_join;
}

template <int kMode, bool kTmaEpilogue, bool kAMn, bool kBMn, bool kMx = false, class Maps = StoreMaps>
cudaError_t launch_variant(const Operands& maps, const Maps& stores, const FusedParams& p,
                           int block_n, const DeviceInfo& info, cudaStream_t stream) {
  const int64_t tiles = p.order.count();
  const int compute_capacity = info.sm_count - p.num_comm_ctas;
  const int compute = int(tiles < compute_capacity ? tiles : compute_capacity);
  const int grid = p.num_comm_ctas + compute;
  const bool cooperative = kMode != kModePlain || kMx;
  if (block_n == 256) {
    using Layout = SmemLayout<256, 4, kMx>;
    return host::launch_kernel(fused_gemm_kernel<256, 4, kMode, kTmaEpilogue, kAMn, kBMn, kMx, Maps>, grid, kThreads,
                               Layout::kDynamicBytes, cooperative, stream, maps.a, maps.b, stores, p);
  }
  using Layout = SmemLayout<128, 6, kMx>;
  return host::launch_kernel(fused_gemm_kernel<128, 6, kMode, kTmaEpilogue, kAMn, kBMn, kMx, Maps>, grid, kThreads,
                             Layout::kDynamicBytes, cooperative, stream, maps.a, maps.b, stores, p);
}

// The epilogue writes the local output through the copy engine unless the caller asked for the
// 16-byte vector epilogue or the mode needs it (beta != 0, tile publication to communication
// CTAs).
template <int kMode, bool kAMn = false, bool kBMn = false, bool kMx = false, class Maps = StoreMaps>
cudaError_t launch_mode(const Operands& maps, Maps& stores, const FusedParams& p, int block_n,
                        const DeviceInfo& info, cudaStream_t stream, bool tma_epilogue) {
  if constexpr (kMode != kModeQkvPush) {
    if (tma_epilogue) {
      const cudaError_t status = encode_store_map(&stores.local, p.d, uint64_t(p.m), uint64_t(p.n), p.ldd);
      if (status != cudaSuccess) return status;
      return launch_variant<kMode, true, kAMn, kBMn, kMx, Maps>(maps, stores, p, block_n, info, stream);
    }
  }
  return launch_variant<kMode, false, kAMn, kBMn, kMx, Maps>(maps, stores, p, block_n, info, stream);
}

// Row-major [rows, cols] tensor of `element_bytes`-wide elements boxed box_rows x box_cols
// without swizzle: the copy boxes of the gradient routes.
inline cudaError_t encode_copy_map(CUtensorMap* map, const void* base, uint32_t element_bytes, uint64_t rows,
                                   uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
  return host::encode_tensor_map_2d(map, base,
                                    element_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                                    element_bytes, rows, cols, cols * element_bytes, box_rows, box_cols,
                                    CU_TENSOR_MAP_SWIZZLE_NONE);
}

// Tensor maps of the forward lhs pull (LhsPullPolicy).  False when the geometry does not fit the
// tensor copies (the caller then runs the bulk-copy pull with one gate per shard): a slice must
// be a whole number of power-of-two pieces of at most 1 KiB, and the rows of one chunk must be
// consecutive in the peer's tensor.
inline bool encode_lhs_pull_maps(LhsPullMaps* maps, const FusedParams& f, uint64_t source_rows) {
  const LhsRoute& r = f.lhs;
  const uint32_t unit_bytes = uint32_t(r.virt_width) * uint32_t(r.element_bytes);
  const uint64_t shard_bytes = uint64_t(r.shard_width) * uint64_t(r.element_bytes);
  const uint64_t staging_pitch = uint64_t(r.lda) * uint64_t(r.element_bytes);
  uint32_t piece = 1024;
  while (piece >= 128 && unit_bytes % piece != 0) piece /= 2;
  if (piece < 128 || shard_bytes % 16 != 0 || staging_pitch % 16 != 0) return false;
  const uint32_t rows_per_chunk = kPullStageBytes / piece < uint32_t(kBlockM) ? kPullStageBytes / piece : uint32_t(kBlockM);
  const int32_t row_block = r.causal ? r.seq_local / 2 : r.seq_local;
  if (row_block % int32_t(rows_per_chunk) != 0) return false;
  maps->piece_bytes = int32_t(piece);
  maps->rows_per_chunk = int32_t(rows_per_chunk);
  for (int peer = 0; peer < r.world; ++peer)
    if (host::encode_tensor_map_2d(&maps->peer[peer], r.peer_input[peer], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, source_rows,
                                   shard_bytes / 4, shard_bytes, rows_per_chunk, piece / 4,
                                   CU_TENSOR_MAP_SWIZZLE_NONE) != cudaSuccess)
      return false;
  return host::encode_tensor_map_2d(&maps->staging, r.staging, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, uint64_t(f.m),
                                    uint64_t(f.k) * uint64_t(r.element_bytes) / 4, staging_pitch, rows_per_chunk,
                                    piece / 4, CU_TENSOR_MAP_SWIZZLE_NONE) == cudaSuccess;
}

// Launches pair_gemm_kernel (CTA pairs, 256 x 256 tiles) over `k`, whose tile order is re-planned
// for those tiles.  `maps.b` must box half a tile's B rows (kPairBRows /
// kPairMxBRows); sfa / sfb are only read by the block-scaled variant.
constexpr int kPairBRows = PairLayoutT<false>::kBlockN / 2;
constexpr int kPairMxBlockN = PairLayoutT<true>::kBlockN;
constexpr int kPairMxBRows = kPairMxBlockN / 2;

template <int kMode, class Maps, bool kMx, bool kAMn = false, bool kBMn = false, bool kEmbedded = false>
cudaError_t launch_pair_kernel(const Operands& maps, const CUtensorMap& sfa, const CUtensorMap& sfb, Maps& stores,
                               FusedParams k, int max_swizzle, const DeviceInfo& info, cudaStream_t stream,
                               double comm_bytes) {
  using Layout = PairLayoutT<kMx, kEmbedded>;
  if (kEmbedded) k.num_comm_ctas = 0;  // every CTA computes; its copy warp pulls
  cudaError_t status = encode_store_map(&stores.local, k.d, uint64_t(k.m), uint64_t(k.n), k.ldd);
  if (status != cudaSuccess) return status;
  k.order.m_tiles = host::ceil_div(k.m, 2 * kBlockM);
  k.order.n_tiles = host::ceil_div(k.n, Layout::kBlockN);
  k.order.swizzle = select_swizzle(max_swizzle, k.order.m_tiles, k.order.n_tiles);
  if (kMode == kModeQkvDirect) k.order.n_shift = int32_t(int64_t(k.qkv.rank) * k.order.n_tiles / k.qkv.world);
  k.join_tile = k.order.count();
  if (!kEmbedded && (kMode == kModeLhsPull || kMode == kModeGradPull || kMode == kModeHeadGate)) plan_join(&k, Layout::kBlockN, info.sm_count, comm_bytes, kMx, 2);
  const int64_t tiles = k.order.count();
  const int compute_pairs = int(tiles < (info.sm_count - k.num_comm_ctas) / 2 ? tiles : (info.sm_count - k.num_comm_ctas) / 2);
  return host::launch_kernel(pair_gemm_kernel<kMode, Maps, kMx, kAMn, kBMn, kEmbedded>, k.num_comm_ctas + 2 * compute_pairs, kThreads,
                             Layout::kDynamicBytes, kMode != kModePlain || kMx, stream, maps.a, maps.b, sfa, sfb, stores, k);
}

// Scale storage of a block-scaled operand ([rows, K] elements) as a tensor of 512-byte atoms,
// one atom per row of 128 32-bit words.
inline cudaError_t encode_scale_atoms(CUtensorMap* map, const void* scales, int64_t rows, int64_t k) {
  const uint64_t atoms = uint64_t((rows + 127) / 128) * uint64_t((k + 127) / 128);
  return host::encode_tensor_map_2d(map, scales, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, atoms, 128, 512, 1, 128,
                                    CU_TENSOR_MAP_SWIZZLE_NONE);
}

// Who moves the data of a pull / push operator on CTA pairs: an explicit `num_comm_ctas` means that
// many communication CTAs, exactly; Auto (0) follows the planner, which on B200 picks the copy
// warp embedded in every compute CTA (no SM given up) wherever the geometry allows it.
// FUSE_B200_EMBEDDED_PULL=1 / 0 (read on every launch) overrides both.
inline bool embedded_copy_selected(int explicit_comm_ctas, const planner::Choice& plan) {
  if (const char* text = std::getenv("FUSE_B200_EMBEDDED_PULL")) return std::atoi(text) != 0;
  return explicit_comm_ctas == 0 && plan.embedded != 0;
}

// The plan of a transfer-fed GEMM on this device: `tiles` of 256 x 256 (CTA pairs).
inline planner::Choice plan_transfer(planner::Kind kind, int64_t m, int64_t n, int64_t k, double bytes, int sm_count,
                                     int explicit_comm_ctas, bool embedded_allowed = true, int world = 1) {
  const int64_t tiles = ((m + 255) / 256) * ((n + 255) / 256);
  return planner::choose(kind, 2.0 * double(m) * double(n) * double(k), bytes, tiles, sm_count, 2, explicit_comm_ctas,
                         embedded_allowed, world > 1 ? double(world - 1) / double(world) : 0.0);
}

// CTA-pair tiles are used wherever the shape allows; the environment switch FUSE_B200_PAIR=0
// (read on every launch) selects the one-CTA tiles.
inline bool pair_tiles_requested() {
  const char* text = std::getenv("FUSE_B200_PAIR");
  return text == nullptr || std::atoi(text) != 0;
}

inline bool vector_epilogue_requested(const fuse_b200_options* options) {
  return options != nullptr && (options->flags & FUSE_B200_VECTOR_EPILOGUE) != 0;
}

inline cudaError_t check_device(DeviceInfo* info) {
  const cudaError_t status = host::device_info(info);
  if (status != cudaSuccess) return status;
  // Compiled for sm_100a only: tcgen05 / TMEM kernels exist for no other target.
  return info->cc_major == 10 ? cudaSuccess : cudaErrorNotSupported;
}

inline int choose_block_n(int n, const fuse_b200_options* options) {
  if (options && (options->block_n == 128 || options->block_n == 256)) return options->block_n;
  return n % 256 == 0 || n > 1024 ? 256 : 128;
}

// Fills the (peer, segment) store maps of a head-sharded planar destination; false when a map
// cannot be encoded.
inline bool encode_peer_store_maps(StoreMaps* stores, fuse_bf16* const* peer_output, int world,
                                   uint64_t rows_total, int64_t q_local, int64_t kv_local) {
  for (int peer = 0; peer < world; ++peer)
    for (int segment = 0; segment < (kv_local > 0 ? 3 : 1); ++segment) {
      const int64_t width = segment == 0 ? q_local : kv_local;
      const int64_t offset =
          segment == 0 ? 0 : int64_t(rows_total) * q_local + (segment == 2 ? int64_t(rows_total) * kv_local : 0);
      if (encode_store_map(&stores->peer[peer][segment], peer_output[peer] + offset, rows_total,
                           uint64_t(width), width) != cudaSuccess)
        return false;
    }
  return true;
}

inline void copy_trace(FusedParams* k, const fuse_b200_options* options) {
  if (options != nullptr) {
    k->trace = options->trace;
    k->trace_capacity = options->trace_capacity;
    k->trace_cta = options->trace_cta;
  }
}

}  // namespace launch
}  // namespace fuse_b200
