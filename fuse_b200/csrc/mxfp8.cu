// MXFP8 (E4M3 data, one UE8M0 scale per 32 K values, FP32 accumulate, BF16 out): standalone
// quantisers and the block-scaled forward entry points.
//
// Interface: include/fuse/operators/primitives/gemm_a2a_mxfp8.h and a2a_gemm_mxfp8.h of the
// reference; quantisation arithmetic and scale storage: csrc/operators/sm103/detail/
// quantization.cuh:91-141,350-450 and benchmarks/sm103/fused_mxfp8.cuh:13-16.
#include <cstdio>
#include <mutex>

#include "launch.cuh"

namespace fuse_b200 {
namespace {

using namespace launch;

size_t align256(size_t n) { return (n + 255) & ~size_t{255}; }
size_t scale_bytes(int64_t rows, int64_t k) { return size_t((rows + 127) / 128) * size_t((k + 127) / 128) * 512; }

// Row-major BF16 [rows, k] -> E4M3 [rows, k] + native scales.  One thread per K32 group.
__global__ void quantize_rows_kernel(const uint16_t* source, int64_t stride, int32_t rows, int32_t k,
                                     uint8_t* data, uint8_t* scales) {
  mxfp8_quantize_rows(source, stride, rows, k, data, scales, int64_t(blockIdx.x) * blockDim.x + threadIdx.x,
                      int64_t(gridDim.x) * blockDim.x);
}

// BF16 [rows, cols] -> E4M3 [cols, rows] quantised along the source ROW axis (the new K axis)
// + native scales of the [cols, rows] operand.  A block stages a 32 x 256 source tile in shared
// memory with coalesced loads; each thread then owns one column: reduces its 32 values, writes
// 32 contiguous output bytes and one scale byte.
constexpr int kTransposeCols = 256;
__global__ void quantize_transposed_kernel(const uint16_t* source, int64_t stride, int32_t rows, int32_t cols,
                                           uint8_t* data, uint8_t* scales) {
  __shared__ uint16_t tile[32][kTransposeCols + 2];
  const int32_t col_tiles = (cols + kTransposeCols - 1) / kTransposeCols;
  const int32_t row_groups = rows / 32;
  const int64_t k_atoms = (int64_t(rows) + 127) >> 7;
  const int64_t padded_cols = (int64_t(cols) + 127) & ~int64_t(127);
  const bool vector_loads = cols % 8 == 0 && stride % 8 == 0 && reinterpret_cast<uintptr_t>(source) % 16 == 0;
  for (int64_t t = blockIdx.x; t < int64_t(col_tiles) * row_groups; t += gridDim.x) {
    const int32_t group = int32_t(t / col_tiles), col0 = int32_t(t % col_tiles) * kTransposeCols;
    __syncthreads();
    if (vector_loads) {
      // 16-byte loads: four per thread in flight
      for (int i = threadIdx.x; i < 32 * (kTransposeCols / 8); i += blockDim.x) {
        const int r = i / (kTransposeCols / 8), c8 = (i % (kTransposeCols / 8)) * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (col0 + c8 < cols) v = ptx::ld_cg_v4(source + int64_t(group * 32 + r) * stride + col0 + c8);
        uint32_t* row = reinterpret_cast<uint32_t*>(&tile[r][c8]);
        row[0] = v.x;
        row[1] = v.y;
        row[2] = v.z;
        row[3] = v.w;
      }
    } else {
      for (int i = threadIdx.x; i < 32 * (kTransposeCols / 2); i += blockDim.x) {
        const int r = i / (kTransposeCols / 2), c2 = (i % (kTransposeCols / 2)) * 2;
        uint32_t pair = 0;
        if (col0 + c2 < cols)
          pair = *reinterpret_cast<const uint32_t*>(source + int64_t(group * 32 + r) * stride + col0 + c2);
        tile[r][c2] = uint16_t(pair);
        tile[r][c2 + 1] = uint16_t(pair >> 16);
      }
    }
    __syncthreads();
    const int32_t col = col0 + threadIdx.x;
    if (threadIdx.x < kTransposeCols && col < cols) {
      float f[32];
      float amax = 0.0f;
#pragma unroll
      for (int r = 0; r < 32; ++r) {
        f[r] = __uint_as_float(uint32_t(tile[r][threadIdx.x]) << 16);
        amax = fmaxf(amax, fabsf(f[r]));
      }
      const int exponent = mxfp8_scale_exponent(amax);
      const float inverse = mxfp8_inverse_scale(exponent);
      uint4 o[2];
      uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        ow[i] = pack_e4m3x4(f[4 * i] * inverse, f[4 * i + 1] * inverse, f[4 * i + 2] * inverse, f[4 * i + 3] * inverse);
      uint4* out = reinterpret_cast<uint4*>(data + int64_t(col) * rows + group * 32);
      out[0] = o[0];
      out[1] = o[1];
      scales[mxfp8_scale_offset(col, int64_t(group) * 32, k_atoms)] = uint8_t(exponent + 127);
    }
    // neutral scales for the padding rows of the last 128-row atom
    if (col0 + kTransposeCols >= cols)
      for (int64_t pad = cols + threadIdx.x; pad < padded_cols; pad += blockDim.x)
        scales[mxfp8_scale_offset(pad, int64_t(group) * 32, k_atoms)] = 127;
  }
}

// The same operation for the common geometry (rows a multiple of 128, cols a multiple of 64,
// 16-byte rows), arranged for full-line traffic in both directions.  A block works on tiles of 128
// source rows x 64 columns: coalesced 16-byte loads into shared memory (rows padded to 144 bytes);
// thread (column c, group g) reduces 32 values down its column -- the lanes of a warp read
// consecutive halfwords -- and puts its 32 output bytes into a second shared tile laid out as the
// DESTINATION ([64 output rows][128 bytes], rows padded to 144); the block then writes that tile
// with 16-byte stores, eight consecutive threads per 128-byte output line, and one 32-bit word of
// four scale bytes per column (a 128 x 64 tile covers exactly one K atom of half a row atom).
// HBM-bound: 2 bytes read and 1.03 written per element.
constexpr int kTqRows = 128, kTqCols = 64, kTqInPitch = 144, kTqOutPitch = 144;
__global__ void __launch_bounds__(256, 4) quantize_transposed_tiled_kernel(const uint16_t* source, int64_t stride, int32_t rows,
                                                                     int32_t cols, uint8_t* data, uint8_t* scales) {
  __shared__ __align__(16) uint8_t tile_in[kTqRows * kTqInPitch];
  __shared__ __align__(16) uint8_t tile_out[kTqCols * kTqOutPitch];
  __shared__ uint32_t scale_words[kTqCols];
  const int32_t col_tiles = cols / kTqCols, row_tiles = rows / kTqRows;
  const int64_t k_atoms = int64_t(rows) >> 7;
  const int tid = threadIdx.x;
  if (tid < kTqCols) scale_words[tid] = 0u;
  const int64_t tiles = int64_t(col_tiles) * row_tiles;
  // this thread's four 16-byte pieces of a tile; the NEXT tile's are in flight while one is worked on
  auto fetch = [&](int64_t t, uint4 (&v)[4]) {
    const int32_t row0 = int32_t(t / col_tiles) * kTqRows, col0 = int32_t(t % col_tiles) * kTqCols;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = tid + 256 * j, r = i >> 3, chunk = i & 7;
      v[j] = ptx::ld_cg_v4(source + int64_t(row0 + r) * stride + col0 + chunk * 8);
    }
  };
  uint4 v[4];
  if (int64_t(blockIdx.x) < tiles) fetch(blockIdx.x, v);
  for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
    // column tiles fastest: consecutive blocks read consecutive 128-byte pieces of the same rows
    const int32_t row0 = int32_t(t / col_tiles) * kTqRows, col0 = int32_t(t % col_tiles) * kTqCols;
    __syncthreads();  // the previous tile's readers are done
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = tid + 256 * j, r = i >> 3, chunk = i & 7;
      *reinterpret_cast<uint4*>(tile_in + r * kTqInPitch + chunk * 16) = v[j];
    }
    if (t + gridDim.x < tiles) fetch(t + gridDim.x, v);
    __syncthreads();
    {
      const int c = tid & 63, g = tid >> 6;
      float f[32];
      float amax = 0.0f;
#pragma unroll
      for (int r = 0; r < 32; ++r) {
        const uint16_t bits = *reinterpret_cast<const uint16_t*>(tile_in + (g * 32 + r) * kTqInPitch + c * 2);
        f[r] = __uint_as_float(uint32_t(bits) << 16);
        amax = fmaxf(amax, fabsf(f[r]));
      }
      const int exponent = mxfp8_scale_exponent(amax);
      const float inverse = mxfp8_inverse_scale(exponent);
      uint4 o[2];
      uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        ow[i] = pack_e4m3x4(f[4 * i] * inverse, f[4 * i + 1] * inverse, f[4 * i + 2] * inverse, f[4 * i + 3] * inverse);
      uint4* out = reinterpret_cast<uint4*>(tile_out + c * kTqOutPitch + g * 32);
      out[0] = o[0];
      out[1] = o[1];
      atomicOr(&scale_words[c], uint32_t(exponent + 127) << (8 * g));  // byte g of the column's word
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int i = tid + 256 * j, c = i >> 3, chunk = i & 7;
      const uint4 v = *reinterpret_cast<const uint4*>(tile_out + c * kTqOutPitch + chunk * 16);
      *reinterpret_cast<uint4*>(data + int64_t(col0 + c) * rows + row0 + chunk * 16) = v;
    }
    if (tid < kTqCols) {
      // the four scale bytes of (output row col0 + tid, this K atom) are one aligned word
      *reinterpret_cast<uint32_t*>(scales + mxfp8_scale_offset(col0 + tid, row0, k_atoms)) = scale_words[tid];
      scale_words[tid] = 0u;
      // neutral scales for the other half of a row atom the operand does not fill
      if (col0 + kTqCols == cols && (cols & 127) != 0)
        *reinterpret_cast<uint32_t*>(scales + mxfp8_scale_offset(cols + tid, row0, k_atoms)) = 0x7f7f7f7fu;
    }
  }
}

cudaError_t quantize_rows(const fuse_bf16* source, int64_t stride, int rows, int k, uint8_t* data,
                          uint8_t* scales, cudaStream_t stream) {
  if (source == nullptr || data == nullptr || scales == nullptr || rows <= 0 || k <= 0 || k % 32 != 0 ||
      stride % 8 != 0 || !host::aligned16(source) || !host::aligned16(data))
    return cudaErrorInvalidValue;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  quantize_rows_kernel<<<info.sm_count * 8, 256, 0, stream>>>(source, stride, rows, k, data, scales);
  status = cudaGetLastError();
  if (status == cudaSuccess) host::count_launch();
  return status;
}

cudaError_t quantize_transposed(const fuse_bf16* source, int64_t stride, int rows, int cols, uint8_t* data,
                                uint8_t* scales, cudaStream_t stream) {
  if (source == nullptr || data == nullptr || scales == nullptr || rows <= 0 || cols <= 0 || rows % 32 != 0 ||
      stride % 2 != 0 || cols % 2 != 0 || !host::aligned16(data) || !host::aligned4(source))
    return cudaErrorInvalidValue;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  if (rows % kTqRows == 0 && cols % kTqCols == 0 && stride % 8 == 0 && host::aligned16(source))
    quantize_transposed_tiled_kernel<<<info.sm_count * 4, 256, 0, stream>>>(source, stride, rows, cols, data, scales);
  else
    quantize_transposed_kernel<<<info.sm_count * 8, 256, 0, stream>>>(source, stride, rows, cols, data, scales);
  status = cudaGetLastError();
  if (status == cudaSuccess) host::count_launch();
  return status;
}

// detail/gemm.cuh supported_problem + the MXFP8 geometry domain (api/forward_mxfp8.cuh:95-145):
// K a multiple of 128 (whole scale atoms), 16-byte rows.
bool supported_mx_problem(const fuse_gemm_problem& g) {
  return g.m > 0 && g.n > 0 && g.k > 0 && g.l == 1 && !g.transpose_a && !g.transpose_b && g.k % 128 == 0 &&
         g.n % 8 == 0 && (g.stride_d.row < 0 || (g.stride_d.row >= g.n && g.stride_d.row % 8 == 0)) &&
         (g.stride_b.row < 0 || (g.stride_b.row >= g.k && g.stride_b.row % 8 == 0)) &&
         (g.max_swizzle_size == 1 || g.max_swizzle_size == 2 || g.max_swizzle_size == 4 ||
          g.max_swizzle_size == 8) &&
         g.raster >= FUSE_RASTER_HEURISTIC && g.raster <= FUSE_RASTER_ALONG_N;
}

struct WeightScratch {
  uint8_t* data;
  uint8_t* scales;
  size_t bytes;
};
WeightScratch weight_scratch(const fuse_gemm_problem& g, void* memory) {
  WeightScratch w;
  const size_t data = align256(size_t(g.n) * size_t(g.k));
  w.data = static_cast<uint8_t*>(memory);
  w.scales = w.data ? w.data + data : nullptr;
  w.bytes = data + align256(scale_bytes(g.n, g.k));
  return w;
}

enum class MxPhase { kFull, kPrepareOnly, kPrequantized, kComputeOnly };

cudaError_t qkv_forward_mxfp8(const fuse_mxfp8_gemm_a2a_params& mp, const fuse_b200_options* options,
                              cudaStream_t stream, MxPhase phase) {
  const fuse_gemm_a2a_params& p = mp.projection;
  const fuse_gemm_problem& g = p.gemm;
  if (!supported_mx_problem(g) || !std::isfinite(p.alpha) || p.epoch == 0 || p.num_comm_ctas < 0)
    return cudaErrorInvalidValue;
  // num_comm_ctas == 0: Auto -- the epilogue push (no communication CTA), or the planned budget
  // when the caller asks for the communication-CTA route; the GEMM-only launch then uses every SM
  if (mp.postprocess.q_gamma != nullptr || mp.postprocess.cos != nullptr) return cudaErrorNotSupported;
  const WeightScratch w = weight_scratch(g, mp.workspace);
  if (mp.workspace == nullptr || reinterpret_cast<uintptr_t>(mp.workspace) % 256 != 0 ||
      mp.workspace_bytes < w.bytes)
    return cudaErrorInvalidValue;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  if (p.num_comm_ctas >= info.sm_count) return cudaErrorInvalidValue;
  const int64_t ldb = packed_or(g.stride_b.row, g.k);
  if (phase == MxPhase::kPrepareOnly)
    return quantize_rows(p.rhs_nt, ldb, g.n, g.k, w.data, w.scales, stream);
  if (mp.activation.data == nullptr || mp.activation.scales == nullptr ||
      mp.activation.data_bytes < size_t(g.m) * size_t(g.k) ||
      mp.activation.scale_bytes < scale_bytes(g.m, g.k) || !host::aligned16(mp.activation.data) ||
      !host::aligned16(mp.activation.scales) || !host::aligned16(p.rhs_nt) || !host::aligned16(p.local_output))
    return cudaErrorInvalidValue;

  const fuse_ulysses_route& r = p.route;
  const bool routed = phase != MxPhase::kComputeOnly;
  if (routed) {
    if (r.world_size <= 0 || r.world_size > FUSE_MAX_WORLD_SIZE || r.rank < 0 || r.rank >= r.world_size ||
        r.batch <= 0 || r.seq_local <= 0 || r.q_heads <= 0 || r.kv_heads <= 0 || r.head_dim <= 0 ||
        r.kind != FUSE_ROUTE_QKV_GQA_PACK || r.direction != FUSE_ROUTE_FORWARD || r.qkv_peer_interleaved ||
        r.defer_v_a2a || r.cyclic_peer_order || r.q_heads % r.world_size != 0 ||
        r.kv_heads % r.world_size != 0 || r.q_heads % r.kv_heads != 0 || r.head_dim % 8 != 0 ||
        int64_t(r.seq_local) * r.world_size != r.global_seq || int64_t(r.batch) * r.seq_local != g.m ||
        (int64_t(r.q_heads) + 2 * int64_t(r.kv_heads)) * r.head_dim != g.n)
      return cudaErrorNotSupported;
    for (int peer = 0; peer < r.world_size; ++peer)
      if (!host::aligned16(p.peer_output[peer]) || !host::aligned4(p.peer_route_done_epoch[peer]))
        return cudaErrorNotSupported;
  }

  const int block_n = launch::choose_block_n(g.n, options);
  Operands maps;
  if ((status = encode_operand_u8(&maps.a, mp.activation.data, g.m, g.k, g.k, kBlockM)) != cudaSuccess) return status;
  if ((status = encode_operand_u8(&maps.b, w.data, g.n, g.k, g.k, block_n)) != cudaSuccess) return status;

  // Epilogue push by default; communication CTAs when asked for (they need the tile flags).
  const bool direct = routed && !(options && (options->flags & FUSE_B200_QKV_ROUTE_COMM_CTAS) &&
                                  host::aligned4(p.ready));
  const int planned_comm =
      p.num_comm_ctas ? p.num_comm_ctas
                      : planner::choose(planner::kQkvPushMx, 2.0 * double(g.m) * g.n * g.k, double(g.m) * g.n * 2.0,
                                        int64_t(host::ceil_div(g.m, kBlockM)) * host::ceil_div(g.n, 256), info.sm_count, 1,
                                        0, false)
                            .comm_ctas;
  FusedParams f{};
  launch::fill_core(&f, g.m, g.n, g.k, block_n, (routed && !direct) ? planned_comm : 0, p.alpha, 0.0f,
                    p.local_output, packed_or(g.stride_d.row, g.n),
                    g.raster == FUSE_RASTER_ALONG_N ? FUSE_RASTER_ALONG_N : FUSE_RASTER_ALONG_M,
                    g.max_swizzle_size);
  f.sfa = mp.activation.scales;
  f.sfb = w.scales;
  f.k_atoms = g.k / 128;
  f.ready = p.ready;
  f.flags = options ? options->flags : 0u;
  f.wait = host::make_wait(info, p.epoch, options ? options->wait_budget_ns : 0);
  copy_trace(&f, options);
  if (phase == MxPhase::kFull) {  // the master weight is quantised inside the kernel, every call
    f.wq_source = p.rhs_nt;
    f.wq_data = w.data;
    f.wq_scales = w.scales;
    f.wq_rows = g.n;
    f.wq_k = g.k;
    f.wq_stride = ldb;
  }
  StoreMaps stores{};
  if (!routed) {
    DeviceInfo reduced = info;
    reduced.sm_count = info.sm_count - p.num_comm_ctas;  // compute budget of the fused kernel
    if (block_n == 256 && g.k % 128 == 0 && reduced.sm_count % 2 == 0 && launch::pair_tiles_requested()) {
      Operands pair_maps = maps;
      CUtensorMap sfa_map, sfb_map;
      if (encode_operand_u8(&pair_maps.b, w.data, g.n, g.k, g.k, launch::kPairMxBRows) == cudaSuccess &&
          launch::encode_scale_atoms(&sfa_map, f.sfa, g.m, g.k) == cudaSuccess &&
          launch::encode_scale_atoms(&sfb_map, f.sfb, g.n, g.k) == cudaSuccess)
        return launch::launch_pair_kernel<kModePlain, StoreMaps, true>(pair_maps, sfa_map, sfb_map, stores, f,
                                                                       g.max_swizzle_size, reduced, stream, 0.0);
    }
    return launch_mode<kModePlain, false, false, true>(maps, stores, f, block_n, reduced, stream, true);
  }
  f.qkv.world = r.world_size;
  f.qkv.rank = r.rank;
  f.qkv.batch = r.batch;
  f.qkv.seq_local = r.seq_local;
  f.qkv.global_seq = r.global_seq;
  f.qkv.q_heads = r.q_heads;
  f.qkv.kv_heads = r.kv_heads;
  f.qkv.head_dim = r.head_dim;
  for (int peer = 0; peer < r.world_size; ++peer) {
    f.qkv.peer_output[peer] = p.peer_output[peer];
    f.qkv.peer_done[peer] = p.peer_route_done_epoch[peer];
  }
  if (!direct) return launch_mode<kModeQkvPush, false, false, true>(maps, stores, f, block_n, info, stream, false);
  bool tma = !vector_epilogue_requested(options) && r.head_dim % 64 == 0 && r.seq_local % kBlockM == 0;
  if (tma)
    tma = encode_peer_store_maps(&stores, p.peer_output, r.world_size, uint64_t(r.batch) * uint64_t(r.global_seq),
                                 int64_t(r.q_heads) / r.world_size * r.head_dim,
                                 int64_t(r.kv_heads) / r.world_size * r.head_dim);
  if (tma && block_n == 256 && g.k % 128 == 0 && info.sm_count % 2 == 0 && launch::pair_tiles_requested()) {
    Operands pair_maps = maps;
    CUtensorMap sfa_map, sfb_map;
    if (encode_operand_u8(&pair_maps.b, w.data, g.n, g.k, g.k, launch::kPairMxBRows) == cudaSuccess &&
        launch::encode_scale_atoms(&sfa_map, f.sfa, g.m, g.k) == cudaSuccess &&
        launch::encode_scale_atoms(&sfb_map, f.sfb, g.n, g.k) == cudaSuccess)
      return launch::launch_pair_kernel<kModeQkvDirect, StoreMaps, true>(pair_maps, sfa_map, sfb_map, stores, f,
                                                                         g.max_swizzle_size, info, stream, 0.0);
  }
  return launch_mode<kModeQkvDirect, false, false, true>(maps, stores, f, block_n, info, stream, tma);
}

struct LhsScratch {
  WeightScratch weights;
  uint8_t* a;
  uint8_t* sfa;
  uint32_t* ready;
  size_t ready_words, bytes;
};
// Scratch of the output-projection operator: quantised weight, gathered lhs bytes and scales,
// and the invocation-private (M tile, K shard) flags (sized for every supported world size, as
// csrc/operators/sm103/detail/quantization.cuh:50-83 does).
LhsScratch lhs_scratch(const fuse_gemm_problem& g, void* memory) {
  LhsScratch w;
  w.weights = weight_scratch(g, memory);
  const size_t data = align256(size_t(g.m) * size_t(g.k));
  const size_t scales = align256(scale_bytes(g.m, g.k));
  w.ready_words = size_t(host::ceil_div(g.m, kBlockM)) * FUSE_MAX_WORLD_SIZE * FUSE_READY_FLAG_STRIDE;
  uint8_t* base = memory ? static_cast<uint8_t*>(memory) + w.weights.bytes : nullptr;
  w.a = base;
  w.sfa = base ? base + data : nullptr;
  w.ready = base ? reinterpret_cast<uint32_t*>(base + data + scales) : nullptr;
  w.bytes = w.weights.bytes + data + scales + align256(w.ready_words * sizeof(uint32_t));
  return w;
}

cudaError_t oproj_forward_mxfp8(const fuse_mxfp8_a2a_gemm_params& mp, const fuse_b200_options* options,
                                cudaStream_t stream) {
  const fuse_a2a_gemm_params& p = mp.projection;
  const fuse_gemm_problem& g = p.gemm;
  const fuse_ulysses_route& r = p.route;
  if (!supported_mx_problem(g) || !std::isfinite(p.alpha) || p.epoch == 0 || p.num_comm_ctas < 0 ||
      p.lhs_policy != 0)
    return cudaErrorInvalidValue;
  if (mp.postprocess.residual != nullptr || mp.overlap_postnorm) return cudaErrorNotSupported;
  // m_window_tiles / n_group_tiles shape the reference scheduler's tile windows
  // (csrc/operators/sm103/detail/persistent_gemm.cuh:55-59: both powers of two when either is set).
  // They do not change results; this library walks its own order, so valid values are accepted as
  // hints and an invalid pair is refused as the reference refuses it.
  if (mp.m_window_tiles != 0 || mp.n_group_tiles != 0) {
    auto power_of_two = [](int32_t v) { return v > 0 && (v & (v - 1)) == 0; };
    if (!power_of_two(mp.m_window_tiles) || !power_of_two(mp.n_group_tiles)) return cudaErrorNotSupported;
  }
  const LhsScratch w = lhs_scratch(g, mp.workspace);
  if (mp.workspace == nullptr || reinterpret_cast<uintptr_t>(mp.workspace) % 256 != 0 ||
      mp.workspace_bytes < w.bytes)
    return cudaErrorInvalidValue;
  DeviceInfo info;
  cudaError_t status = check_device(&info);
  if (status != cudaSuccess) return status;
  if (p.num_comm_ctas >= info.sm_count) return cudaErrorInvalidValue;
  // Auto: the planner's choice (embedded copy warps, or a communication budget); explicit: exactly that
  const planner::Choice plan = launch::plan_transfer(planner::kLhsPullMx, g.m, g.n, g.k, double(g.m) * g.k * (1.0 + 1.0 / 32),
                                                     info.sm_count, p.num_comm_ctas, true, p.route.world_size);
  const int num_comm_ctas = p.num_comm_ctas ? p.num_comm_ctas : (plan.comm_ctas ? plan.comm_ctas : 16);
  if (r.world_size <= 0 || r.world_size > FUSE_MAX_WORLD_SIZE || r.rank < 0 || r.rank >= r.world_size ||
      r.batch <= 0 || r.seq_local <= 0 || r.kind != FUSE_ROUTE_HEAD_TO_SEQUENCE ||
      r.direction != FUSE_ROUTE_INVERSE || int64_t(r.seq_local) * r.world_size != r.global_seq ||
      int64_t(r.batch) * r.seq_local != g.m || g.k % r.world_size != 0 ||
      // whole scale atoms per shard (api/forward_mxfp8.cuh: peer K shard a multiple of 128) and
      // 128-row groups that map to one aligned source group
      (g.k / r.world_size) % 128 != 0 || r.seq_local % 128 != 0 ||
      (r.causal_load_balanced && (r.seq_local / 2) % 128 != 0))
    return cudaErrorNotSupported;
  const int shard = g.k / r.world_size;
  const size_t rows_global = size_t(r.batch) * size_t(r.global_seq);
  for (int peer = 0; peer < r.world_size; ++peer) {
    const fuse_mxfp8_activation& a = mp.activation[peer];
    if (!host::aligned16(a.data) || !host::aligned16(a.scales) || a.data_bytes < rows_global * size_t(shard) ||
        a.scale_bytes < scale_bytes(int64_t(rows_global), shard))
      return cudaErrorInvalidValue;
  }
  if (!host::aligned16(p.rhs_nt) || !host::aligned16(p.output)) return cudaErrorInvalidValue;

  const int block_n = launch::choose_block_n(g.n, options);
  Operands maps;
  if ((status = encode_operand_u8(&maps.a, w.a, g.m, g.k, g.k, kBlockM)) != cudaSuccess) return status;
  if ((status = encode_operand_u8(&maps.b, w.weights.data, g.n, g.k, g.k, block_n)) != cudaSuccess) return status;

  FusedParams f{};
  launch::fill_core(&f, g.m, g.n, g.k, block_n, num_comm_ctas, p.alpha, 0.0f, p.output,
                    packed_or(g.stride_d.row, g.n),
                    g.raster == FUSE_RASTER_ALONG_M ? FUSE_RASTER_ALONG_M : FUSE_RASTER_ALONG_N,
                    g.max_swizzle_size);
  f.sfa = w.sfa;
  f.sfb = w.weights.scales;
  f.k_atoms = g.k / 128;
  f.ready = w.ready;
  f.flags = options ? options->flags : 0u;
  f.wait = host::make_wait(info, p.epoch, options ? options->wait_budget_ns : 0);
  copy_trace(&f, options);
  f.wq_source = p.rhs_nt;
  f.wq_data = w.weights.data;
  f.wq_scales = w.weights.scales;
  f.wq_rows = g.n;
  f.wq_k = g.k;
  f.wq_stride = packed_or(g.stride_b.row, g.k);
  f.clear_words = w.ready;
  f.clear_count = int64_t(host::ceil_div(g.m, kBlockM)) * r.world_size * FUSE_READY_FLAG_STRIDE;
  f.lhs.world = r.world_size;
  f.lhs.rank = r.rank;
  f.lhs.seq_local = r.seq_local;
  f.lhs.global_seq = r.global_seq;
  f.lhs.shard_width = shard;
  f.lhs.causal = r.causal_load_balanced ? 1 : 0;
  f.lhs.cyclic = r.cyclic_peer_order ? 1 : 0;
  f.lhs.input_epoch = p.input_epoch;
  f.lhs.staging = reinterpret_cast<uint16_t*>(w.a);
  f.lhs.lda = g.k;
  f.lhs.element_bytes = 1;
  f.lhs.local_scales = w.sfa;
  f.lhs.k_atoms = g.k / 128;
  f.lhs.shard_atoms = shard / 128;
  for (int peer = 0; peer < r.world_size; ++peer) {
    f.lhs.peer_input[peer] = reinterpret_cast<const uint16_t*>(mp.activation[peer].data);
    f.lhs.peer_scales[peer] = mp.activation[peer].scales;
    f.lhs.peer_input_ready[peer] = p.peer_input_ready[peer];
  }
  plan_lhs_slices(&f, info.sm_count);
  plan_join(&f, block_n, info.sm_count, double(g.m) * g.k * (1.0 + 1.0 / 32), true);
  if (!(f.flags & kFlagVectorPull)) {
    LhsPullMaps pull{};
    if (launch::encode_lhs_pull_maps(&pull, f, uint64_t(r.batch) * uint64_t(r.global_seq))) {
      if (block_n == 256 && g.k % 128 == 0 && num_comm_ctas % 2 == 0 && info.sm_count % 2 == 0 &&
          launch::pair_tiles_requested()) {
        // CTA pairs: whole pairs of communication CTAs, 256-row tiles
        Operands pair_maps = maps;
        CUtensorMap sfa_map, sfb_map;
        FusedParams pf = f;
        pf.lhs.m_group = 2 * launch::wave_m_group_pairs(pf, info.sm_count, launch::kPairMxBlockN);
        if (encode_operand_u8(&pair_maps.b, w.weights.data, g.n, g.k, g.k, launch::kPairMxBRows) == cudaSuccess &&
            launch::encode_scale_atoms(&sfa_map, f.sfa, g.m, g.k) == cudaSuccess &&
            launch::encode_scale_atoms(&sfb_map, f.sfb, g.n, g.k) == cudaSuccess)
        {
          if (launch::embedded_copy_selected(p.num_comm_ctas, plan))
            return launch::launch_pair_kernel<kModeLhsPull, LhsPullMaps, true, false, false, true>(
                pair_maps, sfa_map, sfb_map, pull, pf, g.max_swizzle_size, info, stream, 0.0);
          return launch::launch_pair_kernel<kModeLhsPull, LhsPullMaps, true>(
              pair_maps, sfa_map, sfb_map, pull, pf, g.max_swizzle_size, info, stream, double(g.m) * g.k * (1.0 + 1.0 / 32));
        }
      }
    }
    if (launch::encode_lhs_pull_maps(&pull, f, uint64_t(r.batch) * uint64_t(r.global_seq)))
      return launch_mode<kModeLhsPull, false, false, true, LhsPullMaps>(maps, pull, f, block_n, info, stream,
                                                                        !vector_epilogue_requested(options));
  }
  f.lhs.virt = 1;  // bulk-copy or vector pull: one gate per shard
  f.lhs.virt_width = f.lhs.shard_width;
  if (f.lhs.gate_start != 0) f.lhs.gate_start = f.lhs.rank;
  StoreMaps stores{};
  return launch_mode<kModeLhsPull, false, false, true>(maps, stores, f, block_n, info, stream,
                                                       !vector_epilogue_requested(options));
}

}  // namespace
}  // namespace fuse_b200

extern "C" {

using namespace fuse_b200;

int fuse_gemm_a2a_mxfp8_activation_size(const fuse_gemm_problem* g, size_t* data_bytes, size_t* scale_bytes_out) {
  if (g == nullptr || data_bytes == nullptr || scale_bytes_out == nullptr || g->m <= 0 || g->k <= 0 ||
      g->k % 32 != 0)
    return int(cudaErrorInvalidValue);
  *data_bytes = size_t(g->m) * size_t(g->k);
  *scale_bytes_out = scale_bytes(g->m, g->k);
  return 0;
}

int fuse_quantize_gemm_a2a_mxfp8_activation(const fuse_gemm_problem* g, const fuse_bf16* source,
                                            const fuse_mxfp8_activation* output, fuse_stream stream) {
  if (g == nullptr || output == nullptr || output->data_bytes < size_t(g->m) * size_t(g->k) ||
      output->scale_bytes < scale_bytes(g->m, g->k))
    return int(cudaErrorInvalidValue);
  return int(quantize_rows(source, launch::packed_or(g->stride_a.row, g->k), g->m, g->k,
                           const_cast<uint8_t*>(output->data), const_cast<uint8_t*>(output->scales),
                           reinterpret_cast<cudaStream_t>(stream)));
}

int fuse_gemm_a2a_mxfp8_workspace_size(const fuse_gemm_problem* g, size_t* bytes) {
  if (g == nullptr || bytes == nullptr || g->n <= 0 || g->k <= 0) return int(cudaErrorInvalidValue);
  *bytes = weight_scratch(*g, nullptr).bytes;
  return 0;
}

int fuse_launch_gemm_a2a_mxfp8_cutlass_ex(const fuse_mxfp8_gemm_a2a_params* p, const fuse_b200_options* o,
                                          fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  return int(qkv_forward_mxfp8(*p, o, reinterpret_cast<cudaStream_t>(s), MxPhase::kFull));
}
int fuse_launch_gemm_a2a_mxfp8_cutlass(const fuse_mxfp8_gemm_a2a_params* p, fuse_stream s) {
  return fuse_launch_gemm_a2a_mxfp8_cutlass_ex(p, nullptr, s);
}
int fuse_prepare_gemm_a2a_mxfp8(const fuse_mxfp8_gemm_a2a_params* p, fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  return int(qkv_forward_mxfp8(*p, nullptr, reinterpret_cast<cudaStream_t>(s), MxPhase::kPrepareOnly));
}
int fuse_launch_gemm_a2a_mxfp8_prequantized_ex(const fuse_mxfp8_gemm_a2a_params* p, const fuse_b200_options* o,
                                               fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  return int(qkv_forward_mxfp8(*p, o, reinterpret_cast<cudaStream_t>(s), MxPhase::kPrequantized));
}
int fuse_launch_gemm_a2a_mxfp8_prequantized(const fuse_mxfp8_gemm_a2a_params* p, fuse_stream s) {
  return fuse_launch_gemm_a2a_mxfp8_prequantized_ex(p, nullptr, s);
}
int fuse_launch_gemm_a2a_mxfp8_compute_reference(const fuse_mxfp8_gemm_a2a_params* p, fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  return int(qkv_forward_mxfp8(*p, nullptr, reinterpret_cast<cudaStream_t>(s), MxPhase::kComputeOnly));
}

int fuse_b200_quantize_mxfp8(const fuse_bf16* source, int64_t row_stride, int32_t rows, int32_t k, uint8_t* data,
                             uint8_t* scales, fuse_stream s) {
  return int(quantize_rows(source, row_stride, rows, k, data, scales, reinterpret_cast<cudaStream_t>(s)));
}
int fuse_b200_quantize_mxfp8_transposed(const fuse_bf16* source, int64_t row_stride, int32_t rows, int32_t cols,
                                        uint8_t* data, uint8_t* scales, fuse_stream s) {
  return int(quantize_transposed(source, row_stride, rows, cols, data, scales, reinterpret_cast<cudaStream_t>(s)));
}
size_t fuse_b200_mxfp8_scale_bytes(int64_t rows, int64_t k) { return scale_bytes(rows, k); }

}  // extern "C"

extern "C" {

int fuse_a2a_gemm_mxfp8_activation_size(const fuse_gemm_problem* g, const fuse_ulysses_route* r, size_t* data_bytes,
                                        size_t* scale_bytes_out) {
  if (g == nullptr || r == nullptr || data_bytes == nullptr || scale_bytes_out == nullptr || r->world_size <= 0 ||
      g->k <= 0 || g->k % r->world_size != 0 || r->batch <= 0 || r->global_seq <= 0)
    return int(cudaErrorInvalidValue);
  const int64_t rows = int64_t(r->batch) * r->global_seq, shard = g->k / r->world_size;
  *data_bytes = size_t(rows) * size_t(shard);
  *scale_bytes_out = scale_bytes(rows, shard);
  return 0;
}
int fuse_a2a_gemm_mxfp8_workspace_size(const fuse_gemm_problem* g, size_t* bytes) {
  if (g == nullptr || bytes == nullptr || g->m <= 0 || g->n <= 0 || g->k <= 0) return int(cudaErrorInvalidValue);
  *bytes = lhs_scratch(*g, nullptr).bytes;
  return 0;
}
int fuse_a2a_gemm_mxfp8_workspace_size_for_params(const fuse_mxfp8_a2a_gemm_params* p, size_t* bytes) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  return fuse_a2a_gemm_mxfp8_workspace_size(&p->projection.gemm, bytes);
}
static void mx_traits(int32_t epilogue_n, fuse_kernel_traits* out) {
  if (out == nullptr) return;
  *out = {};
  if (epilogue_n != 32 && epilogue_n != 64) return;
  using Layout = fuse_b200::SmemLayout<256, 4, true>;
  *out = {fuse_b200::kBlockM, 256, 128, fuse_b200::kThreads, int32_t(Layout::kDynamicBytes)};
}
void fuse_mxfp8_qkv_cutlass_kernel_traits(int32_t epilogue_n, fuse_kernel_traits* out) { mx_traits(epilogue_n, out); }
void fuse_mxfp8_oproj_cutlass_kernel_traits(int32_t epilogue_n, uint8_t overlap_postnorm, fuse_kernel_traits* out) {
  (void)overlap_postnorm;
  mx_traits(epilogue_n, out);
}
int fuse_a2a_gemm_mxfp8_staging_view(const fuse_mxfp8_a2a_gemm_params* p, fuse_mxfp8_activation* out) {
  if (p == nullptr || out == nullptr || p->workspace == nullptr) return int(cudaErrorInvalidValue);
  const LhsScratch w = lhs_scratch(p->projection.gemm, p->workspace);
  out->data = w.a;
  out->scales = w.sfa;
  out->data_bytes = size_t(p->projection.gemm.m) * size_t(p->projection.gemm.k);
  out->scale_bytes = scale_bytes(p->projection.gemm.m, p->projection.gemm.k);
  return 0;
}
int fuse_launch_a2a_gemm_mxfp8_cutlass_ex(const fuse_mxfp8_a2a_gemm_params* p, const fuse_b200_options* o,
                                          fuse_stream s) {
  if (p == nullptr) return int(cudaErrorInvalidValue);
  return int(oproj_forward_mxfp8(*p, o, reinterpret_cast<cudaStream_t>(s)));
}
int fuse_launch_a2a_gemm_mxfp8_cutlass(const fuse_mxfp8_a2a_gemm_params* p, fuse_stream s) {
  return fuse_launch_a2a_gemm_mxfp8_cutlass_ex(p, nullptr, s);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Entry point that allocates nothing.
//
// Some callers of the MXFP8 QKV operator cannot hand over scratch memory: code running inside a
// CUDA-graph capture or a real-time serving loop must not call cudaMalloc (it synchronises the
// device and is illegal during capture), and plug-ins whose host framework owns the device
// allocator have nothing of their own to carve scratch from.  For them the quantised-weight
// scratch lives in this fixed array inside the library image.  Every GPU that loads the library
// holds these bytes until the process exits, which is why the limit is modest.
// ------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_weight_scratch[FUSE_B200_STATIC_SCRATCH_BYTES];

namespace fuse_b200 {
namespace {

// Device address of the array on each device.  In host code the array's name is only a
// stand-in for the symbol: the address a kernel can use comes from cudaGetSymbolAddress, asked
// once per device with that device current.
std::mutex g_static_scratch_mutex;
void* g_static_scratch_address[64] = {};

cudaError_t static_scratch(void** address) {
  int device = -1;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess) return status;
  if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_address[device] == nullptr) {
    void* ptr = nullptr;
    status = cudaGetSymbolAddress(&ptr, g_static_weight_scratch);
    if (status != cudaSuccess) return status;
    g_static_scratch_address[device] = ptr;
  }
  *address = g_static_scratch_address[device];
  return cudaSuccess;
}

}  // namespace
}  // namespace fuse_b200

extern "C" int fuse_b200_launch_gemm_a2a_mxfp8_static(const fuse_mxfp8_gemm_a2a_params* params, fuse_stream stream) {
  if (params == nullptr) return int(cudaErrorInvalidValue);
  const fuse_gemm_problem& g = params->projection.gemm;
  if (g.n <= 0 || g.k <= 0) return int(cudaErrorInvalidValue);
  const size_t need = fuse_b200::weight_scratch(g, nullptr).bytes;
  if (need > size_t(FUSE_B200_STATIC_SCRATCH_BYTES)) {
    std::fprintf(stderr,
                 "fuse_b200_launch_gemm_a2a_mxfp8_static: weight [%d, %d] needs %zu bytes of scratch, the "
                 "built-in scratch holds %zu; use fuse_launch_gemm_a2a_mxfp8_cutlass with caller scratch\n",
                 g.n, g.k, need, size_t(FUSE_B200_STATIC_SCRATCH_BYTES));
    return int(cudaErrorInvalidValue);
  }
  void* scratch = nullptr;
  const cudaError_t status = fuse_b200::static_scratch(&scratch);
  if (status != cudaSuccess) return int(status);
  fuse_mxfp8_gemm_a2a_params with_scratch = *params;
  with_scratch.workspace = scratch;
  with_scratch.workspace_bytes = size_t(FUSE_B200_STATIC_SCRATCH_BYTES);
  return int(fuse_b200::qkv_forward_mxfp8(with_scratch, nullptr, reinterpret_cast<cudaStream_t>(stream),
                                          fuse_b200::MxPhase::kFull));
}
