// One persistent kernel per fused operator.
//
// CTAs [0, num_comm_ctas) are communication CTAs; the rest are compute CTAs that walk the
// static tile order round-robin.  A compute CTA is warp-specialised:
//
//   warp 0  TMA producer   global -> 128B-swizzled shared tiles, `kStages` deep ring of
//                          full/empty mbarriers
//   warp 1  UMMA issuer    one thread issues tcgen05.mma (cta_group::1, 128 x kBlockN x 16)
//                          into one of two TMEM accumulator stages and commits to mbarriers
//   warp 2  TMEM allocator
//   warps 4-7 epilogue     tcgen05.ld -> alpha/beta -> BF16 -> 16-byte global stores, then
//                          (when the operator routes its output) publishes the tile's epoch
//
// The operator-specific parts are three hooks selected at compile time by `kMode`:
//   * a load gate      (wait until the rows of A this K block reads have arrived),
//   * a tile publisher (release flag after the tile's stores),
//   * the communication role run by the communication CTAs.
//
// Replaces the role-dispatch kernel and CUTLASS collectives of the reference
// (csrc/operators/sm103/detail/persistent_gemm.cuh:186-263, detail/gemm.cuh:112-188,
// detail/cutlass_pipeline.cuh:335-814) with hand-written tcgen05/TMEM code.
#pragma once

#include <type_traits>

#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"
#include "sync.cuh"
#include "tile_order.cuh"

namespace fuse_b200 {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;        // 64 BF16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 256;
constexpr int kEpilogueThreads = 128;
constexpr uint32_t kMnGroupBytes = 64 * kBlockK * 2;  // one [64 K rows x 64 MN] box of an MN-major tile

enum FusedMode : int {
  kModePlain = 0,     // GEMM only
  kModeQkvPush = 1,   // GEMM -> publish tiles -> comm CTAs push to peers' planar Q|K|V
  kModeLhsPull = 2,   // comm CTAs pull the lhs shards from peers -> gated GEMM
  kModeQkvDirect = 3, // GEMM whose epilogue stores each vector to local_output AND to its place
                      // in the owning peer's planar Q|K|V; no communication CTAs, no tile flags
  kModeHeadGate = 4,  // QKV backward data: comm CTAs push this rank's planar dQ/dK/dV into every
                      // destination's packed staging; the GEMM's K loop is gated per (M tile, head)
  kModeGradPull = 5,  // MXFP8 QKV backward data: comm CTAs pull the owners' prequantised planar
                      // gradients (bytes + scale atoms) into the packed lhs, and their BF16
                      // masters into the staging kept for the weight gradient; same head gate
};

enum LaunchFlags : uint32_t {
  // Skip the wait for the peers' completion epochs (single-GPU emulation of several ranks,
  // where the "peers" are later launches on the same stream).
  kFlagSkipPeerWait = 1u,
  // Communication CTAs of the lhs pull move data with 16-byte loads/stores instead of the
  // bulk-copy pipeline (kept for comparison and as the fallback).
  kFlagVectorPull = 8u,
  // Run only one of the two roles of a fused kernel (single-GPU emulation of operators whose
  // GEMM waits for data pushed by other ranks: all ranks push first, then all ranks compute).
  kFlagCommOnly = 32u,
  kFlagComputeOnly = 64u,
};

// Tensor maps of the TMA-store epilogue: the local output and, for the direct QKV push, every
// (peer, segment) planar tensor.  Boxes are 64 columns x 128 rows, 128-byte swizzle.
struct alignas(64) StoreMaps {
  CUtensorMap local;
  CUtensorMap peer[kMaxWorldSize][3];
};
// Tensor maps of the QKV backward sender push: this rank's planar dQ, dK, dV
// ([B*S_global, local_heads*128] BF16, boxes of 128 columns x 64 rows, no swizzle) and every
// destination's packed staging ([M, (q+2kv)*128], same boxes).
struct alignas(64) GradPushMaps {
  CUtensorMap local;
  CUtensorMap plane[3];
  CUtensorMap staging[kMaxWorldSize];
};
// Tensor maps of the MXFP8 QKV backward receiver pull: every owner's planes as E4M3 bytes
// (boxes of 128 bytes x 128 rows) and as BF16 masters (128 columns x 64 rows), the local packed
// lhs bytes and the local packed BF16 staging.
struct alignas(64) GradPullMaps {
  CUtensorMap local;
  CUtensorMap lhs, master;
  CUtensorMap bytes[kMaxWorldSize][3];
  CUtensorMap masters[kMaxWorldSize][3];
};

// Tensor maps of the forward lhs pull: every peer's head shard ([B*S_global, K/world]) and the
// local staging ([M, K]), both typed as 32-bit words so that a box row can be 1 KiB wide; boxes of
// `piece_bytes` x `rows_per_chunk` (one pipeline stage), no swizzle.
struct alignas(64) LhsPullMaps {
  CUtensorMap local;
  CUtensorMap staging;
  CUtensorMap peer[kMaxWorldSize];
  int32_t piece_bytes, rows_per_chunk;
};

struct QkvRoute {
  int32_t world, rank, batch, seq_local, global_seq;
  int32_t q_heads, kv_heads, head_dim;
  int32_t causal;  // head-only (output-projection backward) routes may use the causal row map
  // defer_v (UlyssesRoute::defer_v_a2a, csrc/operators/sm103/detail/gemm_a2a.cuh:199-215,521-533):
  // V stays in the local output; Q and K of a destination's heads share ONE row-major tensor
  // [B*S_global, q_local + kv_local] there (Q columns, then K columns).
  int32_t defer_v;
  // interleaved (UlyssesRoute::qkv_peer_interleaved, csrc/operators/sm103/detail/gemm_a2a.cuh:404-415):
  // the projection weight was prepacked offline so that inside Q and inside K physical head p belongs
  // to owner p % world as its local head p / world; V and the routed layout are unchanged.
  int32_t interleaved;
  uint16_t* peer_output[kMaxWorldSize];
  uint32_t* peer_done[kMaxWorldSize];
  uint32_t* completion_epoch;  // local word: the epoch, once this rank's whole local output (V included) is written
};

struct LhsRoute {
  int32_t world, rank, seq_local, global_seq;
  int32_t shard_width;        // K / world, elements
  int32_t causal, cyclic;
  const uint16_t* peer_input[kMaxWorldSize];
  const uint32_t* peer_input_ready[kMaxWorldSize];
  uint32_t input_epoch;
  uint16_t* staging;          // [M, lda]
  int64_t lda;
  // Block-scaled lhs: one-byte elements plus the native scale atoms of every peer's shard
  // ([B*S_global, K/world]) which are re-homed into the local [M, K] scale storage.
  int32_t element_bytes;      // 2 (BF16) or 1 (E4M3)
  const uint8_t* peer_scales[kMaxWorldSize];
  uint8_t* local_scales;
  int32_t k_atoms, shard_atoms;  // K/128 and (K/world)/128
  // Gate granularity: every shard is cut into `virt` column slices of virt_width elements, each
  // with its own flag (word 2v of the shard's flag line) and arrival counter (word 2v + 1), so
  // that a GEMM tile starts on the first slice instead of the whole shard.  m_group: M tiles one
  // GEMM wave works on together; their slices are delivered side by side.
  int32_t virt, virt_width, m_group;
  // The GEMM walks K starting at this rank's own shard (gate_start = first column slice of it,
  // k_block_start the matching K block) and wraps around: the first K blocks need no transfer,
  // and at any moment every rank pulls from a different peer.
  int32_t gate_start, k_block_start;
};

// QKV backward reverse route (head -> sequence), sender side: this rank holds planar
// dQ, dK, dV for its local heads and all global rows, and writes each destination's rows into
// that destination's packed staging [M, (q + 2 kv) * head_dim].
struct GradRoute {
  int32_t world, rank, seq_local, global_seq, m;   // m = rows per rank (same on every rank)
  int32_t q_heads, kv_heads, head_dim, causal;
  int32_t m_group;                                  // M tiles one GEMM wave works on together (>= 1)
  const uint16_t* grad[3];                          // dQ, dK, dV planes of this rank
  uint16_t* peer_staging[kMaxWorldSize];
  uint32_t* peer_ready[kMaxWorldSize];              // [m_tiles * (q + 2 kv)] flags on each peer
  // Receiver pull of prequantised gradients (head_dim == 128: one scale atom per head and
  // 128-row group): every owner's planes as E4M3 bytes, native scales and BF16 masters.
  const uint8_t* peer_bytes[kMaxWorldSize][3];
  const uint8_t* peer_scales[kMaxWorldSize][3];
  const uint16_t* peer_master[kMaxWorldSize][3];
  uint8_t* lhs_bytes;                               // packed [M, (q + 2 kv) * 128] E4M3
  uint8_t* lhs_scales;                              // its native scale storage
  uint16_t* master_staging;                         // packed BF16 [M, (q + 2 kv) * 128]
};

struct FusedParams {
  int32_t m, n, k;
  TileOrder order;
  int32_t num_comm_ctas;
  float alpha, beta;
  uint16_t* d;
  int64_t ldd;
  // Block-scaled operands: native K32 scale storage of A ([M,K]) and B ([N,K]) -- 512-byte
  // atoms of 128 rows x 4 K-blocks, K atoms before row atoms -- and K/128.
  const uint8_t* sfa;
  const uint8_t* sfb;
  int32_t k_atoms;
  // In-kernel preparation run by every CTA before the roles start (block-scaled kernels):
  // quantise the BF16 master weight [wq_rows, wq_k] into B's E4M3 bytes + scales, and clear
  // invocation-private flag words that live in caller scratch.
  const uint16_t* wq_source;
  uint8_t* wq_data;
  uint8_t* wq_scales;
  int32_t wq_rows, wq_k;
  int64_t wq_stride;
  uint32_t* clear_words;
  int64_t clear_count;
  uint32_t* ready;            // tile flags (QkvPush) or (m-tile, k-shard) flags (LhsPull)
  // Tiles [join_tile, tiles) are dealt round-robin to ALL CTAs of the grid: communication CTAs
  // whose transfers are finished by then run the GEMM pipeline on their share (pull and
  // gradient modes).  join_tile == tiles: communication CTAs never compute.
  int64_t join_tile;
  uint32_t flags;
  // Optional %globaltimer trace: CTA `trace_cta` appends (site, timestamp) pairs until the
  // buffer holds trace_capacity records; word 0 of the buffer is the record count.
  unsigned long long* trace;
  uint32_t trace_capacity;
  int32_t trace_cta;
  WaitContext wait;
  QkvRoute qkv;
  LhsRoute lhs;
  GradRoute grad;
};

// Geometry of the bulk-copy pull pipeline run by communication CTAs (lhs_pull_bulk_role).
constexpr int kPullWarps = 7;
constexpr int kPullStages = 2;
constexpr uint32_t kPullStageBytes = 16384;
constexpr int kPullLag = 4;
constexpr int kPullEagerChunks = 4;  // chunks per warp reported without lag at start-up
constexpr int kPullSubRows = 32;
constexpr int kPullSubsPerTile = kBlockM / kPullSubRows;
// Shared memory a communication CTA needs for it: the warps' rings plus their mbarriers.
constexpr uint32_t kPullSmemBytes = kPullWarps * kPullStages * (kPullStageBytes + 8u) + 512u;  // + unit queues

// kMx: block-scaled E4M3 operands (one UE8M0 scale per 32 K values).  A K block is then 128
// one-byte elements (the same 128-byte swizzle rows), each stage also carries the 512-byte scale
// atoms of its A rows and B rows, the accumulator is single-buffered (TMEM also holds the
// scales) and the epilogue stages through one buffer.
template <int kBlockN, int kStages, bool kMx = false>
struct SmemLayout {
  static constexpr uint32_t kABytes = kBlockM * kBlockK * 2;
  static constexpr uint32_t kBBytes = kBlockN * kBlockK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  // Scale atoms per stage: one for the 128 A rows, one per 128 B rows.
  static constexpr uint32_t kSfaBytes = kMx ? 512u : 0u;
  static constexpr uint32_t kSfbBytes = kMx ? 512u * ((kBlockN + 127) / 128) : 0u;
  static constexpr uint32_t kSfOffset = kStages * kStageBytes;
  static constexpr uint32_t kSfStageBytes = kSfaBytes + kSfbBytes;
  // Epilogue staging for TMA stores: 128-row x 64-column BF16 blocks (16 KiB each).
  static constexpr uint32_t kStagingBuffers = kMx ? 1u : 2u;
  static constexpr uint32_t kStagingOffset = kSfOffset + ((kStages * kSfStageBytes + 1023u) & ~1023u);
  static constexpr uint32_t kStagingBlockBytes = kBlockM * 64 * 2;
  static constexpr uint32_t kBarrierOffset = kStagingOffset + kStagingBuffers * kStagingBlockBytes;
  static constexpr uint32_t kAccumStages = (kMx && kBlockN > 240) ? 1u : 2u;
  // + 1: the barrier the UMMA issuer drains on while unwinding (an accumulator-full barrier
  // only ever completes for a finished tile)
  static constexpr uint32_t kNumBarriers = 2 * kStages + 2 * kAccumStages + 1;
  static constexpr uint32_t kTmemSlotOffset = kBarrierOffset + kNumBarriers * 8;
  // Two per-tile route tables (column chunk -> destination base pointer, row pitch) used by
  // the direct-push epilogue, double-buffered by tile parity.
  static constexpr uint32_t kRouteTableOffset = kTmemSlotOffset + 16;
  static constexpr uint32_t kRouteTableBytes = 2 * (kBlockN / 8) * 16;
  static constexpr uint32_t kComputeBytes = kRouteTableOffset + kRouteTableBytes;
  // Communication CTAs of the same launch lay their own pipeline over the same allocation.
  static constexpr uint32_t kBytes = kComputeBytes > kPullSmemBytes ? kComputeBytes : kPullSmemBytes;
  // + 1024 so the kernel can align the base itself; total is above half of the SM's shared
  // memory, which pins residency at exactly one CTA per SM.
  static constexpr uint32_t kDynamicBytes = kBytes + 1024;
  static_assert(kDynamicBytes <= 227 * 1024, "shared memory budget");
  static_assert(kDynamicBytes > 114 * 1024, "must force one CTA per SM");
  // TMEM: accumulators, then (kMx) two sets of scale columns: 4 for A, 4 per 128 B rows.
  static constexpr uint32_t kSfColumns = kMx ? 4u + 4u * ((kBlockN + 127) / 128) : 0u;
  static constexpr uint32_t kTmemSfOffset = kAccumStages * kBlockN;
  static constexpr uint32_t kTmemUsed = kTmemSfOffset + 2 * kSfColumns;
  static constexpr uint32_t kTmemColumns = kTmemUsed <= 256 ? 256u : 512u;
  static_assert(kTmemUsed <= 512, "TMEM budget");
};

__device__ __forceinline__ void trace_event(const FusedParams& p, uint32_t site) {
  if (p.trace == nullptr || int32_t(blockIdx.x) != p.trace_cta) return;
  const unsigned long long slot = atomicAdd(p.trace, 1ull);
  if (slot < p.trace_capacity) {
    p.trace[1 + 2 * slot] = (static_cast<unsigned long long>(threadIdx.x) << 32) | site;
    p.trace[2 + 2 * slot] = ptx::globaltimer();
  }
}

// ------------------------------------------------------------------------------------------
// Row mapping shared by the routes: rank-local row -> row of the global [batch, S] axis.
// Contiguous shards (csrc/operators/sm103/detail/gemm_a2a.cuh:115-132) or the causal
// two-chunk assignment (csrc/operators/sm103/detail/a2a_gemm.cuh:410-420).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ int64_t global_row(int32_t world, int32_t rank, int32_t seq_local,
                                              int32_t global_seq, bool causal, int32_t local_row) {
  const int32_t batch = local_row / seq_local;
  const int32_t seq = local_row - batch * seq_local;
  if (causal) {
    const int32_t half = seq_local / 2;
    const int32_t chunk = seq < half ? rank : 2 * world - rank - 1;
    return int64_t(batch) * global_seq + int64_t(chunk) * half + seq % half;
  }
  return int64_t(batch) * global_seq + int64_t(rank) * seq_local + seq;
}

// Owner rank and column inside the owner's segment of position `within` of segment `segment`
// (0 Q, 1 K, 2 V; `local_width` = the segment's width per rank).
__device__ __forceinline__ void qkv_owner_column(const QkvRoute& r, int32_t segment, int32_t within,
                                                 int32_t local_width, int32_t& owner, int32_t& local_col) {
  if (r.interleaved && segment < 2) {
    const int32_t head = within / r.head_dim;
    owner = head % r.world;
    local_col = head / r.world * r.head_dim + (within - head * r.head_dim);
  } else {
    owner = within / local_width;
    local_col = within - owner * local_width;
  }
}

// Destination of one 8-column chunk of the packed QKV feature axis: base pointer of row 0 in
// the owning rank's planar Q | K | V tensor and that tensor's row pitch
// (include/fuse/layout/ulysses.h:77-107; csrc/operators/sm103/detail/gemm_a2a.cuh:190-215).
__device__ __forceinline__ void qkv_chunk_destination(const QkvRoute& r, int32_t feature,
                                                      uint16_t*& base, int64_t& stride) {
  const int64_t rows_total = int64_t(r.batch) * r.global_seq;
  const int32_t q_width = r.q_heads * r.head_dim, kv_width = r.kv_heads * r.head_dim;
  const int32_t q_local = q_width / r.world, kv_local = kv_width / r.world;
  const int32_t segment = feature < q_width ? 0 : (feature < q_width + kv_width ? 1 : 2);
  const int32_t within = feature - (segment == 0 ? 0 : q_width + (segment == 2 ? kv_width : 0));
  const int32_t local_width = segment == 0 ? q_local : kv_local;
  int32_t owner, local_col;
  qkv_owner_column(r, segment, within, local_width, owner, local_col);
  if (r.defer_v) {
    if (segment == 2) return;  // V is not routed: base stays null and the chunk is skipped
    base = r.peer_output[owner] + (segment == 1 ? q_local : 0) + local_col;
    stride = q_local + kv_local;
    return;
  }
  const int64_t segment_base =
      segment == 0 ? 0 : rows_total * q_local + (segment == 2 ? rows_total * kv_local : 0);
  base = r.peer_output[owner] + segment_base + local_col;
  stride = local_width;
}

// ------------------------------------------------------------------------------------------
// Communication role: forward QKV push.
//
// For each published output tile (same linear order as the producers), copy every 16-byte
// chunk of the tile from the local GEMM output (L2-resident, just written) to its place in
// the owning rank's planar Q | K | V tensor.  Column chunks and rows are mapped once per tile
// into shared-memory tables; the copy itself is 8 independent 16-byte loads followed by 8
// stores per thread.  Address map: include/fuse/layout/ulysses.h:77-107 (feature -> owner,
// local feature) and csrc/operators/sm103/detail/gemm_a2a.cuh:190-215 (planar bases).
// ------------------------------------------------------------------------------------------
template <int kBlockN>
__device__ __forceinline__ void qkv_push_role(const FusedParams& p, uint8_t* smem) {
  constexpr int kChunks = kBlockN / 8;
  uint16_t** col_base = reinterpret_cast<uint16_t**>(smem);                 // [kChunks]
  int64_t* col_stride = reinterpret_cast<int64_t*>(smem + 8 * kChunks);     // [kChunks]
  int64_t* row_dest = reinterpret_cast<int64_t*>(smem + 16 * kChunks);      // [kBlockM]
  uint32_t* ok_slot = reinterpret_cast<uint32_t*>(smem + 16 * kChunks + 8 * kBlockM);
  const QkvRoute& r = p.qkv;
  const int tid = threadIdx.x;
  const int64_t tiles = p.order.count();

  for (int64_t t = blockIdx.x; t < tiles; t += p.num_comm_ctas) {
    int32_t mt, nt;
    p.order.decode(t, mt, nt);
    const int32_t m0 = mt * kBlockM, n0 = nt * kBlockN;
    __syncthreads();  // the previous tile's table readers are done
    if (tid < kChunks) {
      const int32_t feature = n0 + tid * 8;
      uint16_t* base = nullptr;
      int64_t stride = 0;
      if (feature < p.n) qkv_chunk_destination(r, feature, base, stride);
      col_base[tid] = base;
      col_stride[tid] = stride;
    } else if (tid >= 128) {
      const int32_t row = m0 + (tid - 128);
      row_dest[tid - 128] =
          row < p.m ? global_row(r.world, r.rank, r.seq_local, r.global_seq, r.causal != 0, row) : -1;
    }
    if (tid == 0) {
      const int64_t flag = (int64_t(mt) * p.order.n_tiles + nt) * kReadyFlagStride;
      *ok_slot = flag_wait<false>(p.ready + flag, p.wait.epoch, p.wait, kSiteTileReady,
                                  uint32_t(flag / kReadyFlagStride))
                     ? 1u : 0u;
    }
    __syncthreads();
    if (*ok_slot == 0u) break;

    constexpr int kPerThread = kBlockM * kChunks / kThreads;
    constexpr int kUnroll = 8;
    static_assert(kPerThread % kUnroll == 0, "copy unroll");
    for (int j0 = 0; j0 < kPerThread; j0 += kUnroll) {
      uint4 value[kUnroll];
      uint16_t* dst[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int i = tid + (j0 + u) * kThreads;
        const int row = i / kChunks, chunk = i % kChunks;
        uint16_t* base = col_base[chunk];
        const int64_t dest_row = row_dest[row];
        dst[u] = (base != nullptr && dest_row >= 0) ? base + dest_row * col_stride[chunk] : nullptr;
        if (dst[u] != nullptr)
          value[u] = ptx::ld_cg_v4(p.d + int64_t(m0 + row) * p.ldd + n0 + chunk * 8);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (dst[u] != nullptr) ptx::st_v4(dst[u], value[u]);
    }
  }
  __threadfence_system();  // this thread's peer stores are performed before the CTA joins
}

// Cross-rank completion after the grid has joined: tell every destination that this rank's
// pushes into it are complete, then wait until every source has said the same to this rank
// (protocol of csrc/operators/sm103/detail/gemm_a2a.cuh:760-786, with a bounded wait).
__device__ __forceinline__ void qkv_finalize(const FusedParams& p) {
  if (blockIdx.x != 0 || threadIdx.x >= 32) return;
  const QkvRoute& r = p.qkv;
  const int lane = threadIdx.x;
  // A launch in which any wait gave up publishes nothing: its transfers may be incomplete, so
  // the peers must run out their own bounded wait (and record kSitePeerDone) instead of reading
  // half-written rows behind a fresh epoch.
  const bool failed = __shfl_sync(0xffffffffu, lane == 0 && aborted(p.wait) ? 1 : 0, 0) != 0;
  if (failed) return;
  if (lane == 0) ptx::fence_sc_sys();
  __syncwarp();
  if (lane < r.world)
    ptx::st_release_sys(r.peer_done[lane] + r.rank * kReadyFlagStride, p.wait.epoch);
  __syncwarp();
  // (the grid has joined: the whole local output, the deferred V included, is written)
  if (lane == 0 && r.completion_epoch != nullptr) ptx::st_release_sys(r.completion_epoch, p.wait.epoch);
  if (lane < r.world && !(p.flags & kFlagSkipPeerWait))
    flag_wait<true>(r.peer_done[r.rank] + lane * kReadyFlagStride, p.wait.epoch, p.wait,
                    kSitePeerDone, uint32_t(lane));
  __syncwarp();
}

// ------------------------------------------------------------------------------------------
// Communication role: inverse (head -> sequence) pull feeding the output projection.
//
// Unit of work = (M tile, K shard): 128 rows x (K / world) columns read from the owning
// peer's head-sharded tensor [B*S_global, K/world] and written into the local row-major lhs
// staging [M, K] at column shard*K/world.  One warp moves one row at a time with 16-byte
// accesses, four rows in flight per warp.  When the unit is in place the CTA publishes
// ready[(m_tile*world + shard)*32] = epoch.  Address map: benchmarks/sm103/fused_inputs.cuh:79-104;
// unit/flag layout: csrc/operators/sm103/api/policy.cuh:312-329.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void lhs_pull_role(const FusedParams& p, uint8_t* smem) {
  uint32_t* ok_slot = reinterpret_cast<uint32_t*>(smem);
  const LhsRoute& r = p.lhs;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t units = int64_t(p.order.m_tiles) * r.world;
  const int32_t chunks_per_row = r.shard_width / 8;  // 16-byte chunks
  uint32_t upstream_seen = 0;                        // bit per peer (thread 0 only)

  for (int64_t u = blockIdx.x; u < units; u += p.num_comm_ctas) {
    const int32_t mt = int32_t(u / r.world), shard = int32_t(u % r.world);
    const int32_t peer = r.cyclic ? (r.rank + shard) % r.world : shard;
    const int32_t m0 = mt * kBlockM;
    bool ok = true;
    if (r.peer_input_ready[peer] != nullptr) {
      // Upstream producer (attention on the peer) publishes one epoch per tensor.
      __syncthreads();
      if (tid == 0) {
        uint32_t good = 1u;
        if (!((upstream_seen >> peer) & 1u)) {
          good = flag_wait<true>(r.peer_input_ready[peer], r.input_epoch, p.wait,
                                 kSiteUpstreamReady, uint32_t(peer))
                     ? 1u : 0u;
          upstream_seen |= good << peer;
        }
        *ok_slot = good;
      }
      __syncthreads();
      ok = *ok_slot != 0u;
    }
    if (!ok) break;

    const uint16_t* src_base = r.peer_input[peer];
    uint16_t* dst_base = r.staging + int64_t(shard) * r.shard_width;
    const int32_t rows = p.m - m0 < kBlockM ? p.m - m0 : kBlockM;
    constexpr int kRowsInFlight = 4;
    for (int32_t row0 = warp * kRowsInFlight; row0 < rows; row0 += (kThreads / 32) * kRowsInFlight) {
      for (int32_t c0 = lane; c0 < chunks_per_row; c0 += 32 * 2) {
        uint4 value[kRowsInFlight][2];
        bool valid[kRowsInFlight][2];
#pragma unroll
        for (int i = 0; i < kRowsInFlight; ++i) {
          const int32_t row = m0 + row0 + i;
          const int64_t src_row =
              row0 + i < rows
                  ? global_row(r.world, r.rank, r.seq_local, r.global_seq, r.causal != 0, row)
                  : -1;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int32_t c = c0 + j * 32;
            valid[i][j] = src_row >= 0 && c < chunks_per_row;
            if (valid[i][j]) value[i][j] = ptx::ld_cg_v4(src_base + src_row * r.shard_width + c * 8);
          }
        }
#pragma unroll
        for (int i = 0; i < kRowsInFlight; ++i)
#pragma unroll
          for (int j = 0; j < 2; ++j)
            if (valid[i][j])
              ptx::st_v4(dst_base + int64_t(m0 + row0 + i) * r.lda + (c0 + j * 32) * 8, value[i][j]);
      }
    }
    __syncthreads();  // every thread's stores of this unit are issued ...
    if (tid == 0) {
      __threadfence();                    // ... and ordered before the flag at GPU scope,
      ptx::fence_proxy_async_global();    // also for the TMA (async proxy) reads that follow
      for (int32_t v = 0; v < r.virt; ++v)
        ptx::st_release_gpu(p.ready + (int64_t(mt) * r.world + shard) * kReadyFlagStride + 2 * v, p.wait.epoch);
    }
  }
}

// ------------------------------------------------------------------------------------------
// Communication role: the same pull with the copy engine.
//
// A (M tile, K shard) unit is cut into sub-units of kPullSubRows rows, dealt round-robin in unit
// order to the kPullWarps x num_comm_ctas pull warps, so the rows the first GEMM wave needs
// arrive first and through every warp at once.  A warp walks its sub-units in chunks of at most
// kPullStageBytes (whole rows, or pieces of a row wider than a stage) through its own pipeline:
// one thread starts bulk copies peer -> shared memory (kPullStages chunks in flight per warp, so
// NVLink latency is covered by shared memory rather than registers); as a chunk lands the lanes
// start one bulk copy per row shared -> local staging.  Addresses are derived once per sub-unit;
// the per-chunk work of the single issuing warp is a few adds.  When the stores of a sub-unit's
// last chunk have completed (checked kPullLag chunks late, a bulk store's completion takes
// microseconds) the warp counts an arrival in word 1 of the unit's flag line, and the arrival
// that completes the unit publishes word 0 = epoch (arrival counting as in
// csrc/operators/sm103/detail/a2a_gemm.cuh:466-642, but the epoch need not advance by one).
// ------------------------------------------------------------------------------------------

struct PullCursor {
  int32_t sub;        // global sub-unit index; advances by the number of pull warps
  int32_t chunk;      // chunk inside the sub-unit
  int32_t chunks;     // chunks of this sub-unit
  int32_t rows;       // rows of this sub-unit
  int32_t row;        // rank-local row of its first row
  int32_t flag, needed, peer;
  bool contiguous;    // its source rows are consecutive in the peer's tensor
  uint32_t src_col;   // byte offset of its column slice inside a source row
  const uint8_t* src; // source of its first row (valid when contiguous)
  uint8_t* dst;       // destination of its first row
  int32_t data_chunks;       // chunks [data_chunks, chunks) carry the unit's scale atoms
  const uint8_t* scale_src;  // first scale atom of the unit at the source / in local storage
  uint8_t* scale_dst;
};

__device__ __forceinline__ void lhs_pull_bulk_role(const FusedParams& p, uint32_t smem_base) {
  const LhsRoute& r = p.lhs;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp >= kPullWarps) return;
  const uint32_t ring = smem_base + uint32_t(warp) * kPullStages * kPullStageBytes;
  const uint32_t bars = smem_base + kPullWarps * kPullStages * kPullStageBytes +
                        uint32_t(warp) * kPullStages * 8u;
  if (lane == 0) {
    for (int s = 0; s < kPullStages; ++s) ptx::mbar_init(bars + 8u * s, 1);
    ptx::fence_mbar_init();
  }
  __syncwarp();

  const int32_t workers = p.num_comm_ctas * kPullWarps;
  const int32_t worker = warp * p.num_comm_ctas + int32_t(blockIdx.x);  // neighbours on different SMs
  const uint32_t shard_bytes = uint32_t(r.shard_width) * uint32_t(r.element_bytes);  // source row pitch
  const uint32_t unit_bytes = uint32_t(r.virt_width) * uint32_t(r.element_bytes);    // one column slice
  const int32_t unit_atoms = r.virt_width / 128;
  const int32_t gates = r.world * r.virt;  // column slices of one M tile
  const int32_t pieces = int32_t((unit_bytes + kPullStageBytes - 1) / kPullStageBytes);
  // Scale atoms of one unit travel as extra chunks of its first sub-unit: the K atoms of one
  // 128-row group are contiguous at the source and at the destination.
  const bool with_scales = r.local_scales != nullptr;
  constexpr int32_t kAtomsPerChunk = int32_t(kPullStageBytes / 512);
  const int32_t scale_chunks = with_scales ? (unit_atoms + kAtomsPerChunk - 1) / kAtomsPerChunk : 0;
  const int32_t rows_per_chunk =
      pieces == 1 ? (int32_t(kPullStageBytes / unit_bytes) < kPullSubRows ? int32_t(kPullStageBytes / unit_bytes)
                                                                         : kPullSubRows)
                  : 1;
  // A sub-unit is at most two chunks, so that the first units the GEMM waits for are spread
  // over every pull warp (wide rows: a few rows; 1 KiB rows: 32 rows).
  int32_t sub_rows = 2 * rows_per_chunk < kPullSubRows ? 2 * rows_per_chunk : kPullSubRows;
  while (kBlockM % sub_rows != 0) --sub_rows;
  const int32_t subs_per_tile = kBlockM / sub_rows;
  const int32_t subs_total = p.order.m_tiles * gates * subs_per_tile;
  const int32_t row_block = r.causal ? r.seq_local / 2 : r.seq_local;  // rows consecutive at the source
  const int64_t dst_pitch = r.lda * r.element_bytes;

  // Positions `c` on the first sub-unit at or after c.sub that has rows; false past the end.
  auto seek = [&](PullCursor& c) {
    for (; c.sub < subs_total; c.sub += workers) {
      const int32_t unit = c.sub / subs_per_tile, quarter = c.sub - unit * subs_per_tile;
      // unit order: group of m_group M tiles, then column slice, then M tile of the group
      const int32_t per_group = r.m_group * gates;
      const int32_t group = unit / per_group, mt0 = group * r.m_group;
      const int32_t group_size = p.order.m_tiles - mt0 < r.m_group ? p.order.m_tiles - mt0 : r.m_group;
      const int32_t within = unit - group * per_group;
      const int32_t position = within / group_size, mt = mt0 + within - position * group_size;
      const int32_t gate = position + r.gate_start < gates ? position + r.gate_start : position + r.gate_start - gates;
      const int32_t shard = gate / r.virt, slice = gate - shard * r.virt;
      const int32_t rows_in_unit = p.m - mt * kBlockM < kBlockM ? p.m - mt * kBlockM : kBlockM;
      const int32_t row0 = quarter * sub_rows;
      if (row0 >= rows_in_unit) continue;
      c.rows = rows_in_unit - row0 < sub_rows ? rows_in_unit - row0 : sub_rows;
      c.row = mt * kBlockM + row0;
      c.chunk = 0;
      c.data_chunks = ((c.rows + rows_per_chunk - 1) / rows_per_chunk) * pieces;
      c.chunks = c.data_chunks + (quarter == 0 ? scale_chunks : 0);
      c.flag = (mt * r.world + shard) * kReadyFlagStride + 2 * slice;  // word offset of the slice's flag
      c.needed = (rows_in_unit + sub_rows - 1) / sub_rows;
      c.peer = r.cyclic ? (r.rank + shard) % r.world : shard;
      c.contiguous = r.virt == 1 && (c.row % row_block) + c.rows <= row_block;
      c.src_col = uint32_t(slice) * unit_bytes;
      c.src = reinterpret_cast<const uint8_t*>(r.peer_input[c.peer]) +
              global_row(r.world, r.rank, r.seq_local, r.global_seq, r.causal != 0, c.row) * shard_bytes + c.src_col;
      c.dst = reinterpret_cast<uint8_t*>(r.staging) + int64_t(c.row) * dst_pitch +
              int64_t(shard) * shard_bytes + c.src_col;
      if (with_scales) {
        const int64_t src_row = global_row(r.world, r.rank, r.seq_local, r.global_seq, r.causal != 0, mt * kBlockM);
        c.scale_src = r.peer_scales[c.peer] + ((src_row >> 7) * int64_t(r.shard_atoms) + int64_t(slice) * unit_atoms) * 512;
        c.scale_dst = r.local_scales +
                      (int64_t(mt) * r.k_atoms + int64_t(shard) * r.shard_atoms + int64_t(slice) * unit_atoms) * 512;
      }
      return true;
    }
    return false;
  };
  auto advance = [&](PullCursor& c) {
    if (++c.chunk < c.chunks) return true;
    c.sub += workers;
    return seek(c);
  };
  // Geometry of the chunk under a cursor: first row inside the sub-unit, rows, byte range.
  struct Chunk { int32_t row_off, rows; uint32_t col_off, bytes_per_row; };
  auto chunk_of = [&](const PullCursor& c) {
    Chunk k;
    if (c.chunk >= c.data_chunks) {  // scale atoms: one contiguous run, described as a single row
      const int32_t first_atom = (c.chunk - c.data_chunks) * kAtomsPerChunk;
      const int32_t atoms = unit_atoms - first_atom < kAtomsPerChunk ? unit_atoms - first_atom : kAtomsPerChunk;
      k.row_off = 0;
      k.rows = 1;
      k.col_off = uint32_t(first_atom) * 512u;
      k.bytes_per_row = uint32_t(atoms) * 512u;
      return k;
    }
    if (pieces == 1) {
      k.row_off = c.chunk * rows_per_chunk;
      k.rows = c.rows - k.row_off < rows_per_chunk ? c.rows - k.row_off : rows_per_chunk;
      k.col_off = 0;
      k.bytes_per_row = unit_bytes;
    } else {
      k.row_off = c.chunk / pieces;
      k.rows = 1;
      k.col_off = uint32_t(c.chunk - k.row_off * pieces) * kPullStageBytes;
      k.bytes_per_row = unit_bytes - k.col_off < kPullStageBytes ? unit_bytes - k.col_off : kPullStageBytes;
    }
    return k;
  };

  uint32_t upstream_seen = 0;
  bool ok = true;
  auto start_load = [&](const PullCursor& c, int stage) {  // whole warp
    if (r.peer_input_ready[c.peer] != nullptr && !((upstream_seen >> c.peer) & 1u)) {
      uint32_t good = 1u;
      if (lane == 0)
        good = flag_wait<true>(r.peer_input_ready[c.peer], r.input_epoch, p.wait, kSiteUpstreamReady,
                               uint32_t(c.peer)) ? 1u : 0u;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { ok = false; return; }
      upstream_seen |= 1u << c.peer;
    }
    const Chunk k = chunk_of(c);
    const uint32_t dst = ring + uint32_t(stage) * kPullStageBytes;
    const uint32_t bar = bars + 8u * stage;
    if (lane == 0) ptx::mbar_expect_tx(bar, uint32_t(k.rows) * k.bytes_per_row);
    __syncwarp();
    if (c.chunk >= c.data_chunks) {
      if (lane == 0) ptx::bulk_load(dst, c.scale_src + k.col_off, k.bytes_per_row, bar);
    } else if (c.contiguous) {
      // consecutive source rows: one copy for the whole chunk (rows are shard_bytes apart)
      if (pieces == 1) {
        if (lane == 0)
          ptx::bulk_load(dst, c.src + int64_t(k.row_off) * shard_bytes, uint32_t(k.rows) * shard_bytes, bar);
      } else if (lane == 0) {
        ptx::bulk_load(dst, c.src + int64_t(k.row_off) * shard_bytes + k.col_off, k.bytes_per_row, bar);
      }
    } else {
      for (int32_t row = lane; row < k.rows; row += 32) {
        const int64_t src_row = global_row(r.world, r.rank, r.seq_local, r.global_seq, r.causal != 0,
                                           c.row + k.row_off + row);
        ptx::bulk_load(dst + uint32_t(row) * k.bytes_per_row,
                       reinterpret_cast<const uint8_t*>(r.peer_input[c.peer]) + src_row * shard_bytes + c.src_col + k.col_off,
                       k.bytes_per_row, bar);
      }
    }
  };

  // Arrival counting, split in two so that the atomic's round trip overlaps later chunks:
  // `count` adds one finished sub-unit to word 1 of the unit's flag line, `publish` (at the
  // next count) writes word 0 = epoch if that arrival completed the unit.  The rows were
  // written by completed bulk copies and are only read by TMA (the consumer fences the proxies
  // after its acquire); the acq_rel RMW orders them before the count.
  uint32_t counted_before = 0;
  int32_t counted_flag = -1, counted_needed = 1;
  auto publish = [&]() {
    if (lane == 0 && counted_flag >= 0 && (counted_before + 1u) % uint32_t(counted_needed) == 0u)
      ptx::st_release_gpu(p.ready + counted_flag, p.wait.epoch);
    counted_flag = -1;
  };
  auto count = [&](int32_t flag, int32_t needed) {
    publish();
    if (lane == 0)
      counted_before = ptx::atom_acq_rel_gpu_add(p.ready + flag + 1, 1u);
    counted_flag = flag;
    counted_needed = needed;
  };

  PullCursor load_cursor{};
  load_cursor.sub = worker;
  bool more_loads = seek(load_cursor);
  if (!more_loads) return;
  PullCursor store_cursor = load_cursor;
  int32_t issued = 0, consumed = 0;
  while (issued < kPullStages && more_loads) {
    start_load(load_cursor, issued % kPullStages);
    if (!ok) break;
    more_loads = advance(load_cursor);
    ++issued;
  }
  // Sub-units closed by the newest store groups (newest first; -1 = that chunk closed nothing).
  int32_t lag_flag[kPullLag], lag_needed[kPullLag];
#pragma unroll
  for (int i = 0; i < kPullLag; ++i) { lag_flag[i] = -1; lag_needed[i] = 1; }
  bool more_stores = true;
  while (ok && more_stores) {
    const int stage = consumed % kPullStages;
    uint32_t landed = 1u;
    if (lane == 0)
      landed = mbar_wait(bars + 8u * stage, uint32_t(consumed / kPullStages) & 1u, p.wait,
                         kSiteCommStage) ? 1u : 0u;
    landed = __shfl_sync(0xffffffffu, landed, 0);
    if (!landed) { ok = false; break; }
    if (lane == 0) trace_event(p, 1);  // chunk landed
    const Chunk k = chunk_of(store_cursor);
    const uint32_t src = ring + uint32_t(stage) * kPullStageBytes;
    uint8_t* dst = store_cursor.chunk >= store_cursor.data_chunks
                       ? store_cursor.scale_dst + k.col_off
                       : store_cursor.dst + int64_t(k.row_off) * dst_pitch + k.col_off;
    for (int32_t row = lane; row < k.rows; row += 32)
      ptx::bulk_store(dst + int64_t(row) * dst_pitch, src + uint32_t(row) * k.bytes_per_row, k.bytes_per_row);
    ptx::bulk_commit();
    ++consumed;
    if (lane == 0) trace_event(p, 2);  // stores issued
    // Once these stores have finished READING shared memory the stage takes the next load.
    ptx::bulk_wait_read<0>();
    __syncwarp();
    if (more_loads && issued < consumed + kPullStages) {
      start_load(load_cursor, issued % kPullStages);
      if (ok) {
        more_loads = advance(load_cursor);
        ++issued;
      }
    }
    if (lane == 0) trace_event(p, 3);  // next load issued
    ptx::bulk_wait<kPullLag>();  // all but the kPullLag newest store groups are complete ...
    __syncwarp();                // ... for every lane's rows, before lane 0 counts the arrival
    if (lag_flag[kPullLag - 1] >= 0) count(lag_flag[kPullLag - 1], lag_needed[kPullLag - 1]);
#pragma unroll
    for (int i = kPullLag - 1; i > 0; --i) { lag_flag[i] = lag_flag[i - 1]; lag_needed[i] = lag_needed[i - 1]; }
    const bool closes = store_cursor.chunk + 1 == store_cursor.chunks;
    lag_flag[0] = closes ? store_cursor.flag : -1;
    lag_needed[0] = store_cursor.needed;
    more_stores = advance(store_cursor);
    if (lane == 0) trace_event(p, 4);  // bookkeeping done
  }
  ptx::bulk_wait<0>();
  __syncwarp();
  if (ok) {
#pragma unroll
    for (int i = kPullLag - 1; i >= 0; --i)
      if (lag_flag[i] >= 0) count(lag_flag[i], lag_needed[i]);
    publish();
  }
  if (!ok && lane == 0) {
    // Unwinding: loads started but not consumed must land before shared memory goes away.
    for (int32_t i = consumed; i < issued; ++i)
      mbar_wait(bars + 8u * uint32_t(i % kPullStages), uint32_t(i / kPullStages) & 1u, p.wait,
                kSiteDrain, false);
  }
}

// ------------------------------------------------------------------------------------------
// Communication role: QKV backward reverse route, sender push.
//
// Unit of work = (destination rank, destination M tile, one of this rank's local heads of
// dQ / dK / dV): 128 rows x head_dim columns copied with 16-byte accesses from the local plane
// [B*S_global, local_heads*head_dim] into the destination's packed staging at the head's place
// in [all Q, all K, all V] order, then ready[m_tile * heads + head] = epoch is released at
// system scope on the destination (csrc/operators/sm103/detail/backward.cuh:208-279).
// Destinations are visited starting from the next rank so that ranks do not all write to the
// same peer at once.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void grad_push_role(const FusedParams& p) {
  const GradRoute& g = p.grad;
  const int tid = threadIdx.x;
  const int32_t m_tiles = (g.m + kBlockM - 1) / kBlockM;
  const int32_t q_local = g.q_heads / g.world, kv_local = g.kv_heads / g.world;
  const int32_t local_heads = q_local + 2 * kv_local;
  const int32_t heads_total = g.q_heads + 2 * g.kv_heads;
  const int32_t width = heads_total * g.head_dim;
  const int32_t chunks_per_row = g.head_dim / 8;
  const int64_t units = int64_t(m_tiles) * g.world * local_heads;
  for (int64_t u = blockIdx.x; u < units; u += p.num_comm_ctas) {
    const int32_t head_slot = int32_t(u % local_heads);
    const int32_t rest = int32_t(u / local_heads);
    const int32_t dest = (g.rank + 1 + rest % g.world) % g.world;
    const int32_t mt = rest / g.world;
    const int32_t segment = head_slot < q_local ? 0 : (head_slot < q_local + kv_local ? 1 : 2);
    const int32_t local_head = head_slot - (segment == 0 ? 0 : q_local + (segment == 2 ? kv_local : 0));
    const int32_t seg_local_heads = segment == 0 ? q_local : kv_local;
    const int32_t seg_heads = segment == 0 ? g.q_heads : g.kv_heads;
    const int32_t head = (segment == 0 ? 0 : g.q_heads + (segment == 2 ? g.kv_heads : 0)) +
                         g.rank * seg_local_heads + local_head;
    (void)seg_heads;
    const int64_t plane_width = int64_t(seg_local_heads) * g.head_dim;
    const uint16_t* src = g.grad[segment] + int64_t(local_head) * g.head_dim;
    uint16_t* dst = g.peer_staging[dest] + int64_t(head) * g.head_dim;
    const int32_t m0 = mt * kBlockM;
    const int32_t rows = g.m - m0 < kBlockM ? g.m - m0 : kBlockM;
    const int32_t total = rows * chunks_per_row;
    for (int32_t i0 = tid; i0 < total; i0 += kThreads * 4) {
      uint4 value[4];
      uint16_t* out[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int32_t i = i0 + j * kThreads;
        out[j] = nullptr;
        if (i < total) {
          const int32_t row = i / chunks_per_row, chunk = i - row * chunks_per_row;
          const int64_t src_row = global_row(g.world, dest, g.seq_local, g.global_seq, g.causal != 0, m0 + row);
          value[j] = *reinterpret_cast<const uint4*>(src + src_row * plane_width + chunk * 8);
          out[j] = dst + int64_t(m0 + row) * width + chunk * 8;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (out[j] != nullptr) ptx::st_v4(out[j], value[j]);
    }
    __syncthreads();  // every thread's stores of this unit are issued ...
    if (tid == 0) {
      __threadfence_system();  // ... and performed before the destination sees the flag
      ptx::fence_proxy_async_global();
      ptx::st_release_sys(g.peer_ready[dest] + (int64_t(mt) * heads_total + head) * kReadyFlagStride,
                          p.wait.epoch);
    }
  }
  __threadfence_system();
}

// ------------------------------------------------------------------------------------------
// Communication role: MXFP8 QKV backward reverse route, receiver pull.
//
// Unit of work = (M tile, logical head): from the owner's planar gradient the 128 x 128 E4M3
// block, its 512-byte scale atom and the 128 x 128 BF16 master block are copied with 16-byte
// accesses into the packed lhs bytes / scale storage (consumed by the block-scaled GEMM) and
// the packed BF16 staging (kept for the weight gradient), then ready[m_tile*heads + head] =
// epoch is released (csrc/operators/sm103/detail/backward.cuh:423-552).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void grad_pull_role(const FusedParams& p) {
  const GradRoute& g = p.grad;
  const int tid = threadIdx.x;
  const int32_t m_tiles = (g.m + kBlockM - 1) / kBlockM;
  const int32_t heads_total = g.q_heads + 2 * g.kv_heads;
  const int32_t width = heads_total * 128;
  const int64_t units = int64_t(m_tiles) * heads_total;
  for (int64_t u = blockIdx.x; u < units; u += p.num_comm_ctas) {
    const int32_t mt = int32_t(u / heads_total), head = int32_t(u % heads_total);
    const int32_t segment = head < g.q_heads ? 0 : (head < g.q_heads + g.kv_heads ? 1 : 2);
    const int32_t seg_head = head - (segment == 0 ? 0 : g.q_heads + (segment == 2 ? g.kv_heads : 0));
    const int32_t seg_local = (segment == 0 ? g.q_heads : g.kv_heads) / g.world;
    const int32_t owner = seg_head / seg_local, local_head = seg_head - owner * seg_local;
    const int64_t plane_width = int64_t(seg_local) * 128;
    const int32_t m0 = mt * kBlockM;
    const int32_t rows = g.m - m0 < kBlockM ? g.m - m0 : kBlockM;
    const uint8_t* src8 = g.peer_bytes[owner][segment] + int64_t(local_head) * 128;
    const uint16_t* src16 = g.peer_master[owner][segment] + int64_t(local_head) * 128;
    // E4M3 bytes: 8 chunks per row; BF16 masters: 16 chunks per row
    for (int32_t i = tid; i < rows * 24; i += kThreads) {
      const int32_t row = i / 24, c = i - row * 24;
      const int64_t src_row = global_row(g.world, g.rank, g.seq_local, g.global_seq, g.causal != 0, m0 + row);
      if (c < 8) {
        const uint4 v = ptx::ld_cg_v4(src8 + src_row * plane_width + c * 16);
        ptx::st_v4(g.lhs_bytes + int64_t(m0 + row) * width + int64_t(head) * 128 + c * 16, v);
      } else {
        const uint4 v = ptx::ld_cg_v4(src16 + src_row * plane_width + (c - 8) * 8);
        ptx::st_v4(g.master_staging + int64_t(m0 + row) * width + int64_t(head) * 128 + (c - 8) * 8, v);
      }
    }
    if (tid < 32) {  // the (128-row group, head) scale atom
      const int64_t src_row0 = global_row(g.world, g.rank, g.seq_local, g.global_seq, g.causal != 0, m0);
      const uint4 v = ptx::ld_cg_v4(g.peer_scales[owner][segment] + ((src_row0 >> 7) * seg_local + local_head) * 512 + tid * 16);
      ptx::st_v4(g.lhs_scales + (int64_t(mt) * heads_total + head) * 512 + tid * 16, v);
    }
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      ptx::fence_proxy_async_global();
      ptx::st_release_gpu(p.ready + (int64_t(mt) * heads_total + head) * kReadyFlagStride, p.wait.epoch);
    }
  }
}

// ------------------------------------------------------------------------------------------
// Chunk pipeline shared by the tensor-copy communication roles.
//
// Warps 0..kPullWarps-1 of a communication CTA each walk their units chunk by chunk (a chunk
// fits one kPullStageBytes stage): loads run kPullStages ahead into the warp's shared-memory
// ring and complete on mbarriers; as a chunk lands its store is issued and committed as one bulk
// group; the stage is reused once that store has read it; a unit is complete when the group
// holding its last chunk has completed, checked kPullLag chunks late.  Completed units go into a
// small per-warp queue in shared memory; the last warp of the CTA (the publisher) drains the
// queues and releases the units' flags -- one memory fence per batch of units, so the
// microseconds a GPU- or system-scope fence takes are never on a copy warp's path.  The policy
// supplies the unit/chunk walk, the copy instructions, the fence and the flag store.
// ------------------------------------------------------------------------------------------
constexpr int kPublishDepth = 16;                 // queue entries per copy warp
constexpr uint32_t kPublishSentinel = 0xffffffffu;  // "this warp has no more units"
constexpr uint32_t kPublishQueueBytes = kPullWarps * (kPublishDepth + 2) * 4u;
static_assert(kPublishQueueBytes <= 512u, "the unit queues live in the 512 bytes after the copy rings");
static_assert(kThreads / 32 > kPullWarps, "one warp beyond the copy warps publishes");

template <class Policy>
__device__ __forceinline__ void run_unit_publisher(Policy& policy, const WaitContext& w, uint32_t queue,
                                                   uint32_t heads, uint32_t tails, int lane) {
  uint32_t tail = 0, idle = 0;
  bool finished = lane >= kPullWarps;  // lane l drains the queue of copy warp l
  uint64_t idle_since = 0;
  for (;;) {
    uint32_t units[4];
    int n = 0;
    if (!finished) {
      const uint32_t head = ptx::ld_acquire_cta_shared(heads + 4u * uint32_t(lane));
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        units[i] = 0u;
        if (!finished && tail != head) {
          const uint32_t u = ptx::ld_acquire_cta_shared(queue + (uint32_t(lane) * kPublishDepth + tail % kPublishDepth) * 4u);
          ++tail;
          if (u == kPublishSentinel) finished = true;
          else { units[i] = u; n = i + 1; }
        }
      }
    }
    if (__any_sync(0xffffffffu, n > 0)) {
      policy.publish_fence();
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (i < n) policy.publish_flag(int64_t(units[i]));
      if (lane < kPullWarps) ptx::st_release_cta_shared(tails + 4u * uint32_t(lane), tail);
      idle = 0;
      continue;
    }
    if (lane < kPullWarps) ptx::st_release_cta_shared(tails + 4u * uint32_t(lane), tail);
    if (__all_sync(0xffffffffu, finished)) break;
    if (idle == 0u) idle_since = ptx::globaltimer();
    __nanosleep(100);
    if ((++idle & 63u) == 0u) {
      // Copy warps end with a sentinel whatever happens to them; this limit only covers a warp
      // that never ran.
      uint32_t stop = 0u;
      if (lane == 0) {
        if (aborted(w) && ptx::globaltimer() - idle_since > w.budget_ns) stop = 1u;
        if (ptx::globaltimer() - idle_since > 2 * w.budget_ns) {
          report_timeout(w, kStatusFlagTimeout, kSiteCommStage, 0u, 0u, 0u);
          stop = 1u;
        }
      }
      if (__shfl_sync(0xffffffffu, stop, 0)) break;
    }
  }
}

template <class Policy>
__device__ __forceinline__ void run_chunk_pipeline(Policy& policy, const WaitContext& w, uint32_t smem_base,
                                                   int32_t num_comm_ctas) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t queue = smem_base + kPullWarps * kPullStages * (kPullStageBytes + 8u);
  const uint32_t heads = queue + kPullWarps * kPublishDepth * 4u, tails = heads + kPullWarps * 4u;
  if (threadIdx.x < kPullWarps) {
    ptx::st_release_cta_shared(heads + 4u * threadIdx.x, 0u);
    ptx::st_release_cta_shared(tails + 4u * threadIdx.x, 0u);
  }
  __syncthreads();  // every thread of the communication CTA comes through here
  if (warp == kPullWarps) {
    run_unit_publisher(policy, w, queue, heads, tails, lane);
    return;
  }
  if (warp > kPullWarps) return;
  const uint32_t ring = smem_base + uint32_t(warp) * kPullStages * kPullStageBytes;
  const uint32_t bars = smem_base + kPullWarps * kPullStages * kPullStageBytes + uint32_t(warp) * kPullStages * 8u;
  if (lane == 0) {
    for (int s = 0; s < kPullStages; ++s) ptx::mbar_init(bars + 8u * s, 1);
    ptx::fence_mbar_init();
  }
  __syncwarp();
  const int32_t workers = num_comm_ctas * kPullWarps;
  const int32_t worker = warp * num_comm_ctas + int32_t(blockIdx.x);

  // Lane 0 appends a completed unit (or the sentinel) to this warp's queue; a full queue waits
  // for the publisher, giving up only when the launch is being aborted.
  uint32_t posted = 0;
  auto post = [&](uint32_t unit) {
    if (lane != 0) return;
    const uint32_t my_tail = tails + 4u * uint32_t(warp);
    if (posted - ptx::ld_acquire_cta_shared(my_tail) >= uint32_t(kPublishDepth)) {
      if (!progress_wait(my_tail, posted - uint32_t(kPublishDepth) + 1u, w, kSiteCommStage, uint32_t(warp))) return;
    }
    ptx::st_release_cta_shared(queue + (uint32_t(warp) * kPublishDepth + posted % kPublishDepth) * 4u, unit);
    ++posted;
    ptx::st_release_cta_shared(heads + 4u * uint32_t(warp), posted);
  };

  // The cursor of every chunk in flight is kept from its load to its store (one per stage), so
  // the unit walk is decoded once per chunk.
  static_assert(kPullStages == 2, "two cursors in flight");
  typename Policy::Cursor load_cursor, in_flight0, in_flight1;
  bool more_loads = policy.first(load_cursor, worker, workers);
  if (!more_loads) {
    post(kPublishSentinel);
    return;
  }
  int32_t issued = 0, consumed = 0;
  bool ok = true;
  // Starts the copy of the chunk under the load cursor; false when the policy had to give up
  // (an upstream flag that never came), in which case nothing was started.
  auto start_load = [&]() {
    uint32_t good = policy.load(load_cursor, ring + uint32_t(issued % kPullStages) * kPullStageBytes,
                                bars + 8u * uint32_t(issued % kPullStages), lane) ? 1u : 0u;
    good = __shfl_sync(0xffffffffu, good, 0);
    if (!good) { ok = false; return; }
    if (issued % kPullStages == 0) in_flight0 = load_cursor;
    else in_flight1 = load_cursor;
    more_loads = policy.next(load_cursor, workers);
    ++issued;
  };
  while (ok && issued < kPullStages && more_loads) start_load();
  int64_t lag_unit[kPullLag];
#pragma unroll
  for (int i = 0; i < kPullLag; ++i) lag_unit[i] = -1;
  while (ok && consumed < issued) {
    const int stage = consumed % kPullStages;
    const typename Policy::Cursor store_cursor = stage == 0 ? in_flight0 : in_flight1;
    uint32_t landed = 1u;
    if (lane == 0) {
      trace_event(policy.p, 30);  // waiting for the chunk to land
      landed = mbar_wait(bars + 8u * stage, uint32_t(consumed / kPullStages) & 1u, w, kSiteCommStage) ? 1u : 0u;
      trace_event(policy.p, 31);
    }
    landed = __shfl_sync(0xffffffffu, landed, 0);
    if (!landed) { ok = false; break; }
    policy.store(store_cursor, ring + uint32_t(stage) * kPullStageBytes, lane);
    ptx::bulk_commit();
    ++consumed;
    if (lane == 0) trace_event(policy.p, 32);  // store issued
    ptx::bulk_wait_read<0>();
    __syncwarp();
    if (lane == 0) trace_event(policy.p, 33);  // store has read the stage
    if (more_loads && issued < consumed + kPullStages) start_load();
    if (consumed <= kPullEagerChunks) {
      // The first chunks feed GEMM tiles that are already waiting: report them as soon as their
      // stores have completed instead of kPullLag chunks later.
      ptx::bulk_wait<0>();
      __syncwarp();
#pragma unroll
      for (int i = kPullLag - 1; i >= 0; --i) {
        if (lag_unit[i] >= 0) post(uint32_t(lag_unit[i]));
        lag_unit[i] = -1;
      }
      if (policy.closes(store_cursor)) post(uint32_t(policy.unit(store_cursor)));
    } else {
      ptx::bulk_wait<kPullLag>();
      __syncwarp();
      if (lane == 0) trace_event(policy.p, 34);  // older stores complete
      if (lag_unit[kPullLag - 1] >= 0) post(uint32_t(lag_unit[kPullLag - 1]));
      if (lane == 0) trace_event(policy.p, 35);  // unit queued for publication
#pragma unroll
      for (int i = kPullLag - 1; i > 0; --i) lag_unit[i] = lag_unit[i - 1];
      lag_unit[0] = policy.closes(store_cursor) ? policy.unit(store_cursor) : -1;
    }
  }
  ptx::bulk_wait<0>();
  __syncwarp();
  if (ok) {
#pragma unroll
    for (int i = kPullLag - 1; i >= 0; --i)
      if (lag_unit[i] >= 0) post(uint32_t(lag_unit[i]));
  }
  if (!ok && lane == 0)
    for (int32_t i = consumed; i < issued; ++i)
      mbar_wait(bars + 8u * uint32_t(i % kPullStages), uint32_t(i / kPullStages) & 1u, w, kSiteDrain, false);
  post(kPublishSentinel);
}

// The same pipeline run by ONE thread with its own two stages (the copy warp embedded in a compute
// CTA): chunks are dealt to `workers` such threads, a finished unit is published by the thread
// itself (fence + flag, kPullLag chunks late except at start-up).  `bars`: two mbarriers of count 1.
template <class Policy>
__device__ __forceinline__ void run_chunk_pipeline_thread(Policy& policy, const WaitContext& w, uint32_t ring,
                                                          uint32_t bars, int32_t worker, int32_t workers) {
  static_assert(kPullStages == 2, "two cursors in flight");
  typename Policy::Cursor load_cursor, in_flight0, in_flight1;
  bool more_loads = policy.first(load_cursor, worker, workers);
  if (!more_loads) return;
  int32_t issued = 0, consumed = 0;
  bool ok = true;
  auto publish = [&](int64_t unit) {
    policy.publish_fence();
    policy.publish_flag(unit);
  };
  auto start_load = [&]() {
    if (!policy.load(load_cursor, ring + uint32_t(issued % kPullStages) * kPullStageBytes,
                     bars + 8u * uint32_t(issued % kPullStages), 0)) {
      ok = false;
      return;
    }
    if (issued % kPullStages == 0) in_flight0 = load_cursor;
    else in_flight1 = load_cursor;
    more_loads = policy.next(load_cursor, workers);
    ++issued;
  };
  while (ok && issued < kPullStages && more_loads) start_load();
  int64_t lag_unit[kPullLag];
#pragma unroll
  for (int i = 0; i < kPullLag; ++i) lag_unit[i] = -1;
  while (ok && consumed < issued) {
    const int stage = consumed % kPullStages;
    const typename Policy::Cursor store_cursor = stage == 0 ? in_flight0 : in_flight1;
    if (!mbar_wait(bars + 8u * stage, uint32_t(consumed / kPullStages) & 1u, w, kSiteCommStage)) {
      ok = false;
      break;
    }
    policy.store(store_cursor, ring + uint32_t(stage) * kPullStageBytes, 0);
    ptx::bulk_commit();
    ++consumed;
    ptx::bulk_wait_read<0>();
    if (more_loads && issued < consumed + kPullStages) start_load();
    if (consumed <= kPullEagerChunks) {
      ptx::bulk_wait<0>();
#pragma unroll
      for (int i = kPullLag - 1; i >= 0; --i) {
        if (lag_unit[i] >= 0) publish(lag_unit[i]);
        lag_unit[i] = -1;
      }
      if (policy.closes(store_cursor)) publish(policy.unit(store_cursor));
    } else {
      ptx::bulk_wait<kPullLag>();
      if (lag_unit[kPullLag - 1] >= 0) publish(lag_unit[kPullLag - 1]);
#pragma unroll
      for (int i = kPullLag - 1; i > 0; --i) lag_unit[i] = lag_unit[i - 1];
      lag_unit[0] = policy.closes(store_cursor) ? policy.unit(store_cursor) : -1;
    }
  }
  ptx::bulk_wait<0>();
  if (ok) {
#pragma unroll
    for (int i = kPullLag - 1; i >= 0; --i)
      if (lag_unit[i] >= 0) publish(lag_unit[i]);
  } else {
    for (int32_t i = consumed; i < issued; ++i)
      mbar_wait(bars + 8u * uint32_t(i % kPullStages), uint32_t(i / kPullStages) & 1u, w, kSiteDrain, false);
  }
}

// Forward lhs pull with tensor copies.  A (M tile, column slice) unit -- 128 rows of one slice of
// one peer's shard, plus (block-scaled operands) the slice's scale atoms -- is cut into chunks of
// rows_per_chunk rows x piece_bytes (one stage) and the chunks into sub-units of two, dealt round
// robin to the copy warps in the GEMM's first-use order (wave group, slice, M tile).  Each
// chunk is one tensor load from the peer and one tensor store into the staging; a finished
// sub-unit is counted in word 2v+1 of the shard's flag line and the arrival that completes the
// unit publishes word 2v = epoch (arrival counting as in
// csrc/operators/sm103/detail/a2a_gemm.cuh:466-642, but the epoch need not advance by one).
struct LhsPullPolicy {
  struct Cursor {
    int32_t sub, chunk;                       // global sub-unit index, chunk inside it (0 or 1)
    int32_t mt, shard, slice, peer;           // decoded unit
    int32_t first_chunk, chunks_here, data_chunks, flag, needed;
    int64_t src_row0;                         // source row of the M tile's first row
  };
  const FusedParams& p;
  const LhsPullMaps& maps;
  int32_t gates, pieces, rows_per_chunk, piece_bytes, unit_bytes, unit_atoms, scale_chunks;
  int32_t subs_per_unit, subs_total, m_tiles;  // m_tiles: 128-row tiles (the launch's tile order may use taller ones)
  uint32_t shard_bytes;
  bool tile_rows_consecutive;  // the 128 rows of every M tile are consecutive at the source
  mutable uint32_t upstream_seen = 0;
  static constexpr int32_t kAtomsPerChunk = int32_t(kPullStageBytes / 512);
  __device__ LhsPullPolicy(const FusedParams& params, const LhsPullMaps& m) : p(params), maps(m) {
    const LhsRoute& r = p.lhs;
    shard_bytes = uint32_t(r.shard_width) * uint32_t(r.element_bytes);
    unit_bytes = r.virt_width * r.element_bytes;
    unit_atoms = r.virt_width / 128;
    gates = r.world * r.virt;
    piece_bytes = m.piece_bytes;
    rows_per_chunk = m.rows_per_chunk;
    pieces = unit_bytes / piece_bytes;
    scale_chunks = r.local_scales != nullptr ? (unit_atoms + kAtomsPerChunk - 1) / kAtomsPerChunk : 0;
    const int32_t chunks_full = (kBlockM / rows_per_chunk) * pieces + scale_chunks;
    subs_per_unit = (chunks_full + 1) / 2;
    m_tiles = (p.m + kBlockM - 1) / kBlockM;
    subs_total = m_tiles * gates * subs_per_unit;
    tile_rows_consecutive = (r.causal ? r.seq_local / 2 : r.seq_local) % kBlockM == 0;
  }
  // Decodes sub-unit c.sub; false when it holds no chunk (a short last M tile).
  __device__ bool decode(Cursor& c) const {
    const LhsRoute& r = p.lhs;
    const int32_t unit = c.sub / subs_per_unit, q = c.sub - unit * subs_per_unit;
    const int32_t per_group = r.m_group * gates;
    const int32_t group = unit / per_group, mt0 = group * r.m_group;
    const int32_t group_size = m_tiles - mt0 < r.m_group ? m_tiles - mt0 : r.m_group;
    const int32_t within = unit - group * per_group;
    const int32_t position = within / group_size;  // in the GEMM's (rotated) K order
    c.mt = mt0 + within - position * group_size;
    const int32_t gate = position + r.gate_start < gates ? position + r.gate_start : position + r.gate_start - gates;
    c.shard = gate / r.virt;
    c.slice = gate - c.shard * r.virt;
    const int32_t rows = p.m - c.mt * kBlockM < kBlockM ? p.m - c.mt * kBlockM : kBlockM;
    c.data_chunks = ((rows + rows_per_chunk - 1) / rows_per_chunk) * pieces;
    const int32_t total = c.data_chunks + scale_chunks;
    c.first_chunk = 2 * q;
    if (c.first_chunk >= total) return false;
    c.chunks_here = total - c.first_chunk < 2 ? total - c.first_chunk : 2;
    c.needed = (total + 1) / 2;
    c.flag = (c.mt * r.world + c.shard) * kReadyFlagStride + 2 * c.slice;
    c.peer = r.cyclic ? (r.rank + c.shard) % r.world : c.shard;
    c.src_row0 = global_row(r.world, r.rank, r.seq_local, r.global_seq, r.causal != 0, c.mt * kBlockM);
    c.chunk = 0;
    return true;
  }
  __device__ bool seek(Cursor& c, int32_t workers) const {
    for (; c.sub < subs_total; c.sub += workers)
      if (decode(c)) return true;
    return false;
  }
  __device__ bool first(Cursor& c, int32_t worker, int32_t workers) const {
    c.sub = worker;
    return seek(c, workers);
  }
  __device__ bool next(Cursor& c, int32_t workers) const {
    if (++c.chunk < c.chunks_here) return true;
    c.sub += workers;
    return seek(c, workers);
  }
  __device__ bool load(const Cursor& c, uint32_t smem, uint32_t bar, int lane) const {
    if (lane != 0) return true;
    const LhsRoute& r = p.lhs;
    if (r.peer_input_ready[c.peer] != nullptr && !((upstream_seen >> c.peer) & 1u)) {
      // the peer's producer (attention) publishes one epoch per tensor
      if (!flag_wait<true>(r.peer_input_ready[c.peer], r.input_epoch, p.wait, kSiteUpstreamReady, uint32_t(c.peer)))
        return false;
      upstream_seen |= 1u << c.peer;
    }
    const int32_t k = c.first_chunk + c.chunk;
    if (k < c.data_chunks) {
      const int32_t row_block = pieces == 1 ? k : k / pieces, piece = k - row_block * pieces;
      // rows of one chunk are consecutive at the source: chunks never straddle a sequence block
      const int64_t src_row = tile_rows_consecutive
                                  ? c.src_row0 + row_block * rows_per_chunk
                                  : global_row(r.world, r.rank, r.seq_local, r.global_seq, r.causal != 0,
                                               c.mt * kBlockM + row_block * rows_per_chunk);
      ptx::mbar_expect_tx(bar, uint32_t(rows_per_chunk) * uint32_t(piece_bytes));
      ptx::tma_load_2d(smem, &maps.peer[c.peer], bar, (c.slice * unit_bytes + piece * piece_bytes) / 4, int32_t(src_row));
    } else {
      const int32_t first_atom = (k - c.data_chunks) * kAtomsPerChunk;
      const int32_t atoms = unit_atoms - first_atom < kAtomsPerChunk ? unit_atoms - first_atom : kAtomsPerChunk;
      ptx::mbar_expect_tx(bar, uint32_t(atoms) * 512u);
      ptx::bulk_load(smem,
                     r.peer_scales[c.peer] +
                         ((c.src_row0 >> 7) * int64_t(r.shard_atoms) + int64_t(c.slice) * unit_atoms + first_atom) * 512,
                     uint32_t(atoms) * 512u, bar);
    }
    return true;
  }
  __device__ void store(const Cursor& c, uint32_t smem, int lane) const {
    if (lane != 0) return;
    const LhsRoute& r = p.lhs;
    const int32_t k = c.first_chunk + c.chunk;
    if (k < c.data_chunks) {
      const int32_t row_block = pieces == 1 ? k : k / pieces, piece = k - row_block * pieces;
      ptx::tma_store_2d(&maps.staging, smem,
                        int32_t((uint32_t(c.shard) * shard_bytes + uint32_t(c.slice * unit_bytes + piece * piece_bytes)) / 4u),
                        c.mt * kBlockM + row_block * rows_per_chunk);
    } else {
      const int32_t first_atom = (k - c.data_chunks) * kAtomsPerChunk;
      const int32_t atoms = unit_atoms - first_atom < kAtomsPerChunk ? unit_atoms - first_atom : kAtomsPerChunk;
      ptx::bulk_store(r.local_scales + (int64_t(c.mt) * r.k_atoms + int64_t(c.shard) * r.shard_atoms +
                                        int64_t(c.slice) * unit_atoms + first_atom) * 512,
                      smem, uint32_t(atoms) * 512u);
    }
  }
  __device__ bool closes(const Cursor& c) const { return c.chunk + 1 == c.chunks_here; }
  __device__ int64_t unit(const Cursor& c) const { return c.sub; }
  __device__ void publish_fence() const {}
  // The acq_rel read-modify-write orders the completed copies (observed by the copy warp and
  // handed over through shared memory) before the count; the consumer fences the proxies after
  // its acquire.
  __device__ void publish_flag(int64_t sub) const {
    Cursor c;
    c.sub = int32_t(sub);
    if (!decode(c)) return;
    const uint32_t before = ptx::atom_acq_rel_gpu_add(p.ready + c.flag + 1, 1u);
    if ((before + 1u) % uint32_t(c.needed) == 0u) ptx::st_release_gpu(p.ready + c.flag, p.wait.epoch);
  }
};

// QKV backward sender push with tensor copies (head_dim 128): unit = (destination M tile,
// destination, local head), two chunks of 64 rows x 128 columns.  Destinations rotate from the
// next rank on.  The destination's flag is released at system scope once both chunks' stores
// have completed.
struct GradPushPolicy {
  struct Where { int32_t dest, mt, segment, local_head, head; };
  struct Cursor { int64_t unit; int32_t chunk; Where x; };
  const FusedParams& p;
  const GradPushMaps& maps;
  int32_t m_tiles, local_heads, heads_total, q_local, kv_local;
  int64_t units;
  __device__ GradPushPolicy(const FusedParams& params, const GradPushMaps& m) : p(params), maps(m) {
    const GradRoute& g = p.grad;
    m_tiles = (g.m + kBlockM - 1) / kBlockM;
    q_local = g.q_heads / g.world;
    kv_local = g.kv_heads / g.world;
    local_heads = q_local + 2 * kv_local;
    heads_total = g.q_heads + 2 * g.kv_heads;
    units = int64_t(m_tiles) * g.world * local_heads;
  }
  // Units are ordered so that the M tiles one GEMM wave works on (a group of m_group tiles)
  // advance through the heads together: group, then local head, then destination, then M tile.
  __device__ Where where(int64_t u) const {
    const GradRoute& g = p.grad;
    Where x;
    const int64_t per_group = int64_t(g.m_group) * g.world * local_heads;
    const int32_t group = int32_t(u / per_group);
    const int32_t mt0 = group * g.m_group;
    const int32_t size = m_tiles - mt0 < g.m_group ? m_tiles - mt0 : g.m_group;
    const int32_t within = int32_t(u - group * per_group);
    const int32_t slot = within / (g.world * size), rest = within - slot * (g.world * size);
    x.dest = (g.rank + 1 + rest / size) % g.world;
    x.mt = mt0 + rest % size;
    x.segment = slot < q_local ? 0 : (slot < q_local + kv_local ? 1 : 2);
    x.local_head = slot - (x.segment == 0 ? 0 : q_local + (x.segment == 2 ? kv_local : 0));
    const int32_t seg_local = x.segment == 0 ? q_local : kv_local;
    x.head = (x.segment == 0 ? 0 : g.q_heads + (x.segment == 2 ? g.kv_heads : 0)) + g.rank * seg_local + x.local_head;
    return x;
  }
  __device__ bool first(Cursor& c, int32_t worker, int32_t) const {
    c.unit = worker;
    c.chunk = 0;
    if (c.unit >= units) return false;
    c.x = where(c.unit);
    return true;
  }
  __device__ bool next(Cursor& c, int32_t workers) const {
    if (++c.chunk < 2 && p.grad.m - c.x.mt * kBlockM > 64) return true;
    c.chunk = 0;
    c.unit += workers;
    if (c.unit >= units) return false;
    c.x = where(c.unit);
    return true;
  }
  __device__ bool load(const Cursor& c, uint32_t smem, uint32_t bar, int lane) const {
    if (lane != 0) return true;
    const GradRoute& g = p.grad;
    const int64_t src_row = global_row(g.world, c.x.dest, g.seq_local, g.global_seq, g.causal != 0, c.x.mt * kBlockM + c.chunk * 64);
    ptx::mbar_expect_tx(bar, 64u * 256u);
    ptx::tma_load_2d(smem, &maps.plane[c.x.segment], bar, c.x.local_head * 128, int32_t(src_row));
    return true;
  }
  __device__ void store(const Cursor& c, uint32_t smem, int lane) const {
    if (lane != 0) return;
    ptx::tma_store_2d(&maps.staging[c.x.dest], smem, c.x.head * 128, c.x.mt * kBlockM + c.chunk * 64);
  }
  __device__ bool closes(const Cursor& c) const { return c.chunk == 1 || p.grad.m - c.x.mt * kBlockM <= 64; }
  __device__ int64_t unit(const Cursor& c) const { return c.unit; }
  __device__ void publish_fence() const { ptx::fence_acq_rel_sys(); }
  __device__ void publish_flag(int64_t u) const {
    const Where x = where(u);
    ptx::st_relaxed_sys(p.grad.peer_ready[x.dest] + (int64_t(x.mt) * heads_total + x.head) * kReadyFlagStride,
                        p.wait.epoch);
  }
};

// MXFP8 QKV backward receiver pull with tensor copies: unit = (M tile, logical head), four
// chunks: the 128 x 128 E4M3 block, two 64-row halves of the BF16 master block, the scale atom.
struct GradPullPolicy {
  struct Where { int32_t mt, head, segment, owner, local_head, seg_local; int64_t src_row; };
  struct Cursor { int64_t unit; int32_t chunk; Where x; };
  const FusedParams& p;
  const GradPullMaps& maps;
  int32_t heads_total;
  int64_t units;
  __device__ GradPullPolicy(const FusedParams& params, const GradPullMaps& m) : p(params), maps(m) {
    heads_total = p.grad.q_heads + 2 * p.grad.kv_heads;
    units = int64_t((p.grad.m + kBlockM - 1) / kBlockM) * heads_total;
  }
  __device__ Where where(int64_t u) const {
    const GradRoute& g = p.grad;
    Where x;
    // group of m_group M tiles, then head, then M tile: a GEMM wave's tiles advance together
    const int32_t m_tiles = (g.m + kBlockM - 1) / kBlockM;
    const int64_t per_group = int64_t(g.m_group) * heads_total;
    const int32_t group = int32_t(u / per_group);
    const int32_t mt0 = group * g.m_group;
    const int32_t size = m_tiles - mt0 < g.m_group ? m_tiles - mt0 : g.m_group;
    const int32_t within = int32_t(u - group * per_group);
    x.head = within / size;
    x.mt = mt0 + within % size;
    x.segment = x.head < g.q_heads ? 0 : (x.head < g.q_heads + g.kv_heads ? 1 : 2);
    const int32_t seg_head = x.head - (x.segment == 0 ? 0 : g.q_heads + (x.segment == 2 ? g.kv_heads : 0));
    x.seg_local = (x.segment == 0 ? g.q_heads : g.kv_heads) / g.world;
    x.owner = seg_head / x.seg_local;
    x.local_head = seg_head - x.owner * x.seg_local;
    x.src_row = global_row(g.world, g.rank, g.seq_local, g.global_seq, g.causal != 0, x.mt * kBlockM);
    return x;
  }
  __device__ bool first(Cursor& c, int32_t worker, int32_t) const {
    c.unit = worker;
    c.chunk = 0;
    if (c.unit >= units) return false;
    c.x = where(c.unit);
    return true;
  }
  __device__ bool next(Cursor& c, int32_t workers) const {
    if (++c.chunk < 4) return true;
    c.chunk = 0;
    c.unit += workers;
    if (c.unit >= units) return false;
    c.x = where(c.unit);
    return true;
  }
  __device__ bool load(const Cursor& c, uint32_t smem, uint32_t bar, int lane) const {
    if (lane != 0) return true;
    const Where& x = c.x;
    if (c.chunk == 0) {
      ptx::mbar_expect_tx(bar, 128u * 128u);
      ptx::tma_load_2d(smem, &maps.bytes[x.owner][x.segment], bar, x.local_head * 128, int32_t(x.src_row));
    } else if (c.chunk < 3) {
      ptx::mbar_expect_tx(bar, 64u * 256u);
      ptx::tma_load_2d(smem, &maps.masters[x.owner][x.segment], bar, x.local_head * 128,
                       int32_t(x.src_row) + (c.chunk - 1) * 64);
    } else {
      ptx::mbar_expect_tx(bar, 512u);
      ptx::bulk_load(smem, p.grad.peer_scales[x.owner][x.segment] + ((x.src_row >> 7) * x.seg_local + x.local_head) * 512,
                     512u, bar);
    }
    return true;
  }
  __device__ void store(const Cursor& c, uint32_t smem, int lane) const {
    if (lane != 0) return;
    const Where& x = c.x;
    if (c.chunk == 0) ptx::tma_store_2d(&maps.lhs, smem, x.head * 128, x.mt * kBlockM);
    else if (c.chunk < 3) ptx::tma_store_2d(&maps.master, smem, x.head * 128, x.mt * kBlockM + (c.chunk - 1) * 64);
    else ptx::bulk_store(p.grad.lhs_scales + (int64_t(x.mt) * heads_total + x.head) * 512, smem, 512u);
  }
  __device__ bool closes(const Cursor& c) const { return c.chunk == 3; }
  __device__ int64_t unit(const Cursor& c) const { return c.unit; }
  __device__ void publish_fence() const { ptx::fence_acq_rel_gpu(); }
  __device__ void publish_flag(int64_t u) const {
    const Where x = where(u);
    ptx::st_relaxed_gpu(p.ready + (int64_t(x.mt) * heads_total + x.head) * kReadyFlagStride, p.wait.epoch);
  }
};

// 32 FP32 accumulators of one output row -> alpha (and beta * old D) -> BF16 -> four 16-byte
// stores.  `col` is the global column of acc[0]; vectors past N are skipped (N % 8 == 0).
struct PeerRow {
  uint16_t* const* col_base;   // per 8-column chunk of the tile: destination base (row 0)
  const int64_t* col_stride;   // per chunk: destination row pitch in elements
  int64_t dest_row;            // destination row of this thread's output row
  int32_t chunk0;              // chunk index of acc[0] inside the tile
};

template <bool kPushToPeer>
__device__ __forceinline__ void store_accumulators(const uint32_t (&acc)[32], uint16_t* dst,
                                                   int32_t col, bool row_ok, const FusedParams& p,
                                                   const PeerRow& peer) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    if (row_ok && col + v * 8 < p.n) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = p.alpha * __uint_as_float(acc[v * 8 + e]);
      if (p.beta != 0.0f) {
        const uint4 old = *reinterpret_cast<const uint4*>(dst + v * 8);
        f[0] += p.beta * __uint_as_float(old.x << 16);
        f[1] += p.beta * __uint_as_float(old.x & 0xffff0000u);
        f[2] += p.beta * __uint_as_float(old.y << 16);
        f[3] += p.beta * __uint_as_float(old.y & 0xffff0000u);
        f[4] += p.beta * __uint_as_float(old.z << 16);
        f[5] += p.beta * __uint_as_float(old.z & 0xffff0000u);
        f[6] += p.beta * __uint_as_float(old.w << 16);
        f[7] += p.beta * __uint_as_float(old.w & 0xffff0000u);
      }
      uint4 out;
      __nv_bfloat162 pair = __floats2bfloat162_rn(f[0], f[1]);
      out.x = *reinterpret_cast<const uint32_t*>(&pair);
      pair = __floats2bfloat162_rn(f[2], f[3]);
      out.y = *reinterpret_cast<const uint32_t*>(&pair);
      pair = __floats2bfloat162_rn(f[4], f[5]);
      out.z = *reinterpret_cast<const uint32_t*>(&pair);
      pair = __floats2bfloat162_rn(f[6], f[7]);
      out.w = *reinterpret_cast<const uint32_t*>(&pair);
      ptx::st_v4(dst + v * 8, out);
      if constexpr (kPushToPeer) {
        uint16_t* base = peer.col_base[peer.chunk0 + v];  // null: a chunk that is not routed (deferred V)
        if (base != nullptr) ptx::st_v4(base + peer.dest_row * peer.col_stride[peer.chunk0 + v], out);
      }
    }
  }
}

// 32 FP32 accumulators of one row -> alpha -> BF16 -> four 16-byte chunks of that row inside a
// 128B-swizzled staging block (chunk index XOR row%8, the layout TMA's SWIZZLE_128B expects).
__device__ __forceinline__ void stage_accumulators(const uint32_t (&acc)[32], uint32_t row_addr,
                                                   int32_t first_chunk, int32_t row, float alpha) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    uint4 out;
    __nv_bfloat162 pair = __floats2bfloat162_rn(alpha * __uint_as_float(acc[v * 8 + 0]),
                                                alpha * __uint_as_float(acc[v * 8 + 1]));
    out.x = *reinterpret_cast<const uint32_t*>(&pair);
    pair = __floats2bfloat162_rn(alpha * __uint_as_float(acc[v * 8 + 2]), alpha * __uint_as_float(acc[v * 8 + 3]));
    out.y = *reinterpret_cast<const uint32_t*>(&pair);
    pair = __floats2bfloat162_rn(alpha * __uint_as_float(acc[v * 8 + 4]), alpha * __uint_as_float(acc[v * 8 + 5]));
    out.z = *reinterpret_cast<const uint32_t*>(&pair);
    pair = __floats2bfloat162_rn(alpha * __uint_as_float(acc[v * 8 + 6]), alpha * __uint_as_float(acc[v * 8 + 7]));
    out.w = *reinterpret_cast<const uint32_t*>(&pair);
    ptx::st_shared_v4(row_addr + uint32_t(((first_chunk + v) ^ (row & 7)) * 16), out);
  }
}

// ------------------------------------------------------------------------------------------
// The kernel.
// ------------------------------------------------------------------------------------------
// ------------------------------------------------------------------------------------------
// MXFP8 K32 quantisation of one group of 32 consecutive K values (device side).
// exponent: csrc/operators/sm103/detail/quantization.cuh:91-105 (integer form, 448 = 1.75*2^8);
// scaling by an exact power of two: :107-118; E4M3 conversion round-to-nearest-even,
// saturating; scale byte exponent+127 at the native offset
// (benchmarks/sm103/fused_mxfp8.cuh:13-16).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ int mxfp8_scale_exponent(float amax) {
  if (!(amax > 0.0f)) return 0;
  const int exponent = int((__float_as_uint(amax) + 0x001fffffu) >> 23) - 127 - 8;
  return exponent < -127 ? -127 : exponent > 127 ? 127 : exponent;
}
__device__ __forceinline__ float mxfp8_inverse_scale(int exponent) {
  return __uint_as_float(exponent == 127 ? 0x00400000u : uint32_t(127 - exponent) << 23);
}
__device__ __forceinline__ int64_t mxfp8_scale_offset(int64_t row, int64_t k, int64_t k_atoms) {
  return ((row >> 7) * k_atoms + (k >> 7)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + ((k & 127) >> 5);
}
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
// One thread quantises one K32 group read as four 16-byte vectors.
__device__ __forceinline__ void mxfp8_quantize_group(const uint16_t* in, uint8_t* out, uint8_t* scale_byte) {
  uint4 v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = reinterpret_cast<const uint4*>(in)[i];
  const uint32_t* w = reinterpret_cast<const uint32_t*>(v);
  float f[32];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    amax = fmaxf(amax, fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1])));
  }
  const int exponent = mxfp8_scale_exponent(amax);
  const float inverse = mxfp8_inverse_scale(exponent);
  uint4 o[2];
  uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
  for (int i = 0; i < 8; ++i)
    ow[i] = pack_e4m3x4(f[4 * i] * inverse, f[4 * i + 1] * inverse, f[4 * i + 2] * inverse, f[4 * i + 3] * inverse);
  reinterpret_cast<uint4*>(out)[0] = o[0];
  reinterpret_cast<uint4*>(out)[1] = o[1];
  *scale_byte = uint8_t(exponent + 127);
}
// Grid-stride quantisation of a row-major BF16 [rows, k] operand; rows up to the next multiple
// of 128 get the neutral scale (2^0), as the reference's quantiser writes them.
__device__ __forceinline__ void mxfp8_quantize_rows(const uint16_t* source, int64_t stride, int32_t rows,
                                                    int32_t k, uint8_t* data, uint8_t* scales,
                                                    int64_t first, int64_t step) {
  const int32_t groups_per_row = k >> 5;
  const int64_t k_atoms = (k + 127) >> 7;
  const int64_t padded_rows = (int64_t(rows) + 127) & ~int64_t(127);
  const int64_t total = padded_rows * groups_per_row;
  for (int64_t g = first; g < total; g += step) {
    const int64_t row = g / groups_per_row;
    const int32_t group = int32_t(g - row * groups_per_row);
    uint8_t* scale = scales + mxfp8_scale_offset(row, int64_t(group) << 5, k_atoms);
    if (row < rows)
      mxfp8_quantize_group(source + row * stride + (group << 5), data + row * k + (group << 5), scale);
    else
      *scale = 127;
  }
}

// The tile sequence of one CTA: compute CTAs first take every compute_ctas-th tile below
// join_tile, then every CTA of the grid (communication CTAs included) takes every
// all_ctas-th tile from join_tile on.
// Gate scout, one tile: the lanes of one warp acquire the flags of the tile's K groups (32 at a
// time, in the GEMM's K order, which starts at `gate_start` and wraps) and lane 0 posts the
// complete prefix, plus `progress_base`, to the shared-memory word the TMA producer watches.
// `virt` groups share one flag line (words 0, 2, 4, ...).  False when the wait gave up.
constexpr uint32_t kGateSeqStep = 65536u;  // progress word = tiles walked * step + complete groups
template <bool kRemoteWriter>
__device__ __forceinline__ bool scout_tile(const WaitContext& w, const uint32_t* flags, int32_t groups, int32_t virt,
                                           int32_t gate_start, uint32_t gate_word, uint32_t progress_base, int lane,
                                           uint32_t index_base) {
  int32_t prefix = 0;
  uint32_t spin = 0;
  uint64_t start = 0;
  while (prefix < groups) {
    // while stalled only the next few flags are polled
    const int32_t g = prefix + lane;
    uint32_t seen = 0u;
    if (g < groups && (spin == 0u || lane < 4)) {
      int32_t gate = g + gate_start;  // position g of the K order -> gate index
      if (gate >= groups) gate -= groups;
      const uint32_t* flag = flags + int64_t(gate / virt) * kReadyFlagStride + 2 * (gate % virt);
      seen = kRemoteWriter ? ptx::ld_acquire_sys(flag) : ptx::ld_acquire_gpu(flag);
    }
    const uint32_t complete = __ballot_sync(0xffffffffu, seen >= w.epoch);
    const int32_t n = complete == 0xffffffffu ? 32 : __ffs(int(~complete)) - 1;
    if (n > 0) {
      prefix = prefix + n < groups ? prefix + n : groups;
      __syncwarp();  // every lane's acquire is ordered before the release below
      if (lane == 0) ptx::st_release_cta_shared(gate_word, progress_base + uint32_t(prefix));
      spin = 0u;
      continue;
    }
    if (spin == 0u) start = ptx::globaltimer();
    __nanosleep(64);
    if ((++spin & 15u) == 0u) {
      uint32_t stop = 0u;
      if (lane == 0) {
        if (aborted(w)) {
          stop = 1u;
        } else if (ptx::globaltimer() - start > w.budget_ns) {
          report_timeout(w, kRemoteWriter ? kStatusPeerTimeout : kStatusFlagTimeout, kSiteLhsReady,
                         index_base + uint32_t(prefix), seen, w.epoch);
          stop = 1u;
        }
      }
      if (__shfl_sync(0xffffffffu, stop, 0)) return false;
    }
  }
  return true;
}

struct TileWalk {
  int64_t t, join_tile, tiles;
  int32_t compute_id, all_id, compute_ctas, all_ctas;
  bool joined;
  __device__ int64_t first() {
    joined = compute_id < 0;
    t = joined ? join_tile + all_id : compute_id;
    if (!joined && t >= join_tile) {
      joined = true;
      t = join_tile + all_id;
    }
    return t < tiles ? t : -1;
  }
  __device__ int64_t next() {
    if (!joined) {
      t += compute_ctas;
      if (t < join_tile) return t;
      joined = true;
      t = join_tile + all_id;
    } else {
      t += all_ctas;
    }
    return t < tiles ? t : -1;
  }
};

// kAMn / kBMn: the operand is stored with its M (resp. N) axis contiguous -- [K, M] / [K, N]
// row-major -- and is fed to the tensor core as an MN-major tile: 64-element groups along MN,
// each a [64 K rows x 128 bytes] swizzled box (the data-gradient GEMMs read the forward weight
// as stored, the weight-gradient GEMMs read both operands along the token axis).
template <int kBlockN, int kStages, int kMode, bool kTmaEpilogue, bool kAMn = false, bool kBMn = false,
          bool kMx = false, class Maps = StoreMaps>
__global__ void __launch_bounds__(kThreads, 1)
fused_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ Maps store_maps, const FusedParams p) {
  using Layout = SmemLayout<kBlockN, kStages, kMx>;
  constexpr uint32_t kAccumStages = Layout::kAccumStages;
  static_assert(!kMx || (!kAMn && !kBMn), "block-scaled operands are K-major");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool is_comm = int(blockIdx.x) < p.num_comm_ctas;
  const bool skip_role = (p.flags & (is_comm ? kFlagComputeOnly : kFlagCommOnly)) != 0u;

  if constexpr (kMx) {
    // Preparation by every CTA of the (cooperative) grid, then one grid-wide join.
    if (p.wq_source != nullptr || p.clear_words != nullptr) {
      const int64_t first = int64_t(blockIdx.x) * kThreads + threadIdx.x;
      const int64_t step = int64_t(gridDim.x) * kThreads;
      if (p.wq_source != nullptr)
        mxfp8_quantize_rows(p.wq_source, p.wq_stride, p.wq_rows, p.wq_k, p.wq_data, p.wq_scales, first, step);
      for (int64_t i = first; i < p.clear_count; i += step) p.clear_words[i] = 0u;
      __threadfence();
      ptx::fence_proxy_async_global();  // the quantised bytes are read by TMA after the join
      cooperative_groups::this_grid().sync();
    }
  }

  constexpr bool kCommJoins = kMode == kModeLhsPull || kMode == kModeHeadGate || kMode == kModeGradPull;
  const bool joins_compute = kCommJoins && is_comm && p.join_tile < p.order.count();
  if (is_comm && !skip_role) {
    if constexpr (kMode == kModeQkvPush) qkv_push_role<kBlockN>(p, smem);
    if constexpr (kMode == kModeLhsPull) {
      if constexpr (std::is_same<Maps, LhsPullMaps>::value) {
        LhsPullPolicy policy(p, store_maps);
        run_chunk_pipeline(policy, p.wait, base, p.num_comm_ctas);
      } else {
        if (p.flags & kFlagVectorPull) lhs_pull_role(p, smem);
        else lhs_pull_bulk_role(p, base);
      }
    }
    if constexpr (kMode == kModeHeadGate) {
      if constexpr (std::is_same<Maps, GradPushMaps>::value) {
        GradPushPolicy policy(p, store_maps);
        run_chunk_pipeline(policy, p.wait, base, p.num_comm_ctas);
        __threadfence_system();
      } else {
        grad_push_role(p);
      }
    }
    if constexpr (kMode == kModeGradPull) {
      if constexpr (std::is_same<Maps, GradPullMaps>::value) {
        GradPullPolicy policy(p, store_maps);
        run_chunk_pipeline(policy, p.wait, base, p.num_comm_ctas);
      } else {
        grad_pull_role(p);
      }
    }
  }
  if (joins_compute) __syncthreads();  // the transfer pipeline's shared memory is free again
  if ((!is_comm || joins_compute) && !(p.flags & kFlagCommOnly)) {
    const uint32_t bar_base = base + Layout::kBarrierOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tmem_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
    auto tmem_empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + kAccumStages + s); };
    const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 2 * kAccumStages);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Layout::kTmemSlotOffset);
    constexpr uint32_t kTmemColumns = Layout::kTmemColumns;

    if (threadIdx.x == 0) {
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_b);
      for (int s = 0; s < kStages; ++s) {
        ptx::mbar_init(full_bar(s), 1);
        ptx::mbar_init(empty_bar(s), 1);
      }
      for (int s = 0; s < kAccumStages; ++s) {
        ptx::mbar_init(tmem_full_bar(s), 1);
        ptx::mbar_init(tmem_empty_bar(s), kEpilogueThreads);
      }
      ptx::mbar_init(drain_bar, 1);
      ptx::fence_mbar_init();
      *reinterpret_cast<volatile uint32_t*>(smem + Layout::kTmemSlotOffset + 8) = 0u;  // gate progress
    }
    if (warp == 2) {
      ptx::tmem_alloc(base + Layout::kTmemSlotOffset, kTmemColumns);
      ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int32_t compute_ctas = int32_t(gridDim.x) - p.num_comm_ctas;
    const int32_t compute_id = int32_t(blockIdx.x) - p.num_comm_ctas;  // negative on communication CTAs
    const int64_t tiles = p.order.count();
    TileWalk walk_template;
    walk_template.join_tile = p.join_tile < tiles ? p.join_tile : tiles;
    walk_template.tiles = tiles;
    walk_template.compute_id = compute_id;
    walk_template.all_id = compute_id >= 0 ? compute_id : compute_ctas + int32_t(blockIdx.x);
    walk_template.compute_ctas = compute_ctas;
    walk_template.all_ctas = int32_t(gridDim.x);
    constexpr int32_t kBlockElems = kMx ? 2 * kBlockK : kBlockK;  // K elements per 128-byte row
    constexpr bool kGated = kMode == kModeLhsPull || kMode == kModeHeadGate || kMode == kModeGradPull;
    // Gate progress word: (tiles this CTA has walked) * kGateSeqStep + complete groups of the current one.
    const uint32_t gate_word = base + Layout::kTmemSlotOffset + 8u;
    (void)gate_word;
    const int32_t k_blocks = (p.k + kBlockElems - 1) / kBlockElems;

    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        uint32_t stage = 0, phase = 0;
        uint32_t issued_mask = 0, issued_parity = 0;  // last armed phase per stage (for the drain)
        bool ok = true;
        TileWalk walk = walk_template;
        uint32_t tile_seq = 0;
        for (int64_t t = walk.first(); ok && t >= 0; t = walk.next(), ++tile_seq) {
          int32_t mt, nt;
          p.order.decode(t, mt, nt);
          // K blocks of this tile whose groups the scout has posted complete; the group a block
          // needs is worked out (a division) only when the walk reaches a block that is not open.
          int32_t open_blocks = 0;
          for (int32_t ki = 0; ki < k_blocks; ++ki) {
            // K block loaded at step ki: the lhs pull starts at this rank's own shard and wraps.
            int32_t kb = ki;
            if constexpr (kMode == kModeLhsPull) {
              kb += p.lhs.k_block_start;
              if (kb >= k_blocks) kb -= k_blocks;
            }
            if constexpr (kGated) {
              // K groups whose rows arrive separately: peers' shards (forward pull) or Q/K/V heads
              // (backward).  The gate scout (warp 3) polls the flags, 32 at a time and ahead of
              // this thread, and posts how far this tile's groups are complete.
              if (ki >= open_blocks) {
                constexpr bool kHeads = kMode != kModeLhsPull;
                const int32_t group_width = kHeads ? p.grad.head_dim : p.lhs.virt_width;
                const int32_t groups = kHeads ? p.grad.q_heads + 2 * p.grad.kv_heads : p.lhs.world * p.lhs.virt;
                int32_t last = (ki * kBlockElems + kBlockElems - 1) / group_width;  // position in K order
                if (last >= groups) last = groups - 1;
                if (ki == 0) trace_event(p, 10);  // first gate wait of the tile begins
                uint32_t seen = 0;
                ok = progress_wait(gate_word, tile_seq * kGateSeqStep + uint32_t(last) + 1u, p.wait, kSiteLhsReady,
                                   uint32_t(mt * groups + last), &seen);
                // One proxy fence covers every group the scout has posted so far.
                ptx::fence_proxy_async_global();
                if (ki == 0) trace_event(p, 11);  // first gate passed
                if (!ok) break;
                const int32_t upto = (seen / kGateSeqStep) > tile_seq ? groups - 1 : int32_t(seen % kGateSeqStep) - 1;
                open_blocks = upto >= groups - 1 ? k_blocks
                                                 : int32_t((int64_t(upto + 1) * group_width) / kBlockElems);
              }
            }
            ok = mbar_wait(empty_bar(stage), phase ^ 1u, p.wait, kSiteSmemEmpty);
            if (!ok) break;
            const uint32_t a_dst = base + stage * Layout::kStageBytes;
            if constexpr (kMx) {
              // scale atoms of this K block: one for the A rows, one per 128 B rows that exist
              constexpr int kBAtoms = (kBlockN + 127) / 128;
              const int32_t n_atoms_total = (p.n + 127) / 128;
              const int32_t first_b_atom = nt * kBAtoms;
              const int32_t b_atoms = n_atoms_total - first_b_atom < kBAtoms ? n_atoms_total - first_b_atom : kBAtoms;
              ptx::mbar_expect_tx(full_bar(stage), Layout::kStageBytes + 512u * uint32_t(1 + b_atoms));
              const uint32_t sf_dst = base + Layout::kSfOffset + stage * Layout::kSfStageBytes;
              ptx::bulk_load(sf_dst, p.sfa + (int64_t(mt) * p.k_atoms + kb) * 512, 512u, full_bar(stage));
              for (int32_t j = 0; j < b_atoms; ++j)
                ptx::bulk_load(sf_dst + 512u * uint32_t(1 + j),
                               p.sfb + (int64_t(first_b_atom + j) * p.k_atoms + kb) * 512, 512u, full_bar(stage));
            } else {
              ptx::mbar_expect_tx(full_bar(stage), Layout::kStageBytes);
            }
            if constexpr (!kAMn) {
              ptx::tma_load_2d(a_dst, &tmap_a, full_bar(stage), kb * kBlockElems, mt * kBlockM);
            } else {
#pragma unroll
              for (int g = 0; g < kBlockM / 64; ++g)
                ptx::tma_load_2d(a_dst + g * kMnGroupBytes, &tmap_a, full_bar(stage),
                                 mt * kBlockM + g * 64, kb * kBlockK);
            }
            if constexpr (!kBMn) {
              ptx::tma_load_2d(a_dst + Layout::kABytes, &tmap_b, full_bar(stage), kb * kBlockElems,
                               nt * kBlockN);
            } else {
#pragma unroll
              for (int g = 0; g < kBlockN / 64; ++g)
                ptx::tma_load_2d(a_dst + Layout::kABytes + g * kMnGroupBytes, &tmap_b, full_bar(stage),
                                 nt * kBlockN + g * 64, kb * kBlockK);
            }
            issued_mask |= 1u << stage;
            issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
          (void)open_blocks;
        }
        (void)tile_seq;
        if (!ok) {
          // Unwinding: let every copy this thread started land before shared memory goes away.
          for (int s = 0; s < kStages; ++s)
            if ((issued_mask >> s) & 1u)
              mbar_wait(full_bar(s), (issued_parity >> s) & 1u, p.wait, kSiteDrain, false);
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ UMMA issuer
      if (lane == 0) {
        constexpr uint32_t kIdesc = ptx::idesc_bf16_f32(kBlockM, kBlockN, kAMn ? 1 : 0, kBMn ? 1 : 0);
        // Descriptor address step per UMMA (16 K values): 32 bytes inside the swizzle row of a
        // K-major tile, 16 rows of 128 bytes in an MN-major tile.
        constexpr uint64_t kAStep = kAMn ? (kUmmaK * 128) >> 4 : (kUmmaK * 2) >> 4;
        constexpr uint64_t kBStep = kBMn ? (kUmmaK * 128) >> 4 : (kUmmaK * 2) >> 4;
        uint32_t stage = 0, phase = 0, accum = 0, accum_phase = 0;
        uint32_t sf_parity = 0;
        (void)sf_parity;
        // high words of the operand and scale-atom descriptors (constant), low words of stage 0
        constexpr uint32_t kDescHigh = (1024u >> 4) | (1u << 14) | (2u << 29);
        constexpr uint32_t kSfDescHigh = (128u >> 4) | (1u << 14);
        constexpr uint32_t kMnStride = (kMnGroupBytes >> 4) << 16, kKStride = 1u << 16;  // the low word's second field
        constexpr uint32_t kAStride = kAMn ? kMnStride : kKStride, kBStride = kBMn ? kMnStride : kKStride;
        const uint32_t a_low0 = (base & 0x3FFFFu) >> 4;
        const uint32_t sf_low0 = ((base + Layout::kSfOffset) & 0x3FFFFu) >> 4;
        uint32_t a_low = a_low0, sf_low = sf_low0;
        (void)kSfDescHigh;
        (void)sf_low;
        bool ok = true;
        TileWalk walk = walk_template;
        for (int64_t t = walk.first(); ok && t >= 0; t = walk.next()) {
          ok = mbar_wait(tmem_empty_bar(accum), accum_phase ^ 1u, p.wait, kSiteTmemEmpty);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t d_tmem = tmem_base + accum * kBlockN;
          for (int32_t kb = 0; kb < k_blocks; ++kb) {
            ok = mbar_wait(full_bar(stage), phase, p.wait, kSiteSmemFull);
            if (!ok) break;
            // The descriptors of a stage differ from the previous stage's by a constant in their
            // low word: this thread's instruction stream per K block bounds the kernel, so they
            // are stepped, not rebuilt.
            const uint64_t a_desc = (uint64_t(kDescHigh) << 32) | (a_low + kAStride);
            const uint64_t b_desc = (uint64_t(kDescHigh) << 32) | (a_low + ((Layout::kABytes >> 4) + kBStride));
            const uint32_t accumulate = kb != 0 ? 1u : 0u;
            if constexpr (kMx) {
              // Copy this K block's scale atoms shared -> TMEM (32 lanes x 16 bytes each, broadcast
              // to the four lane quarters), then four K=32 UMMAs; UMMA k reads byte k of every
              // 32-bit scale column.  tcgen05.cp and tcgen05.mma of one thread execute in order;
              // two sets of scale columns alternate anyway.
              constexpr int kBAtoms = (kBlockN + 127) / 128;
              const uint64_t sf_desc = (uint64_t(kSfDescHigh) << 32) | sf_low;
              const uint32_t sf_tmem = tmem_base + Layout::kTmemSfOffset + (sf_parity ? Layout::kSfColumns : 0u);
              sf_parity ^= 1u;
              ptx::tmem_cp_32x128b_warpx4(sf_tmem, sf_desc);
#pragma unroll
              for (int j = 0; j < kBAtoms; ++j)
                ptx::tmem_cp_32x128b_warpx4(sf_tmem + 4u + 4u * j, sf_desc + ((512u * (1 + j)) >> 4));
#pragma unroll
              for (int k = 0; k < 4; ++k)
                ptx::umma_mxf8(d_tmem, a_desc + 2u * k, b_desc + 2u * k,
                               ptx::idesc_mxf8_e4m3(kBlockM, kBlockN, k, k), sf_tmem, sf_tmem + 4u,
                               k == 0 ? accumulate : 1u);
              sf_low += Layout::kSfStageBytes >> 4;
            } else {
              ptx::umma_f16(d_tmem, a_desc, b_desc, kIdesc, accumulate);
#pragma unroll
              for (int k = 1; k < kBlockK / kUmmaK; ++k)
                ptx::umma_f16_accumulate(d_tmem, a_desc + kAStep * k, b_desc + kBStep * k, kIdesc);
            }
            ptx::umma_commit(empty_bar(stage));  // frees the stage when these UMMAs retire
            a_low += Layout::kStageBytes >> 4;
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
              a_low = a_low0;
              sf_low = sf_low0;
            }
          }
          if (!ok) break;
          ptx::umma_commit(tmem_full_bar(accum));
          if (++accum == kAccumStages) { accum = 0; accum_phase ^= 1u; }
        }
        if (!ok) {
          // Unwinding: UMMAs already issued must retire before TMEM is released.  They retire on
          // a barrier of their own, so the epilogue never takes a partial tile for a finished one.
          ptx::umma_commit(drain_bar);
          mbar_wait(drain_bar, 0u, p.wait, kSiteDrain, false);
        }
      }
    } else if (warp == 3) {
      // ------------------------------------------------------------------ gate scout
      // Walks this CTA's tiles in the producer's order; every lane acquires one group's flag of
      // the current tile, the complete prefix is posted to shared memory for the producer.  The
      // scout runs ahead of the producer, so in steady state the producer never sees flag latency.
      if constexpr (kGated) {
        constexpr bool kRemoteWriter = kMode == kModeHeadGate;  // flags released by the sending GPUs
        constexpr bool kHeads = kMode != kModeLhsPull;
        const int32_t groups = kHeads ? p.grad.q_heads + 2 * p.grad.kv_heads : p.lhs.world * p.lhs.virt;
        const int32_t virt = kHeads ? 1 : p.lhs.virt;  // column slices sharing one flag line
        TileWalk walk = walk_template;
        uint32_t tile_seq = 0;
        bool ok = true;
        for (int64_t t = walk.first(); ok && t >= 0; t = walk.next(), ++tile_seq) {
          int32_t mt, nt;
          p.order.decode(t, mt, nt);
          const uint32_t* flags = p.ready + int64_t(mt) * (groups / virt) * kReadyFlagStride;
          ok = scout_tile<kRemoteWriter>(p.wait, flags, groups, virt, kHeads ? 0 : p.lhs.gate_start, gate_word,
                                         tile_seq * kGateSeqStep, lane, uint32_t(mt * groups));
        }
      }
    } else if (warp >= 4) {
      // ------------------------------------------------------------------ epilogue
      const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
      const int epi_tid = threadIdx.x - 128;
      uint32_t accum = 0, accum_phase = 0;
      bool ok = true;
      constexpr bool kDirect = kMode == kModeQkvDirect;
      constexpr bool kVectorPush = kDirect && !kTmaEpilogue;
      constexpr int kChunks = kBlockN / 8;
      uint32_t table = 0;  // which of the two route tables this tile uses
      uint32_t staged_blocks = 0;  // 64-column blocks staged so far (selects the staging buffer)
      TileWalk walk = walk_template;
      for (int64_t t = walk.first(); ok && t >= 0; t = walk.next()) {
        int32_t mt, nt;
        p.order.decode(t, mt, nt);
        PeerRow peer{};
        if constexpr (kDirect && !kTmaEpilogue) {
          uint16_t** col_base =
              reinterpret_cast<uint16_t**>(smem + Layout::kRouteTableOffset + table * kChunks * 16);
          int64_t* col_stride = reinterpret_cast<int64_t*>(col_base + kChunks);
          if (epi_tid < kChunks) {
            const int32_t feature = nt * kBlockN + epi_tid * 8;
            uint16_t* base = nullptr;
            int64_t stride = 0;
            if (feature < p.n) qkv_chunk_destination(p.qkv, feature, base, stride);
            col_base[epi_tid] = base;
            col_stride[epi_tid] = stride;
          }
          peer.col_base = col_base;
          peer.col_stride = col_stride;
          const int32_t local_row = mt * kBlockM + quarter * 32 + lane;
          peer.dest_row = local_row < p.m ? global_row(p.qkv.world, p.qkv.rank, p.qkv.seq_local,
                                                       p.qkv.global_seq, p.qkv.causal != 0, local_row)
                                          : 0;
          table ^= 1u;
        }
        ok = mbar_wait(tmem_full_bar(accum), accum_phase, p.wait, kSiteTmemFull);
        // The four epilogue warps leave together or not at all (they share a named barrier).
        ok = ptx::named_bar_all(2, kEpilogueThreads, ok);
        if (!ok) break;
        ptx::tc_fence_after();
        const int32_t row = mt * kBlockM + quarter * 32 + lane;
        const bool row_ok = row < p.m;
        uint16_t* d_row = p.d + int64_t(row) * p.ldd + nt * kBlockN;
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + accum * kBlockN;
        if constexpr (kTmaEpilogue) {
          // Stage 64-column blocks in 128B-swizzled shared memory and let the copy engine write
          // them: one tensor store into the local output and, for the direct QKV push, one into
          // the owning peer's planar tensor (full-line writes over NVLink).
          const int32_t row_in_tile = quarter * 32 + lane;
          // One thread hands a staged 64-column block to the copy engine.
          auto issue_stores = [&](int c, uint32_t staging) {
            const int32_t col = nt * kBlockN + c;
            if (col < p.n) {
              ptx::tma_store_2d(&store_maps.local, staging, col, mt * kBlockM);
              if constexpr (kMode == kModeQkvDirect) {
                const QkvRoute& r = p.qkv;
                const int32_t q_width = r.q_heads * r.head_dim, kv_width = r.kv_heads * r.head_dim;
                const int32_t segment = col < q_width ? 0 : (col < q_width + kv_width ? 1 : 2);
                const int32_t within = col - (segment == 0 ? 0 : q_width + (segment == 2 ? kv_width : 0));
                const int32_t local_width = (segment == 0 ? q_width : kv_width) / r.world;
                int32_t owner, local_col;  // segment > 0 only when kv_heads > 0
                qkv_owner_column(r, segment, within, local_width, owner, local_col);
                // defer_v: one [rows, q_local + kv_local] tensor per destination (map 0), V not routed
                const int32_t map = r.defer_v ? 0 : segment;
                const int32_t dest_col = local_col + (r.defer_v && segment == 1 ? q_width / r.world : 0);
                if (!(r.defer_v && segment == 2))
                  ptx::tma_store_2d(&store_maps.peer[owner][map], staging, dest_col,
                                    int32_t(global_row(r.world, r.rank, r.seq_local, r.global_seq,
                                                       r.causal != 0, mt * kBlockM)));
              }
            }
            ptx::bulk_commit();
          };
          if constexpr (kAccumStages == 1) {
            // Single accumulator: the first 64 columns go straight to the staging block (its store is
            // in flight while the rest is read), the other 192 into packed BF16 registers; TMEM is
            // handed back before those are staged, so the next tile's UMMAs overlap the stores.
            {
              const uint32_t staging =
                  base + Layout::kStagingOffset + (staged_blocks % Layout::kStagingBuffers) * Layout::kStagingBlockBytes;
              ++staged_blocks;
              if (epi_tid == 0) ptx::bulk_wait_read<Layout::kStagingBuffers - 1>();
              ptx::named_bar_sync(1, kEpilogueThreads);
              uint32_t acc0[32], acc1[32];
              ptx::tmem_ld_32x32b_x32(taddr, acc0);
              ptx::tmem_ld_32x32b_x32(taddr + 32, acc1);
              ptx::tmem_wait_ld();
              const uint32_t row_addr = staging + uint32_t(row_in_tile) * 128u;
              stage_accumulators(acc0, row_addr, 0, row_in_tile, p.alpha);
              stage_accumulators(acc1, row_addr, 4, row_in_tile, p.alpha);
              ptx::fence_proxy_async_shared();
              ptx::named_bar_sync(1, kEpilogueThreads);
              if (epi_tid == 0) issue_stores(0, staging);
            }
            uint32_t packed[(kBlockN - 64) / 2];
#pragma unroll
            for (int c = 64; c < kBlockN; c += 64) {
              uint32_t acc0[32], acc1[32];
              ptx::tmem_ld_32x32b_x32(taddr + c, acc0);
              ptx::tmem_ld_32x32b_x32(taddr + c + 32, acc1);
              ptx::tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                __nv_bfloat162 pair = __floats2bfloat162_rn(p.alpha * __uint_as_float(acc0[2 * e]),
                                                            p.alpha * __uint_as_float(acc0[2 * e + 1]));
                packed[(c - 64) / 2 + e] = *reinterpret_cast<const uint32_t*>(&pair);
                pair = __floats2bfloat162_rn(p.alpha * __uint_as_float(acc1[2 * e]),
                                             p.alpha * __uint_as_float(acc1[2 * e + 1]));
                packed[(c - 64) / 2 + 16 + e] = *reinterpret_cast<const uint32_t*>(&pair);
              }
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive(tmem_empty_bar(accum));
#pragma unroll
            for (int c = 64; c < kBlockN; c += 64) {
              const uint32_t staging =
                  base + Layout::kStagingOffset + (staged_blocks % Layout::kStagingBuffers) * Layout::kStagingBlockBytes;
              ++staged_blocks;
              if (epi_tid == 0) ptx::bulk_wait_read<Layout::kStagingBuffers - 1>();
              ptx::named_bar_sync(1, kEpilogueThreads);
              const uint32_t row_addr = staging + uint32_t(row_in_tile) * 128u;
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                const uint4 out = make_uint4(packed[(c - 64) / 2 + v * 4], packed[(c - 64) / 2 + v * 4 + 1],
                                             packed[(c - 64) / 2 + v * 4 + 2], packed[(c - 64) / 2 + v * 4 + 3]);
                ptx::st_shared_v4(row_addr + uint32_t((v ^ (row_in_tile & 7)) * 16), out);
              }
              ptx::fence_proxy_async_shared();
              ptx::named_bar_sync(1, kEpilogueThreads);
              if (epi_tid == 0) issue_stores(c, staging);
            }
          } else {
#pragma unroll 1
            for (int c = 0; c < kBlockN; c += 64) {
              const uint32_t staging =
                  base + Layout::kStagingOffset + (staged_blocks % Layout::kStagingBuffers) * Layout::kStagingBlockBytes;
              ++staged_blocks;
              // the block that last used this staging buffer has been read out by its tensor stores
              if (epi_tid == 0) ptx::bulk_wait_read<Layout::kStagingBuffers - 1>();
              ptx::named_bar_sync(1, kEpilogueThreads);
              uint32_t acc0[32], acc1[32];
              ptx::tmem_ld_32x32b_x32(taddr + c, acc0);
              ptx::tmem_ld_32x32b_x32(taddr + c + 32, acc1);
              ptx::tmem_wait_ld();
              if (c + 64 >= kBlockN) {
                ptx::tc_fence_before();
                ptx::mbar_arrive(tmem_empty_bar(accum));
              }
              const uint32_t row_addr = staging + uint32_t(row_in_tile) * 128u;
              stage_accumulators(acc0, row_addr, 0, row_in_tile, p.alpha);
              stage_accumulators(acc1, row_addr, 4, row_in_tile, p.alpha);
              ptx::fence_proxy_async_shared();
              ptx::named_bar_sync(1, kEpilogueThreads);
              if (epi_tid == 0) issue_stores(c, staging);
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < kBlockN; c += 64) {
            uint32_t acc0[32], acc1[32];
            ptx::tmem_ld_32x32b_x32(taddr + c, acc0);
            ptx::tmem_ld_32x32b_x32(taddr + c + 32, acc1);
            ptx::tmem_wait_ld();
            if (c + 64 >= kBlockN) {
              // Accumulator fully read: hand the TMEM stage back to the UMMA issuer.
              ptx::tc_fence_before();
              ptx::mbar_arrive(tmem_empty_bar(accum));
            }
            peer.chunk0 = c / 8;
            store_accumulators<kVectorPush>(acc0, d_row + c, nt * kBlockN + c, row_ok, p, peer);
            peer.chunk0 = c / 8 + 4;
            store_accumulators<kVectorPush>(acc1, d_row + c + 32, nt * kBlockN + c + 32, row_ok, p, peer);
          }
        }
        if constexpr (kMode == kModeQkvPush) {
          // Publish the tile: all 128 epilogue threads' stores, then one release at GPU scope
          // (flag index m*n_tiles+n, csrc/operators/sm103/detail/producer_consumer.cuh:42-48).
          ptx::named_bar_sync(1, kEpilogueThreads);
          if (epi_tid == 0) {
            __threadfence();
            ptx::st_release_gpu(
                p.ready + (int64_t(mt) * p.order.n_tiles + nt) * kReadyFlagStride, p.wait.epoch);
          }
        }
        if (epi_tid == 0) trace_event(p, 13);  // tile handed to the copy engine
        if (++accum == kAccumStages) { accum = 0; accum_phase ^= 1u; }
      }
      if constexpr (kTmaEpilogue) {
        if (epi_tid == 0) ptx::bulk_wait<0>();  // every tensor store of this CTA is performed
      }
    }

    if constexpr (kMode == kModeQkvDirect) __threadfence_system();  // peer stores performed
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 2) {
      ptx::tc_fence_after();
      ptx::tmem_dealloc(tmem_base, kTmemColumns);
    }
  }

  if constexpr (kMode == kModeQkvPush || kMode == kModeQkvDirect || kMode == kModeHeadGate ||
                kMode == kModeGradPull) {
    cooperative_groups::this_grid().sync();
    qkv_finalize(p);
  }
}

}  // namespace fuse_b200
