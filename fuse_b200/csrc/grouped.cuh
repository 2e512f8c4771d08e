// MoE grouped GEMMs: dispatch -> expert FC1, and expert FC2 -> combine; one persistent kernel each.
//
// For every local expert e, A_e[M_e, K] is gathered row by row from the ranks that hold the
// routed tokens (source[row] = {rank, token, slot} -> peer_input[rank][token, :]) into the
// expert's lhs slab, and D_e[M_e, N] = A_e W_e[N, K]^T.  M_e comes from the DEVICE row_offsets on
// every launch, so a captured launch can be replayed with new routes.
//
//   communication CTAs: the bulk-copy pull pipeline (one row = one chunk) over sub-units of 32
//       rows of a (expert, 128-row panel), dealt round-robin to the pull warps in panel order;
//       a panel's flag is published by the arrival that completes it;
//       on CTA pairs with an Auto budget there are none: one thread of EVERY compute CTA runs the
//       same pull (a pull over NVLink is bounded by what one SM may have in flight, so 148 SMs
//       pulling a little each move more than 20 CTAs pulling flat out), its two 16 KiB stages over
//       the epilogue staging this kernel's register epilogue leaves unused;
//   compute CTAs: the tcgen05 pipeline of fused_gemm.cuh with a grouped tile decode -- tile ->
//       (expert, m, n) through the per-launch prefix of tile counts, N fastest so the CTAs of a
//       wave share a freshly arrived panel -- per-expert tensor maps read from global memory,
//       the TMA producer gated on the panel flag, and an epilogue that writes only rows < M_e
//       (the caller's poison in the unused capacity stays).
//
// Combine (kCombine): A_e is local and complete at launch; D_e[M_e, N] = A_e W_e^T goes to the
// expert's output slab AND row by row to the rank that owns the token,
// peer_output[source.rank][(source.token * topk + source.slot), :].  No communication CTAs: the
// epilogue of every compute CTA stages each 64-column block in shared memory and its four warps
// write whole 128-byte row pieces -- eight lanes per row -- to the local slab and over NVLink to
// the owner, so the scatter of tile i overlaps the UMMAs of tile i+1.  Every rank has entered the
// invocation before anything is written into it (its started epoch), and the kernel ends with
// the done handshake: when it returns, every source has finished writing into this rank.
//
// Replaces csrc/operators/sm103/detail/grouped/{a2a_gemm,gemm_a2a,persistent_gemm,cutlass_pipeline,
// communication}.cuh of the reference.
#pragma once

#include "fused_gemm.cuh"
#include "pair_gemm.cuh"

namespace fuse_b200 {

struct GroupedTokenSource {
  int32_t rank, token, slot;
};

struct GroupedParams {
  int32_t experts, n, k, capacity, lhs_rows;
  int32_t rank, world;
  int32_t n_tiles, cap_tiles, num_comm_ctas;
  int32_t embedded;            // dispatch on CTA pairs: one thread of every compute CTA pulls, no communication CTAs
  const CUtensorMap* maps_a;   // [experts], lhs slabs   [lhs_rows, K]
  const CUtensorMap* maps_b;   // [experts], weights     [N, K]
  uint16_t* const* lhs;        // device array of per-expert slab pointers
  uint16_t* const* output;     // device array of per-expert output pointers [capacity, N]
  const int64_t* row_offsets;  // device [experts + 1]
  const GroupedTokenSource* source;
  const uint16_t* peer_input[kMaxWorldSize];
  uint16_t* peer_output[kMaxWorldSize];  // combine: every rank's [tokens * topk, N] branch outputs
  int32_t topk;
  uint32_t* peer_started[kMaxWorldSize];
  uint32_t* peer_done[kMaxWorldSize];
  uint32_t* ready;             // [experts * cap_tiles] flag lines: word 0 epoch, word 1 arrivals
  uint32_t* epoch_word;        // device epoch, advanced by the prepare kernel
  int32_t* tile_prefix;        // [experts + 1] tiles before each expert, written by prepare
  uint32_t flags;
  int32_t tile_m;              // rows of one GEMM tile: 128 (one CTA) or 256 (a CTA pair)
  WaitContext wait;            // wait.epoch is read from epoch_word on the device
};

// One block per launch: advances the device epoch, derives the tile prefix from the device row
// counts, clears the panels' arrival counters and tells every peer that this rank's inputs for
// this invocation are in place (everything earlier on the stream has completed).
// csrc/operators/sm103/detail/grouped/communication.cuh:137-207.
__global__ void grouped_prepare_kernel(GroupedParams p) {
  __shared__ uint32_t epoch;
  if (threadIdx.x == 0) {
    epoch = *p.epoch_word + 1u;
    if (epoch == 0u) epoch = 1u;
    *p.epoch_word = epoch;
    int32_t tiles = 0;
    for (int32_t e = 0; e < p.experts; ++e) {
      p.tile_prefix[e] = tiles;
      int64_t rows = p.row_offsets[e + 1] - p.row_offsets[e];
      if (rows < 0) rows = 0;
      if (rows > p.capacity) rows = p.capacity;
      tiles += int32_t((rows + p.tile_m - 1) / p.tile_m) * p.n_tiles;
    }
    p.tile_prefix[p.experts] = tiles;
  }
  for (int32_t i = threadIdx.x; i < p.experts * p.cap_tiles; i += blockDim.x)
    p.ready[int64_t(i) * kReadyFlagStride + 1] = 0u;
  __syncthreads();
  if (threadIdx.x < p.world) {
    __threadfence_system();
    ptx::st_release_sys(p.peer_started[threadIdx.x] + p.rank * kReadyFlagStride, epoch);
  }
}

// ------------------------------------------------------------------------------------------
// Dispatch pull (communication CTAs).
// ------------------------------------------------------------------------------------------
struct DispatchCursor {
  int32_t sub;       // sub-unit index over (expert, panel, quarter); advances by the pull warps
  int32_t row;       // row inside the sub-unit = chunk (one row per chunk), times pieces
  int32_t rows;      // rows of this sub-unit
  int32_t pieces_done;
  int32_t flag, needed;
  int64_t first_row; // index of its first row in `source`
  uint8_t* dst;      // destination of its first row
};

// One worker of the pull: a whole warp of a communication CTA (kWarp: lane 0 issues, the warp keeps
// in step) or the single copy thread embedded in a compute CTA.  `ring`: kPullStages stages of
// kPullStageBytes; `bars`: their mbarriers; sub-units are dealt round-robin to `workers` workers.
template <bool kWarp>
__device__ __forceinline__ void dispatch_pull(const GroupedParams& p, const WaitContext& w, uint32_t ring,
                                              uint32_t bars, int32_t worker, int32_t workers, int lane) {
  auto broadcast = [&](uint32_t value) { return kWarp ? __shfl_sync(0xffffffffu, value, 0) : value; };
  auto in_step = [&] {
    if (kWarp) __syncwarp();
  };
  if (lane == 0) {
    for (int s = 0; s < kPullStages; ++s) ptx::mbar_init(bars + 8u * s, 1);
    ptx::fence_mbar_init();
  }
  in_step();

  const uint32_t row_bytes = uint32_t(p.k) * 2u;
  const int32_t pieces = int32_t((row_bytes + kPullStageBytes - 1) / kPullStageBytes);
  const int32_t subs_per_expert = p.cap_tiles * kPullSubsPerTile;
  const int32_t subs_total = p.experts * subs_per_expert;

  auto seek = [&](DispatchCursor& c) {
    for (; c.sub < subs_total; c.sub += workers) {
      const int32_t e = c.sub / subs_per_expert, within = c.sub - e * subs_per_expert;
      const int32_t panel = within / kPullSubsPerTile, quarter = within - panel * kPullSubsPerTile;
      const int64_t begin = p.row_offsets[e];
      int64_t expert_rows = p.row_offsets[e + 1] - begin;
      if (expert_rows > p.capacity) expert_rows = p.capacity;
      const int32_t row0 = panel * kBlockM + quarter * kPullSubRows;
      if (row0 >= expert_rows) continue;
      const int32_t panel_rows = int32_t(expert_rows - panel * kBlockM < kBlockM ? expert_rows - panel * kBlockM : kBlockM);
      c.rows = int32_t(expert_rows - row0 < kPullSubRows ? expert_rows - row0 : kPullSubRows);
      c.row = 0;
      c.pieces_done = 0;
      c.flag = e * p.cap_tiles + panel;
      c.needed = (panel_rows + kPullSubRows - 1) / kPullSubRows;
      c.first_row = begin + row0;
      c.dst = reinterpret_cast<uint8_t*>(p.lhs[e]) + int64_t(row0 % p.lhs_rows) * row_bytes;
      return true;
    }
    return false;
  };
  auto advance = [&](DispatchCursor& c) {
    if (++c.pieces_done < pieces) return true;
    c.pieces_done = 0;
    if (++c.row < c.rows) return true;
    c.sub += workers;
    return seek(c);
  };

  uint32_t started_seen = 0;
  bool ok = true;
  auto start_load = [&](const DispatchCursor& c, int stage) {  // whole warp
    GroupedTokenSource src{0, 0, 0};
    if (lane == 0) src = p.source[c.first_row + c.row];
    const int32_t src_rank = int32_t(broadcast(uint32_t(src.rank)));
    if (src_rank != p.rank && !(p.flags & kFlagSkipPeerWait) && !((started_seen >> src_rank) & 1u)) {
      // the peer's tokens are valid once it has entered this invocation
      uint32_t good = 1u;
      if (lane == 0)
        good = flag_wait<true>(p.peer_started[p.rank] + src_rank * kReadyFlagStride, w.epoch, w,
                               kSitePeerStarted, uint32_t(src_rank)) ? 1u : 0u;
      good = broadcast(good);
      if (!good) { ok = false; return; }
      started_seen |= 1u << src_rank;
    }
    if (lane == 0) {
      const uint32_t offset = uint32_t(c.pieces_done) * kPullStageBytes;
      const uint32_t bytes = row_bytes - offset < kPullStageBytes ? row_bytes - offset : kPullStageBytes;
      const uint32_t bar = bars + 8u * stage;
      ptx::mbar_expect_tx(bar, bytes);
      ptx::bulk_load(ring + uint32_t(stage) * kPullStageBytes,
                     reinterpret_cast<const uint8_t*>(p.peer_input[src.rank]) + int64_t(src.token) * row_bytes + offset,
                     bytes, bar);
    }
  };

  uint32_t counted_before = 0;
  int32_t counted_flag = -1, counted_needed = 1;
  auto publish = [&]() {
    if (lane == 0 && counted_flag >= 0 && counted_before + 1u == uint32_t(counted_needed))
      ptx::st_release_gpu(p.ready + int64_t(counted_flag) * kReadyFlagStride, w.epoch);
    counted_flag = -1;
  };
  auto count = [&](int32_t flag, int32_t needed) {
    publish();
    if (lane == 0)
      counted_before = ptx::atom_acq_rel_gpu_add(p.ready + int64_t(flag) * kReadyFlagStride + 1, 1u);
    counted_flag = flag;
    counted_needed = needed;
  };

  DispatchCursor load_cursor{};
  load_cursor.sub = worker;
  bool more_loads = seek(load_cursor);
  if (!more_loads) return;
  DispatchCursor store_cursor = load_cursor;
  int32_t issued = 0, consumed = 0;
  while (issued < kPullStages && more_loads) {
    start_load(load_cursor, issued % kPullStages);
    if (!ok) break;
    more_loads = advance(load_cursor);
    ++issued;
  }
  int32_t lag_flag[kPullLag], lag_needed[kPullLag];
#pragma unroll
  for (int i = 0; i < kPullLag; ++i) { lag_flag[i] = -1; lag_needed[i] = 1; }
  bool more_stores = true;
  while (ok && more_stores) {
    const int stage = consumed % kPullStages;
    uint32_t landed = 1u;
    if (lane == 0)
      landed = mbar_wait(bars + 8u * stage, uint32_t(consumed / kPullStages) & 1u, w, kSiteCommStage) ? 1u : 0u;
    landed = broadcast(landed);
    if (!landed) { ok = false; break; }
    if (lane == 0) {
      const uint32_t offset = uint32_t(store_cursor.pieces_done) * kPullStageBytes;
      const uint32_t bytes = row_bytes - offset < kPullStageBytes ? row_bytes - offset : kPullStageBytes;
      ptx::bulk_store(store_cursor.dst + int64_t(store_cursor.row) * row_bytes + offset,
                      ring + uint32_t(stage) * kPullStageBytes, bytes);
    }
    ptx::bulk_commit();
    ++consumed;
    ptx::bulk_wait_read<0>();
    in_step();
    if (more_loads && issued < consumed + kPullStages) {
      start_load(load_cursor, issued % kPullStages);
      if (ok) {
        more_loads = advance(load_cursor);
        ++issued;
      }
    }
    ptx::bulk_wait<kPullLag>();
    in_step();
    if (lag_flag[kPullLag - 1] >= 0) count(lag_flag[kPullLag - 1], lag_needed[kPullLag - 1]);
#pragma unroll
    for (int i = kPullLag - 1; i > 0; --i) { lag_flag[i] = lag_flag[i - 1]; lag_needed[i] = lag_needed[i - 1]; }
    const bool closes = store_cursor.row + 1 == store_cursor.rows && store_cursor.pieces_done + 1 == pieces;
    lag_flag[0] = closes ? store_cursor.flag : -1;
    lag_needed[0] = store_cursor.needed;
    more_stores = advance(store_cursor);
  }
  ptx::bulk_wait<0>();
  in_step();
  if (ok) {
#pragma unroll
    for (int i = kPullLag - 1; i >= 0; --i)
      if (lag_flag[i] >= 0) count(lag_flag[i], lag_needed[i]);
    publish();
  }
  if (!ok && lane == 0) {
    for (int32_t i = consumed; i < issued; ++i)
      mbar_wait(bars + 8u * uint32_t(i % kPullStages), uint32_t(i / kPullStages) & 1u, w, kSiteDrain, false);
  }
}

// Communication CTAs: seven pull warps each.
__device__ __forceinline__ void dispatch_pull_role(const GroupedParams& p, const WaitContext& w,
                                                   uint32_t smem_base) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp >= kPullWarps) return;
  dispatch_pull<true>(p, w, smem_base + uint32_t(warp) * kPullStages * kPullStageBytes,
                      smem_base + kPullWarps * kPullStages * kPullStageBytes + uint32_t(warp) * kPullStages * 8u,
                      warp * p.num_comm_ctas + int32_t(blockIdx.x), p.num_comm_ctas * kPullWarps, lane);
}

// ------------------------------------------------------------------------------------------
// Combine epilogue (csrc/operators/sm103/detail/grouped/gemm_a2a.cuh:15-93 of the reference: one
// row of the expert's output per routed branch, no weighting or top-k reduction).
// ------------------------------------------------------------------------------------------
// Before the first remote write: every destination has entered this invocation (its buffers may
// be overwritten).  Called by the four epilogue warps together; false when a wait gave up.
__device__ __forceinline__ bool combine_wait_started(const GroupedParams& p, const WaitContext& w, int warp, int lane) {
  bool ok = true;
  if (warp == 4 && lane < p.world && !(p.flags & kFlagSkipPeerWait))
    ok = flag_wait<true>(p.peer_started[p.rank] + lane * kReadyFlagStride, w.epoch, w, kSitePeerStarted, uint32_t(lane));
  return ptx::named_bar_all(2, kEpilogueThreads, ok);
}

// One accumulator tile (this CTA's 128 rows x kBlockN columns at TMEM address `taddr`) -> BF16 ->
// the expert's output slab and the owners' branch rows.  `release` hands the accumulator back
// once its last column has been read.
template <int kBlockN, class Release>
__device__ __forceinline__ void combine_store_tile(const GroupedParams& p, int32_t expert, int32_t mt, int32_t nt,
                                                   int64_t expert_rows, uint32_t taddr, uint32_t staging_base,
                                                   uint32_t& staged_blocks, int warp, int lane, Release release) {
  const int quarter = warp & 3;
  const int32_t row_in_tile = quarter * 32 + lane;
  const int64_t begin = p.row_offsets[expert];
  // the rows this lane writes in the cooperative phase: 8 lanes per row, 4 rows per warp and step
  const int32_t piece = lane & 7;
  uint16_t* local_row[8];
  uint16_t* remote_row[8];
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int32_t r = mt * kBlockM + it * 16 + quarter * 4 + (lane >> 3);
    local_row[it] = nullptr;
    remote_row[it] = nullptr;
    if (r < expert_rows) {  // rows past M_e keep the caller's contents everywhere
      const GroupedTokenSource src = p.source[begin + r];
      local_row[it] = p.output[expert] + int64_t(r) * p.n;
      remote_row[it] = p.peer_output[src.rank] + (int64_t(src.token) * p.topk + src.slot) * p.n;
    }
  }
#pragma unroll 1
  for (int c = 0; c < kBlockN; c += 64) {
    const uint32_t staging = staging_base + (staged_blocks & 1u) * uint32_t(kBlockM * 128);
    ++staged_blocks;
    uint32_t acc0[32], acc1[32];
    ptx::tmem_ld_32x32b_x32(taddr + c, acc0);
    ptx::tmem_ld_32x32b_x32(taddr + c + 32, acc1);
    ptx::tmem_wait_ld();
    if (c + 64 >= kBlockN) release();
    const uint32_t row_addr = staging + uint32_t(row_in_tile) * 128u;
    stage_accumulators(acc0, row_addr, 0, row_in_tile, 1.0f);
    stage_accumulators(acc1, row_addr, 4, row_in_tile, 1.0f);
    // one barrier per block: a buffer is written again two blocks later, behind the barrier that
    // every thread reaches only after it has read this one
    ptx::named_bar_sync(1, kEpilogueThreads);
    const int32_t col = nt * kBlockN + c + piece * 8;
    if (col < p.n) {
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        if (local_row[it] == nullptr) continue;
        const int32_t rloc = it * 16 + quarter * 4 + (lane >> 3);
        const uint4 v = ptx::ld_shared_v4(staging + uint32_t(rloc) * 128u + uint32_t((piece ^ (rloc & 7)) * 16));
        ptx::st_v4(local_row[it] + col, v);
        ptx::st_v4(remote_row[it] + col, v);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// The grouped kernel.
// ------------------------------------------------------------------------------------------
template <int kBlockN, int kStages, bool kCombine = false>
__global__ void __launch_bounds__(kThreads, 1) grouped_gemm_kernel(const GroupedParams p) {
  using Layout = SmemLayout<kBlockN, kStages, false>;
  constexpr uint32_t kAccumStages = Layout::kAccumStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool is_comm = int(blockIdx.x) < p.num_comm_ctas;
  WaitContext w = p.wait;
  w.epoch = *p.epoch_word;  // advanced by the prepare kernel earlier on the stream

  if (is_comm) {
    dispatch_pull_role(p, w, base);
  } else {
    const uint32_t bar_base = base + Layout::kBarrierOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tmem_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
    auto tmem_empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + kAccumStages + s); };
    const uint32_t drain_bar = bar_base + 8u * (Layout::kNumBarriers - 1);  // unwinding UMMAs retire here
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Layout::kTmemSlotOffset);
    constexpr uint32_t kTmemColumns = Layout::kTmemColumns;
    if (threadIdx.x == 0) {
      for (int s = 0; s < kStages; ++s) {
        ptx::mbar_init(full_bar(s), 1);
        ptx::mbar_init(empty_bar(s), 1);
      }
      for (int s = 0; s < int(kAccumStages); ++s) {
        ptx::mbar_init(tmem_full_bar(s), 1);
        ptx::mbar_init(tmem_empty_bar(s), kEpilogueThreads);
      }
      ptx::mbar_init(drain_bar, 1);
      ptx::fence_mbar_init();
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
    const int32_t compute_id = int32_t(blockIdx.x) - p.num_comm_ctas;
    const int32_t tiles = p.tile_prefix[p.experts];
    const int32_t k_blocks = (p.k + kBlockK - 1) / kBlockK;
    // tile -> (expert, m, n); experts only move forward for one CTA
    auto decode = [&](int32_t t, int32_t& expert, int32_t& mt, int32_t& nt) {
      while (t >= p.tile_prefix[expert + 1]) ++expert;
      const int32_t local = t - p.tile_prefix[expert];
      mt = local / p.n_tiles;
      nt = local - mt * p.n_tiles;
    };

    if (warp == 0) {
      if (lane == 0) {
        uint32_t stage = 0, phase = 0, issued_mask = 0, issued_parity = 0;
        int32_t expert = 0;
        bool ok = true;
        for (int32_t t = compute_id; ok && t < tiles; t += compute_ctas) {
          int32_t mt, nt;
          decode(t, expert, mt, nt);
          if constexpr (!kCombine) {
            // the whole panel (all of K) arrives as one unit
            const int64_t flag = (int64_t(expert) * p.cap_tiles + mt) * kReadyFlagStride;
            ok = flag_wait<false>(p.ready + flag, w.epoch, w, kSitePanelReady, uint32_t(flag / kReadyFlagStride));
            ptx::fence_proxy_async_global();
            if (!ok) break;
          }
          const CUtensorMap* map_a = p.maps_a + expert;
          const CUtensorMap* map_b = p.maps_b + expert;
          for (int32_t kb = 0; kb < k_blocks; ++kb) {
            ok = mbar_wait(empty_bar(stage), phase ^ 1u, w, kSiteSmemEmpty);
            if (!ok) break;
            ptx::mbar_expect_tx(full_bar(stage), Layout::kStageBytes);
            const uint32_t a_dst = base + stage * Layout::kStageBytes;
            ptx::tma_load_2d(a_dst, map_a, full_bar(stage), kb * kBlockK, (mt * kBlockM) % p.lhs_rows);
            ptx::tma_load_2d(a_dst + Layout::kABytes, map_b, full_bar(stage), kb * kBlockK, nt * kBlockN);
            issued_mask |= 1u << stage;
            issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
        if (!ok)
          for (int s = 0; s < kStages; ++s)
            if ((issued_mask >> s) & 1u) mbar_wait(full_bar(s), (issued_parity >> s) & 1u, w, kSiteDrain, false);
      }
    } else if (warp == 1) {
      if (lane == 0) {
        constexpr uint32_t kIdesc = ptx::idesc_bf16_f32(kBlockM, kBlockN, 0, 0);
        constexpr uint32_t kDescHigh = (1024u >> 4) | (1u << 14) | (2u << 29);  // K-major, 128-byte swizzle
        const uint32_t a_low0 = ((base & 0x3FFFFu) >> 4) | (1u << 16);
        uint32_t a_low = a_low0;
        uint32_t stage = 0, phase = 0, accum = 0, accum_phase = 0;
        bool ok = true;
        for (int32_t t = compute_id; ok && t < tiles; t += compute_ctas) {
          ok = mbar_wait(tmem_empty_bar(accum), accum_phase ^ 1u, w, kSiteTmemEmpty);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t d_tmem = tmem_base + accum * kBlockN;
          for (int32_t kb = 0; kb < k_blocks; ++kb) {
            ok = mbar_wait(full_bar(stage), phase, w, kSiteSmemFull);
            if (!ok) break;
            // descriptors stepped from stage to stage (this thread's instruction stream bounds the kernel)
            const uint64_t a_desc = (uint64_t(kDescHigh) << 32) | a_low;
            const uint64_t b_desc = a_desc + (Layout::kABytes >> 4);
            ptx::umma_f16(d_tmem, a_desc, b_desc, kIdesc, kb != 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < kBlockK / kUmmaK; ++k)
              ptx::umma_f16_accumulate(d_tmem, a_desc + uint64_t(2 * k), b_desc + uint64_t(2 * k), kIdesc);
            ptx::umma_commit(empty_bar(stage));
            a_low += Layout::kStageBytes >> 4;
            if (++stage == kStages) { stage = 0; phase ^= 1u; a_low = a_low0; }
          }
          if (!ok) break;
          ptx::umma_commit(tmem_full_bar(accum));
          if (++accum == kAccumStages) { accum = 0; accum_phase ^= 1u; }
        }
        if (!ok) {
          ptx::umma_commit(drain_bar);
          mbar_wait(drain_bar, 0u, w, kSiteDrain, false);
        }
      }
    } else if (warp >= 4) {
      const int quarter = warp & 3;
      uint32_t accum = 0, accum_phase = 0;
      int32_t expert = 0;
      bool ok = true;
      uint32_t staged_blocks = 0;
      (void)staged_blocks;
      if constexpr (kCombine) ok = combine_wait_started(p, w, warp, lane);
      for (int32_t t = compute_id; ok && t < tiles; t += compute_ctas) {
        int32_t mt, nt;
        decode(t, expert, mt, nt);
        ok = mbar_wait(tmem_full_bar(accum), accum_phase, w, kSiteTmemFull);
        ok = ptx::named_bar_all(2, kEpilogueThreads, ok);
        if (!ok) break;
        ptx::tc_fence_after();
        int64_t expert_rows = p.row_offsets[expert + 1] - p.row_offsets[expert];
        if (expert_rows > p.capacity) expert_rows = p.capacity;
        if constexpr (kCombine) {
          const uint32_t bar = tmem_empty_bar(accum);
          combine_store_tile<kBlockN>(p, expert, mt, nt, expert_rows,
                                      tmem_base + (uint32_t(quarter * 32) << 16) + accum * kBlockN,
                                      base + Layout::kStagingOffset, staged_blocks, warp, lane, [&] {
                                        ptx::tc_fence_before();
                                        ptx::mbar_arrive(bar);
                                      });
          if (++accum == kAccumStages) { accum = 0; accum_phase ^= 1u; }
          continue;
        }
        const int32_t row = mt * kBlockM + quarter * 32 + lane;
        const bool row_ok = row < expert_rows;  // rows past M_e keep the caller's contents
        uint16_t* d_row = p.output[expert] + int64_t(row) * p.n + nt * kBlockN;
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + accum * kBlockN;
#pragma unroll 1
        for (int c = 0; c < kBlockN; c += 64) {
          uint32_t acc0[32], acc1[32];
          ptx::tmem_ld_32x32b_x32(taddr + c, acc0);
          ptx::tmem_ld_32x32b_x32(taddr + c + 32, acc1);
          ptx::tmem_wait_ld();
          if (c + 64 >= kBlockN) {
            ptx::tc_fence_before();
            ptx::mbar_arrive(tmem_empty_bar(accum));
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int32_t col = nt * kBlockN + c + half * 32 + v * 8;
              if (row_ok && col < p.n) {
                const uint32_t* a = half == 0 ? &acc0[v * 8] : &acc1[v * 8];
                uint4 out;
                __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(a[0]), __uint_as_float(a[1]));
                out.x = *reinterpret_cast<const uint32_t*>(&pair);
                pair = __floats2bfloat162_rn(__uint_as_float(a[2]), __uint_as_float(a[3]));
                out.y = *reinterpret_cast<const uint32_t*>(&pair);
                pair = __floats2bfloat162_rn(__uint_as_float(a[4]), __uint_as_float(a[5]));
                out.z = *reinterpret_cast<const uint32_t*>(&pair);
                pair = __floats2bfloat162_rn(__uint_as_float(a[6]), __uint_as_float(a[7]));
                out.w = *reinterpret_cast<const uint32_t*>(&pair);
                ptx::st_v4(d_row + c + half * 32 + v * 8, out);
              }
            }
          }
        }
        if (++accum == kAccumStages) { accum = 0; accum_phase ^= 1u; }
      }
    }
    if constexpr (kCombine) __threadfence_system();  // this thread's remote rows are performed before the grid joins
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 2) {
      ptx::tc_fence_after();
      ptx::tmem_dealloc(tmem_base, kTmemColumns);
    }
  }

  // Every rank tells its peers that it has finished reading their tokens (combine: writing their
  // branch rows), and leaves only when all of them have finished with its own
  // (communication.cuh:237-250).
  cooperative_groups::this_grid().sync();
  if (blockIdx.x == 0 && threadIdx.x < 32) {
    // Combine: "done" tells a peer that its branch rows are complete, so a launch in which a wait
    // gave up publishes nothing (the peers run out their own bounded wait and record it).  Dispatch:
    // "done" only says that this rank no longer reads the peer's tokens, true after a failure too.
    if constexpr (kCombine) {
      uint32_t failed = lane == 0 && aborted(w) ? 1u : 0u;
      failed = __shfl_sync(0xffffffffu, failed, 0);
      if (failed) return;
    }
    if (lane == 0) ptx::fence_sc_sys();
    __syncwarp();
    if (lane < p.world) ptx::st_release_sys(p.peer_done[lane] + p.rank * kReadyFlagStride, w.epoch);
    __syncwarp();
    if (lane < p.world && !(p.flags & kFlagSkipPeerWait))
      flag_wait<true>(p.peer_done[p.rank] + lane * kReadyFlagStride, w.epoch, w, kSitePeerDone, uint32_t(lane));
  }
}

// ------------------------------------------------------------------------------------------
// The grouped kernel on CTA pairs (policy.mma_sm_count == 2): clusters of two CTAs work on
// 256 x 256 tiles of one expert with tcgen05.mma.cta_group::2 -- each CTA holds its own 128 lhs
// rows and half of the weight tile per K block, six stages; barriers and TMEM as in
// pair_gemm.cuh.  Each CTA gates its own 128-row panel; a panel past M_e has no rows to wait
// for (its accumulator rows are never stored).  Communication CTAs come in whole pairs.
// ------------------------------------------------------------------------------------------
template <bool kCombine = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) grouped_pair_kernel(const GroupedParams p) {
  using Layout = PairLayoutT<false>;
  constexpr int kStages = Layout::kStages;
  constexpr int kBlockN = Layout::kBlockN;
  constexpr uint32_t kAccumStages = Layout::kAccumStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool is_comm = int(blockIdx.x) < p.num_comm_ctas;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool leader = rank == 0;
  WaitContext w = p.wait;
  w.epoch = *p.epoch_word;  // advanced by the prepare kernel earlier on the stream

  if (is_comm) {
    dispatch_pull_role(p, w, base);
  } else {
    const uint32_t bar_base = base + Layout::kBarrierOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tmem_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
    auto tmem_empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + kAccumStages + s); };
    const uint32_t drain_bar = bar_base + 8u * (Layout::kNumBarriers - 1);  // the leader's; unwinding UMMAs retire here
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Layout::kTmemSlotOffset);
    if (threadIdx.x == 0) {
      for (int s = 0; s < kStages; ++s) {
        ptx::mbar_init(full_bar(s), 1);
        ptx::mbar_init(empty_bar(s), 1);
      }
      for (int s = 0; s < int(kAccumStages); ++s) {
        ptx::mbar_init(tmem_full_bar(s), 1);
        ptx::mbar_init(tmem_empty_bar(s), 2 * kEpilogueThreads);
      }
      ptx::mbar_init(drain_bar, 1);
      ptx::fence_mbar_init();
    }
    if (warp == 2) {
      ptx::tmem_alloc_pair(base + Layout::kTmemSlotOffset, Layout::kTmemColumns);
      ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int32_t pairs = (int32_t(gridDim.x) - p.num_comm_ctas) / 2;
    const int32_t pair_id = (int32_t(blockIdx.x) - p.num_comm_ctas) / 2;
    const int32_t tiles = p.tile_prefix[p.experts];  // 256-row tiles
    const int32_t k_blocks = (p.k + kBlockK - 1) / kBlockK;
    auto decode = [&](int32_t t, int32_t& expert, int32_t& mp, int32_t& nt) {
      while (t >= p.tile_prefix[expert + 1]) ++expert;
      const int32_t local = t - p.tile_prefix[expert];
      mp = local / p.n_tiles;
      nt = local - mp * p.n_tiles;
    };
    auto rows_of = [&](int32_t expert) {
      int64_t rows = p.row_offsets[expert + 1] - p.row_offsets[expert];
      if (rows > p.capacity) rows = p.capacity;
      return rows < 0 ? int64_t(0) : rows;
    };
    bool unwound = false;

    if (warp == 0) {
      if (lane == 0) {
        uint32_t stage = 0, phase = 0;
        int32_t expert = 0;
        bool ok = true;
        // The flag of the NEXT tile's panel is looked at late in this tile's K loop, when the ring is
        // full and a global round trip costs the GEMM nothing; a panel seen complete then needs no
        // wait (and no bubble) at the tile boundary.
        bool panel_seen = false;
        for (int32_t t = pair_id; ok && t < tiles; t += pairs) {
          int32_t mp, nt;
          decode(t, expert, mp, nt);
          const int32_t mt = mp * 2 + int32_t(rank);  // this CTA's 128-row panel
          if (!kCombine && !panel_seen && int64_t(mt) * kBlockM < rows_of(expert)) {
            const int64_t flag = (int64_t(expert) * p.cap_tiles + mt) * kReadyFlagStride;
            ok = flag_wait<false>(p.ready + flag, w.epoch, w, kSitePanelReady, uint32_t(flag / kReadyFlagStride));
            ptx::fence_proxy_async_global();
            if (!ok) break;
          }
          panel_seen = false;
          const CUtensorMap* map_a = p.maps_a + expert;
          const CUtensorMap* map_b = p.maps_b + expert;
          const int32_t look_at = k_blocks > 16 ? k_blocks - 8 : -1;
          for (int32_t kb = 0; kb < k_blocks; ++kb) {
            if (!kCombine && kb == look_at && t + pairs < tiles) {
              int32_t next_expert = expert, next_mp, next_nt;
              decode(t + pairs, next_expert, next_mp, next_nt);
              const int32_t next_mt = next_mp * 2 + int32_t(rank);
              if (next_expert != expert) {  // the next tile's operand maps, on their way into the descriptor cache
                ptx::prefetch_tensormap(p.maps_a + next_expert);
                ptx::prefetch_tensormap(p.maps_b + next_expert);
              }
              if (int64_t(next_mt) * kBlockM >= rows_of(next_expert)) {
                panel_seen = true;  // no rows in this half: nothing to wait for
              } else if (ptx::ld_acquire_gpu(p.ready + (int64_t(next_expert) * p.cap_tiles + next_mt) * kReadyFlagStride) >=
                         w.epoch) {
                ptx::fence_proxy_async_global();
                panel_seen = true;
              }
            }
            ok = mbar_wait(empty_bar(stage), phase ^ 1u, w, kSiteSmemEmpty);
            if (!ok) break;
            const uint32_t a_dst = base + stage * Layout::kStageBytes;
            const uint32_t leader_full = ptx::map_to_cta(full_bar(stage), 0);
            if (leader) ptx::mbar_expect_tx(full_bar(stage), 2 * Layout::kStageBytes);
            ptx::tma_load_2d_pair(a_dst, map_a, leader_full, kb * kBlockK, mt * kBlockM);
            ptx::tma_load_2d_pair(a_dst + Layout::kABytes, map_b, leader_full, kb * kBlockK,
                                  nt * kBlockN + int32_t(rank) * (kBlockN / 2));
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
        unwound = !ok;
      }
    } else if (warp == 1) {
      if (lane == 0 && leader) {
        constexpr uint32_t kIdesc = ptx::idesc_bf16_f32(2 * kBlockM, kBlockN, 0, 0);
        constexpr uint32_t kDescHigh = (1024u >> 4) | (1u << 14) | (2u << 29);  // K-major, 128-byte swizzle
        const uint32_t a_low0 = ((base & 0x3FFFFu) >> 4) | (1u << 16);
        uint32_t a_low = a_low0;
        uint32_t stage = 0, phase = 0, accum = 0, accum_phase = 0;
        bool ok = true;
        for (int32_t t = pair_id; ok && t < tiles; t += pairs) {
          ok = mbar_wait(tmem_empty_bar(accum), accum_phase ^ 1u, w, kSiteTmemEmpty);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t d_tmem = tmem_base + accum * kBlockN;
          for (int32_t kb = 0; kb < k_blocks; ++kb) {
            ok = mbar_wait(full_bar(stage), phase, w, kSiteSmemFull);
            if (!ok) break;
            // descriptors stepped from stage to stage (this thread's instruction stream bounds the kernel)
            const uint64_t a_desc = (uint64_t(kDescHigh) << 32) | a_low;
            const uint64_t b_desc = a_desc + (Layout::kABytes >> 4);
            ptx::umma_f16_pair(d_tmem, a_desc, b_desc, kIdesc, kb != 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < kBlockK / kUmmaK; ++k)
              ptx::umma_f16_pair_accumulate(d_tmem, a_desc + uint64_t(2 * k), b_desc + uint64_t(2 * k), kIdesc);
            ptx::umma_commit_pair(empty_bar(stage), 3);
            a_low += Layout::kStageBytes >> 4;
            if (++stage == kStages) { stage = 0; phase ^= 1u; a_low = a_low0; }
          }
          if (!ok) break;
          ptx::umma_commit_pair(tmem_full_bar(accum), 3);
          if (++accum == kAccumStages) { accum = 0; accum_phase ^= 1u; }
        }
        if (!ok) {
          ptx::umma_commit_pair(drain_bar, 1);
          mbar_wait(drain_bar, 0u, w, kSiteDrain, false);
        }
        unwound = !ok;
      }
    } else if (warp == 2) {
      // embedded dispatch pull: the ring lies over the epilogue staging (unused by this kernel's
      // register epilogue), its two mbarriers behind the TMEM slot
      if constexpr (!kCombine) {
        static_assert(Layout::kStagingBuffers * Layout::kStagingBlockBytes >= kPullStages * kPullStageBytes, "ring");
        static_assert(Layout::kTmemSlotOffset + 16 + 8 * kPullStages <= Layout::kBytes, "ring barriers");
        if (p.embedded && lane == 0)
          dispatch_pull<false>(p, w, base + Layout::kStagingOffset, base + Layout::kTmemSlotOffset + 16u,
                               int32_t(blockIdx.x), int32_t(gridDim.x), 0);
        __syncwarp();
      }
    } else if (warp >= 4) {
      const int quarter = warp & 3;
      const uint32_t leader_tmem_empty0 = ptx::map_to_cta(tmem_empty_bar(0), 0);
      const uint32_t leader_tmem_empty1 = ptx::map_to_cta(tmem_empty_bar(1), 0);
      uint32_t accum = 0, accum_phase = 0;
      int32_t expert = 0;
      bool ok = true;
      uint32_t staged_blocks = 0;
      (void)staged_blocks;
      if constexpr (kCombine) ok = combine_wait_started(p, w, warp, lane);
      for (int32_t t = pair_id; ok && t < tiles; t += pairs) {
        int32_t mp, nt;
        decode(t, expert, mp, nt);
        const int32_t mt = mp * 2 + int32_t(rank);
        ok = mbar_wait(tmem_full_bar(accum), accum_phase, w, kSiteTmemFull);
        ok = ptx::named_bar_all(2, kEpilogueThreads, ok);
        if (!ok) break;
        ptx::tc_fence_after();
        const int64_t expert_rows = rows_of(expert);
        if constexpr (kCombine) {
          const uint32_t bar = accum ? leader_tmem_empty1 : leader_tmem_empty0;
          combine_store_tile<kBlockN>(p, expert, mt, nt, expert_rows,
                                      tmem_base + (uint32_t(quarter * 32) << 16) + accum * kBlockN,
                                      base + Layout::kStagingOffset, staged_blocks, warp, lane, [&] {
                                        ptx::tc_fence_before();
                                        ptx::mbar_arrive_cluster(bar);
                                      });
          if (++accum == kAccumStages) { accum = 0; accum_phase ^= 1u; }
          continue;
        }
        const int32_t row = mt * kBlockM + quarter * 32 + lane;
        const bool row_ok = row < expert_rows;  // rows past M_e keep the caller's contents
        uint16_t* d_row = p.output[expert] + int64_t(row) * p.n + nt * kBlockN;
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + accum * kBlockN;
#pragma unroll 1
        for (int c = 0; c < kBlockN; c += 64) {
          uint32_t acc0[32], acc1[32];
          ptx::tmem_ld_32x32b_x32(taddr + c, acc0);
          ptx::tmem_ld_32x32b_x32(taddr + c + 32, acc1);
          ptx::tmem_wait_ld();
          if (c + 64 >= kBlockN) {
            ptx::tc_fence_before();
            ptx::mbar_arrive_cluster(accum ? leader_tmem_empty1 : leader_tmem_empty0);
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int32_t col = nt * kBlockN + c + half * 32 + v * 8;
              if (row_ok && col < p.n) {
                const uint32_t* a = half == 0 ? &acc0[v * 8] : &acc1[v * 8];
                uint4 out;
                __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(a[0]), __uint_as_float(a[1]));
                out.x = *reinterpret_cast<const uint32_t*>(&pair);
                pair = __floats2bfloat162_rn(__uint_as_float(a[2]), __uint_as_float(a[3]));
                out.y = *reinterpret_cast<const uint32_t*>(&pair);
                pair = __floats2bfloat162_rn(__uint_as_float(a[4]), __uint_as_float(a[5]));
                out.z = *reinterpret_cast<const uint32_t*>(&pair);
                pair = __floats2bfloat162_rn(__uint_as_float(a[6]), __uint_as_float(a[7]));
                out.w = *reinterpret_cast<const uint32_t*>(&pair);
                ptx::st_v4(d_row + c + half * 32 + v * 8, out);
              }
            }
          }
        }
        if (++accum == kAccumStages) { accum = 0; accum_phase ^= 1u; }
      }
      unwound = !ok;
    }
    if (unwound) {
      // error path: copies that were started may still be landing in either CTA's shared memory
      const uint64_t start = ptx::globaltimer();
      while (ptx::globaltimer() - start < 200000ull) __nanosleep(1000);
    }
    if constexpr (kCombine) __threadfence_system();  // this thread's remote rows are performed before the grid joins
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();
    if (warp == 2) {
      ptx::tc_fence_after();
      ptx::tmem_dealloc_pair(tmem_base, Layout::kTmemColumns);
    }
  }

  cooperative_groups::this_grid().sync();
  if (blockIdx.x == 0 && threadIdx.x < 32) {
    // Combine: "done" tells a peer that its branch rows are complete, so a launch in which a wait
    // gave up publishes nothing (the peers run out their own bounded wait and record it).  Dispatch:
    // "done" only says that this rank no longer reads the peer's tokens, true after a failure too.
    if constexpr (kCombine) {
      uint32_t failed = lane == 0 && aborted(w) ? 1u : 0u;
      failed = __shfl_sync(0xffffffffu, failed, 0);
      if (failed) return;
    }
    if (lane == 0) ptx::fence_sc_sys();
    __syncwarp();
    if (lane < p.world) ptx::st_release_sys(p.peer_done[lane] + p.rank * kReadyFlagStride, w.epoch);
    __syncwarp();
    if (lane < p.world && !(p.flags & kFlagSkipPeerWait))
      flag_wait<true>(p.peer_done[p.rank] + lane * kReadyFlagStride, w.epoch, w, kSitePeerDone, uint32_t(lane));
  }
}

}  // namespace fuse_b200
