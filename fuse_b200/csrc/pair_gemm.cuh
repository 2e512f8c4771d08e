// BF16 NT GEMM on CTA pairs: two CTAs of a cluster, resident on the two SMs of one TPC, work on
// one 256 x 256 output tile with `tcgen05.mma.cta_group::2`.
//
// Each CTA keeps the A rows of its half of the tile (128 x 64 per K block) and HALF of the B tile
// (128 of the 256 weight rows); the tensor cores of both SMs read both halves, so a CTA moves and
// holds 32 KiB per K block instead of 48 KiB -- six pipeline stages instead of four, and a third
// less shared-memory traffic per FLOP, which is what bounds the one-CTA 128 x 256 tile.  The
// accumulator rows of each CTA stay in its own TMEM (two stages of 256 columns).
//
// Roles per CTA: warp 0 TMA producer (its own A and B halves; the byte counts of both CTAs land
// on the LEADER's full barrier), warp 1 UMMA issuer (leader CTA only; its commits arrive on the
// empty / accumulator-full barriers of both CTAs), warp 2 TMEM allocator (same warp in both
// CTAs), warps 4-7 epilogue (both CTAs; the peer's epilogue threads release the accumulator on
// the leader's barrier through the cluster's shared-memory window).
//
// Modes: plain GEMM; the QKV projection whose epilogue stores every 64-column block into the
// local output and into the owning peer's planar Q | K | V tensor (no communication CTAs); and
// the output projection fed by the lhs pull (communication CTAs, launched as whole pairs, run the
// tensor-copy pull and join the GEMM afterwards; each compute CTA gates its own A rows on the
// column-slice flags through its gate scout warp).
// Replaces the 2-SM instances of csrc/operators/sm103/detail/cutlass_pipeline.cuh of the
// reference (tile m256n256k64), written directly against the instructions.
#pragma once

#include <cooperative_groups.h>

#include "fused_gemm.cuh"

namespace fuse_b200 {

// kMx: block-scaled E4M3 operands.  A K block is then 128 one-byte elements (the same 128-byte
// rows); every stage also carries the 512-byte scale atom of this CTA's A rows and the two atoms
// of ALL 256 B rows (each CTA's tensor core needs the scales of the whole B tile); the
// accumulator is single-buffered (TMEM also holds the scales) and drained whole by the epilogue.
// kEmbedded: one warp of every compute CTA runs the copy pipeline of the mode -- the lhs pull, the
// gradient push or the gradient pull -- and there are no communication CTAs at all; its two 16 KiB
// stages take the place of the sixth GEMM stage.
template <bool kMx, bool kEmbedded = false>
struct PairLayoutT {
  static constexpr int kStages = kEmbedded ? 5 : 6;
  static constexpr int kAccumStages = kMx ? 1 : 2;
  static constexpr int kBlockN = 256;                                  // of the pair's tile
  static constexpr uint32_t kABytes = kBlockM * kBlockK * 2;           // this CTA's 128 rows
  static constexpr uint32_t kBBytes = (kBlockN / 2) * kBlockK * 2;     // this CTA's half of B
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kSfStageBytes = kMx ? 512u * 3u : 0u;      // SFA, SFB rows 0-127, SFB rows 128-255
  static constexpr uint32_t kSfOffset = kStages * kStageBytes;
  static constexpr uint32_t kStagingBuffers = kMx ? 1 : 2;
  static constexpr uint32_t kStagingBlockBytes = kBlockM * 64 * 2;
  static constexpr uint32_t kStagingOffset = kSfOffset + ((kStages * kSfStageBytes + 1023u) & ~1023u);
  static constexpr uint32_t kCopyRingOffset = kStagingOffset + kStagingBuffers * kStagingBlockBytes;
  static constexpr uint32_t kCopyRingBytes = kEmbedded ? kPullStages * kPullStageBytes : 0u;
  static constexpr uint32_t kBarrierOffset = kCopyRingOffset + kCopyRingBytes;
  // + 1: the leader's drain barrier (UMMAs of an unwinding launch retire on it, never on an
  // accumulator-full barrier)
  static constexpr uint32_t kNumBarriers = 2 * kStages + 2 * kAccumStages + (kEmbedded ? kPullStages : 0) + 1;
  static constexpr uint32_t kTmemSlotOffset = kBarrierOffset + kNumBarriers * 8;
  static constexpr uint32_t kComputeBytes = kTmemSlotOffset + 16;
  // communication pairs lay the copy pipeline over the same allocation
  static constexpr uint32_t kBytes = kComputeBytes > kPullSmemBytes ? kComputeBytes : kPullSmemBytes;
  static constexpr uint32_t kDynamicBytes = kBytes + 1024;
  static constexpr uint32_t kTmemColumns = 512;
  // TMEM: accumulator stage(s), then (kMx) two alternating sets of scale columns: 4 for A, 8 for B.
  static constexpr uint32_t kSfColumns = kMx ? 12u : 0u;
  static constexpr uint32_t kTmemSfOffset = kAccumStages * kBlockN;
  static_assert(kTmemSfOffset + 2 * kSfColumns <= kTmemColumns, "TMEM budget");
  static_assert(kDynamicBytes <= 227 * 1024, "shared memory budget");
  static_assert(kDynamicBytes > 114 * 1024, "must force one CTA per SM");
};
using PairLayout = PairLayoutT<false>;

// kMode: kModePlain, kModeQkvDirect (FusedParams::qkv, StoreMaps::peer) or kModeLhsPull
// (FusedParams::lhs, LhsPullMaps; num_comm_ctas even).
// kMx: block-scaled E4M3 (tmap_sfa / tmap_sfb: the operands' scale storage as rows of one 512-byte
// atom, 128 32-bit words); FusedParams::wq_* / clear_* request the weight quantisation prologue.
// kAMn / kBMn (BF16 only): the operand is stored with its M (resp. N) axis contiguous and is fed to
// the tensor core as an MN-major tile -- 64-element groups along MN, each a [64 K rows x 128 bytes]
// swizzled box; a CTA then holds two groups of A and two groups of its half of B per K block.
template <int kMode, class Maps, bool kMx = false, bool kAMn = false, bool kBMn = false, bool kEmbedded = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
pair_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                 const __grid_constant__ Maps store_maps, const FusedParams p) {
  static_assert(kMode == kModePlain || kMode == kModeQkvDirect || kMode == kModeLhsPull || kMode == kModeGradPull ||
                    kMode == kModeHeadGate,
                "modes of the pair kernel");
  static_assert(kMode != kModeGradPull || kMx, "the gradient pull feeds the block-scaled GEMM");
  static_assert(!kMx || (!kAMn && !kBMn), "block-scaled operands are K-major");
  constexpr bool kDirect = kMode == kModeQkvDirect;
  constexpr bool kGated = kMode == kModeLhsPull || kMode == kModeGradPull || kMode == kModeHeadGate;
  constexpr bool kHeads = kMode == kModeGradPull || kMode == kModeHeadGate;  // K groups are Q/K/V heads
  constexpr bool kRemoteWriter = kMode == kModeHeadGate;  // flags released by the sending GPUs
  static_assert(!kEmbedded || kGated, "the embedded copy warp serves the pull and push modes");
  using Layout = PairLayoutT<kMx, kEmbedded>;
  constexpr int kStages = Layout::kStages;
  constexpr int32_t kBlockElems = kMx ? 2 * kBlockK : kBlockK;  // K elements per 128-byte row
  constexpr int kBlockN = Layout::kBlockN;
  constexpr uint32_t kAccumStages = Layout::kAccumStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // the same offset in both CTAs of the pair
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0: leader (issues the UMMAs)
  const bool leader = rank == 0;

  const uint32_t bar_base = base + Layout::kBarrierOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
  auto tmem_empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + kAccumStages + s); };
  const uint32_t drain_bar = bar_base + 8u * (Layout::kNumBarriers - 1);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Layout::kTmemSlotOffset);
  const uint32_t gate_word = base + Layout::kTmemSlotOffset + 8u;

  if constexpr (kMx) {
    // Preparation by every CTA of the (cooperative) grid, then one grid-wide join: quantise the
    // BF16 master weight into the workspace, clear the library-owned flag words.
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

  // Communication pairs first move the lhs; they take part in the GEMM afterwards when the
  // host planned a share of tiles for them, and leave otherwise.
  const bool is_comm = int(blockIdx.x) < p.num_comm_ctas;
  const int64_t tiles = p.order.count();  // tiles of 256 x 256
  bool do_compute = true;
  if constexpr (kGated) {
    if (is_comm) {
      if (!(p.flags & kFlagComputeOnly)) {
        if constexpr (kMode == kModeHeadGate) {
          GradPushPolicy policy(p, store_maps);
          run_chunk_pipeline(policy, p.wait, base, p.num_comm_ctas);
          __threadfence_system();
        } else if constexpr (kHeads) {
          GradPullPolicy policy(p, store_maps);
          run_chunk_pipeline(policy, p.wait, base, p.num_comm_ctas);
        } else {
          LhsPullPolicy policy(p, store_maps);
          run_chunk_pipeline(policy, p.wait, base, p.num_comm_ctas);
        }
      }
      if (p.join_tile >= tiles || (p.flags & kFlagCommOnly)) do_compute = false;  // both CTAs of the pair alike
      // The copy pipelines of BOTH CTAs of the pair are done before either re-uses its shared
      // memory for the GEMM: the pair's TMEM allocation and barriers involve both CTAs.
      __syncthreads();
      ptx::cluster_sync();
    } else if ((p.flags & kFlagCommOnly) && !kEmbedded) {
      do_compute = false;  // (with embedded copy warps every CTA still has its transfers to run)
    }
  }
  if (do_compute) {

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);   // the leader's expect_tx arrival; bytes from both CTAs
      ptx::mbar_init(empty_bar(s), 1);  // one commit arrival per phase, in each CTA
    }
    for (int s = 0; s < int(kAccumStages); ++s) {
      ptx::mbar_init(tmem_full_bar(s), 1);                      // commit arrival, in each CTA
      ptx::mbar_init(tmem_empty_bar(s), 2 * kEpilogueThreads);  // both CTAs' epilogues (leader's copy is used)
    }
    if constexpr (kEmbedded)
      for (int s = 0; s < kPullStages; ++s) ptx::mbar_init(bar_base + 8u * (2 * kStages + 2 * kAccumStages + s), 1);
    ptx::mbar_init(drain_bar, 1);
    ptx::fence_mbar_init();
    *reinterpret_cast<volatile uint32_t*>(smem + Layout::kTmemSlotOffset + 8) = 0u;  // gate progress
  }
  if (warp == 2) {
    ptx::tmem_alloc_pair(base + Layout::kTmemSlotOffset, Layout::kTmemColumns);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // barriers of both CTAs exist before anything arrives on them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Tile walk in units of pairs: compute pairs own the tiles before join_tile, every pair shares
  // the rest.
  TileWalk walk_template;
  walk_template.join_tile = p.join_tile < tiles ? p.join_tile : tiles;
  walk_template.tiles = tiles;
  walk_template.compute_ctas = (int32_t(gridDim.x) - p.num_comm_ctas) / 2;
  walk_template.all_ctas = int32_t(gridDim.x) / 2;
  walk_template.compute_id = is_comm ? -1 : (int32_t(blockIdx.x) - p.num_comm_ctas) / 2;
  walk_template.all_id = is_comm ? walk_template.compute_ctas + int32_t(blockIdx.x) / 2 : walk_template.compute_id;
  const int32_t k_blocks = (p.k + kBlockElems - 1) / kBlockElems;
  bool unwound = false;

  // Role-only launches (several ranks emulated on one GPU): with embedded copy warps every CTA
  // runs its copy warp unless kFlagComputeOnly and its GEMM roles unless kFlagCommOnly.
  const bool gemm_roles = !(kEmbedded && (p.flags & kFlagCommOnly));
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && gemm_roles) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      TileWalk walk = walk_template;
      uint32_t tile_seq = 0;
      for (int64_t t = walk.first(); ok && t >= 0; t = walk.next(), ++tile_seq) {
        int32_t mp, nt;
        p.order.decode(t, mp, nt);
        const int32_t row0 = mp * 2 * kBlockM + int32_t(rank) * kBlockM;          // this CTA's A rows
        const int32_t wrow0 = nt * kBlockN + int32_t(rank) * (kBlockN / 2);      // this CTA's half of B
        // K blocks of this tile whose groups the scout has posted complete.  The group a block needs
        // is worked out (a division) only when the walk reaches a block that is not open yet: this
        // thread's time between a stage falling free and its loads going out is what the GEMM
        // feels, so the common step carries no arithmetic beyond the compare.
        int32_t open_blocks = 0;
        for (int32_t ki = 0; ki < k_blocks; ++ki) {
          int32_t kb = ki;
          if constexpr (kGated) {
            // forward pull: K starts at this rank's own shard and wraps; this CTA's rows arrive
            // slice by slice.  Gradient pull: head by head, in order.
            if constexpr (!kHeads) {
              kb += p.lhs.k_block_start;
              if (kb >= k_blocks) kb -= k_blocks;
            }
            if (ki >= open_blocks) {
              const int32_t groups = kHeads ? p.grad.q_heads + 2 * p.grad.kv_heads : p.lhs.world * p.lhs.virt;
              const int32_t group_width = kHeads ? p.grad.head_dim : p.lhs.virt_width;
              int32_t last = (ki * kBlockElems + kBlockElems - 1) / group_width;
              if (last >= groups) last = groups - 1;
              uint32_t seen = 0;
              ok = progress_wait(gate_word, tile_seq * kGateSeqStep + uint32_t(last) + 1u, p.wait, kSiteLhsReady,
                                 uint32_t((mp * 2 + int32_t(rank)) * groups + last), &seen);
              ptx::fence_proxy_async_global();
              if (!ok) break;
              const int32_t upto = (seen / kGateSeqStep) > tile_seq ? groups - 1 : int32_t(seen % kGateSeqStep) - 1;
              open_blocks = upto >= groups - 1 ? k_blocks
                                               : int32_t((int64_t(upto + 1) * group_width) / kBlockElems);
            }
          }
          const uint32_t a_dst = base + stage * Layout::kStageBytes;
          const uint32_t leader_full = ptx::map_to_cta(full_bar(stage), 0);
          const int32_t k_elem = kb * kBlockElems;
          ok = mbar_wait(empty_bar(stage), phase ^ 1u, p.wait, kSiteSmemEmpty);
          if (!ok) break;
          if (leader) ptx::mbar_expect_tx(full_bar(stage), 2 * (Layout::kStageBytes + Layout::kSfStageBytes));
          if constexpr (!kAMn) {
            ptx::tma_load_2d_pair(a_dst, &tmap_a, leader_full, k_elem, row0);
          } else {
#pragma unroll
            for (int g = 0; g < kBlockM / 64; ++g)
              ptx::tma_load_2d_pair(a_dst + g * kMnGroupBytes, &tmap_a, leader_full, row0 + g * 64, kb * kBlockK);
          }
          if constexpr (!kBMn) {
            ptx::tma_load_2d_pair(a_dst + Layout::kABytes, &tmap_b, leader_full, k_elem, wrow0);
          } else {
#pragma unroll
            for (int g = 0; g < kBlockN / 2 / 64; ++g)
              ptx::tma_load_2d_pair(a_dst + Layout::kABytes + g * kMnGroupBytes, &tmap_b, leader_full, wrow0 + g * 64,
                                    kb * kBlockK);
          }
          if constexpr (kMx) {
            // scale atoms of this K block: this CTA's A rows, and both 128-row halves of the B tile
            // (rows past the operand read zeros: the tensor map clips)
            const uint32_t sf_dst = base + Layout::kSfOffset + stage * Layout::kSfStageBytes;
            const int32_t mt = mp * 2 + int32_t(rank);
            ptx::tma_load_2d_pair(sf_dst, &tmap_sfa, leader_full, 0, mt * p.k_atoms + kb);
            ptx::tma_load_2d_pair(sf_dst + 512u, &tmap_sfb, leader_full, 0, (nt * 2) * p.k_atoms + kb);
            ptx::tma_load_2d_pair(sf_dst + 1024u, &tmap_sfb, leader_full, 0, (nt * 2 + 1) * p.k_atoms + kb);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        (void)open_blocks;
      }
      (void)tile_seq;
      unwound = !ok;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer (leader CTA)
    if (lane == 0 && leader && gemm_roles) {
      constexpr uint32_t kIdesc = ptx::idesc_bf16_f32(2 * kBlockM, kBlockN, kAMn ? 1 : 0, kBMn ? 1 : 0);
      // descriptor step per UMMA (16 K values): 32 bytes inside the swizzle row of a K-major tile,
      // 16 rows of 128 bytes in an MN-major tile
      constexpr uint64_t kAStep = kAMn ? (kUmmaK * 128) >> 4 : (kUmmaK * 2) >> 4;
      constexpr uint64_t kBStep = kBMn ? (kUmmaK * 128) >> 4 : (kUmmaK * 2) >> 4;
      uint32_t stage = 0, phase = 0, accum = 0, accum_phase = 0;
      uint32_t sf_parity = 0;
      (void)sf_parity;
      (void)kIdesc;
      // high words of the operand and scale-atom descriptors (constant), low words of stage 0
      constexpr uint32_t kKMajorHigh = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kADescHigh = kKMajorHigh, kBDescHigh = kKMajorHigh;
      constexpr uint32_t kSfDescHigh = (128u >> 4) | (1u << 14);
      constexpr uint32_t kMnStride = (kMnGroupBytes >> 4) << 16, kKStride = 1u << 16;  // the low word's second field
      constexpr uint32_t kAStride = kAMn ? kMnStride : kKStride, kBStride = kBMn ? kMnStride : kKStride;
      const uint32_t a_low0 = (base & 0x3FFFFu) >> 4;  // start address field of stage 0's A tile
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
          // (no tcgen05 fence: the operands were written by the copy engine and their arrival is
          // acquired through the mbarrier; the fence after the accumulator wait above orders this
          // tile's UMMAs behind the epilogue's TMEM loads)
          // The descriptors of a stage differ from the previous stage's by a constant in their low
          // word: this thread's instruction stream per K block is what bounds the kernel, so they
          // are stepped, not rebuilt.
          const uint64_t a_desc = (uint64_t(kADescHigh) << 32) | (a_low + kAStride);
          const uint64_t b_desc = (uint64_t(kBDescHigh) << 32) | (a_low + ((Layout::kABytes >> 4) + kBStride));
          const uint32_t accumulate = kb != 0 ? 1u : 0u;
          if constexpr (kMx) {
            // scale atoms shared -> TMEM in both CTAs, then four K = 32 UMMAs; UMMA k reads byte k
            // of every 32-bit scale column; two sets of scale columns alternate
            const uint64_t sf_desc = (uint64_t(kSfDescHigh) << 32) | sf_low;
            const uint32_t sf_tmem = tmem_base + Layout::kTmemSfOffset + sf_parity;
            sf_parity ^= Layout::kSfColumns;  // alternates 0 and kSfColumns (12 = 0b1100)
            ptx::tmem_cp_32x128b_warpx4_pair(sf_tmem, sf_desc);
            ptx::tmem_cp_32x128b_warpx4_pair(sf_tmem + 4u, sf_desc + (512u >> 4));
            ptx::tmem_cp_32x128b_warpx4_pair(sf_tmem + 8u, sf_desc + (1024u >> 4));
            ptx::umma_mxf8_pair(d_tmem, a_desc, b_desc, ptx::idesc_mxf8_e4m3(2 * kBlockM, kBlockN, 0, 0), sf_tmem,
                                sf_tmem + 4u, accumulate);
#pragma unroll
            for (int k = 1; k < 4; ++k)
              ptx::umma_mxf8_pair_accumulate(d_tmem, a_desc + 2u * k, b_desc + 2u * k,
                                             ptx::idesc_mxf8_e4m3(2 * kBlockM, kBlockN, k, k), sf_tmem, sf_tmem + 4u);
            sf_low += Layout::kSfStageBytes >> 4;
          } else {
            ptx::umma_f16_pair(d_tmem, a_desc, b_desc, kIdesc, accumulate);
#pragma unroll
            for (int k = 1; k < kBlockK / kUmmaK; ++k)
              ptx::umma_f16_pair_accumulate(d_tmem, a_desc + kAStep * k, b_desc + kBStep * k, kIdesc);
          }
          ptx::umma_commit_pair(empty_bar(stage), 3);  // frees the stage in both CTAs
          a_low += Layout::kStageBytes >> 4;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
            a_low = a_low0;
            sf_low = sf_low0;
          }
        }
        if (!ok) break;
        ptx::umma_commit_pair(tmem_full_bar(accum), 3);
        if (++accum == kAccumStages) { accum = 0; accum_phase ^= 1u; }
      }
      if (!ok) {
        // Unwinding: UMMAs already issued must retire before TMEM is released.  They retire on the
        // leader's own drain barrier, so neither CTA's epilogue takes a partial tile for a finished one.
        ptx::umma_commit_pair(drain_bar, 1);
        mbar_wait(drain_bar, 0u, p.wait, kSiteDrain, false);
      }
      unwound = !ok;
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ embedded copy warp
    if constexpr (kEmbedded) {
      if (lane == 0 && !(p.flags & kFlagComputeOnly)) {
        using Policy = std::conditional_t<kMode == kModeHeadGate, GradPushPolicy,
                                          std::conditional_t<kMode == kModeGradPull, GradPullPolicy, LhsPullPolicy>>;
        Policy policy(p, store_maps);
        run_chunk_pipeline_thread(policy, p.wait, base + Layout::kCopyRingOffset,
                                  bar_base + 8u * (2 * kStages + 2 * kAccumStages), int32_t(blockIdx.x),
                                  int32_t(gridDim.x));
        if constexpr (kMode == kModeHeadGate) __threadfence_system();  // this thread's peer stores are performed
      }
      __syncwarp();
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------ gate scout (both CTAs)
    if constexpr (kGated) {
      const int32_t groups = kHeads ? p.grad.q_heads + 2 * p.grad.kv_heads : p.lhs.world * p.lhs.virt;
      const int32_t virt = kHeads ? 1 : p.lhs.virt;
      TileWalk walk = walk_template;
      uint32_t tile_seq = 0;
      bool ok = gemm_roles;
      for (int64_t t = walk.first(); ok && t >= 0; t = walk.next(), ++tile_seq) {
        int32_t mp, nt;
        p.order.decode(t, mp, nt);
        const int32_t mt = mp * 2 + int32_t(rank);
        if (mt * kBlockM >= p.m) {  // no rows in this half: nothing to wait for, the loads read zeros
          if (lane == 0) ptx::st_release_cta_shared(gate_word, (tile_seq + 1u) * kGateSeqStep);
          continue;
        }
        const uint32_t* flags = p.ready + int64_t(mt) * (groups / virt) * kReadyFlagStride;
        ok = scout_tile<kRemoteWriter>(p.wait, flags, groups, virt, kHeads ? 0 : p.lhs.gate_start, gate_word,
                               tile_seq * kGateSeqStep, lane, uint32_t(mt * groups));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int quarter = warp & 3;
    const int epi_tid = threadIdx.x - 128;
    const uint32_t leader_tmem_empty0 = ptx::map_to_cta(tmem_empty_bar(0), 0);
    const uint32_t leader_tmem_empty1 = ptx::map_to_cta(tmem_empty_bar(kAccumStages - 1), 0);
    (void)leader_tmem_empty1;
    uint32_t accum = 0, accum_phase = 0, staged_blocks = 0;
    bool ok = true;
    TileWalk walk = walk_template;
    for (int64_t t = gemm_roles ? walk.first() : -1; ok && t >= 0; t = walk.next()) {
      int32_t mp, nt;
      p.order.decode(t, mp, nt);
      const int32_t mt = mp * 2 + int32_t(rank);  // this CTA's 128-row tile
      ok = mbar_wait(tmem_full_bar(accum), accum_phase, p.wait, kSiteTmemFull);
      ok = ptx::named_bar_all(2, kEpilogueThreads, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + accum * kBlockN;
      const int32_t row_in_tile = quarter * 32 + lane;
      // One thread hands a staged 64-column block to the copy engine.
      auto issue_stores = [&](int c, uint32_t staging) {
        const int32_t col = nt * kBlockN + c;
        if (col < p.n && mt * kBlockM < p.m) {
          ptx::tma_store_2d(&store_maps.local, staging, col, mt * kBlockM);
          if constexpr (kDirect) {
            const QkvRoute& r = p.qkv;
            const int32_t q_width = r.q_heads * r.head_dim, kv_width = r.kv_heads * r.head_dim;
            const int32_t segment = col < q_width ? 0 : (col < q_width + kv_width ? 1 : 2);
            const int32_t within = col - (segment == 0 ? 0 : q_width + (segment == 2 ? kv_width : 0));
            const int32_t local_width = (segment == 0 ? q_width : kv_width) / r.world;
            int32_t owner, local_col;
            qkv_owner_column(r, segment, within, local_width, owner, local_col);
            // defer_v: one [rows, q_local + kv_local] tensor per destination (map 0), V not routed
            const int32_t map = r.defer_v ? 0 : segment;
            const int32_t dest_col = local_col + (r.defer_v && segment == 1 ? q_width / r.world : 0);
            if (!(r.defer_v && segment == 2))
              ptx::tma_store_2d(&store_maps.peer[owner][map], staging, dest_col,
                                int32_t(global_row(r.world, r.rank, r.seq_local, r.global_seq, r.causal != 0,
                                                   mt * kBlockM)));
          }
        }
        ptx::bulk_commit();
      };
      if constexpr (kAccumStages == 1) {
        // Single accumulator: the first 64 columns go straight to the staging block (its store is
        // in flight while the rest is read), the other 192 into packed BF16 registers; TMEM is handed
        // back before those are staged, so the next tile's UMMAs overlap the stores.  (Draining all
        // 256 columns into registers first spilled ~230 bytes per thread and measured 2 % slower.)
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
            pair = __floats2bfloat162_rn(p.alpha * __uint_as_float(acc1[2 * e]), p.alpha * __uint_as_float(acc1[2 * e + 1]));
            packed[(c - 64) / 2 + 16 + e] = *reinterpret_cast<const uint32_t*>(&pair);
          }
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive_cluster(leader_tmem_empty0);
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
          if (epi_tid == 0) ptx::bulk_wait_read<Layout::kStagingBuffers - 1>();
          ptx::named_bar_sync(1, kEpilogueThreads);
          uint32_t acc0[32], acc1[32];
          ptx::tmem_ld_32x32b_x32(taddr + c, acc0);
          ptx::tmem_ld_32x32b_x32(taddr + c + 32, acc1);
          ptx::tmem_wait_ld();
          if (c + 64 >= kBlockN) {
            // Accumulator read: hand the stage back to the leader's UMMA issuer.
            ptx::tc_fence_before();
            ptx::mbar_arrive_cluster(accum ? leader_tmem_empty1 : leader_tmem_empty0);
          }
          const uint32_t row_addr = staging + uint32_t(row_in_tile) * 128u;
          stage_accumulators(acc0, row_addr, 0, row_in_tile, p.alpha);
          stage_accumulators(acc1, row_addr, 4, row_in_tile, p.alpha);
          ptx::fence_proxy_async_shared();
          ptx::named_bar_sync(1, kEpilogueThreads);
          if (epi_tid == 0) issue_stores(c, staging);
        }
      }
      if (++accum == kAccumStages) { accum = 0; accum_phase ^= 1u; }
    }
    if (epi_tid == 0) ptx::bulk_wait<0>();  // every tensor store of this CTA is performed
    unwound = !ok;
  }

  if (unwound) {
    // A wait gave up: copies that were started may still be landing in either CTA's shared
    // memory.  Give them time before the pair is torn down (error path only).
    const uint64_t start = ptx::globaltimer();
    while (ptx::globaltimer() - start < 200000ull) __nanosleep(1000);
  }
  if constexpr (kDirect) __threadfence_system();  // peer stores performed
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // neither CTA leaves (or frees TMEM) while the other may still touch it
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, Layout::kTmemColumns);
  }
  }  // do_compute
  if constexpr (kDirect || kMode == kModeGradPull || kMode == kModeHeadGate) {
    // every rank's transfers are complete before any rank's inputs or outputs may change
    cooperative_groups::this_grid().sync();
    qkv_finalize(p);
  }
}

}  // namespace fuse_b200
