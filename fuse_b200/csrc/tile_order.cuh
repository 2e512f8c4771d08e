// Static tile order shared by the compute CTAs (which produce or consume tiles in this order)
// and the communication CTAs (which deliver data in the same order), so that the first data a
// GEMM wave needs is the first data moved.
//
// The linear index walks bands of `swizzle` tiles along the minor axis: with the M raster a
// band is `swizzle` N-tiles wide and the index runs down M inside it, so one wave of CTAs
// touches few distinct weight panels; the N raster is the transpose.  Same knobs as the
// reference scheduler (csrc/operators/sm103/detail/persistent_gemm.cuh:27-182: raster
// AlongM/AlongN, power-of-two swizzle), independent decode.
#pragma once

#include <cstdint>

namespace fuse_b200 {

struct TileOrder {
  int32_t m_tiles = 0;
  int32_t n_tiles = 0;
  int32_t swizzle = 1;    // 1, 2, 4 or 8
  int32_t along_n = 0;    // 0: linear index runs along M first; 1: along N first
  // Every rank of a context-parallel group walks the same order; shifting the N coordinate by a
  // rank-dependent number of tiles makes the ranks work on different column ranges -- and thus
  // push to different owners -- at any moment, instead of all writing to the same peer.
  int32_t n_shift = 0;

  __host__ __device__ int64_t count() const { return int64_t(m_tiles) * n_tiles; }

  __host__ __device__ void decode(int64_t linear, int32_t& m, int32_t& n) const {
    const int32_t major = along_n ? n_tiles : m_tiles;  // axis the index runs along
    const int32_t minor = along_n ? m_tiles : n_tiles;  // axis cut into bands
    const int64_t band_tiles = int64_t(swizzle) * major;
    const int32_t band = int32_t(linear / band_tiles);
    const int32_t within = int32_t(linear - band * band_tiles);
    const int32_t band_begin = band * swizzle;
    const int32_t width = minor - band_begin < swizzle ? minor - band_begin : swizzle;
    const int32_t a = within / width;               // position along the major axis
    const int32_t b = band_begin + within % width;  // position along the minor axis
    m = along_n ? b : a;
    n = along_n ? a : b;
    if (n_shift != 0) {
      n += n_shift;
      if (n >= n_tiles) n -= n_tiles;
    }
  }

  __host__ __device__ int64_t linear(int32_t m, int32_t n) const {
    const int32_t major = along_n ? n_tiles : m_tiles;
    const int32_t minor = along_n ? m_tiles : n_tiles;
    if (n_shift != 0) {
      n -= n_shift;
      if (n < 0) n += n_tiles;
    }
    const int32_t a = along_n ? n : m, b = along_n ? m : n;
    const int32_t band = b / swizzle, band_begin = band * swizzle;
    const int32_t width = minor - band_begin < swizzle ? minor - band_begin : swizzle;
    return int64_t(band) * swizzle * major + int64_t(a) * width + (b - band_begin);
  }
};

// Largest power-of-two swizzle allowed by the caller's cap and by the smaller grid dimension
// (selection rule of benchmarks/sm103/fused_bf16.cu:196-206).
__host__ __device__ inline int32_t select_swizzle(int32_t max_swizzle, int32_t m_tiles,
                                                  int32_t n_tiles) {
  const int32_t smaller = m_tiles < n_tiles ? m_tiles : n_tiles;
  if (max_swizzle >= 8 && smaller >= 6) return 8;
  if (max_swizzle >= 4 && smaller >= 3) return 4;
  if (max_swizzle >= 2 && smaller >= 2) return 2;
  return 1;
}

}  // namespace fuse_b200
