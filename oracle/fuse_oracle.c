/*
 * CPU oracle for the fused Ulysses projection / MoE dispatch hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's algorithm (routing address maps, MXFP8 K32 quantisation, dense and
 * grouped GEMM arithmetic) used as the checker by tests/, by the smoke entry and
 * by the CPU-baseline leg of bench.py.  Nothing in the product path links, loads
 * or calls it; the product fails when its CUDA library is missing.
 *
 * Parity pin: every routing function below is compared, in tests/, against the
 * reference's own host-compilable headers (include/fuse/layout/ulysses.h,
 * benchmarks/sm103/fused_validation.cuh, benchmarks/sm103/fused_inputs.cuh)
 * compiled in place by oracle/Makefile into oracle/_ref/, and against golden
 * vectors generated from that build (tests/golden/).  The E4M3 conversion is
 * pinned against CUTLASS host numerics (cutlass::float_e4m3_t, CUTLASS 4.5.0 as
 * shipped in the image; the reference pins NVIDIA/cutlass @ 57e3cfb which is
 * not vendored).
 *
 * Every function cites the reference file:line it restates (paths are relative
 * to the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define FO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* scalar formats                                                            */
/* ------------------------------------------------------------------------- */

static inline float bits_to_f32(uint32_t bits) {
  float value;
  memcpy(&value, &bits, sizeof value);
  return value;
}
static inline uint32_t f32_to_bits(float value) {
  uint32_t bits;
  memcpy(&bits, &value, sizeof bits);
  return bits;
}

/* benchmarks/sm103/fused_validation.cuh:22-31 (bf16 decode is a 16-bit shift). */
FO_API float fo_bf16_to_f32(uint16_t value) { return bits_to_f32((uint32_t)value << 16); }

/* Round-to-nearest-even FP32 -> BF16, NaN kept quiet (what __float2bfloat16_rn
 * and cutlass::bfloat16_t(float) do; benchmarks/sm103/fused_inputs.cuh:133). */
FO_API uint16_t fo_f32_to_bf16(float value) {
  uint32_t bits = f32_to_bits(value);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040u);
  bits += 0x7fffu + ((bits >> 16) & 1u);
  return (uint16_t)(bits >> 16);
}

/* E4M3 (1-4-3, bias 7, max 448, 0x7f = NaN, no infinity).  Round to nearest
 * even, saturating to +-448: the behaviour of
 * cutlass::NumericArrayConverter<float_e4m3_t,float,32> used by
 * csrc/operators/sm103/detail/quantization.cuh:130-131. */
FO_API uint8_t fo_f32_to_e4m3(float value) {
  const uint32_t bits = f32_to_bits(value);
  const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
  const uint32_t magnitude = bits & 0x7fffffffu;
  if (magnitude > 0x7f800000u) return (uint8_t)(sign | 0x7fu);
  const float a = bits_to_f32(magnitude);
  if (a >= 448.0f) return (uint8_t)(sign | 0x7eu);
  int code;
  if (a < 0.015625f) { /* below 2^-6: subnormal grid of 2^-9 */
    code = (int)nearbyintf(a * 512.0f);
  } else {
    int exponent;
    const float fraction = frexpf(a, &exponent); /* a = fraction * 2^exponent, fraction in [0.5,1) */
    const int q = (int)nearbyintf(fraction * 16.0f); /* 8..16 */
    code = ((exponent - 1 + 7) << 3) + (q - 8);      /* q==16 carries into the exponent */
  }
  if (code > 0x7e) code = 0x7e;
  return (uint8_t)(sign | (uint8_t)code);
}

FO_API float fo_e4m3_to_f32(uint8_t value) {
  const int exponent = (value >> 3) & 0xf, mantissa = value & 7;
  float result;
  if (exponent == 0xf && mantissa == 7) result = NAN;
  else if (exponent == 0) result = ldexpf((float)mantissa, -9);
  else result = ldexpf(1.0f + (float)mantissa / 8.0f, exponent - 7);
  return (value & 0x80u) ? -result : result;
}

/* ------------------------------------------------------------------------- */
/* input generators                                                          */
/* ------------------------------------------------------------------------- */

/* benchmarks/sm103/fused_inputs.cuh:22-29. */
FO_API float fo_uniform_value(uint32_t bits, float magnitude) {
  const float unit = (float)(bits >> 8) / 16777216.0f;
  return (unit - 0.5f) * (2 * magnitude);
}

/* benchmarks/sm103/backward/validation.cuh:11-17 (splitmix-style hash -> BF16). */
FO_API uint16_t fo_backward_random_value(int64_t index, int seed) {
  uint64_t x = (uint64_t)index + ((uint64_t)(int64_t)seed << 32);
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
  x ^= x >> 31;
  return fo_f32_to_bf16(((int)(x & 65535) - 32768) / 131072.0f);
}

/* ------------------------------------------------------------------------- */
/* Ulysses route maps                                                        */
/* ------------------------------------------------------------------------- */

/* include/fuse/layout/ulysses.h:77-107.  out = {owner_rank, local_feature,
 * segment, logical_head, head_offset}; returns 0 when the reference returns an
 * invalid address. */
FO_API int fo_map_qkv_gqa_feature(int world, int q_heads, int kv_heads, int head_dim,
                                  int global_feature, int32_t out[5]) {
  for (int i = 0; i < 5; ++i) out[i] = -1;
  if (world <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || q_heads % world != 0 ||
      kv_heads % world != 0 || global_feature < 0 ||
      global_feature >= (q_heads + 2 * kv_heads) * head_dim)
    return 0;
  const int q_width = q_heads * head_dim, kv_width = kv_heads * head_dim;
  const int segment = global_feature < q_width ? 0 : (global_feature < q_width + kv_width ? 1 : 2);
  const int within = global_feature - (segment == 0 ? 0 : q_width + (segment == 2 ? kv_width : 0));
  const int head = within / head_dim, offset = within % head_dim;
  const int heads_per_rank = (segment == 0 ? q_heads : kv_heads) / world;
  const int owner = head / heads_per_rank, local_head = head % heads_per_rank;
  const int q_local = q_heads / world * head_dim, kv_local = kv_heads / world * head_dim;
  const int base = segment == 0 ? 0 : q_local + (segment == 2 ? kv_local : 0);
  out[0] = owner;
  out[1] = base + local_head * head_dim + offset;
  out[2] = segment;
  out[3] = head;
  out[4] = offset;
  return 1;
}

/* include/fuse/layout/ulysses.h:109-137 (inverse of the map above). */
FO_API int fo_qkv_gqa_global_feature(int world, int q_heads, int kv_heads, int head_dim,
                                     int owner_rank, int local_feature) {
  if (world <= 0 || owner_rank < 0 || owner_rank >= world || q_heads % world != 0 ||
      kv_heads % world != 0 || head_dim <= 0)
    return -1;
  const int q_local = q_heads / world * head_dim, kv_local = kv_heads / world * head_dim;
  if (local_feature < 0 || local_feature >= q_local + 2 * kv_local) return -1;
  const int segment = local_feature < q_local ? 0 : (local_feature < q_local + kv_local ? 1 : 2);
  const int within = local_feature - (segment == 0 ? 0 : q_local + (segment == 2 ? kv_local : 0));
  const int heads_per_rank = (segment == 0 ? q_heads : kv_heads) / world;
  const int head = owner_rank * heads_per_rank + within / head_dim;
  const int q_width = q_heads * head_dim, kv_width = kv_heads * head_dim;
  const int base = segment == 0 ? 0 : q_width + (segment == 2 ? kv_width : 0);
  return base + head * head_dim + within % head_dim;
}

/* Rank-local row -> row of the global [batch, global_seq] sequence axis.
 * Contiguous sharding: csrc/operators/sm103/detail/gemm_a2a.cuh:115-132;
 * causal two-chunk sharding: csrc/operators/sm103/detail/a2a_gemm.cuh:410-420. */
FO_API int64_t fo_global_row(int world, int rank, int seq_local, int causal, int64_t local_row) {
  const int64_t batch = local_row / seq_local, seq = local_row % seq_local;
  const int64_t global_seq = (int64_t)seq_local * world;
  if (causal) {
    const int64_t half = seq_local / 2;
    const int64_t chunk = seq < half ? rank : 2 * world - rank - 1;
    return batch * global_seq + chunk * half + seq % half;
  }
  return batch * global_seq + (int64_t)rank * seq_local + seq;
}

/* Forward QKV route, sender view: element (source row, packed feature) of rank
 * `rank`'s GEMM output -> (destination rank, element offset inside that rank's
 * planar Q|K|V buffer).  csrc/operators/sm103/detail/gemm_a2a.cuh:115-132
 * (row), :190-215 (segment bases), :404-415 (owner), :505-533 (column).  The
 * packed QKV route is rank-major even under causal CP
 * (benchmarks/sm103/fused_bf16.cu:2464-2466). */
FO_API int fo_qkv_forward_destination(int world, int rank, int batch, int seq_local, int q_heads,
                                      int kv_heads, int head_dim, int64_t source_row,
                                      int global_feature, int32_t* dest_rank,
                                      int64_t* dest_offset) {
  int32_t address[5];
  if (!fo_map_qkv_gqa_feature(world, q_heads, kv_heads, head_dim, global_feature, address))
    return 0;
  const int64_t rows = (int64_t)batch * seq_local * world;
  const int64_t q_local = q_heads / world * head_dim, kv_local = kv_heads / world * head_dim;
  const int segment = address[2];
  const int64_t width = segment == 0 ? q_local : kv_local;
  const int64_t base = segment == 0 ? 0 : rows * q_local + (segment == 2 ? rows * kv_local : 0);
  const int64_t column = address[1] - (segment == 0 ? 0 : q_local + (segment == 2 ? kv_local : 0));
  *dest_rank = address[0];
  *dest_offset = base + fo_global_row(world, rank, seq_local, 0, source_row) * width + column;
  return 1;
}

/* The same with UlyssesRoute::defer_v_a2a: V is not routed (returns 2), and Q and K of the
 * destination's heads share one row-major tensor [B*S_global, q_local + kv_local] there, Q
 * columns first.  csrc/operators/sm103/detail/gemm_a2a.cuh:199-215 (one descriptor of width
 * q_local + kv_local, offset 0), :408 (V tasks skipped), :505-533 (destination feature = local
 * feature: Q at head*d, K at q_local + head*d). */
FO_API int fo_qkv_forward_destination_defer_v(int world, int rank, int batch, int seq_local, int q_heads,
                                              int kv_heads, int head_dim, int64_t source_row,
                                              int global_feature, int32_t* dest_rank,
                                              int64_t* dest_offset) {
  int32_t address[5];
  if (!fo_map_qkv_gqa_feature(world, q_heads, kv_heads, head_dim, global_feature, address))
    return 0;
  (void)batch;
  const int64_t q_local = q_heads / world * head_dim, kv_local = kv_heads / world * head_dim;
  if (address[2] == 2) return 2;
  *dest_rank = address[0];
  *dest_offset = fo_global_row(world, rank, seq_local, 0, source_row) * (q_local + kv_local) + address[1];
  return 1;
}

/* The route with its two variants as flags: defer_v (above) and interleaved
 * (UlyssesRoute::qkv_peer_interleaved, csrc/operators/sm103/detail/gemm_a2a.cuh:404-415: inside Q and
 * inside K, physical head p of the prepacked projection belongs to owner p % world as its local head
 * p / world; V and the routed layout are unchanged).  Returns 1 (routed), 2 (not routed) or 0. */
FO_API int fo_qkv_forward_destination_variant(int world, int rank, int batch, int seq_local, int q_heads,
                                              int kv_heads, int head_dim, int defer_v, int interleaved,
                                              int64_t source_row, int global_feature, int32_t* dest_rank,
                                              int64_t* dest_offset) {
  int32_t address[5];
  if (!fo_map_qkv_gqa_feature(world, q_heads, kv_heads, head_dim, global_feature, address))
    return 0;
  const int64_t rows = (int64_t)batch * seq_local * world;
  const int64_t q_local = q_heads / world * head_dim, kv_local = kv_heads / world * head_dim;
  const int segment = address[2];
  int owner = address[0];
  int64_t column = address[1] - (segment == 0 ? 0 : q_local + (segment == 2 ? kv_local : 0));
  if (interleaved && segment < 2) {
    const int q_width = q_heads * head_dim, kv_width = kv_heads * head_dim;
    const int within = global_feature - (segment == 0 ? 0 : q_width);
    (void)kv_width;
    const int head = within / head_dim;
    owner = head % world;
    column = (int64_t)(head / world) * head_dim + within % head_dim;
  }
  if (defer_v && segment == 2) return 2;
  const int64_t row = fo_global_row(world, rank, seq_local, 0, source_row);
  *dest_rank = owner;
  if (defer_v) {
    *dest_offset = row * (q_local + kv_local) + (segment == 1 ? q_local : 0) + column;
  } else {
    const int64_t width = segment == 0 ? q_local : kv_local;
    const int64_t base = segment == 0 ? 0 : rows * q_local + (segment == 2 ? rows * kv_local : 0);
    *dest_offset = base + row * width + column;
  }
  return 1;
}

FO_API void fo_qkv_forward_route_variant(int world, int rank, int batch, int seq_local, int q_heads,
                                         int kv_heads, int head_dim, int defer_v, int interleaved,
                                         const uint16_t* local_output, int64_t ldd,
                                         uint16_t* const* peer_output) {
  const int64_t m = (int64_t)batch * seq_local;
  const int n = (q_heads + 2 * kv_heads) * head_dim;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < m; ++row)
    for (int feature = 0; feature < n; ++feature) {
      int32_t dest;
      int64_t offset;
      if (fo_qkv_forward_destination_variant(world, rank, batch, seq_local, q_heads, kv_heads, head_dim, defer_v,
                                             interleaved, row, feature, &dest, &offset) == 1)
        peer_output[dest][offset] = local_output[row * ldd + feature];
    }
}

/* Forward QKV route, receiver view: element `index` of destination rank's
 * planar Q|K|V buffer -> (source rank, element offset in that rank's [M,N] GEMM
 * output).  benchmarks/sm103/fused_validation.cuh:104-138 (batch == 1). */
FO_API void fo_qkv_oracle_source(int world, int destination, uint64_t seq_local, uint64_t q_width,
                                 uint64_t kv_width, uint64_t index, int32_t* source_rank,
                                 uint64_t* source_offset) {
  const uint64_t rows = seq_local * world;
  const uint64_t local_q = q_width / world, local_kv = kv_width / world;
  uint64_t local_width = local_q, feature_base = 0;
  if (index >= rows * local_q) {
    index -= rows * local_q;
    local_width = local_kv;
    feature_base = q_width;
    if (index >= rows * local_kv) {
      index -= rows * local_kv;
      feature_base += kv_width;
    }
  }
  const uint64_t row = index / local_width;
  *source_rank = (int32_t)(row / seq_local);
  *source_offset = (row % seq_local) * (q_width + 2 * kv_width) + feature_base +
                   destination * local_width + index % local_width;
}

/* Inverse (head -> sequence) route feeding the output projection: element
 * `index` of destination rank's gathered lhs [M, K] -> (source rank, element
 * offset in that rank's head-sharded attention output [B*S_global, K/world]).
 * benchmarks/sm103/fused_inputs.cuh:79-104 extended with batch and cyclic peer
 * order as in benchmarks/sm103/fused_mxfp8.cuh:30-41. */
FO_API void fo_oproj_gather_source(int world, int destination, int seq_local, int64_t width,
                                   int causal, int cyclic, uint64_t index, int32_t* source_rank,
                                   uint64_t* source_offset) {
  const uint64_t row = index / (uint64_t)width, feature = index % (uint64_t)width;
  const uint64_t shard_width = (uint64_t)width / world;
  const int shard = (int)(feature / shard_width);
  *source_rank = cyclic ? (destination + shard) % world : shard;
  *source_offset =
      (uint64_t)fo_global_row(world, destination, seq_local, causal, (int64_t)row) * shard_width +
      feature % shard_width;
}

/* QKV backward reverse route, receiver view: element (row, feature) of rank's
 * packed gradient staging [M, (q+2kv)*d] -> (owner rank, segment, element offset
 * in the owner's planar dQ / dK / dV [B*S_global, local_heads*d]).
 * benchmarks/sm103/backward/validation.cuh:27-46 and
 * benchmarks/sm103/backward/mxfp8_reference.cuh:38-57. */
FO_API void fo_qkv_backward_source(int world, int rank, int seq_local, int q_heads, int kv_heads,
                                   int head_dim, int causal, int64_t row, int feature,
                                   int32_t* owner, int32_t* segment, int64_t* offset) {
  const int head = feature / head_dim;
  const int seg = head < q_heads ? 0 : (head < q_heads + kv_heads ? 1 : 2);
  const int heads = seg == 0 ? q_heads : kv_heads;
  const int segment_head = head - (seg == 0 ? 0 : q_heads + (seg - 1) * kv_heads);
  const int heads_per_rank = heads / world;
  *owner = segment_head / heads_per_rank;
  *segment = seg;
  *offset = fo_global_row(world, rank, seq_local, causal, row) * heads_per_rank * head_dim +
            (int64_t)(segment_head % heads_per_rank) * head_dim + feature % head_dim;
}

/* Output-projection backward route (sequence -> head), receiver view: element
 * `index` of rank's head-sharded gradient [B*S_global, width/world] -> (source
 * rank, element offset in the source's dA [M, width]).
 * benchmarks/sm103/backward/validation.cuh:47-57. */
FO_API void fo_oproj_backward_source(int world, int rank, int batch, int seq_local, int64_t width,
                                     int causal, uint64_t index, int32_t* source_rank,
                                     uint64_t* source_offset) {
  (void)batch;
  const int64_t shard = width / world;
  const int64_t global_seq = (int64_t)seq_local * world;
  const int64_t row = (int64_t)(index / (uint64_t)shard), column = (int64_t)(index % (uint64_t)shard);
  const int64_t b = row / global_seq, seq = row % global_seq;
  int64_t source = seq / seq_local, local_row = seq % seq_local;
  if (causal) {
    const int64_t half = seq_local / 2, chunk = seq / half;
    source = chunk < world ? chunk : 2 * world - chunk - 1;
    local_row = (chunk < world ? 0 : half) + seq % half;
  }
  *source_rank = (int32_t)source;
  *source_offset = (uint64_t)((b * seq_local + local_row) * width + rank * shard + column);
}

/* benchmarks/sm103/fused_bf16.cu:196-206: largest power-of-two swizzle allowed
 * by the cap and by the smaller tile-grid dimension. */
FO_API int fo_swizzle_size(int max_swizzle, int m_tiles, int n_tiles) {
  const int smaller = m_tiles < n_tiles ? m_tiles : n_tiles;
  if (max_swizzle >= 8 && smaller >= 6) return 8;
  if (max_swizzle >= 4 && smaller >= 3) return 4;
  if (max_swizzle >= 2 && smaller >= 2) return 2;
  return 1;
}

/* ------------------------------------------------------------------------- */
/* MXFP8 (E4M3 data, UE8M0 scale per 32 K values)                            */
/* ------------------------------------------------------------------------- */

/* csrc/operators/sm103/detail/quantization.cuh:91-105. */
FO_API int fo_mxfp8_scale_exponent(float amax) {
  if (!(amax > 0)) return 0;
  const int exponent = (int)((f32_to_bits(amax) + 0x001fffffu) >> 23) - 127 - 8;
  return exponent < -127 ? -127 : exponent > 127 ? 127 : exponent;
}

/* csrc/operators/sm103/detail/quantization.cuh:107-118. */
FO_API float fo_mxfp8_scaled_value(float value, int exponent) {
  const uint32_t bits = exponent == 127 ? 0x00400000u : (uint32_t)(127 - exponent) << 23;
  return value * bits_to_f32(bits);
}

/* The independent formulation the reference's validators use
 * (benchmarks/sm103/fused_mxfp8.cuh:64-71, backward/mxfp8_smoke.cu:89-110):
 * frexp + boundary comparison instead of integer exponent arithmetic. */
FO_API int fo_mxfp8_scale_exponent_frexp(float amax) {
  int exponent = 0;
  if (amax > 0) {
    frexpf(amax, &exponent);
    exponent -= 9;
    if (amax > ldexpf(448.0f, exponent)) ++exponent;
  }
  return exponent < -127 ? -127 : exponent > 127 ? 127 : exponent;
}

/* Byte offset of the scale of (row, k) in the native K32 scale storage of a
 * [rows, width] operand (512-byte atoms of 128 rows x 4 K-blocks, K atoms before
 * row atoms).  benchmarks/sm103/fused_mxfp8.cuh:13-16. */
FO_API int64_t fo_mxfp8_scale_offset(int64_t row, int64_t k, int64_t width) {
  return ((row / 128) * ((width + 127) / 128) + k / 128) * 512 + (row % 32) * 16 +
         ((row % 128) / 32) * 4 + (k % 128) / 32;
}

FO_API int64_t fo_mxfp8_scale_bytes(int64_t rows, int64_t width) {
  return ((rows + 127) / 128) * ((width + 127) / 128) * 512;
}

/* Row-major BF16 [rows, k] (row stride in elements) -> E4M3 [rows, k] + native
 * scales.  csrc/operators/sm103/detail/quantization.cuh:120-141. */
FO_API void fo_mxfp8_quantize(const uint16_t* source, int64_t rows, int64_t k, int64_t row_stride,
                              uint8_t* data, uint8_t* scales) {
  /* rows past the end of the last 128-row atom quantise zeros: scale 2^0 (quantization.cuh:128) */
  for (int64_t row = rows; row < ((rows + 127) / 128) * 128; ++row)
    for (int64_t group = 0; group < k / 32; ++group) scales[fo_mxfp8_scale_offset(row, group * 32, k)] = 127;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < rows; ++row) {
    for (int64_t group = 0; group < k / 32; ++group) {
      const uint16_t* in = source + row * row_stride + group * 32;
      float amax = 0;
      for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(fo_bf16_to_f32(in[i])));
      const int exponent = fo_mxfp8_scale_exponent(amax);
      for (int i = 0; i < 32; ++i)
        data[row * k + group * 32 + i] =
            fo_f32_to_e4m3(fo_mxfp8_scaled_value(fo_bf16_to_f32(in[i]), exponent));
      scales[fo_mxfp8_scale_offset(row, group * 32, k)] = (uint8_t)(exponent + 127);
    }
  }
}

/* BF16 [rows, cols] (row stride) -> E4M3 [cols, rows] quantised along the
 * source ROW axis (the new K axis) + native scales of the [cols, rows] operand.
 * csrc/operators/sm103/detail/quantization.cuh:350-450: every backward operand
 * orientation is re-quantised from its BF16 master along its own K axis. */
FO_API void fo_mxfp8_quantize_transposed(const uint16_t* source, int64_t rows, int64_t cols,
                                         int64_t row_stride, uint8_t* data, uint8_t* scales) {
  for (int64_t col = cols; col < ((cols + 127) / 128) * 128; ++col)
    for (int64_t group = 0; group < rows / 32; ++group) scales[fo_mxfp8_scale_offset(col, group * 32, rows)] = 127;
#pragma omp parallel for schedule(static)
  for (int64_t col = 0; col < cols; ++col) {
    for (int64_t group = 0; group < rows / 32; ++group) {
      float amax = 0;
      for (int i = 0; i < 32; ++i)
        amax = fmaxf(amax, fabsf(fo_bf16_to_f32(source[(group * 32 + i) * row_stride + col])));
      const int exponent = fo_mxfp8_scale_exponent(amax);
      for (int i = 0; i < 32; ++i)
        data[col * rows + group * 32 + i] = fo_f32_to_e4m3(fo_mxfp8_scaled_value(
            fo_bf16_to_f32(source[(group * 32 + i) * row_stride + col]), exponent));
      scales[fo_mxfp8_scale_offset(col, group * 32, rows)] = (uint8_t)(exponent + 127);
    }
  }
}

/* E4M3 + native scales -> FP32 represented values [rows, k]. */
FO_API void fo_mxfp8_dequantize(const uint8_t* data, const uint8_t* scales, int64_t rows,
                                int64_t k, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < rows; ++row)
    for (int64_t col = 0; col < k; ++col) {
      const int exponent = (int)scales[fo_mxfp8_scale_offset(row, col, k)] - 127;
      out[row * k + col] = ldexpf(fo_e4m3_to_f32(data[row * k + col]), exponent);
    }
}

/* Quantise -> dequantise in one step with the validators' independent exponent
 * rule: the "represented operand" of benchmarks/sm103/fused_mxfp8.cuh:54-73. */
FO_API void fo_mxfp8_represented(const uint16_t* source, int64_t count, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t group = 0; group < count / 32; ++group) {
    float amax = 0;
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(fo_bf16_to_f32(source[group * 32 + i])));
    const int exponent = fo_mxfp8_scale_exponent_frexp(amax);
    for (int i = 0; i < 32; ++i)
      out[group * 32 + i] = ldexpf(
          fo_e4m3_to_f32(fo_f32_to_e4m3(ldexpf(fo_bf16_to_f32(source[group * 32 + i]), -exponent))),
          exponent);
  }
}

/* ------------------------------------------------------------------------- */
/* GEMM arithmetic (FP32 accumulate, BF16 out)                               */
/* ------------------------------------------------------------------------- */

static float dot_f32(const float* a, const float* b, int64_t k) {
  float lanes[16] = {0};
  int64_t i = 0;
  for (; i + 16 <= k; i += 16)
    for (int j = 0; j < 16; ++j) lanes[j] += a[i + j] * b[i + j];
  float sum = 0;
  for (int j = 0; j < 16; ++j) sum += lanes[j];
  for (; i < k; ++i) sum += a[i] * b[i];
  return sum;
}

/* D[m,n] = alpha * sum_k A[m,k] * B[n,k] (+ beta * D), FP32 operands, BF16 out.
 * The arithmetic contract of csrc/operators/sm103/detail/gemm.cuh:112-188
 * (BF16 in, FP32 accumulate, BF16 out); the reference checks it against
 * cublasGemmEx with FP32 compute (benchmarks/sm103/fused_bf16.cu:2099-2106). */
FO_API void fo_gemm_f32_nt(const float* a, const float* b, uint16_t* d, int64_t m, int64_t n,
                           int64_t k, int64_t ldd, float alpha, float beta) {
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t row = 0; row < m; ++row)
    for (int64_t col = 0; col < n; ++col) {
      float value = alpha * dot_f32(a + row * k, b + col * k, k);
      if (beta != 0) value += beta * fo_bf16_to_f32(d[row * ldd + col]);
      d[row * ldd + col] = fo_f32_to_bf16(value);
    }
}

static float* widen(const uint16_t* source, int64_t rows, int64_t cols, int64_t stride,
                    int transpose) {
  float* out = (float*)malloc(sizeof(float) * (size_t)rows * (size_t)cols);
  if (!out) return NULL;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) {
      const float value = fo_bf16_to_f32(source[r * stride + c]);
      if (transpose) out[c * rows + r] = value;
      else out[r * cols + c] = value;
    }
  return out;
}

/* BF16 GEMM in the three operand orientations of the hot path:
 *   mode 0 (NT, forward):    A[m,k] row-major,  B[n,k] row-major
 *   mode 1 (NN, data grad):  A[m,k] row-major,  B[k,n] row-major
 *       (csrc/operators/sm103/api/backward.cuh:12-119: W is read as stored)
 *   mode 2 (TN, weight grad):A stored [k,m] row-major, B stored [k,n] row-major,
 *       D[m,n] = alpha * A^T B + beta * D   (api/backward.cuh:252-268)
 * Leading dimensions are in elements.  Returns 0 on success. */
FO_API int fo_gemm_bf16(int mode, const uint16_t* a, int64_t lda, const uint16_t* b, int64_t ldb,
                        uint16_t* d, int64_t ldd, int64_t m, int64_t n, int64_t k, float alpha,
                        float beta) {
  float* fa = mode == 2 ? widen(a, k, m, lda, 1) : widen(a, m, k, lda, 0);
  float* fb = mode == 0 ? widen(b, n, k, ldb, 0) : widen(b, k, n, ldb, 1);
  if (!fa || !fb) {
    free(fa);
    free(fb);
    return 1;
  }
  fo_gemm_f32_nt(fa, fb, d, m, n, k, ldd, alpha, beta);
  free(fa);
  free(fb);
  return 0;
}

/* MXFP8 GEMM on represented operands: D = bf16(alpha * deq(A) deq(B)^T).
 * benchmarks/sm103/backward/mxfp8_smoke.cu:87-134 (represented + multiply). */
FO_API int fo_gemm_mxfp8_nt(const uint8_t* a, const uint8_t* a_scales, const uint8_t* b,
                            const uint8_t* b_scales, uint16_t* d, int64_t ldd, int64_t m,
                            int64_t n, int64_t k, float alpha) {
  float* fa = (float*)malloc(sizeof(float) * (size_t)m * (size_t)k);
  float* fb = (float*)malloc(sizeof(float) * (size_t)n * (size_t)k);
  if (!fa || !fb) {
    free(fa);
    free(fb);
    return 1;
  }
  fo_mxfp8_dequantize(a, a_scales, m, k, fa);
  fo_mxfp8_dequantize(b, b_scales, n, k, fb);
  fo_gemm_f32_nt(fa, fb, d, m, n, k, ldd, alpha, 0.0f);
  free(fa);
  free(fb);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Multi-rank simulators (all ranks in one address space)                    */
/* ------------------------------------------------------------------------- */

/* Scatter one rank's GEMM output [m, n] into every destination's planar Q|K|V
 * buffer, element by element through fo_qkv_forward_destination. */
FO_API void fo_qkv_forward_route(int world, int rank, int batch, int seq_local, int q_heads,
                                 int kv_heads, int head_dim, const uint16_t* local_output,
                                 int64_t ldd, uint16_t* const* peer_output) {
  const int64_t m = (int64_t)batch * seq_local;
  const int n = (q_heads + 2 * kv_heads) * head_dim;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < m; ++row)
    for (int feature = 0; feature < n; ++feature) {
      int32_t dest;
      int64_t offset;
      fo_qkv_forward_destination(world, rank, batch, seq_local, q_heads, kv_heads, head_dim, row,
                                 feature, &dest, &offset);
      peer_output[dest][offset] = local_output[row * ldd + feature];
    }
}

/* The deferred-V variant: Q and K only, into every destination's [rows, q_local + kv_local] tensor. */
FO_API void fo_qkv_forward_route_defer_v(int world, int rank, int batch, int seq_local, int q_heads,
                                         int kv_heads, int head_dim, const uint16_t* local_output,
                                         int64_t ldd, uint16_t* const* peer_output) {
  const int64_t m = (int64_t)batch * seq_local;
  const int n = (q_heads + 2 * kv_heads) * head_dim;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < m; ++row)
    for (int feature = 0; feature < n; ++feature) {
      int32_t dest;
      int64_t offset;
      if (fo_qkv_forward_destination_defer_v(world, rank, batch, seq_local, q_heads, kv_heads, head_dim, row,
                                             feature, &dest, &offset) == 1)
        peer_output[dest][offset] = local_output[row * ldd + feature];
    }
}

/* Gather one rank's output-projection lhs [m, width] from every source's
 * head-sharded tensor, element by element through fo_oproj_gather_source. */
FO_API void fo_oproj_forward_gather(int world, int rank, int batch, int seq_local, int64_t width,
                                    int causal, int cyclic, const uint16_t* const* peer_input,
                                    uint16_t* staging) {
  const int64_t m = (int64_t)batch * seq_local;
#pragma omp parallel for schedule(static)
  for (int64_t index = 0; index < m * width; ++index) {
    int32_t source;
    uint64_t offset;
    fo_oproj_gather_source(world, rank, seq_local, width, causal, cyclic, (uint64_t)index, &source,
                           &offset);
    staging[index] = peer_input[source][offset];
  }
}

/* Gather one rank's packed QKV gradient [m, (q+2kv)*d] from the owners' planar
 * dQ, dK, dV (planes[owner*3 + segment]). */
FO_API void fo_qkv_backward_gather(int world, int rank, int batch, int seq_local, int q_heads,
                                   int kv_heads, int head_dim, int causal,
                                   const uint16_t* const* planes, uint16_t* staging) {
  const int64_t m = (int64_t)batch * seq_local;
  const int width = (q_heads + 2 * kv_heads) * head_dim;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < m; ++row)
    for (int feature = 0; feature < width; ++feature) {
      int32_t owner, segment;
      int64_t offset;
      fo_qkv_backward_source(world, rank, seq_local, q_heads, kv_heads, head_dim, causal, row,
                             feature, &owner, &segment, &offset);
      staging[row * width + feature] = planes[owner * 3 + segment][offset];
    }
}

/* ------------------------------------------------------------------------- */
/* MoE dispatch                                                              */
/* ------------------------------------------------------------------------- */

/* Top-k distinct experts per token by descending score, ties to the lower
 * expert id.  The operator itself takes routing metadata from the caller
 * (include/fuse/operators/primitives/grouped_gemm.h:55-57); this builds it for
 * synthetic workloads. */
FO_API void fo_moe_topk(const float* scores, int64_t tokens, int experts, int topk,
                        int32_t* chosen) {
#pragma omp parallel for schedule(static)
  for (int64_t token = 0; token < tokens; ++token) {
    const float* row = scores + token * experts;
    for (int slot = 0; slot < topk; ++slot) {
      int best = -1;
      for (int e = 0; e < experts; ++e) {
        int taken = 0;
        for (int s = 0; s < slot; ++s) taken |= chosen[token * topk + s] == e;
        if (taken) continue;
        if (best < 0 || row[e] > row[best]) best = e;
      }
      chosen[token * topk + slot] = best;
    }
  }
}

/* Expert-major row lists for one destination rank: for each local expert, rows
 * ordered by (source rank, token, slot); source[row] = {rank, token, slot}
 * (include/fuse/operators/primitives/grouped_gemm.h:10-20;
 * benchmarks/sm103/grouped_validation.cuh:59-79).  chosen[r] is rank r's
 * [tokens, topk] expert table.  row_offsets has experts_local + 1 entries.
 * Returns the total number of rows (sources may be NULL to count only). */
FO_API int64_t fo_moe_build_rows(int world, int dest_rank, int experts_local, int64_t tokens,
                                 int topk, const int32_t* const* chosen, int32_t* row_offsets,
                                 int32_t* sources) {
  int64_t total = 0;
  for (int local = 0; local < experts_local; ++local) {
    const int expert = dest_rank * experts_local + local;
    row_offsets[local] = (int32_t)total;
    for (int rank = 0; rank < world; ++rank)
      for (int64_t token = 0; token < tokens; ++token)
        for (int slot = 0; slot < topk; ++slot)
          if (chosen[rank][token * topk + slot] == expert) {
            if (sources) {
              sources[total * 3 + 0] = rank;
              sources[total * 3 + 1] = (int32_t)token;
              sources[total * 3 + 2] = slot;
            }
            ++total;
          }
  }
  row_offsets[experts_local] = (int32_t)total;
  return total;
}

/* Gather + per-expert GEMM: for local expert e, rows r in [row_offsets[e],
 * row_offsets[e+1]): D_e[r, :] = A_e[r, :] W_e^T with A_e[r, :] =
 * peer_input[source.rank][source.token, :].  lhs / output are per-expert slabs
 * of `capacity` rows (benchmarks/sm103/grouped_validation.cuh:59-144). */
FO_API int fo_moe_dispatch_fc1(int experts_local, const int32_t* row_offsets,
                               const int32_t* sources, const uint16_t* const* peer_input,
                               const uint16_t* weights, int64_t n, int64_t k, int64_t capacity,
                               uint16_t* lhs, uint16_t* output) {
  for (int e = 0; e < experts_local; ++e) {
    const int64_t begin = row_offsets[e], rows = row_offsets[e + 1] - begin;
    if (rows == 0) continue;
    uint16_t* slab = lhs + (int64_t)e * capacity * k;
    for (int64_t r = 0; r < rows; ++r) {
      const int32_t* s = sources + (begin + r) * 3;
      memcpy(slab + r * k, peer_input[s[0]] + (int64_t)s[1] * k, sizeof(uint16_t) * (size_t)k);
    }
    if (fo_gemm_bf16(0, slab, k, weights + (int64_t)e * n * k, k,
                     output + (int64_t)e * capacity * n, n, rows, n, k, 1.0f, 0.0f))
      return 1;
  }
  return 0;
}

/* Per-expert GEMM + scatter (the combine direction): for local expert e, rows r in
 * [row_offsets[e], row_offsets[e+1]): D_e[r, :] = A_e[r, :] W_e^T goes to the expert's output
 * slab and to peer_output[source.rank][(source.token * topk + source.slot), :] -- one row per
 * routed branch, no weighting or top-k reduction
 * (csrc/operators/sm103/detail/grouped/gemm_a2a.cuh:15-93; receiver check:
 * benchmarks/sm103/grouped_validation.cuh:143-157). */
FO_API int fo_moe_fc2_combine(int experts_local, const int32_t* row_offsets, const int32_t* sources,
                              const uint16_t* lhs, const uint16_t* weights, int64_t n, int64_t k,
                              int64_t capacity, int topk, uint16_t* output,
                              uint16_t* const* peer_output) {
  for (int e = 0; e < experts_local; ++e) {
    const int64_t begin = row_offsets[e], rows = row_offsets[e + 1] - begin;
    if (rows == 0) continue;
    uint16_t* slab = output + (int64_t)e * capacity * n;
    if (fo_gemm_bf16(0, lhs + (int64_t)e * capacity * k, k, weights + (int64_t)e * n * k, k, slab, n,
                     rows, n, k, 1.0f, 0.0f))
      return 1;
    for (int64_t r = 0; r < rows; ++r) {
      const int32_t* s = sources + (begin + r) * 3;
      memcpy(peer_output[s[0]] + ((int64_t)s[1] * topk + s[2]) * n, slab + r * n,
             sizeof(uint16_t) * (size_t)n);
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Batch forms of the receiver-view maps (full-size validation samples many   */
/* elements at once; each entry is exactly the scalar map above).             */
/* ------------------------------------------------------------------------- */

FO_API void fo_qkv_oracle_source_batch(int world, int destination, uint64_t seq_local,
                                       uint64_t q_width, uint64_t kv_width, const uint64_t* index,
                                       int64_t count, int32_t* source_rank,
                                       uint64_t* source_offset) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i)
    fo_qkv_oracle_source(world, destination, seq_local, q_width, kv_width, index[i],
                         &source_rank[i], &source_offset[i]);
}

FO_API void fo_oproj_gather_source_batch(int world, int destination, int seq_local, int64_t width,
                                         int causal, int cyclic, const uint64_t* index,
                                         int64_t count, int32_t* source_rank,
                                         uint64_t* source_offset) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i)
    fo_oproj_gather_source(world, destination, seq_local, width, causal, cyclic, index[i],
                           &source_rank[i], &source_offset[i]);
}

FO_API void fo_qkv_backward_source_batch(int world, int rank, int seq_local, int q_heads,
                                         int kv_heads, int head_dim, int causal,
                                         const int64_t* row, const int32_t* feature, int64_t count,
                                         int32_t* owner, int32_t* segment, int64_t* offset) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i)
    fo_qkv_backward_source(world, rank, seq_local, q_heads, kv_heads, head_dim, causal, row[i],
                           feature[i], &owner[i], &segment[i], &offset[i]);
}

FO_API void fo_oproj_backward_source_batch(int world, int rank, int batch, int seq_local,
                                           int64_t width, int causal, const uint64_t* index,
                                           int64_t count, int32_t* source_rank,
                                           uint64_t* source_offset) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i)
    fo_oproj_backward_source(world, rank, batch, seq_local, width, causal, index[i],
                             &source_rank[i], &source_offset[i]);
}

FO_API void fo_global_row_batch(int world, int rank, int seq_local, int causal,
                                const int64_t* local_row, int64_t count, int64_t* global_row) {
  for (int64_t i = 0; i < count; ++i)
    global_row[i] = fo_global_row(world, rank, seq_local, causal, local_row[i]);
}

FO_API void fo_mxfp8_scale_offset_batch(const int64_t* row, const int64_t* k, int64_t width,
                                        int64_t count, int64_t* offset) {
  for (int64_t i = 0; i < count; ++i) offset[i] = fo_mxfp8_scale_offset(row[i], k[i], width);
}

/* Threads the OpenMP loops of this file use from now on (the benchmark's checker shares the
 * host cores with the other ranks' processes). */
FO_API void fo_set_num_threads(int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
}

FO_API int fo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
