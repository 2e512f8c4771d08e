// Checker shim: exposes the reference's OWN host-compilable routing headers and
// CUTLASS host numerics through a C interface so that tests can pin the
// restatement in fuse_oracle.c against them.  It is compiled from the reference
// sources where they lie (REF_ROOT) into oracle/_ref/ and is never shipped, never
// committed as a binary, and never loaded by the product.  Test infrastructure.
#include <cstdint>

#include "fuse/layout/ulysses.h"                     // route maps
#include "benchmarks/sm103/fused_validation.cuh"      // QkvOracle, bf16 decode
#include "benchmarks/sm103/fused_inputs.cuh"          // OprojGather, uniform_value
#include <cutlass/bfloat16.h>
#include <cutlass/float8.h>

extern "C" {

int ref_map_qkv_gqa_feature(int world, int q_heads, int kv_heads, int head_dim, int feature,
                            int32_t out[5]) {
  fuse::UlyssesRoute route;
  route.world_size = world;
  route.q_heads = q_heads;
  route.kv_heads = kv_heads;
  route.head_dim = head_dim;
  const fuse::QkvGqaAddress a = fuse::map_qkv_gqa_feature(route, feature);
  out[0] = a.owner_rank;
  out[1] = a.local_feature;
  out[2] = a.segment;
  out[3] = a.logical_head;
  out[4] = a.head_offset;
  return a.valid() ? 1 : 0;
}

int ref_qkv_gqa_global_feature(int world, int q_heads, int kv_heads, int head_dim, int owner,
                               int local_feature) {
  fuse::UlyssesRoute route;
  route.world_size = world;
  route.q_heads = q_heads;
  route.kv_heads = kv_heads;
  route.head_dim = head_dim;
  return fuse::qkv_gqa_global_feature(route, owner, local_feature);
}

void ref_qkv_oracle_source(int world, int destination, uint64_t seq_local, uint64_t q_width,
                           uint64_t kv_width, uint64_t index, int32_t* rank, uint64_t* offset) {
  fused_validation::QkvOracle oracle{};
  oracle.seq_local = seq_local;
  oracle.q_width = q_width;
  oracle.kv_width = kv_width;
  oracle.world = world;
  oracle.destination = destination;
  const auto a = oracle.address(index);
  *rank = a.rank;
  *offset = a.offset;
}

void ref_oproj_gather_source(int world, int destination, uint64_t seq_local, uint64_t width,
                             int causal, uint64_t index, int32_t* rank, uint64_t* offset) {
  fused_inputs::OprojGather gather{};
  gather.seq_local = seq_local;
  gather.q_width = width;
  gather.world = world;
  gather.destination = destination;
  gather.causal = causal != 0;
  const auto a = gather.address(index);
  *rank = a.rank;
  *offset = a.offset;
}

float ref_uniform_value(uint32_t bits, float magnitude) {
  return fused_inputs::uniform_value(bits, magnitude);
}

float ref_bf16_to_f32(uint16_t value) { return fused_validation::bf16_to_float(value); }

uint16_t ref_f32_to_bf16(float value) { return cutlass::bfloat16_t(value).raw(); }

uint8_t ref_f32_to_e4m3(float value) { return cutlass::float_e4m3_t(value).raw(); }

float ref_e4m3_to_f32(uint8_t value) { return float(cutlass::float_e4m3_t::bitcast(value)); }

}  // extern "C"
