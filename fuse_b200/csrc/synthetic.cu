// Device-side seeded input generators (Philox4x32-10), so that benchmark-size tensors are
// filled in HBM without a host round trip.  Element mapping and the word -> value map follow
// the reference harness (benchmarks/sm103/fused_inputs.cuh:22-29,117-141): 65536 generator
// threads, thread t is subsequence t, its r-th draw of four words fills elements
// 4*(r*65536+t)..+3.  The Philox rounds are written out here (no cuRAND dependency).
#include <cuda_bf16.h>

#include "fuse_b200.h"
#include "host.cuh"

namespace fuse_b200 {
namespace {

constexpr int kGeneratorThreads = 256;
constexpr int kGeneratorBlocks = 256;

__device__ __forceinline__ uint4 philox4x32_10(uint4 counter, uint2 key) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, counter.x), lo0 = 0xD2511F53u * counter.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, counter.z), lo1 = 0xCD9E8D57u * counter.z;
    counter = make_uint4(hi1 ^ counter.y ^ key.x, lo1, hi0 ^ counter.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return counter;
}

__device__ __forceinline__ float uniform_value(uint32_t bits, float magnitude) {
  const float unit = static_cast<float>(bits >> 8) / 16777216.0f;
  return __fmul_rn(__fadd_rn(unit, -0.5f), 2 * magnitude);
}

// mode 0: uniform in [-scale, scale); mode 1: N(0, scale^2) by Box-Muller on word pairs.
__global__ void generate_kernel(uint16_t* out, uint64_t count, uint64_t seed, float scale, int mode) {
  const uint32_t thread = blockIdx.x * blockDim.x + threadIdx.x;
  const uint2 key = make_uint2(uint32_t(seed), uint32_t(seed >> 32));
  uint32_t round = 0;
  for (uint64_t base = 4ull * thread; base < count;
       base += 4ull * kGeneratorBlocks * kGeneratorThreads, ++round) {
    const uint4 w = philox4x32_10(make_uint4(round, 0u, thread, 0u), key);
    float v[4];
    if (mode == 0) {
      v[0] = uniform_value(w.x, scale);
      v[1] = uniform_value(w.y, scale);
      v[2] = uniform_value(w.z, scale);
      v[3] = uniform_value(w.w, scale);
    } else {
      const float u1 = (float(w.x) + 1.0f) * 2.3283064365386963e-10f;
      const float u3 = (float(w.z) + 1.0f) * 2.3283064365386963e-10f;
      const float r0 = sqrtf(-2.0f * logf(fminf(u1, 1.0f))), r1 = sqrtf(-2.0f * logf(fminf(u3, 1.0f)));
      float s0, c0, s1, c1;
      sincospif(2.0f * float(w.y) * 2.3283064365386963e-10f, &s0, &c0);
      sincospif(2.0f * float(w.w) * 2.3283064365386963e-10f, &s1, &c1);
      v[0] = scale * r0 * c0;
      v[1] = scale * r0 * s0;
      v[2] = scale * r1 * c1;
      v[3] = scale * r1 * s1;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (base + i < count) out[base + i] = __bfloat16_as_ushort(__float2bfloat16_rn(v[i]));
  }
}

}  // namespace
}  // namespace fuse_b200

extern "C" int fuse_b200_generate_bf16(fuse_bf16* out, uint64_t count, uint64_t seed, float scale,
                                       int normal, fuse_stream stream) {
  if (out == nullptr || count == 0 || !(scale >= 0.0f)) return int(cudaErrorInvalidValue);
  fuse_b200::generate_kernel<<<fuse_b200::kGeneratorBlocks, fuse_b200::kGeneratorThreads, 0,
                               reinterpret_cast<cudaStream_t>(stream)>>>(out, count, seed, scale,
                                                                         normal ? 1 : 0);
  const cudaError_t status = cudaGetLastError();
  if (status == cudaSuccess) fuse_b200::host::count_launch();
  return int(status);
}
