// Host-side plumbing shared by the entry points: device facts, TMA descriptor encoding
// through the driver entry point (no link-time dependency on libcuda), the per-device status
// record, launch bookkeeping and the cooperative launch helper.
#pragma once

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>

#include <cuda.h>
#include <cuda_runtime.h>

#include "sync.cuh"

namespace fuse_b200 {
namespace host {

struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  uint32_t* status = nullptr;  // device address of the status record on this device
};

// Defined in host.cu.
cudaError_t device_info(DeviceInfo* info);
uint32_t next_launch_id();
void count_launch(uint64_t kernels = 1);
uint64_t default_wait_budget_ns();

// 2-D row-major BF16/byte tensor [rows, cols] with a row pitch, boxed [box_rows, box_cols],
// 128-byte swizzle when box_cols * element_bytes == 128, else no swizzle.
cudaError_t encode_tensor_map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype,
                                 uint32_t element_bytes, uint64_t rows, uint64_t cols,
                                 uint64_t row_pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                                 CUtensorMapSwizzle swizzle);

inline WaitContext make_wait(const DeviceInfo& info, uint32_t epoch, uint64_t budget_ns) {
  WaitContext w;
  w.status = info.status;
  w.launch_id = next_launch_id();
  w.epoch = epoch;
  w.budget_ns = budget_ns ? budget_ns : default_wait_budget_ns();
  return w;
}

template <class Kernel, class... Args>
cudaError_t launch_kernel(Kernel kernel, int grid, int threads, uint32_t dynamic_smem,
                          bool cooperative, cudaStream_t stream, Args... args) {
  cudaError_t status =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dynamic_smem));
  if (status != cudaSuccess) return status;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(unsigned(grid), 1, 1);
  config.blockDim = dim3(unsigned(threads), 1, 1);
  config.dynamicSmemBytes = dynamic_smem;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeCooperative;
  attribute.val.cooperative = cooperative ? 1 : 0;
  config.attrs = &attribute;
  config.numAttrs = 1;
  status = cudaLaunchKernelEx(&config, kernel, args...);
  if (status == cudaSuccess) count_launch();
  return status;
}

inline bool aligned16(const void* p) {
  return p != nullptr && reinterpret_cast<uintptr_t>(p) % 16 == 0;
}
inline bool aligned4(const void* p) {
  return p != nullptr && reinterpret_cast<uintptr_t>(p) % 4 == 0;
}
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace host
}  // namespace fuse_b200
