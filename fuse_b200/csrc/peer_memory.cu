// Harness-side helpers for symmetric buffers between one-process-per-GPU ranks: plain
// cudaMalloc allocations exported and opened through CUDA IPC, as the reference harness does
// in its multi-process mode (benchmarks/sm103/fused_bf16.cu:1080-1139).  Not on the launch path.
#include <cstring>

#include <cuda_runtime.h>

#include "fuse_b200.h"

extern "C" {

int fuse_b200_symmetric_alloc(size_t bytes, void** ptr, unsigned char handle[64]) {
  if (ptr == nullptr || handle == nullptr || bytes == 0) return int(cudaErrorInvalidValue);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaError_t status = cudaMalloc(ptr, bytes);
  if (status != cudaSuccess) return int(status);
  status = cudaMemset(*ptr, 0, bytes);
  if (status != cudaSuccess) return int(status);
  cudaIpcMemHandle_t ipc;
  status = cudaIpcGetMemHandle(&ipc, *ptr);
  if (status != cudaSuccess) return int(status);
  std::memcpy(handle, &ipc, sizeof ipc);
  return int(cudaSuccess);
}

int fuse_b200_symmetric_open(const unsigned char handle[64], void** ptr) {
  if (ptr == nullptr || handle == nullptr) return int(cudaErrorInvalidValue);
  cudaIpcMemHandle_t ipc;
  std::memcpy(&ipc, handle, sizeof ipc);
  return int(cudaIpcOpenMemHandle(ptr, ipc, cudaIpcMemLazyEnablePeerAccess));
}

int fuse_b200_symmetric_close(void* ptr) { return int(cudaIpcCloseMemHandle(ptr)); }

int fuse_b200_symmetric_free(void* ptr) { return int(cudaFree(ptr)); }

}  // extern "C"
