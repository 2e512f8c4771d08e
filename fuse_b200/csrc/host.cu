// Process-wide host state: device facts, status record, launch bookkeeping, TMA encoding.
#include "host.cuh"

#include <mutex>

#include "fuse_b200.h"
#include "tile_order.cuh"

namespace fuse_b200 {

// One status record per device that loads this library (kStatusWords words, zero at load).
__device__ uint32_t g_status_record[kStatusWords];

namespace host {
namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
DeviceInfo g_devices[kMaxDevices];
std::atomic<uint32_t> g_launch_id{0};
std::atomic<uint64_t> g_launch_count{0};

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_entry() {
  static EncodeTiled entry = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &result) !=
            cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeTiled>(fn);
  }();
  return entry;
}

}  // namespace

cudaError_t device_info(DeviceInfo* info) {
  int device = -1;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess) return status;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  // The tensor maps are encoded through the driver API, which needs the device's primary context
  // current on THIS host thread; a thread that has only ever called cudaSetDevice (a framework's
  // backward thread, say) does not have it yet.  cudaFree(nullptr) binds it; once per thread and device.
  thread_local int bound_device = -1;
  if (bound_device != device) {
    if ((status = cudaFree(nullptr)) != cudaSuccess) return status;
    bound_device = device;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& cached = g_devices[device];
  if (cached.device != device) {
    DeviceInfo fresh;
    fresh.device = device;
    if ((status = cudaDeviceGetAttribute(&fresh.sm_count, cudaDevAttrMultiProcessorCount, device)) !=
            cudaSuccess ||
        (status = cudaDeviceGetAttribute(&fresh.cc_major, cudaDevAttrComputeCapabilityMajor, device)) !=
            cudaSuccess ||
        (status = cudaDeviceGetAttribute(&fresh.cc_minor, cudaDevAttrComputeCapabilityMinor, device)) !=
            cudaSuccess)
      return status;
    void* address = nullptr;
    status = cudaGetSymbolAddress(&address, g_status_record);
    if (status != cudaSuccess) return status;
    fresh.status = static_cast<uint32_t*>(address);
    cached = fresh;
  }
  *info = cached;
  return cudaSuccess;
}

uint32_t next_launch_id() {
  uint32_t id = ++g_launch_id;
  if (id == 0) id = ++g_launch_id;  // 0 means "no abort" in the status record
  return id;
}

void count_launch(uint64_t kernels) { g_launch_count += kernels; }

// Read on every launch, like the other environment switches.
uint64_t default_wait_budget_ns() {
  const char* text = std::getenv("FUSE_B200_WAIT_MS");
  double ms = text ? std::atof(text) : 0.0;
  if (!(ms > 0.0)) ms = 2000.0;
  return uint64_t(ms * 1.0e6);
}

cudaError_t encode_tensor_map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype,
                                 uint32_t element_bytes, uint64_t rows, uint64_t cols,
                                 uint64_t row_pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                                 CUtensorMapSwizzle swizzle) {
  EncodeTiled encode = encode_entry();
  if (encode == nullptr) return cudaErrorNotSupported;
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || row_pitch_bytes % 16 != 0 ||
      (uint64_t(box_cols) * element_bytes) % 16 != 0 || box_rows > 256 || box_cols > 256)
    return cudaErrorInvalidValue;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_pitch_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t element_strides[2] = {1, 1};
  const CUresult result =
      encode(map, dtype, 2, const_cast<void*>(base), dims, strides, box, element_strides,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return result == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace host
}  // namespace fuse_b200

extern "C" {

int fuse_b200_read_status(uint32_t out[16], int clear) {
  fuse_b200::host::DeviceInfo info;
  cudaError_t status = fuse_b200::host::device_info(&info);
  if (status != cudaSuccess) return int(status);
  status = cudaMemcpy(out, info.status, sizeof(uint32_t) * fuse_b200::kStatusWords,
                      cudaMemcpyDeviceToHost);
  if (status != cudaSuccess) return int(status);
  if (clear) status = cudaMemset(info.status, 0, sizeof(uint32_t) * fuse_b200::kStatusWords);
  return int(status);
}

int fuse_b200_tile_order_decode(int32_t m_tiles, int32_t n_tiles, int32_t swizzle, int32_t along_n,
                                int64_t linear, int32_t* m, int32_t* n) {
  if (m_tiles <= 0 || n_tiles <= 0 || (swizzle != 1 && swizzle != 2 && swizzle != 4 && swizzle != 8) ||
      linear < 0 || linear >= int64_t(m_tiles) * n_tiles || m == nullptr || n == nullptr)
    return 1;
  fuse_b200::TileOrder order;
  order.m_tiles = m_tiles;
  order.n_tiles = n_tiles;
  order.swizzle = swizzle;
  order.along_n = along_n ? 1 : 0;
  order.decode(linear, *m, *n);
  return order.linear(*m, *n) == linear ? 0 : 1;
}

int32_t fuse_b200_select_swizzle(int32_t max_swizzle, int32_t m_tiles, int32_t n_tiles) {
  return fuse_b200::select_swizzle(max_swizzle, m_tiles, n_tiles);
}

uint64_t fuse_b200_launch_count(void) { return fuse_b200::host::g_launch_count.load(); }

}  // extern "C"
