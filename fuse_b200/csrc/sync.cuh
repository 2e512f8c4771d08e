// Bounded waits and the device status record.
//
// Every wait in this library (mbarrier phase, global epoch flag written by another CTA or by
// another GPU) gives up after a wall-clock budget measured with %globaltimer.  The first
// waiter that gives up claims the status record with an atomic compare-and-swap, writes what
// it was waiting for, and returns false; every other waiter polls the record's owner word and
// returns false as soon as it names the current launch.  Callers unwind to the normal kernel
// exit (in-flight copies drained, TMEM released), so a missing peer or a protocol bug ends as
// an error code on the host instead of a hung GPU.
//
// The reference protocol this restates (include/fuse/arch/common.cuh:35-96) spins without
// limit; the flag layout and scopes are the same.
#pragma once

#include "ptx.cuh"

namespace fuse_b200 {

constexpr int kReadyFlagStride = 32;  // u32 words per flag: one 128-byte line each
constexpr int kMaxWorldSize = 8;
constexpr int kStatusWords = 16;

enum StatusCode : uint32_t {
  kStatusOk = 0,
  kStatusMbarrierTimeout = 1,
  kStatusFlagTimeout = 2,
  kStatusPeerTimeout = 3,
};

// status[0] launch id that aborted (0 = none)   status[1] StatusCode   status[2] wait site
// status[3] blockIdx.x                          status[4] flag index / barrier address
// status[5] last observed value                 status[6] expected value   status[7] epoch
struct WaitContext {
  uint32_t* status;
  uint32_t launch_id;
  uint32_t epoch;
  uint64_t budget_ns;
};

enum WaitSite : uint32_t {
  kSiteSmemEmpty = 1,
  kSiteSmemFull = 2,
  kSiteTmemEmpty = 3,
  kSiteTmemFull = 4,
  kSiteTileReady = 5,
  kSiteLhsReady = 6,
  kSitePeerDone = 7,
  kSiteUpstreamReady = 8,
  kSiteCommStage = 9,
  kSiteWeightReady = 10,
  kSitePanelReady = 11,
  kSitePeerStarted = 12,
  kSiteDrain = 13,
};

__device__ __forceinline__ bool aborted(const WaitContext& w) {
  return ptx::ld_relaxed_gpu(w.status) == w.launch_id;
}

__device__ __noinline__ inline void report_timeout(const WaitContext w, uint32_t code, uint32_t site,
                                            uint32_t index, uint32_t observed, uint32_t expected) {
  // The record goes to the first waiter of THIS launch: a record that an earlier launch left
  // uncleared is overwritten, so that the abort fan-out below still works.
  uint32_t owner = ptx::ld_relaxed_gpu(w.status);
  bool claimed = false;
  while (owner != w.launch_id) {
    const uint32_t seen = atomicCAS(w.status, owner, w.launch_id);
    if (seen == owner) {
      claimed = true;
      break;
    }
    owner = seen;
  }
  if (claimed) {
    w.status[1] = code;
    w.status[2] = site;
    w.status[3] = blockIdx.x;
    w.status[4] = index;
    w.status[5] = observed;
    w.status[6] = expected;
    w.status[7] = w.epoch;
    __threadfence();
  }
}

// Waits for the mbarrier phase with the given parity.  With `honor_abort` the wait also ends
// when another waiter of this launch has given up; the drains that run while unwinding pass
// false so that copies and UMMAs in flight still get their (bounded) time to land.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitContext& w,
                                          uint32_t site, bool honor_abort = true) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t start = ptx::globaltimer();
  for (uint32_t spin = 1;; ++spin) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((spin & 31u) == 0u) {
      if (honor_abort && aborted(w)) return false;
      if (ptx::globaltimer() - start > w.budget_ns) {
        report_timeout(w, kStatusMbarrierTimeout, site, bar, parity, 0);
        return false;
      }
    }
  }
}

// Waits until *flag >= expected with acquire semantics at GPU or system scope.  One thread;
// the caller broadcasts the result (and the acquired ordering) with a CTA/warp barrier.
template <bool kSystemScope>
__device__ __forceinline__ bool flag_wait(const uint32_t* flag, uint32_t expected,
                                          const WaitContext& w, uint32_t site, uint32_t index) {
  uint32_t seen = kSystemScope ? ptx::ld_acquire_sys(flag) : ptx::ld_acquire_gpu(flag);
  if (seen >= expected) return true;
  const uint64_t start = ptx::globaltimer();
  for (uint32_t spin = 1;; ++spin) {
    __nanosleep(40);
    seen = kSystemScope ? ptx::ld_acquire_sys(flag) : ptx::ld_acquire_gpu(flag);
    if (seen >= expected) return true;
    if ((spin & 15u) == 0u) {
      if (aborted(w)) return false;
      if (ptx::globaltimer() - start > w.budget_ns) {
        report_timeout(w, kSystemScope ? kStatusPeerTimeout : kStatusFlagTimeout, site, index, seen,
                       expected);
        return false;
      }
    }
  }
}

// Waits until the shared-memory progress word (written by another warp of this CTA with
// st.release.cta) reaches `expected`.  One thread.  The writer polls global flags under the
// ordinary budget and reports what it was waiting for; this wait learns of that through the
// abort word, and its own (doubled) budget only covers a writer that never ran.
__device__ __forceinline__ bool progress_wait(uint32_t smem_word, uint32_t expected, const WaitContext& w,
                                              uint32_t site, uint32_t index, uint32_t* observed = nullptr) {
  uint32_t seen = ptx::ld_acquire_cta_shared(smem_word);
  if (observed != nullptr) *observed = seen;
  if (seen >= expected) return true;
  const uint64_t start = ptx::globaltimer();
  for (uint32_t spin = 1;; ++spin) {
    seen = ptx::ld_acquire_cta_shared(smem_word);
    if (observed != nullptr) *observed = seen;
    if (seen >= expected) return true;
    if ((spin & 63u) == 0u) {
      if (aborted(w)) return false;
      if (ptx::globaltimer() - start > 2 * w.budget_ns) {
        report_timeout(w, kStatusFlagTimeout, site, index, seen, expected);
        return false;
      }
    }
  }
}

}  // namespace fuse_b200
