// Synchronisation among the thread blocks of one kernel: DeviceSyncer (grid barrier) and
// DeviceSemaphore (counting semaphore). Reference: include/mscclpp/concurrency_device.hpp:28-132.
// Both need every participating block to be co-resident; waits are bounded.
#pragma once

#include <cstdint>

#include "device/ptx.cuh"
#include "poll_device.hpp"

namespace mscclpp {

// Zero-initialise in device memory, then call sync(nBlocks) from every thread of every participating
// block. The counter only grows: the n-th use waits for n * nBlocks arrivals, tracked per block in
// `generation_` kept in registers by the caller through the returned object state.
struct DeviceSyncer {
  uint32_t count_;
  uint32_t pad_[3];

#if defined(__CUDACC__)
  // `generation` is the caller's private count of completed syncs on this syncer (start at 0).
  MSCCLPP_DEVICE_INLINE bool sync(int nBlocks, uint32_t& generation, DeviceStatus* status = nullptr,
                                  uint64_t timeoutNs = 10000000000ull) {
    __shared__ int ok_;
    __syncthreads();
    generation++;
    if (threadIdx.x == 0) {
      ok_ = 1;
      const uint32_t target = generation * static_cast<uint32_t>(nBlocks);
      ptx::fence_acq_rel_gpu();
      ptx::red_release_gpu_add(&count_, 1u);
      SpinGuard g(status, timeoutNs);
      uint32_t v;
      while (static_cast<int32_t>((v = ptx::ld_acquire_gpu(&count_)) - target) < 0) {
        if (!g.keepSpinning()) {
          g.report(kDevTimeoutBarrier, 0, 20, 0, target, v);
          ok_ = 0;
          break;
        }
      }
    }
    __syncthreads();
    return ok_ != 0;
  }
#endif
};

// Counting semaphore between blocks: acquire() takes one unit (waits while the value is <= 0),
// release() gives one back. Call from ONE thread of a block.
struct DeviceSemaphore {
  int value_;
  int pad_[3];

#if defined(__CUDACC__)
  MSCCLPP_DEVICE_INLINE void set(int v) { value_ = v; }
  MSCCLPP_DEVICE_INLINE bool acquire(DeviceStatus* status = nullptr, uint64_t timeoutNs = 10000000000ull) {
    SpinGuard g(status, timeoutNs);
    while (true) {
      int cur = *reinterpret_cast<volatile int*>(&value_);
      if (cur > 0 && atomicCAS(&value_, cur, cur - 1) == cur) {
        __threadfence();
        return true;
      }
      if (!g.keepSpinning()) {
        g.report(kDevTimeoutSemaphore, 0, 21, 0, 1, static_cast<uint64_t>(cur));
        return false;
      }
    }
  }
  MSCCLPP_DEVICE_INLINE void release() {
    __threadfence();
    atomicAdd(&value_, 1);
  }
#endif
};

}  // namespace mscclpp
