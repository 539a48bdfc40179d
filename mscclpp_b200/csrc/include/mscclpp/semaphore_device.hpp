// Device handles of the semaphores. A semaphore is a pair of monotonically increasing 64-bit
// counters: signal() bumps the counter on the receiving side, wait() bumps a private expectation and
// spins until the inbound counter has caught up. Nothing is ever reset, so no ABA and no clearing.
// (Reference: include/mscclpp/semaphore_device.hpp:17-240.) Every wait here is bounded: it returns
// false after `timeoutNs` and records the reason in `status` instead of spinning forever.
#pragma once

#include <cstdint>

#include "device/ptx.cuh"
#include "poll_device.hpp"

namespace mscclpp {

// Host signals, device waits.
struct Host2DeviceSemaphoreDeviceHandle {
  uint64_t* inboundToken;     // written by the host (through the connection), read here
  uint64_t* expectedInboundToken;  // private to the waiting GPU

#if defined(__CUDACC__)
  MSCCLPP_DEVICE_INLINE bool poll() {
    const uint64_t next = *expectedInboundToken + 1;
    if (ptx::ld_acquire_sys(inboundToken) >= next) {
      *expectedInboundToken = next;
      return true;
    }
    return false;
  }
  MSCCLPP_DEVICE_INLINE bool wait(uint64_t timeoutNs = 10000000000ull, DeviceStatus* status = nullptr) {
    const uint64_t next = ++(*expectedInboundToken);
    return waitGreaterEqual(inboundToken, next, status, timeoutNs, kDevTimeoutSemaphore, 0, 1, 0);
  }
  // Building blocks under the names of the reference (include/mscclpp/semaphore_device.hpp:33-49), for kernels that
  // compose their own waits.
  MSCCLPP_DEVICE_INLINE uint64_t loadExpectedInbound() { return *reinterpret_cast<volatile uint64_t*>(expectedInboundToken); }
  MSCCLPP_DEVICE_INLINE uint64_t incExpectedInbound() {
    return atomicAdd(reinterpret_cast<unsigned long long*>(expectedInboundToken), 1ull) + 1;
  }
  MSCCLPP_DEVICE_INLINE uint64_t loadInbound() { return ptx::ld_acquire_sys(inboundToken); }
  MSCCLPP_DEVICE_INLINE uint64_t loadInboundRelaxed() { return ptx::ld_relaxed_sys(inboundToken); }
#endif
};

// Device signals a peer device (peer-mapped token), device waits.
struct MemoryDevice2DeviceSemaphoreDeviceHandle {
  uint64_t* inboundToken;          // local, bumped by the peer
  uint64_t* outboundToken;         // local copy of what we have sent (kept for parity / debugging)
  uint64_t* remoteInboundToken;    // peer's inboundToken, mapped here
  uint64_t* expectedInboundToken;  // private

#if defined(__CUDACC__)
  MSCCLPP_DEVICE_INLINE bool poll() {
    const uint64_t next = *expectedInboundToken + 1;
    if (ptx::ld_acquire_sys(inboundToken) >= next) {
      *expectedInboundToken = next;
      return true;
    }
    return false;
  }
  MSCCLPP_DEVICE_INLINE bool wait(uint64_t timeoutNs = 10000000000ull, DeviceStatus* status = nullptr) {
    const uint64_t next = ++(*expectedInboundToken);
    return waitGreaterEqual(inboundToken, next, status, timeoutNs, kDevTimeoutSemaphore, 0, 2, 0);
  }
  // Acquire-free variant for pure flow control (no data is read after it).
  MSCCLPP_DEVICE_INLINE bool relaxedWait(uint64_t timeoutNs = 10000000000ull, DeviceStatus* status = nullptr) {
    const uint64_t next = ++(*expectedInboundToken);
    SpinGuard g(status, timeoutNs);
    uint64_t v;
    while ((v = ptx::ld_relaxed_sys(inboundToken)) < next) {
      if (!g.keepSpinning()) {
        g.report(kDevTimeoutSemaphore, 0, 3, 0, next, v);
        return false;
      }
    }
    return true;
  }
  // Everything this thread wrote before signal() is visible to the peer once its wait() returns.
  MSCCLPP_DEVICE_INLINE void signal() {
    ++(*outboundToken);
    ptx::red_release_sys_add(remoteInboundToken, 1);
  }
  MSCCLPP_DEVICE_INLINE void relaxedSignal() {
    ++(*outboundToken);
    ptx::red_relaxed_sys_add(remoteInboundToken, 1);
  }
  // Building blocks under the names of the reference (include/mscclpp/semaphore_device.hpp:33-49), for kernels that
  // compose their own waits.
  MSCCLPP_DEVICE_INLINE uint64_t loadExpectedInbound() { return *reinterpret_cast<volatile uint64_t*>(expectedInboundToken); }
  MSCCLPP_DEVICE_INLINE uint64_t incExpectedInbound() {
    return atomicAdd(reinterpret_cast<unsigned long long*>(expectedInboundToken), 1ull) + 1;
  }
  MSCCLPP_DEVICE_INLINE uint64_t loadInbound() { return ptx::ld_acquire_sys(inboundToken); }
  MSCCLPP_DEVICE_INLINE uint64_t loadInboundRelaxed() { return ptx::ld_relaxed_sys(inboundToken); }
#endif
};

// Barrier among all GPUs bound to one multicast object: one multimem.red bumps every member's
// counter, each member waits for `expected += groupSize`.
struct SwitchDevice2DeviceSemaphoreDeviceHandle {
  uint64_t* counter;        // local view of the barrier word
  uint64_t* counterMc;      // multicast alias of the same word
  uint64_t* expected;       // private
  int groupSize;

#if defined(__CUDACC__)
  MSCCLPP_DEVICE_INLINE void signal() { ptx::multimem_red_release_add_u64(counterMc, 1); }
  MSCCLPP_DEVICE_INLINE void relaxedSignal() { ptx::multimem_red_relaxed_add_u64(counterMc, 1); }
  MSCCLPP_DEVICE_INLINE bool wait(uint64_t timeoutNs = 10000000000ull, DeviceStatus* status = nullptr) {
    *expected += static_cast<uint64_t>(groupSize);
    return waitGreaterEqual(counter, *expected, status, timeoutNs, kDevTimeoutBarrier, 0, 4, 0);
  }
#endif
};

}  // namespace mscclpp
