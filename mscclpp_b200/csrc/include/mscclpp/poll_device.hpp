// Bounded device-side waits.
//
// Every spin in this library has a time budget. When it runs out the waiter records what it
// was waiting for in a host-visible DeviceStatus block, raises a "poisoned" flag that other
// waiters observe, and RETURNS false: no trap, no assert, no endless loop. The host reads the
// status after the launch and reports ErrorCode::Timeout.
//
// The reference never gives up in release builds and traps in debug builds
// (include/mscclpp/poll_device.hpp:9-30, include/mscclpp/assert_device.hpp:15-38); on shared GPUs
// neither is acceptable, hence the different contract here.
#pragma once

#include <cstdint>

#include "device/ptx.cuh"

namespace mscclpp {

enum DeviceErrorCode : uint32_t {
  kDevOk = 0,
  kDevTimeoutSemaphore = 1,
  kDevTimeoutPacket = 2,
  kDevTimeoutBarrier = 3,
  kDevTimeoutFifo = 4,
  kDevTimeoutMbarrier = 5,
  kDevTimeoutFlag = 6,
  kDevBadArgument = 7,
  kDevErrorCapacity = 8,  // a receive buffer is too small for the rows routed to it (MoE dispatch)
};

// Lives in host-pinned (mapped) memory or in device memory; 64 bytes.
struct DeviceStatus {
  uint32_t code;      // first error (DeviceErrorCode); 0 = healthy
  uint32_t poisoned;  // non-zero once any waiter gave up; waiters poll it and bail out early
  uint32_t rank;
  uint32_t block;
  uint32_t where;     // caller-defined site id
  uint32_t peer;
  uint64_t expected;
  uint64_t observed;
  uint64_t count;     // number of give-ups (all sites)
  uint64_t reserved[2];
};

#if defined(__CUDACC__)

struct SpinGuard {
  DeviceStatus* status;
  uint64_t budgetNs;
  uint64_t start;
  uint32_t iters;

  MSCCLPP_DEVICE_INLINE SpinGuard(DeviceStatus* s, uint64_t ns) : status(s), budgetNs(ns), start(0), iters(0) {}

  // Call once per failed probe. Returns false when the caller must give up.
  MSCCLPP_DEVICE_INLINE bool keepSpinning() {
    if ((++iters & 0x3f) != 0) return true;
    if (start == 0) {
      start = ptx::globaltimer();
      return true;
    }
    if (status != nullptr && *reinterpret_cast<volatile uint32_t*>(&status->poisoned) != 0) return false;
    return (ptx::globaltimer() - start) < budgetNs;
  }

  MSCCLPP_DEVICE_INLINE void report(uint32_t code, uint32_t rank, uint32_t where, uint32_t peer, uint64_t expected,
                                    uint64_t observed) {
    if (status == nullptr) return;
    if (atomicCAS(&status->code, 0u, code) == 0u) {
      status->rank = rank;
      status->block = blockIdx.x;
      status->where = where;
      status->peer = peer;
      status->expected = expected;
      status->observed = observed;
    }
    atomicAdd(reinterpret_cast<unsigned long long*>(&status->count), 1ull);
    *reinterpret_cast<volatile uint32_t*>(&status->poisoned) = 1u;
    __threadfence_system();
  }
};

// Spin until `*p >= expected` (acquire, system scope). false = gave up.
MSCCLPP_DEVICE_INLINE bool waitGreaterEqual(const uint64_t* p, uint64_t expected, DeviceStatus* st, uint64_t budgetNs,
                                            uint32_t code, uint32_t rank, uint32_t where, uint32_t peer) {
  SpinGuard g(st, budgetNs);
  uint64_t v;
  while ((v = ptx::ld_acquire_sys(p)) < expected) {
    if (!g.keepSpinning()) {
      g.report(code, rank, where, peer, expected, v);
      return false;
    }
  }
  return true;
}
MSCCLPP_DEVICE_INLINE bool waitGreaterEqual(const uint32_t* p, uint32_t expected, DeviceStatus* st, uint64_t budgetNs,
                                            uint32_t code, uint32_t rank, uint32_t where, uint32_t peer) {
  SpinGuard g(st, budgetNs);
  uint32_t v;
  // signed distance so that a wrapping 32-bit epoch still compares correctly
  while (static_cast<int32_t>((v = ptx::ld_acquire_sys(p)) - expected) < 0) {
    if (!g.keepSpinning()) {
      g.report(code, rank, where, peer, expected, v);
      return false;
    }
  }
  return true;
}

// Same contract as waitGreaterEqual, for flags that MANY threads of many blocks poll at once: relaxed
// polls with a short sleep between them (an acquire poll per iteration from thousands of threads keeps
// the flag's L2 slice so busy that the writer's store queues behind the readers), one acquire fence
// after the value has been seen.
MSCCLPP_DEVICE_INLINE bool waitGreaterEqualBackoff(const uint32_t* p, uint32_t expected, DeviceStatus* st, uint64_t budgetNs,
                                                   uint32_t code, uint32_t rank, uint32_t where, uint32_t peer) {
  SpinGuard g(st, budgetNs);
  uint32_t v;
  while (static_cast<int32_t>((v = ptx::ld_relaxed_sys(p)) - expected) < 0) {
    __nanosleep(100);
    if (!g.keepSpinning()) {
      g.report(code, rank, where, peer, expected, v);
      return false;
    }
  }
  // Acquire through a load, not a fence: a system-scope fence would also wait for this thread's earlier peer stores.
  (void)ptx::ld_acquire_sys(p);
  return true;
}

// Bounded mbarrier wait for the hot loops of a pipeline: the common case (the phase has completed, or completes within
// the hardware's own try_wait window) costs one instruction and touches nothing else. `abortFlag` (shared memory, may
// be null) is looked at only while actually waiting. false = gave up or aborted.
MSCCLPP_DEVICE_INLINE bool mbarWaitFast(uint64_t* bar, uint32_t parity, DeviceStatus* st, uint64_t budgetNs, uint32_t where,
                                        const volatile uint32_t* abortFlag) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  SpinGuard g(st, budgetNs);
  while (!ptx::mbar_try_wait(bar, parity)) {
    if (abortFlag != nullptr && *abortFlag != 0) return false;
    if (!g.keepSpinning()) {
      g.report(kDevTimeoutMbarrier, 0, where, 0, parity, 0);
      return false;
    }
  }
  return true;
}

// Bounded mbarrier wait (shared memory). false = gave up.
MSCCLPP_DEVICE_INLINE bool mbarWait(uint64_t* bar, uint32_t parity, DeviceStatus* st, uint64_t budgetNs, uint32_t where) {
  SpinGuard g(st, budgetNs);
  while (!ptx::mbar_try_wait(bar, parity)) {
    if (!g.keepSpinning()) {
      g.report(kDevTimeoutMbarrier, 0, where, 0, parity, 0);
      return false;
    }
  }
  return true;
}

#endif  // __CUDACC__

}  // namespace mscclpp
