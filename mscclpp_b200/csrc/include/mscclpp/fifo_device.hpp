// GPU -> CPU request queue. Many GPU threads push 16-byte triggers into a ring in host-pinned
// memory; one host thread consumes them. The slot's top bit carries the parity of the lap it was
// written in, so the consumer recognises a fresh entry without the slot ever being cleared
// (reference: include/mscclpp/fifo_device.hpp:18-183, src/core/fifo.cc:24-78).
#pragma once

#include <cstdint>

#include "device/ptx.cuh"
#include "poll_device.hpp"

namespace mscclpp {

// fst / snd are opaque to the FIFO except for the top bit of snd (lap parity, set by push()).
struct alignas(16) ProxyTrigger {
  uint64_t fst;
  uint64_t snd;
};

constexpr uint64_t kTriggerParityBit = 1ull << 63;

struct FifoDeviceHandle {
  ProxyTrigger* triggers;   // ring in host-pinned memory (device-visible)
  uint64_t* head;           // device memory: next ticket to hand out
  uint64_t* tail;           // host-pinned memory: tickets consumed so far (written by the host)
  uint64_t* tailCache;      // device memory: last tail value any thread has seen
  int size;                 // number of slots

#if defined(__CUDACC__)
  // Enqueue; returns the ticket (position) of the trigger, or UINT64_MAX if the queue stayed full for
  // the whole budget (the host thread is gone).
  MSCCLPP_DEVICE_INLINE uint64_t push(ProxyTrigger trigger, DeviceStatus* status = nullptr,
                                      uint64_t timeoutNs = 10000000000ull) {
    const uint64_t ticket = atomicAdd(reinterpret_cast<unsigned long long*>(head), 1ull);
    // flow control: slot (ticket % size) is free once ticket - size tickets have been consumed
    if (ticket >= static_cast<uint64_t>(size) + ptx::ld_volatile(tailCache)) {
      SpinGuard g(status, timeoutNs);
      uint64_t seen;
      while (ticket >= static_cast<uint64_t>(size) + (seen = ptx::ld_acquire_sys(tail))) {
        if (!g.keepSpinning()) {
          g.report(kDevTimeoutFifo, 0, 40, 0, ticket, seen);
          return UINT64_MAX;
        }
      }
      atomicMax(reinterpret_cast<unsigned long long*>(tailCache), static_cast<unsigned long long>(seen));
    }
    const uint64_t lap = ticket / static_cast<uint64_t>(size);
    // parity bit = 1 on even laps, 0 on odd laps: a zero-initialised ring reads as "nothing yet"
    trigger.snd = (trigger.snd & ~kTriggerParityBit) | ((lap & 1ull) ? 0ull : kTriggerParityBit);
    ProxyTrigger* slot = &triggers[ticket % static_cast<uint64_t>(size)];
    asm volatile("st.global.release.sys.v2.u64 [%0], {%1, %2};" ::"l"(slot), "l"(trigger.fst), "l"(trigger.snd) : "memory");
    return ticket;
  }

  // Wait until the trigger with this ticket has been consumed by the host. false = budget ran out.
  MSCCLPP_DEVICE_INLINE bool sync(uint64_t ticket, DeviceStatus* status = nullptr, uint64_t timeoutNs = 10000000000ull) {
    if (ticket < ptx::ld_volatile(tailCache)) return true;
    SpinGuard g(status, timeoutNs);
    uint64_t seen;
    while (ticket >= (seen = ptx::ld_acquire_sys(tail))) {
      if (!g.keepSpinning()) {
        g.report(kDevTimeoutFifo, 0, 41, 0, ticket, seen);
        return false;
      }
    }
    atomicMax(reinterpret_cast<unsigned long long*>(tailCache), static_cast<unsigned long long>(seen));
    return true;
  }
#endif
};

}  // namespace mscclpp
