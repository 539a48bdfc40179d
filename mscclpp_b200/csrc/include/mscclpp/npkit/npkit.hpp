// NpKit: a low-overhead event tracer for device kernels and host proxies.
//
// Init(rank) allocates one event buffer per traced thread block (device memory) and per host channel, and
// records a (GPU globaltimer, host clock) pair for aligning the two time lines. Kernels that are handed the
// context array (nullptr when tracing is off) append 16-byte events with `npkitCollectGpuEvent`; Dump(dir) writes
// one binary file per buffer plus the clock files. The reference's NPKit has the same life cycle and file
// names (include/mscclpp/npkit/npkit.hpp:28-109, src/core/npkit/npkit.cc:22-190) but stamps events with the
// SM cycle counter and selects events at compile time; here events carry nanoseconds from %globaltimer (so all
// SMs share one time base) and tracing is switched at run time.
#pragma once

#include <cstdint>
#include <string>

#include "npkit_event.hpp"
#include "npkit_struct.hpp"

#if defined(__CUDACC__)
#include "../device/ptx.cuh"
#endif

class NpKit {
 public:
  static constexpr uint64_t kNumGpuEventBuffers = 256;          // traced thread blocks (blockIdx.x + gridDim.x * blockIdx.y)
  static constexpr uint64_t kNumCpuEventBuffers = 64;           // host channels
  static constexpr uint64_t kMaxNumGpuEventsPerBuffer = 1ull << 14;  // 256 * 16 Ki * 16 B = 64 MiB of device memory
  static constexpr uint64_t kMaxNumCpuEventsPerBuffer = 1ull << 16;

  static void Init(int rank);
  static void Dump(const std::string& dumpDir);
  static void Shutdown();
  static bool Enabled();
  // Device array of kNumGpuEventBuffers contexts, nullptr when tracing is off.
  static NpKitEventCollectContext* GetGpuEventCollectContexts();
  static void CollectCpuEvent(uint8_t type, uint32_t size, uint32_t rsvd, uint64_t timestamp, int channelId);
  // Host time stamp in the unit of the CPU events (nanoseconds of the system clock).
  static uint64_t GetCpuTimestamp();
};

#if defined(__CUDACC__)
// One thread per block calls this (the caller picks the thread). Events beyond the buffer capacity are dropped.
__device__ __forceinline__ void npkitCollectGpuEvent(NpKitEventCollectContext* contexts, uint8_t type, uint32_t size, uint32_t rsvd) {
  if (contexts == nullptr) return;
  const uint64_t buf = blockIdx.x + static_cast<uint64_t>(gridDim.x) * blockIdx.y;
  if (buf >= NpKit::kNumGpuEventBuffers) return;
  NpKitEventCollectContext& ctx = contexts[buf];
  const uint64_t head = ctx.event_buffer_head;
  if (head >= NpKit::kMaxNumGpuEventsPerBuffer) return;
  NpKitEvent e;
  e.bits[0] = static_cast<uint64_t>(type) | (static_cast<uint64_t>(size) << 8) | (static_cast<uint64_t>(rsvd & 0xffffffu) << 40);
  e.bits[1] = mscclpp::ptx::globaltimer();
  ctx.event_buffer[head] = e;
  ctx.event_buffer_head = head + 1;
}
#endif
