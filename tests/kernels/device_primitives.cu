// Test kernels for the header-only device primitives: LL8 / LL16 / LL128 packets (a producer block and a consumer
// block of ONE cooperative launch), byte copies with odd sizes and alignments, the grid syncer, the device semaphore,
// and a packet wait that runs out (nobody writes the flag): it must return an error instead of hanging.
#include <mscclpp/concurrency_device.hpp>
#include <mscclpp/copy_device.hpp>
#include <mscclpp/packet_device.hpp>

using namespace mscclpp;

constexpr unsigned long long kBudget = 2000000000ull;

// block 0 packs `bytes` of src into packets with `flag`; block 1 waits for them and unpacks into dst.
// kind: 8 = LL8, 16 = LL16
extern "C" __global__ void packetPingPong(const void* src, void* packets, void* dst, unsigned long long bytes, unsigned flag, int kind,
                                          int* failed) {
  if (blockIdx.x == 0) {
    if (kind == 8) copyToPackets<LL8Packet>(packets, src, bytes, threadIdx.x, blockDim.x, flag);
    else copyToPackets<LL16Packet>(packets, src, bytes, threadIdx.x, blockDim.x, flag);
  } else {
    bool ok = kind == 8 ? copyFromPackets<LL8Packet>(dst, packets, bytes, threadIdx.x, blockDim.x, flag, nullptr, kBudget)
                        : copyFromPackets<LL16Packet>(dst, packets, bytes, threadIdx.x, blockDim.x, flag, nullptr, kBudget);
    if (!ok) *failed = 1;
  }
}

// LL128: lines of 120 payload bytes; 8 consecutive lanes handle one line. src/dst are arrays of uint4 with 8 per line
// (the 8th carries 8 payload bytes in .x/.y).
extern "C" __global__ void ll128PingPong(const uint4* src, LL128Line* lines, uint4* dst, int numLines, unsigned long long flag, int* failed) {
  const int lane = threadIdx.x & 31, sub = lane & 7;
  const int groupInBlock = threadIdx.x >> 3, groupsPerBlock = blockDim.x >> 3;
  const unsigned mask = 0xffu << (lane & 24);
  for (int l = groupInBlock; l < numLines; l += groupsPerBlock) {
    if (blockIdx.x == 0) {
      ll128Write(&lines[l], sub, src[l * 8 + sub], flag);
    } else {
      uint4 v;
      if (!ll128Read(&lines[l], sub, mask, flag, v, nullptr, kBudget)) {
        *failed = 1;
        return;
      }
      if (sub == 7) v.z = v.w = 0;  // the flag is not payload
      dst[l * 8 + sub] = v;
    }
  }
}

extern "C" __global__ void copyOdd(char* dst, const char* src, unsigned long long bytes) {
  copyBytes(dst, src, bytes, blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x);
}

// Every block adds its id to a slot of `scratch`, syncs, then sums all slots; repeated `rounds` times.
extern "C" __global__ void syncerRounds(DeviceSyncer* syncer, unsigned* scratch, unsigned* sums, int rounds, int* failed) {
  unsigned generation = 0;
  for (int r = 0; r < rounds; r++) {
    if (threadIdx.x == 0) scratch[blockIdx.x] = (r + 1) * (blockIdx.x + 1);
    if (!syncer->sync(gridDim.x, generation, nullptr, kBudget)) {
      if (threadIdx.x == 0) *failed = 1;
      return;
    }
    if (threadIdx.x == 0) {
      unsigned s = 0;
      for (unsigned b = 0; b < gridDim.x; b++) s += reinterpret_cast<volatile unsigned*>(scratch)[b];
      sums[r * gridDim.x + blockIdx.x] = s;
    }
    if (!syncer->sync(gridDim.x, generation, nullptr, kBudget)) {  // nobody overwrites scratch before all have read it
      if (threadIdx.x == 0) *failed = 1;
      return;
    }
  }
}

// Block 0 releases the semaphore `n` times, block 1 acquires it `n` times and counts.
extern "C" __global__ void semaphoreHandOff(DeviceSemaphore* sem, int n, int* acquired, int* failed) {
  if (threadIdx.x != 0) return;
  for (int i = 0; i < n; i++) {
    if (blockIdx.x == 0) {
      sem->release();
    } else {
      if (!sem->acquire(nullptr, kBudget)) {
        *failed = 1;
        return;
      }
      atomicAdd(acquired, 1);
    }
  }
}

// A wait for a packet that nobody sends: returns false after `budgetNs`, records the give-up in `status`.
extern "C" __global__ void packetWaitRunsOut(const LL16Packet* packets, DeviceStatus* status, unsigned long long budgetNs, int* gaveUp) {
  uint2 v;
  if (threadIdx.x == 0 && !packets[0].read(12345u, v, status, budgetNs)) *gaveUp = 1;
}

#include <mscclpp/fifo_device.hpp>

// One thread pushes `n` triggers (fst = i + 1). With nobody consuming, pushes beyond the ring size give up after
// `budgetNs` and return UINT64_MAX: `accepted` counts the ones that went in.
extern "C" __global__ void fifoPush(FifoDeviceHandle fifo, int n, unsigned long long budgetNs, int* accepted) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  for (int i = 0; i < n; i++) {
    ProxyTrigger t;
    t.fst = static_cast<uint64_t>(i + 1);
    t.snd = 0;
    if (fifo.push(t, nullptr, budgetNs) == UINT64_MAX) return;
    atomicAdd(accepted, 1);
  }
}
