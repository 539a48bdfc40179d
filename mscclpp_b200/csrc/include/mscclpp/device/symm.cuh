// Device view of the symmetric heap.
//
// Every rank owns one VMM allocation ("heap") of the same size. All heaps are mapped into every
// rank's address space (peerBase[r]) and, when NVLS is available, bound to one multicast object
// (mcBase). A pointer into the local heap therefore has a peer alias and a multicast alias that
// are computed arithmetically, with no per-buffer registration on the hot path. The first bytes of
// each heap hold a SymmControl block: launch epoch, cross-rank barrier flags and LL packet scratch.
//
// Kernels can also run several "emulated" ranks inside ONE launch on ONE GPU (gridDim.y = world,
// rank = comm.rank + blockIdx.y, cooperative launch). That is how multi-rank protocols are tested
// when fewer GPUs than ranks are available: separate launches that wait on one another are never
// used, because nothing guarantees that they are co-resident.
#pragma once

#include <cstdint>

#include "../poll_device.hpp"
#include "ptx.cuh"

namespace mscclpp {

constexpr int kMaxRanks = 16;
constexpr int kBarrierSlots = 192;   // one slot per thread block taking part in a cross-rank barrier
constexpr int kBarrierPhases = 4;
constexpr uint64_t kAuxFlagBytes = 2u << 20;

struct SymmControl {
  uint32_t epoch;  // number of collective launches completed on this heap
  uint32_t done;   // blocks of the running launch that have finished
  uint32_t gridArrive[2];
  uint32_t pad0[28];
  // barrier[phase][slot][src]: src rank stamps the launch epoch here, with release semantics
  uint32_t barrier[kBarrierPhases][kBarrierSlots][kMaxRanks];
  uint32_t gridSync[64];
  uint64_t userFlags[512];  // free-form signalling words (fused kernels, semaphores for tests)
};

struct DeviceComm {
  uint64_t peerBase[kMaxRanks];  // address of rank r's heap in this process
  uint64_t mcBase;               // multicast alias of the heap, 0 when NVLS is not in use
  uint64_t heapBytes;
  uint64_t llScratchOff;    // heap offset of the LL scratch: 2 buffers x world x llSlotBytes
  uint64_t llSlotBytes;     // bytes of packets one source rank may write per buffer
  uint64_t auxFlagsOff;     // heap offset of kAuxFlagBytes of epoch-stamped flags for fused kernels
  DeviceStatus* status;     // host-visible error block (may be null)
  uint64_t timeoutNs;       // budget of every device-side wait
  int rank;
  int world;
};

#if defined(__CUDACC__)

struct RankView {
  int rank;
  int world;
  uint64_t localBase;
};

MSCCLPP_DEVICE_INLINE int deviceRank(const DeviceComm& c) { return c.rank + static_cast<int>(blockIdx.y); }

MSCCLPP_DEVICE_INLINE SymmControl* control(const DeviceComm& c, int r) {
  return reinterpret_cast<SymmControl*>(c.peerBase[r]);
}

// Alias of local heap pointer `p` (owned by `rank`) inside rank r's heap.
template <typename T>
MSCCLPP_DEVICE_INLINE T* peerPtr(const DeviceComm& c, int rank, int r, T* p) {
  return reinterpret_cast<T*>(c.peerBase[r] + (reinterpret_cast<uint64_t>(p) - c.peerBase[rank]));
}
template <typename T>
MSCCLPP_DEVICE_INLINE T* mcPtr(const DeviceComm& c, int rank, T* p) {
  return reinterpret_cast<T*>(c.mcBase + (reinterpret_cast<uint64_t>(p) - c.peerBase[rank]));
}

// Epoch the running launch stamps into flags and packets. All blocks read the same value because
// it only changes when the last block of a launch retires (finishLaunch).
MSCCLPP_DEVICE_INLINE uint32_t launchEpoch(const DeviceComm& c, int rank) {
  return ptx::ld_volatile(&control(c, rank)->epoch) + 1u;
}

// Called by every block once, after its last use of the epoch. All threads must call it.
MSCCLPP_DEVICE_INLINE void finishLaunch(const DeviceComm& c, int rank, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    SymmControl* ctl = control(c, rank);
    __threadfence();
    uint32_t prev = atomicAdd(&ctl->done, 1u);
    if (prev == gridDim.x - 1) {
      ctl->done = 0;
#pragma unroll
      for (int i = 0; i < 8; i++) ctl->gridSync[i] = 0;  // every block is past its last grid barrier
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&ctl->epoch) = epoch;
    }
  }
}

// The same bookkeeping, done EARLY: for kernels that use none of the grid-barrier counters. All the count decides is when
// the rank's epoch moves on, which only the NEXT launch reads, and that one starts after this one has ended; so a block
// may count itself out as soon as every one of its threads holds its copy of the epoch (the barrier below takes a
// predicate computed from it, which forces the loads to have completed). The last block to get here moves the epoch - by
// then every block has read the old one. At the end of a kernel the round trip of this atomic is exposed; placed before
// a wait (for packets, for copies) it costs nothing. All threads of the block must call it, exactly once.
MSCCLPP_DEVICE_INLINE void retireLaunchEarly(const DeviceComm& c, int rank, uint32_t epoch) {
  (void)__syncthreads_or(epoch == 0u ? 1 : 0);
  if (threadIdx.x == 0) {
    SymmControl* ctl = control(c, rank);
    const uint32_t prev = atomicAdd(&ctl->done, 1u);
    if (prev == gridDim.x - 1) {
      ctl->done = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&ctl->epoch) = epoch;
    }
  }
}

// Cross-rank barrier for block `slot` (same slot index on every rank). All threads of the block
// call it. With `publish` (the default) writes made by this block before the call are visible to peers after their
// barrier returns: one system-scope fence (behind the block's own barrier, so it covers every thread's writes), then a
// relaxed flag store - a release store on top of the fence would pay for a second fence. Without `publish` the flag
// only says "this rank has got here" (an opening barrier, when everything the peers will read was written by earlier
// launches): no fence at all. The wait polls with relaxed loads and takes one acquire when the flag has arrived.
// Returns false if a peer did not show up within the budget.
MSCCLPP_DEVICE_INLINE bool rankBarrier(const DeviceComm& c, int rank, int phase, int slot, uint32_t epoch, bool publish = true) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  const int t = threadIdx.x;
  if (t < c.world && t != rank) {
    if (publish) ptx::fence_acq_rel_sys();
    ptx::st_relaxed_sys(&control(c, t)->barrier[phase][slot][rank], epoch);
    const uint32_t* mine = &control(c, rank)->barrier[phase][slot][t];
    SpinGuard g(c.status, c.timeoutNs);
    uint32_t v;
    bool here = true;
    while (static_cast<int32_t>((v = ptx::ld_relaxed_sys(mine)) - epoch) < 0) {
      if (!g.keepSpinning()) {
        g.report(kDevTimeoutBarrier, rank, phase * 1000 + slot, t, epoch, v);
        here = false;
        break;
      }
    }
    if (here) (void)ptx::ld_acquire_sys(mine);
    else ok_s = 0;
  }
  __syncthreads();
  return ok_s != 0;
}

// Grid-wide barrier among the gridDim.x blocks of ONE rank. `counter` is one of
// SymmControl::gridSync[0..7] (zeroed by finishLaunch); the k-th barrier (k = 0, 1, ...) of a launch
// on that counter passes target = (k + 1) * gridDim.x. The grid must be co-resident.
MSCCLPP_DEVICE_INLINE bool gridBarrier(const DeviceComm& c, int rank, uint32_t* counter, uint32_t target) {
  __shared__ int okg_s;
  __syncthreads();
  if (threadIdx.x == 0) {
    okg_s = 1;
    ptx::fence_acq_rel_gpu();
    ptx::red_release_gpu_add(counter, 1u);
    SpinGuard g(c.status, c.timeoutNs);
    uint32_t v;
    while (static_cast<int32_t>((v = ptx::ld_acquire_gpu(counter)) - target) < 0) {
      if (!g.keepSpinning()) {
        g.report(kDevTimeoutBarrier, rank, 9000, 0, target, v);
        okg_s = 0;
        break;
      }
    }
  }
  __syncthreads();
  return okg_s != 0;
}

#endif  // __CUDACC__

}  // namespace mscclpp
