// Pointer-based bulk-copy (TMA, non-tensor) primitives for sm_90+/sm_100a: shared-memory mbarriers and
// cp.async.bulk loads, stores and reducing stores. They work on raw addresses, including peer-mapped
// ones, which is what MoE dispatch/combine style kernels want (reference:
// include/mscclpp/bulk_device.hpp:16-272). There is deliberately NO cluster-multicast form.
// Rules: both addresses 16-byte aligned, sizes multiples of 16 bytes.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device/ptx.cuh"
#include "poll_device.hpp"

namespace mscclpp {

#if defined(__CUDACC__)

// An mbarrier in shared memory. The phase bit is kept by the caller (start at 0, flip after each wait).
struct BulkBarrier {
  uint64_t word;

  MSCCLPP_DEVICE_INLINE void init(uint32_t arrivals) {
    ptx::mbar_init(&word, arrivals);
    ptx::fence_mbar_init();
  }
  // Announce `bytes` of incoming bulk-copy data and arrive once.
  MSCCLPP_DEVICE_INLINE void arriveExpectTx(uint32_t bytes) { ptx::mbar_expect_tx(&word, bytes); }
  MSCCLPP_DEVICE_INLINE void arrive() { ptx::mbar_arrive(&word); }
  MSCCLPP_DEVICE_INLINE bool tryWait(uint32_t phase) { return ptx::mbar_try_wait(&word, phase); }
  // Bounded wait; false when the budget ran out.
  MSCCLPP_DEVICE_INLINE bool wait(uint32_t phase, DeviceStatus* status = nullptr, uint64_t timeoutNs = 10000000000ull) {
    return mbarWait(&word, phase, status, timeoutNs, 30);
  }
  MSCCLPP_DEVICE_INLINE void invalidate() { ptx::mbar_inval(&word); }

  // The same operations under the names of the reference's BulkBarrier (include/mscclpp/bulk_device.hpp:68-136).
  MSCCLPP_DEVICE_INLINE uint32_t addr() const { return static_cast<uint32_t>(__cvta_generic_to_shared(&word)); }
  // init without the fence that publishes it to the async proxy (the caller fences, e.g. after several barriers)
  MSCCLPP_DEVICE_INLINE void relaxedInit(uint32_t arrivals = 1) { ptx::mbar_init(&word, arrivals); }
  // raise the expected byte count without arriving
  MSCCLPP_DEVICE_INLINE void expect(uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(addr()), "r"(bytes) : "memory");
  }
  MSCCLPP_DEVICE_INLINE void arriveAndExpect(uint32_t bytes) { arriveExpectTx(bytes); }
  MSCCLPP_DEVICE_INLINE bool poll(uint32_t phase) { return tryWait(phase); }
};

// cp.async.bulk wants both addresses on 16-byte boundaries (and sizes in multiples of 16 bytes).
MSCCLPP_DEVICE_INLINE bool bulkAligned(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }

// global -> shared::cta, completion counted on `bar`.
MSCCLPP_DEVICE_INLINE void bulkLoad(void* smemDst, const void* gmemSrc, uint32_t bytes, BulkBarrier& bar) {
  ptx::bulk_g2s(smemDst, gmemSrc, bytes, &bar.word);
}
// shared::cta -> global (local or peer-mapped). Part of the current bulk group.
MSCCLPP_DEVICE_INLINE void bulkStore(void* gmemDst, const void* smemSrc, uint32_t bytes) {
  ptx::bulk_s2g(gmemDst, smemSrc, bytes);
}
// shared::cta -> global with an element-wise add at the destination (atomic per element).
template <typename T>
MSCCLPP_DEVICE_INLINE void bulkReduceStore(void* gmemDst, const void* smemSrc, uint32_t bytes);
template <>
MSCCLPP_DEVICE_INLINE void bulkReduceStore<float>(void* gmemDst, const void* smemSrc, uint32_t bytes) {
  ptx::bulk_reduce_add_f32(gmemDst, smemSrc, bytes);
}
template <>
MSCCLPP_DEVICE_INLINE void bulkReduceStore<__nv_bfloat16>(void* gmemDst, const void* smemSrc, uint32_t bytes) {
  ptx::bulk_reduce_add_bf16(gmemDst, smemSrc, bytes);
}
template <>
MSCCLPP_DEVICE_INLINE void bulkReduceStore<__half>(void* gmemDst, const void* smemSrc, uint32_t bytes) {
  ptx::bulk_reduce_add_f16(gmemDst, smemSrc, bytes);
}
template <>
MSCCLPP_DEVICE_INLINE void bulkReduceStore<uint32_t>(void* gmemDst, const void* smemSrc, uint32_t bytes) {
  ptx::bulk_reduce_add_u32(gmemDst, smemSrc, bytes);
}
MSCCLPP_DEVICE_INLINE void bulkCommit() { ptx::bulk_commit(); }
// Wait until at most N bulk groups of this thread are pending (writes complete / sources readable).
template <int N = 0>
MSCCLPP_DEVICE_INLINE void bulkWait() {
  ptx::bulk_wait<N>();
}
template <int N = 0>
MSCCLPP_DEVICE_INLINE void bulkWaitRead() {
  ptx::bulk_wait_read<N>();
}
// Make generic-proxy writes to shared memory visible to the async proxy before a bulkStore reads them.
MSCCLPP_DEVICE_INLINE void bulkFenceSmem() { ptx::fence_proxy_async_smem(); }

// Names of the reference for the four calls above (include/mscclpp/bulk_device.hpp:242-272).
MSCCLPP_DEVICE_INLINE void bulkFence() { bulkFenceSmem(); }
MSCCLPP_DEVICE_INLINE void bulkStoreCommit() { bulkCommit(); }
template <uint32_t PendingGroups = 0>
MSCCLPP_DEVICE_INLINE void bulkStoreWait() {
  ptx::bulk_wait<static_cast<int>(PendingGroups)>();
}
template <uint32_t PendingGroups = 0>
MSCCLPP_DEVICE_INLINE void bulkStoreWaitSource() {
  ptx::bulk_wait_read<static_cast<int>(PendingGroups)>();
}

#endif  // __CUDACC__

}  // namespace mscclpp
