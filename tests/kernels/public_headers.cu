// Compile check: the device-side public headers can be included together in one translation unit and their templates
// instantiate for sm_100a. Never launched.
#include <mscclpp/assert_device.hpp>
#include <mscclpp/atomic_device.hpp>
#include <mscclpp/device.hpp>
#include <mscclpp/gpu.hpp>
#include <mscclpp/version.hpp>
#include <mscclpp/bulk_device.hpp>
#include <mscclpp/copy_device.hpp>
#include <mscclpp/packet_device.hpp>
#include <mscclpp/semaphore_device.hpp>

#if !defined(MSCCLPP_DEVICE_CUDA) || !defined(CUDA_NVLS_API_AVAILABLE)
#error "device.hpp / gpu.hpp must define their capability macros under nvcc"
#endif

__global__ void touch(unsigned long long* word, int* out) {
  MSCCLPP_ASSERT_DEVICE(word != nullptr, "word must be set");
  mscclpp::atomicStore(word, 1ull, mscclpp::memoryOrderRelaxed);
  const unsigned long long before = mscclpp::atomicFetchAdd<unsigned long long, mscclpp::scopeDevice>(word, 2ull, mscclpp::memoryOrderRelease);
  const unsigned long long now = mscclpp::atomicLoad(word, mscclpp::memoryOrderAcquire);
  *out = static_cast<int>(before + now) + MSCCLPP_VERSION + MSCCLPP_WARP_SIZE;
}

// reference-named members of the bulk-copy and semaphore device API
__global__ void names(mscclpp::MemoryDevice2DeviceSemaphoreDeviceHandle sem, mscclpp::Host2DeviceSemaphoreDeviceHandle h2d, char* gmem,
                      unsigned long long* out) {
  __shared__ mscclpp::BulkBarrier bar;
  __shared__ alignas(128) char tile[256];
  if (threadIdx.x == 0) {
    bar.relaxedInit(1);
    mscclpp::bulkFence();
    if (mscclpp::bulkAligned(gmem) && mscclpp::bulkAligned(tile) && bar.addr() != 0) {
      bar.expect(128);
      mscclpp::bulkLoad(tile, gmem, 128, bar);
      bar.arriveAndExpect(128);
      mscclpp::bulkLoad(tile + 128, gmem + 128, 128, bar);
      if (bar.wait(0, nullptr, 1000000ull) && bar.poll(0)) {
        mscclpp::bulkStore(gmem + 256, tile, 256);
        mscclpp::bulkStoreCommit();
        mscclpp::bulkStoreWaitSource<0>();
        mscclpp::bulkStoreWait<0>();
      }
    }
    out[0] = sem.loadInbound() + sem.loadInboundRelaxed() + sem.loadExpectedInbound() + sem.incExpectedInbound();
    out[1] = h2d.loadInbound() + h2d.loadExpectedInbound();
  }
}

__global__ void copies(float* a, float* b, void* c, void* d, unsigned long long bytes) {
  mscclpp::copy(a, b, bytes / 4, threadIdx.x, blockDim.x);
  mscclpp::copy(c, d, bytes, threadIdx.x, blockDim.x);
  mscclpp::copy<4, false>(c, d, bytes, threadIdx.x, blockDim.x);
}

__global__ void packets(mscclpp::LL16Packet* p16, mscclpp::LL8Packet* p8, unsigned* out) {
  uint2 a;
  unsigned b;
  out[0] = p16->readOnce(1u, a) ? 0u : a.x;
  out[1] = p8->readOnce(1u, b) ? 0u : b;
}
