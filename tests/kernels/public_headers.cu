// Compile check: the device-side public headers can be included together in one translation unit and their templates
// instantiate for sm_100a. Never launched.
#include <mscclpp/assert_device.hpp>
#include <mscclpp/atomic_device.hpp>
#include <mscclpp/device.hpp>
#include <mscclpp/gpu.hpp>
#include <mscclpp/version.hpp>

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
