// GPU memory and stream helpers: RAII guards, plain / host-pinned / VMM ("physical") allocation,
// GpuBuffer<T>, stream pool, capability probes. Covers the reference's include/mscclpp/gpu_utils.hpp
// (41-409) for CUDA on Blackwell; there is no HIP alias layer because this library targets one GPU.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>
#include <memory>
#include <vector>

#include "errors.hpp"

namespace mscclpp {

// Switches the thread to relaxed stream-capture mode for its lifetime, so that set-up calls made
// while another thread captures a CUDA graph do not invalidate the capture.
struct AvoidCudaGraphCaptureGuard {
  AvoidCudaGraphCaptureGuard();
  ~AvoidCudaGraphCaptureGuard();
  cudaStreamCaptureMode mode_;
  bool active_;
};

// Makes `deviceId` current for its lifetime and restores the previous device afterwards.
struct CudaDeviceGuard {
  explicit CudaDeviceGuard(int deviceId);
  ~CudaDeviceGuard();
  int previous_;
};

class CudaStreamWithFlags {
 public:
  CudaStreamWithFlags() : stream_(nullptr), flags_(0) {}
  explicit CudaStreamWithFlags(unsigned int flags);
  ~CudaStreamWithFlags();
  CudaStreamWithFlags(const CudaStreamWithFlags&) = delete;
  CudaStreamWithFlags& operator=(const CudaStreamWithFlags&) = delete;
  void set(unsigned int flags);
  bool empty() const { return stream_ == nullptr; }
  operator cudaStream_t() const { return stream_; }

 private:
  cudaStream_t stream_;
  unsigned int flags_;
};

// Hands out non-blocking streams and takes them back; streams are created on demand.
class GpuStreamPool {
 public:
  std::shared_ptr<CudaStreamWithFlags> getStream();
  void clear();

 private:
  std::vector<std::shared_ptr<CudaStreamWithFlags>> free_;
};
std::shared_ptr<GpuStreamPool> gpuStreamPool();

namespace detail {
void* gpuCalloc(size_t bytes);                       // cudaMalloc + zero
void* gpuCallocHost(size_t bytes, unsigned flags);   // cudaHostAlloc + zero
// cuMemCreate + reserve + map on the current device; exportable as POSIX fd (and multicast-bindable).
// `bytes` is rounded up to `granularity` (0 = recommended multicast/allocation granularity).
void* gpuCallocPhysical(size_t bytes, size_t granularity = 0);
void gpuFree(void* ptr);
void gpuFreeHost(void* ptr);
void gpuFreePhysical(void* ptr);
// If `ptr` lies inside an allocation of gpuCallocPhysical made by this process, give device `dev` read/write access
// to it (VMM allocations are not covered by cudaDeviceEnablePeerAccess). Returns false for other memory.
bool gpuGrantAccessPhysical(const void* ptr, int dev);
size_t physicalGranularity(bool forMulticast);
// MSCCLPP_FABRIC_HANDLES=1 on a GPU that can export fabric handles (multi-node NVLink); off by default.
bool fabricHandlesWanted();
// Allocation granularity that is also valid for binding to a multicast object: the larger of the device's allocation
// granularity and the multicast granularity, both taken as the driver's minimum or recommended value.
size_t multicastGranularity(bool recommended);
}  // namespace detail

// How a GpuBuffer is rounded so that it can be bound to NVLink multicast (NVLS) later.
enum class GpuBufferGranularity {
  MultiCastMinimum,      // smallest granularity the multicast API accepts: least memory
  MultiCastRecommended,  // the driver's recommended granularity (may be larger)
};

template <class T>
struct GpuDeleter {
  void operator()(void* p) const { detail::gpuFree(p); }
};
template <class T>
struct GpuHostDeleter {
  void operator()(void* p) const { detail::gpuFreeHost(p); }
};
template <class T>
struct GpuPhysicalDeleter {
  void operator()(void* p) const { detail::gpuFreePhysical(p); }
};

template <class T>
std::shared_ptr<T> gpuCallocShared(size_t count = 1) {
  return std::shared_ptr<T>(static_cast<T*>(detail::gpuCalloc(count * sizeof(T))), GpuDeleter<T>());
}
template <class T>
std::unique_ptr<T, GpuDeleter<T>> gpuCallocUnique(size_t count = 1) {
  return std::unique_ptr<T, GpuDeleter<T>>(static_cast<T*>(detail::gpuCalloc(count * sizeof(T))));
}
template <class T>
std::shared_ptr<T> gpuCallocHostShared(size_t count = 1, unsigned flags = cudaHostAllocMapped) {
  return std::shared_ptr<T>(static_cast<T*>(detail::gpuCallocHost(count * sizeof(T), flags)), GpuHostDeleter<T>());
}
template <class T>
std::shared_ptr<T> gpuCallocPhysicalShared(size_t count = 1, size_t granularity = 0) {
  return std::shared_ptr<T>(static_cast<T*>(detail::gpuCallocPhysical(count * sizeof(T), granularity)),
                            GpuPhysicalDeleter<T>());
}

// The remaining members of the allocation family (unique_ptr flavours; "uncached" is ordinary device memory on NVIDIA
// GPUs, where fine-grained coherence needs no special allocation - the name exists for source compatibility with
// include/mscclpp/gpu_utils.hpp:205-300 of the reference).
template <class T>
using UniqueGpuPtr = std::unique_ptr<T, GpuDeleter<T>>;
template <class T>
using UniqueGpuHostPtr = std::unique_ptr<T, GpuHostDeleter<T>>;
template <class T>
using UniqueGpuPhysicalPtr = std::unique_ptr<T, GpuPhysicalDeleter<T>>;
template <class T>
UniqueGpuHostPtr<T> gpuCallocHostUnique(size_t count = 1, unsigned flags = cudaHostAllocMapped) {
  return UniqueGpuHostPtr<T>(static_cast<T*>(detail::gpuCallocHost(count * sizeof(T), flags)));
}
template <class T>
UniqueGpuPhysicalPtr<T> gpuCallocPhysicalUnique(size_t count = 1, size_t granularity = 0) {
  return UniqueGpuPhysicalPtr<T>(static_cast<T*>(detail::gpuCallocPhysical(count * sizeof(T), granularity)));
}
template <class T>
std::shared_ptr<T> gpuCallocUncachedShared(size_t count = 1) {
  return gpuCallocShared<T>(count);
}
template <class T>
UniqueGpuPtr<T> gpuCallocUncachedUnique(size_t count = 1) {
  return gpuCallocUnique<T>(count);
}

// Synchronous copy helpers (cudaMemcpy on a private stream, safe during graph capture elsewhere).
void gpuMemcpy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind = cudaMemcpyDefault);
void gpuMemcpyAsync(void* dst, const void* src, size_t bytes, cudaStream_t stream, cudaMemcpyKind kind = cudaMemcpyDefault);
// Synchronous byte fill on the same private stream.
void gpuMemset(void* ptr, int value, size_t bytes);

bool isNvlsSupported();          // multicast objects available and not disabled by MSCCLPP_FORCE_DISABLE_NVLS
bool isBulkSupported();          // cp.async.bulk available (compute capability >= 9)
bool isCuMemMapAllocated(void* ptr);  // true when ptr comes from the VMM path (multicast-bindable)
bool isFp8MultimemSupported();   // multimem fp8 reductions: sm_100a build running on a cc 10.x device

// Zero-initialised device buffer. Uses the VMM path when NVLS is available so that the memory can be
// bound to a multicast object later.
template <class T = char>
class GpuBuffer {
 public:
  // The default is the recommended granularity (what the NVLS paths of this library are measured with); pass
  // MultiCastMinimum to save memory on many small buffers.
  explicit GpuBuffer(size_t nelems, GpuBufferGranularity granularity = GpuBufferGranularity::MultiCastRecommended)
      : nelems_(nelems), bytes_(nelems * sizeof(T)) {
    if (nelems == 0) return;
    MSCCLPP_CUDATHROW(cudaGetDevice(&deviceId_));
    if (isNvlsSupported()) {
      size_t gran = granularity == GpuBufferGranularity::MultiCastRecommended ? detail::physicalGranularity(true)
                                                                              : detail::multicastGranularity(false);
      bytes_ = (bytes_ + gran - 1) / gran * gran;
      memory_ = gpuCallocPhysicalShared<T>(bytes_ / sizeof(T) + (bytes_ % sizeof(T) ? 1 : 0), gran);
    } else {
      memory_ = gpuCallocShared<T>(nelems);
    }
  }
  size_t nelems() const { return nelems_; }
  size_t bytes() const { return bytes_; }  // allocated bytes (>= nelems * sizeof(T))
  std::shared_ptr<T> memory() { return memory_; }
  T* data() { return memory_.get(); }
  const T* data() const { return memory_.get(); }
  int deviceId() const { return deviceId_; }

 private:
  size_t nelems_;
  size_t bytes_;
  int deviceId_ = -1;
  std::shared_ptr<T> memory_;
};

}  // namespace mscclpp
