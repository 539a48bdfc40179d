#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/utils.hpp>

#include <cstdlib>

#include <cstring>
#include <map>
#include <mutex>

#include <mscclpp/env.hpp>

#include "cuda_driver.hpp"
#include "logger.hpp"

namespace mscclpp {

// ------------------------------------------------------------------------------------------ driver table
namespace {

template <typename Fn>
bool resolve(Fn& slot, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      p == nullptr) {
    (void)cudaGetLastError();
    return false;
  }
  slot = reinterpret_cast<Fn>(p);
  return true;
}

CudaDriver* loadDriver() {
  static CudaDriver table{};
  bool ok = true;
#define MSCCLPP_RESOLVE(name) ok = resolve(table.name, #name) && ok
  MSCCLPP_RESOLVE(cuMemCreate);
  MSCCLPP_RESOLVE(cuMemRelease);
  MSCCLPP_RESOLVE(cuMemAddressReserve);
  MSCCLPP_RESOLVE(cuMemAddressFree);
  MSCCLPP_RESOLVE(cuMemMap);
  MSCCLPP_RESOLVE(cuMemUnmap);
  MSCCLPP_RESOLVE(cuMemSetAccess);
  MSCCLPP_RESOLVE(cuMemGetAllocationGranularity);
  MSCCLPP_RESOLVE(cuMemExportToShareableHandle);
  MSCCLPP_RESOLVE(cuMemImportFromShareableHandle);
  MSCCLPP_RESOLVE(cuMemRetainAllocationHandle);
  MSCCLPP_RESOLVE(cuMemGetAddressRange);
  MSCCLPP_RESOLVE(cuMulticastCreate);
  MSCCLPP_RESOLVE(cuMulticastAddDevice);
  MSCCLPP_RESOLVE(cuMulticastBindMem);
  MSCCLPP_RESOLVE(cuMulticastBindAddr);
  MSCCLPP_RESOLVE(cuMulticastUnbind);
  MSCCLPP_RESOLVE(cuMulticastGetGranularity);
  MSCCLPP_RESOLVE(cuDeviceGet);
  MSCCLPP_RESOLVE(cuDeviceGetAttribute);
  MSCCLPP_RESOLVE(cuPointerGetAttribute);
  MSCCLPP_RESOLVE(cuGetErrorString);
  MSCCLPP_RESOLVE(cuModuleLoadData);
  MSCCLPP_RESOLVE(cuModuleUnload);
  MSCCLPP_RESOLVE(cuModuleGetFunction);
  MSCCLPP_RESOLVE(cuFuncSetAttribute);
  MSCCLPP_RESOLVE(cuLaunchKernel);
  MSCCLPP_RESOLVE(cuLaunchCooperativeKernel);
#undef MSCCLPP_RESOLVE
  if (!resolve(table.cuMemGetHandleForAddressRange, "cuMemGetHandleForAddressRange")) table.cuMemGetHandleForAddressRange = nullptr;
  return ok ? &table : nullptr;
}

}  // namespace

const CudaDriver* CudaDriver::tryGet() {
  static const CudaDriver* table = loadDriver();
  return table;
}

const CudaDriver& CudaDriver::get() {
  const CudaDriver* t = tryGet();
  if (t == nullptr) throw Error("the CUDA driver API is not available in this process", ErrorCode::SystemError);
  return *t;
}

// ------------------------------------------------------------------------------------------ guards / streams
AvoidCudaGraphCaptureGuard::AvoidCudaGraphCaptureGuard() : mode_(cudaStreamCaptureModeRelaxed), active_(true) {
  if (cudaThreadExchangeStreamCaptureMode(&mode_) != cudaSuccess) {
    (void)cudaGetLastError();
    active_ = false;
  }
}
AvoidCudaGraphCaptureGuard::~AvoidCudaGraphCaptureGuard() {
  if (active_) (void)cudaThreadExchangeStreamCaptureMode(&mode_);
}

CudaDeviceGuard::CudaDeviceGuard(int deviceId) : previous_(-1) {
  if (deviceId < 0) return;
  MSCCLPP_CUDATHROW(cudaGetDevice(&previous_));
  if (previous_ != deviceId) MSCCLPP_CUDATHROW(cudaSetDevice(deviceId));
  else previous_ = -1;
}
CudaDeviceGuard::~CudaDeviceGuard() {
  if (previous_ >= 0) (void)cudaSetDevice(previous_);
}

CudaStreamWithFlags::CudaStreamWithFlags(unsigned int flags) : stream_(nullptr), flags_(flags) {
  MSCCLPP_CUDATHROW(cudaStreamCreateWithFlags(&stream_, flags));
}
CudaStreamWithFlags::~CudaStreamWithFlags() {
  if (stream_) (void)cudaStreamDestroy(stream_);
}
void CudaStreamWithFlags::set(unsigned int flags) {
  if (stream_) throw Error("CudaStreamWithFlags already holds a stream", ErrorCode::InvalidUsage);
  flags_ = flags;
  MSCCLPP_CUDATHROW(cudaStreamCreateWithFlags(&stream_, flags));
}

std::shared_ptr<CudaStreamWithFlags> GpuStreamPool::getStream() {
  std::shared_ptr<CudaStreamWithFlags> s;
  if (!free_.empty()) {
    s = free_.back();
    free_.pop_back();
  } else {
    s = std::make_shared<CudaStreamWithFlags>(cudaStreamNonBlocking);
  }
  // returns itself to the pool when the last user drops it
  CudaStreamWithFlags* raw = s.get();
  auto keeper = s;
  return std::shared_ptr<CudaStreamWithFlags>(raw, [this, keeper](CudaStreamWithFlags*) mutable {
    free_.push_back(keeper);
  });
}
void GpuStreamPool::clear() { free_.clear(); }
std::shared_ptr<GpuStreamPool> gpuStreamPool() {
  static std::shared_ptr<GpuStreamPool> pool = std::make_shared<GpuStreamPool>();
  return pool;
}

// ------------------------------------------------------------------------------------------ allocation
namespace {

struct PhysicalAlloc {
  CUmemGenericAllocationHandle handle;
  size_t bytes;
};
std::mutex physMutex;
std::map<void*, PhysicalAlloc> physAllocs;

// One set-up stream per (thread, device): a stream belongs to the device that was current when it was made.
cudaStream_t setupStream() {
  static thread_local std::map<int, cudaStream_t> streams;
  int dev = 0;
  MSCCLPP_CUDATHROW(cudaGetDevice(&dev));
  cudaStream_t& s = streams[dev];
  if (s == nullptr) MSCCLPP_CUDATHROW(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  return s;
}

CUmemAllocationProp physicalProp(int deviceId, bool withFabric = false) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = deviceId;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  if (withFabric) {
    prop.requestedHandleTypes = static_cast<CUmemAllocationHandleType>(CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR | CU_MEM_HANDLE_TYPE_FABRIC);
  }
  return prop;
}

}  // namespace

namespace detail {

bool fabricHandlesWanted() {
  static const bool wanted = [] {
    const char* e = std::getenv("MSCCLPP_FABRIC_HANDLES");
    return e != nullptr && e[0] == '1' && isFabricMemHandleAvailable();
  }();
  return wanted;
}

void* gpuCalloc(size_t bytes) {
  AvoidCudaGraphCaptureGuard guard;
  void* p = nullptr;
  MSCCLPP_CUDATHROW(cudaMalloc(&p, bytes));
  cudaStream_t s = setupStream();
  MSCCLPP_CUDATHROW(cudaMemsetAsync(p, 0, bytes, s));
  MSCCLPP_CUDATHROW(cudaStreamSynchronize(s));
  return p;
}

void* gpuCallocHost(size_t bytes, unsigned flags) {
  AvoidCudaGraphCaptureGuard guard;
  void* p = nullptr;
  MSCCLPP_CUDATHROW(cudaHostAlloc(&p, bytes, flags));
  std::memset(p, 0, bytes);
  return p;
}

size_t physicalGranularity(bool forMulticast) {
  const CudaDriver& drv = CudaDriver::get();
  int dev = 0;
  MSCCLPP_CUDATHROW(cudaGetDevice(&dev));
  CUmemAllocationProp prop = physicalProp(dev);
  size_t gran = 0;
  MSCCLPP_CUTHROW(drv.cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  if (forMulticast && isNvlsSupported()) {
    CUmulticastObjectProp mp{};
    mp.numDevices = 2;
    mp.size = gran;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (drv.cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
  }
  return gran;
}

size_t multicastGranularity(bool recommended) {
  if (recommended) return physicalGranularity(true);
  const CudaDriver& drv = CudaDriver::get();
  int dev = 0;
  MSCCLPP_CUDATHROW(cudaGetDevice(&dev));
  CUmemAllocationProp prop = physicalProp(dev);
  size_t gran = 0;
  MSCCLPP_CUTHROW(drv.cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM));
  if (isNvlsSupported()) {
    CUmulticastObjectProp mp{};
    mp.numDevices = 2;
    mp.size = gran;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (drv.cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS && mg > gran) gran = mg;
  }
  return gran;
}

void* gpuCallocPhysical(size_t bytes, size_t granularity) {
  AvoidCudaGraphCaptureGuard guard;
  const CudaDriver& drv = CudaDriver::get();
  int dev = 0;
  MSCCLPP_CUDATHROW(cudaGetDevice(&dev));
  MSCCLPP_CUDATHROW(cudaFree(nullptr));  // make sure the primary context exists
  if (granularity == 0) granularity = physicalGranularity(true);
  const size_t rounded = (bytes + granularity - 1) / granularity * granularity;
  CUmemAllocationProp prop = physicalProp(dev);
  CUmemGenericAllocationHandle handle;
  // Multi-node NVLink: memory that other nodes of the fabric may import has to be created exportable as a fabric handle
  // (it needs the IMEX service; without it the creation fails and the allocation stays node-local).
  bool created = false;
  if (fabricHandlesWanted()) {
    CUmemAllocationProp fabricProp = physicalProp(dev, true);
    created = drv.cuMemCreate(&handle, rounded, &fabricProp, 0) == CUDA_SUCCESS;
  }
  if (!created) MSCCLPP_CUTHROW(drv.cuMemCreate(&handle, rounded, &prop, 0));
  CUdeviceptr va = 0;
  MSCCLPP_CUTHROW(drv.cuMemAddressReserve(&va, rounded, granularity, 0, 0));
  MSCCLPP_CUTHROW(drv.cuMemMap(va, rounded, 0, handle, 0));
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = dev;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  MSCCLPP_CUTHROW(drv.cuMemSetAccess(va, rounded, &access, 1));
  void* p = reinterpret_cast<void*>(va);
  cudaStream_t s = setupStream();
  MSCCLPP_CUDATHROW(cudaMemsetAsync(p, 0, rounded, s));
  MSCCLPP_CUDATHROW(cudaStreamSynchronize(s));
  std::lock_guard<std::mutex> lock(physMutex);
  physAllocs[p] = PhysicalAlloc{handle, rounded};
  return p;
}

void gpuFree(void* ptr) {
  if (ptr == nullptr) return;
  AvoidCudaGraphCaptureGuard guard;
  (void)cudaFree(ptr);
}

void gpuFreeHost(void* ptr) {
  if (ptr == nullptr) return;
  AvoidCudaGraphCaptureGuard guard;
  (void)cudaFreeHost(ptr);
}

bool gpuGrantAccessPhysical(const void* ptr, int dev) {
  std::lock_guard<std::mutex> lock(physMutex);
  auto it = physAllocs.upper_bound(const_cast<void*>(ptr));
  if (it == physAllocs.begin()) return false;
  --it;
  const char* base = static_cast<const char*>(it->first);
  if (static_cast<const char*>(ptr) >= base + it->second.bytes) return false;
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = dev;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  MSCCLPP_CUTHROW(CudaDriver::get().cuMemSetAccess(reinterpret_cast<CUdeviceptr>(base), it->second.bytes, &access, 1));
  return true;
}

void gpuFreePhysical(void* ptr) {
  if (ptr == nullptr) return;
  AvoidCudaGraphCaptureGuard guard;
  PhysicalAlloc a{};
  {
    std::lock_guard<std::mutex> lock(physMutex);
    auto it = physAllocs.find(ptr);
    if (it == physAllocs.end()) return;
    a = it->second;
    physAllocs.erase(it);
  }
  const CudaDriver* drv = CudaDriver::tryGet();
  if (!drv) return;
  (void)drv->cuMemUnmap(reinterpret_cast<CUdeviceptr>(ptr), a.bytes);
  (void)drv->cuMemAddressFree(reinterpret_cast<CUdeviceptr>(ptr), a.bytes);
  (void)drv->cuMemRelease(a.handle);
}

}  // namespace detail

void gpuMemcpyAsync(void* dst, const void* src, size_t bytes, cudaStream_t stream, cudaMemcpyKind kind) {
  MSCCLPP_CUDATHROW(cudaMemcpyAsync(dst, src, bytes, kind, stream));
}

void gpuMemset(void* ptr, int value, size_t bytes) {
  AvoidCudaGraphCaptureGuard guard;
  cudaStream_t s = setupStream();
  MSCCLPP_CUDATHROW(cudaMemsetAsync(ptr, value, bytes, s));
  MSCCLPP_CUDATHROW(cudaStreamSynchronize(s));
}

void gpuMemcpy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind) {
  AvoidCudaGraphCaptureGuard guard;
  cudaStream_t s = setupStream();
  MSCCLPP_CUDATHROW(cudaMemcpyAsync(dst, src, bytes, kind, s));
  MSCCLPP_CUDATHROW(cudaStreamSynchronize(s));
}

// ------------------------------------------------------------------------------------------ probes
bool isNvlsSupported() {
  static int cached = -1;
  if (cached >= 0) return cached == 1;
  cached = 0;
  if (env()->forceDisableNvls) return false;
  const CudaDriver* drv = CudaDriver::tryGet();
  int count = 0;
  if (!drv || cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    (void)cudaGetLastError();
    return false;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  CUdevice cuDev;
  int supported = 0;
  if (drv->cuDeviceGet(&cuDev, dev) == CUDA_SUCCESS &&
      drv->cuDeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cuDev) == CUDA_SUCCESS && supported) {
    cached = 1;
  }
  return cached == 1;
}

bool isBulkSupported() {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return major >= 9;
}

bool isFp8MultimemSupported() {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return major == 10 && isNvlsSupported();  // this library is only ever built for sm_100a
}

bool isCuMemMapAllocated(void* ptr) {
  const CudaDriver* drv = CudaDriver::tryGet();
  if (!drv || ptr == nullptr) return false;
  CUmemGenericAllocationHandle handle;
  if (drv->cuMemRetainAllocationHandle(&handle, ptr) != CUDA_SUCCESS) return false;
  (void)drv->cuMemRelease(handle);
  return true;
}

}  // namespace mscclpp
