// RegisteredMemory and the IPC handles beneath it (reference: src/core/registered_memory.cc:35-187,
// src/core/gpu_ipc_mem.cc:256-506).
#include "registered_memory.hpp"

#include <cstring>
#include <map>
#include <unistd.h>

#include <mscclpp/gpu_utils.hpp>

#include "cuda_driver.hpp"
#include "logger.hpp"
#include "serialize.hpp"
#include "unix_socket.hpp"

namespace mscclpp {

// ------------------------------------------------------------------------------------------ GpuIpcMemHandle
GpuIpcMemHandle GpuIpcMemHandle::create(void* ptr, size_t size) {
  GpuIpcMemHandle h;
  cudaPointerAttributes attr{};
  cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
  if (e != cudaSuccess || attr.type == cudaMemoryTypeUnregistered || attr.type == cudaMemoryTypeHost) {
    (void)cudaGetLastError();
    h.kinds = kHost;
    h.baseAddr = reinterpret_cast<uint64_t>(ptr);
    h.allocSize = size;
    return h;
  }
  h.deviceId = attr.device;
  CudaDeviceGuard onOwner(attr.device);  // the driver queries below want the owning device's context current
  const CudaDriver& drv = CudaDriver::get();
  CUdeviceptr base = 0;
  size_t allocSize = 0;
  MSCCLPP_CUTHROW(drv.cuMemGetAddressRange(&base, &allocSize, reinterpret_cast<CUdeviceptr>(ptr)));
  h.baseAddr = base;
  h.allocSize = allocSize;
  h.offset = reinterpret_cast<uint64_t>(ptr) - base;
  CUmemGenericAllocationHandle vmm;
  if (drv.cuMemRetainAllocationHandle(&vmm, reinterpret_cast<void*>(base)) == CUDA_SUCCESS) {
    if (detail::fabricHandlesWanted()) {
      static_assert(sizeof(CUmemFabricHandle) == sizeof(h.fabric), "fabric handle size");
      // succeeds only for allocations that were created exportable as fabric handles (gpuCallocPhysical does that)
      if (drv.cuMemExportToShareableHandle(h.fabric, vmm, CU_MEM_HANDLE_TYPE_FABRIC, 0) == CUDA_SUCCESS) h.kinds |= kFabric;
    }
    int fd = -1;
    CUresult r = drv.cuMemExportToShareableHandle(&fd, vmm, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    (void)drv.cuMemRelease(vmm);
    if (r == CUDA_SUCCESS) {
      UnixFdServer& server = UnixFdServer::instance();
      std::strncpy(h.fdServer, server.name().c_str(), sizeof(h.fdServer) - 1);
      h.fdId = server.registerFd(fd);
      ::close(fd);
      h.kinds |= kPosixFd;
    }
  } else {
    cudaError_t ie = cudaIpcGetMemHandle(&h.runtimeIpc, reinterpret_cast<void*>(base));
    if (ie == cudaSuccess) {
      h.kinds |= kRuntimeIpc;
    } else {
      (void)cudaGetLastError();
      LOG_WARN(LogSubsys::GPU, "cudaIpcGetMemHandle failed for ", ptr, ": the memory can only be used inside this process");
    }
  }
  return h;
}

GpuIpcMapping::GpuIpcMapping(const GpuIpcMemHandle& h) {
  AvoidCudaGraphCaptureGuard guard;
  if (h.kinds & (GpuIpcMemHandle::kPosixFd | GpuIpcMemHandle::kFabric)) {
    const CudaDriver& drv = CudaDriver::get();
    CUmemGenericAllocationHandle handle;
    bool imported = false;
    if (h.kinds & GpuIpcMemHandle::kFabric) {  // works across the hosts of one NVLink fabric, and inside a host as well
      imported = drv.cuMemImportFromShareableHandle(&handle, const_cast<unsigned char*>(h.fabric), CU_MEM_HANDLE_TYPE_FABRIC) == CUDA_SUCCESS;
    }
    if (!imported) {
      if ((h.kinds & GpuIpcMemHandle::kPosixFd) == 0) throw Error("the fabric handle of this memory could not be imported", ErrorCode::SystemError);
      int fd = requestFdFromPeer(h.fdServer, h.fdId);
      CUresult r = drv.cuMemImportFromShareableHandle(&handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                      CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      ::close(fd);
      MSCCLPP_CUTHROW(r);
    }
    int dev = 0;
    MSCCLPP_CUDATHROW(cudaGetDevice(&dev));
    size_t gran = detail::physicalGranularity(false);
    CUdeviceptr va = 0;
    MSCCLPP_CUTHROW(drv.cuMemAddressReserve(&va, h.allocSize, gran, 0, 0));
    MSCCLPP_CUTHROW(drv.cuMemMap(va, h.allocSize, 0, handle, 0));
    CUmemAccessDesc access{};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = dev;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    MSCCLPP_CUTHROW(drv.cuMemSetAccess(va, h.allocSize, &access, 1));
    base_ = reinterpret_cast<void*>(va);
    size_ = h.allocSize;
    vmm_ = true;
    vmmHandle_ = handle;
  } else if (h.kinds & GpuIpcMemHandle::kRuntimeIpc) {
    MSCCLPP_CUDATHROW(cudaIpcOpenMemHandle(&base_, h.runtimeIpc, cudaIpcMemLazyEnablePeerAccess));
    size_ = h.allocSize;
  } else {
    throw Error("this memory was registered without any handle another process can import", ErrorCode::InvalidUsage);
  }
}

std::shared_ptr<GpuIpcMapping> GpuIpcMapping::acquire(const GpuIpcMemHandle& h) {
  static std::mutex mutex;
  static std::map<std::string, std::weak_ptr<GpuIpcMapping>> cache;
  std::string key;
  if (h.kinds & (GpuIpcMemHandle::kPosixFd | GpuIpcMemHandle::kFabric)) {
    key = std::string("fd:") + h.fdServer + ":" + std::to_string(h.baseAddr) + ":" + std::to_string(h.allocSize);
  } else {
    key = "ipc:" + std::string(reinterpret_cast<const char*>(&h.runtimeIpc), sizeof(h.runtimeIpc));
  }
  std::lock_guard<std::mutex> lock(mutex);
  auto it = cache.find(key);
  if (it != cache.end()) {
    if (auto alive = it->second.lock()) return alive;
  }
  auto fresh = std::make_shared<GpuIpcMapping>(h);
  cache[key] = fresh;
  return fresh;
}

GpuIpcMapping::~GpuIpcMapping() {
  if (base_ == nullptr) return;
  if (vmm_) {
    const CudaDriver* drv = CudaDriver::tryGet();
    if (drv) {
      (void)drv->cuMemUnmap(reinterpret_cast<CUdeviceptr>(base_), size_);
      (void)drv->cuMemAddressFree(reinterpret_cast<CUdeviceptr>(base_), size_);
      (void)drv->cuMemRelease(vmmHandle_);
    }
  } else {
    (void)cudaIpcCloseMemHandle(base_);
  }
}

// ------------------------------------------------------------------------------------------ RegisteredMemory
RegisteredMemory::Impl::~Impl() {
  if (isLocal && registeredFdId != 0) UnixFdServer::instance().unregisterFd(registeredFdId);
}

std::vector<char> RegisteredMemory::Impl::serialize() const {
  Writer w;
  w.put<uint64_t>(reinterpret_cast<uint64_t>(originalDataPtr));
  w.put<uint64_t>(size);
  w.put<uint64_t>(hostHash);
  w.put<uint64_t>(pidHash);
  w.put<uint64_t>(transports.toUlong());
  w.put<uint8_t>(isHostMemory ? 1 : 0);
  w.put<int32_t>(deviceId);
  w.putRaw(&ipc, sizeof(ipc));
  w.put<uint32_t>(static_cast<uint32_t>(ib.size()));
  for (const auto& e : ib) {
    w.put<int32_t>(static_cast<int32_t>(e.transport));
    w.put<uint64_t>(e.info.addr);
    w.put<uint32_t>(e.info.rkey);
  }
  return w.bytes;
}

std::shared_ptr<RegisteredMemory::Impl> RegisteredMemory::Impl::deserialize(const std::vector<char>& data) {
  Reader r(data);
  auto impl = std::make_shared<Impl>();
  impl->originalDataPtr = reinterpret_cast<void*>(r.get<uint64_t>());
  impl->size = r.get<uint64_t>();
  impl->hostHash = r.get<uint64_t>();
  impl->pidHash = r.get<uint64_t>();
  impl->transports = TransportFlags::fromUlong(r.get<uint64_t>());
  impl->isHostMemory = r.get<uint8_t>() != 0;
  impl->deviceId = r.get<int32_t>();
  r.getRaw(&impl->ipc, sizeof(impl->ipc));
  const uint32_t nIb = r.get<uint32_t>();
  for (uint32_t i = 0; i < nIb; i++) {
    IbEntry e;
    e.transport = static_cast<Transport>(r.get<int32_t>());
    e.info.addr = r.get<uint64_t>();
    e.info.rkey = r.get<uint32_t>();
    impl->ib.push_back(std::move(e));
  }
  impl->isLocal = false;
  const bool sameProcess = impl->hostHash == getHostHash() && impl->pidHash == getPidHash();
  if (sameProcess) {
    // self-connections and multi-GPU single-process set-ups: the owner's pointer is usable as is
    impl->data = impl->originalDataPtr;
    if (!impl->isHostMemory && impl->deviceId >= 0) {
      int dev = 0;
      if (cudaGetDevice(&dev) == cudaSuccess && dev != impl->deviceId) {
        // VMM allocations of this process need an explicit access grant; everything else goes through peer access
        (void)detail::gpuGrantAccessPhysical(impl->originalDataPtr, dev);
        cudaError_t e = cudaDeviceEnablePeerAccess(impl->deviceId, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
          (void)cudaGetLastError();
          LOG_WARN(LogSubsys::GPU, "cannot enable peer access from device ", dev, " to ", impl->deviceId);
        } else {
          (void)cudaGetLastError();
        }
      }
    }
  } else if (impl->transports.has(Transport::CudaIpc) && !impl->isHostMemory &&
             (impl->hostHash == getHostHash() || (impl->ipc.kinds & GpuIpcMemHandle::kFabric) != 0)) {
    // this host, or another host of the same NVLink fabric (the handle then carries a fabric export)
    impl->mapping = GpuIpcMapping::acquire(impl->ipc);
    impl->data = static_cast<char*>(impl->mapping->base()) + impl->ipc.offset;
  } else {
    // reachable only through a transport that does not need a local mapping (Ethernet, IB)
    impl->data = nullptr;
  }
  return impl;
}

RegisteredMemory::RegisteredMemory(std::shared_ptr<Impl> pimpl) : pimpl_(std::move(pimpl)) {}
RegisteredMemory::~RegisteredMemory() = default;
void* RegisteredMemory::data() const { return pimpl_->data; }
void* RegisteredMemory::originalDataPtr() const { return pimpl_->originalDataPtr; }
size_t RegisteredMemory::size() const { return pimpl_->size; }
TransportFlags RegisteredMemory::transports() const { return pimpl_->transports; }
bool RegisteredMemory::isLocal() const { return pimpl_->isLocal; }
std::vector<char> RegisteredMemory::serialize() const { return pimpl_->serialize(); }
RegisteredMemory RegisteredMemory::deserialize(const std::vector<char>& data) {
  return RegisteredMemory(Impl::deserialize(data));
}

void validateTransport(const RegisteredMemory& mem, Transport transport, uint64_t offset, uint64_t size) {
  if (!mem.transports().has(transport)) {
    throw Error("RegisteredMemory was not registered for transport " + transportToString(transport), ErrorCode::InvalidUsage);
  }
  if (offset + size > mem.size()) {
    throw Error("access [" + std::to_string(offset) + ", " + std::to_string(offset + size) + ") exceeds the registered size " +
                    std::to_string(mem.size()),
                ErrorCode::InvalidUsage);
  }
}

}  // namespace mscclpp
