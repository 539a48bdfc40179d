#include <mscclpp/switch_channel.hpp>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <unistd.h>

#include <mscclpp/gpu_utils.hpp>

#include "cuda_driver.hpp"
#include "logger.hpp"
#include "range_allocator.hpp"
#include "unix_socket.hpp"

namespace mscclpp {

struct NvlsConnection::Impl {
  std::shared_ptr<Communicator> comm;
  std::vector<int> ranks;
  int deviceId = 0;
  size_t capacity = 0;      // usable bytes (excludes the barrier granule)
  size_t granularity = 0;
  CUmemGenericAllocationHandle mcHandle = 0;
  CUdeviceptr mcVa = 0;     // multicast mapping of the whole object
  size_t mapped = 0;
  RangeAllocator ranges;    // offsets of the object: a range goes back when the last copy of its SwitchChannel is gone
  std::mutex mutex;
  struct Binding {
    size_t offset;
    size_t size;
  };
  std::vector<Binding> bindings;  // what is bound right now (the barrier granule included)
  // group barrier: one granule of this rank's own memory bound at the end of the object
  void* barrierMem = nullptr;
  std::shared_ptr<uint64_t> barrierExpected;
};

NvlsConnection::NvlsConnection(std::unique_ptr<Impl> impl) : pimpl_(std::move(impl)) {}

NvlsConnection::~NvlsConnection() {
  const CudaDriver* drv = CudaDriver::tryGet();
  if (!drv || !pimpl_) return;
  (void)cudaDeviceSynchronize();
  CUdevice dev;
  if (drv->cuDeviceGet(&dev, pimpl_->deviceId) != CUDA_SUCCESS) return;
  if (pimpl_->mcVa) {
    (void)drv->cuMemUnmap(pimpl_->mcVa, pimpl_->mapped);
    (void)drv->cuMemAddressFree(pimpl_->mcVa, pimpl_->mapped);
  }
  for (auto& b : pimpl_->bindings) (void)drv->cuMulticastUnbind(pimpl_->mcHandle, dev, b.offset, b.size);
  if (pimpl_->mcHandle) (void)drv->cuMemRelease(pimpl_->mcHandle);
  if (pimpl_->barrierMem) detail::gpuFreePhysical(pimpl_->barrierMem);
}

size_t NvlsConnection::getMultiCastMinGranularity() { return detail::physicalGranularity(true); }
size_t NvlsConnection::capacity() const { return pimpl_->capacity; }
int NvlsConnection::groupSize() const { return static_cast<int>(pimpl_->ranks.size()); }

SwitchChannel NvlsConnection::bindAllocatedMemory(void* devicePtr, size_t size) {
  const CudaDriver& drv = CudaDriver::get();
  Impl& s = *pimpl_;
  if (!isCuMemMapAllocated(devicePtr)) {
    throw Error("bindAllocatedMemory needs memory from the VMM path (GpuBuffer / gpuCallocPhysical / SymmetricHeap)",
                ErrorCode::InvalidUsage);
  }
  const size_t g = s.granularity;
  if ((reinterpret_cast<uintptr_t>(devicePtr) % g) != 0 || (size % g) != 0) {
    throw Error("bindAllocatedMemory: pointer and size must be multiples of the multicast granularity (" + std::to_string(g) + ")",
                ErrorCode::InvalidUsage);
  }
  size_t offset;
  {
    std::lock_guard<std::mutex> lock(s.mutex);
    offset = s.ranges.allocate(size);
    if (offset == RangeAllocator::npos) {
      throw Error("multicast object has no free range of " + std::to_string(size) + " bytes (" + std::to_string(s.ranges.bytesFree()) +
                      " bytes free, largest piece " + std::to_string(s.ranges.largestFree()) + ")",
                  ErrorCode::InvalidUsage);
    }
  }
  CUresult res = drv.cuMulticastBindAddr(s.mcHandle, offset, reinterpret_cast<CUdeviceptr>(devicePtr), size, 0);
  if (res != CUDA_SUCCESS) {
    std::lock_guard<std::mutex> lock(s.mutex);
    s.ranges.release(offset);
    MSCCLPP_CUTHROW(res);
  }
  {
    std::lock_guard<std::mutex> lock(s.mutex);
    s.bindings.push_back({offset, size});
  }
  // nobody may touch the multicast alias before every member has bound its part
  s.comm->bootstrap()->groupBarrier(s.ranks);
  // The range is unbound and handed back when the last copy of the channel is destroyed. Members have to drop their
  // channels in the same order as well, or their next bindings land at different offsets.
  std::weak_ptr<NvlsConnection> weak = weak_from_this();
  const int deviceId = s.deviceId;
  std::shared_ptr<void> token(nullptr, [weak, offset, size, deviceId](void*) {
    auto conn = weak.lock();
    if (!conn) return;  // the connection went first and has released everything
    const CudaDriver* d = CudaDriver::tryGet();
    if (d == nullptr) return;
    NvlsConnection::Impl& impl = *conn->impl();
    (void)cudaDeviceSynchronize();  // nothing in flight may still use the alias
    CUdevice dev;
    if (d->cuDeviceGet(&dev, deviceId) == CUDA_SUCCESS) (void)d->cuMulticastUnbind(impl.mcHandle, dev, offset, size);
    std::lock_guard<std::mutex> lock(impl.mutex);
    for (auto it = impl.bindings.begin(); it != impl.bindings.end(); ++it) {
      if (it->offset == offset) {
        impl.bindings.erase(it);
        break;
      }
    }
    impl.ranges.release(offset);
  });
  return SwitchChannel(devicePtr, reinterpret_cast<void*>(s.mcVa + offset), size, shared_from_this(), std::move(token));
}

SwitchChannel::DeviceHandle SwitchChannel::deviceHandle() const {
  DeviceHandle h{};
  h.devicePtr = devicePtr_;
  h.mcPtr = mcPtr_;
  h.bufferSize = bufferSize_;
  if (connection_) {
    NvlsConnection::Impl* s = connection_->impl();
    h.barrier.counter = static_cast<uint64_t*>(s->barrierMem);
    h.barrier.counterMc = reinterpret_cast<uint64_t*>(s->mcVa + s->capacity);
    h.barrier.expected = s->barrierExpected.get();
    h.barrier.groupSize = static_cast<int>(s->ranks.size());
  }
  return h;
}

namespace {
struct McAdvert {
  char serverName[96];
  uint32_t fdId;
  uint32_t ok;
  uint64_t totalSize;
};
constexpr int kNvlsTag = 0x7ffd0001;
}  // namespace

std::shared_ptr<NvlsConnection> connectNvlsCollective(std::shared_ptr<Communicator> communicator, std::vector<int> allRanks,
                                                      size_t bufferSize) {
  if (!isNvlsSupported()) throw Error("NVLS (multicast) is not supported or disabled on this device", ErrorCode::InvalidUsage);
  const CudaDriver& drv = CudaDriver::get();
  AvoidCudaGraphCaptureGuard guard;
  auto bootstrap = communicator->bootstrap();
  const int me = bootstrap->getRank();
  if (std::find(allRanks.begin(), allRanks.end(), me) == allRanks.end()) {
    throw Error("connectNvlsCollective: the calling rank is not in the group", ErrorCode::InvalidUsage);
  }
  auto impl = std::make_unique<NvlsConnection::Impl>();
  impl->comm = communicator;
  impl->ranks = allRanks;
  MSCCLPP_CUDATHROW(cudaGetDevice(&impl->deviceId));
  MSCCLPP_CUDATHROW(cudaFree(nullptr));
  const size_t g = detail::physicalGranularity(true);
  impl->granularity = g;
  impl->capacity = (bufferSize + g - 1) / g * g;
  impl->ranges.reset(impl->capacity, g);
  const size_t total = impl->capacity + g;  // + one granule for the group barrier word
  const int root = allRanks[0];

  CUmulticastObjectProp prop{};
  prop.numDevices = static_cast<unsigned>(allRanks.size());
  prop.size = total;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  McAdvert ad{};
  UnixFdServer& server = UnixFdServer::instance();
  if (me == root) {
    MSCCLPP_CUTHROW(drv.cuMulticastCreate(&impl->mcHandle, &prop));
    int fd = -1;
    MSCCLPP_CUTHROW(drv.cuMemExportToShareableHandle(&fd, impl->mcHandle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    std::strncpy(ad.serverName, server.name().c_str(), sizeof(ad.serverName) - 1);
    ad.fdId = server.registerFd(fd);
    ad.ok = 1;
    ad.totalSize = total;
    ::close(fd);
    for (int r : allRanks)
      if (r != root) bootstrap->send(&ad, sizeof(ad), r, kNvlsTag);
  } else {
    bootstrap->recv(&ad, sizeof(ad), root, kNvlsTag);
    int fd = requestFdFromPeer(ad.serverName, ad.fdId);
    CUresult res = drv.cuMemImportFromShareableHandle(&impl->mcHandle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                      CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
    MSCCLPP_CUTHROW(res);
  }
  CUdevice dev;
  MSCCLPP_CUTHROW(drv.cuDeviceGet(&dev, impl->deviceId));
  MSCCLPP_CUTHROW(drv.cuMulticastAddDevice(impl->mcHandle, dev));
  bootstrap->groupBarrier(allRanks);  // all devices added: binding becomes legal
  if (me == root) server.unregisterFd(ad.fdId);

  // barrier word: a granule of my own memory bound at the tail of the object
  impl->barrierMem = detail::gpuCallocPhysical(g, g);
  MSCCLPP_CUTHROW(drv.cuMulticastBindAddr(impl->mcHandle, impl->capacity, reinterpret_cast<CUdeviceptr>(impl->barrierMem), g, 0));
  impl->bindings.push_back({impl->capacity, g});
  impl->barrierExpected = gpuCallocShared<uint64_t>();

  MSCCLPP_CUTHROW(drv.cuMemAddressReserve(&impl->mcVa, total, g, 0, 0));
  MSCCLPP_CUTHROW(drv.cuMemMap(impl->mcVa, total, 0, impl->mcHandle, 0));
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = impl->deviceId;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  MSCCLPP_CUTHROW(drv.cuMemSetAccess(impl->mcVa, total, &access, 1));
  impl->mapped = total;
  bootstrap->groupBarrier(allRanks);
  LOG_INFO(LogSubsys::GPU, "NVLS connection: ", allRanks.size(), " ranks, ", impl->capacity >> 20, " MiB bindable");
  return std::make_shared<NvlsConnection>(std::move(impl));
}

}  // namespace mscclpp
