#include <mscclpp/symmetric_heap.hpp>

#include <cstring>
#include <vector>
#include <unistd.h>

#include <mscclpp/env.hpp>
#include <mscclpp/gpu_utils.hpp>

#include "cuda_driver.hpp"
#include "logger.hpp"
#include "unix_socket.hpp"

namespace mscclpp {

namespace {

size_t roundUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct FdAdvert {
  char serverName[96];
  uint32_t fdId;
  uint32_t ok;
};

}  // namespace

void SymmetricHeap::initLayout(const Options& options) {
  // [SymmControl | LL scratch: 2 buffers x world x llSlotBytes | arena]
  const size_t ctlBytes = roundUp(sizeof(SymmControl), 4096);
  const size_t llBytes = 2 * static_cast<size_t>(world_) * options.llSlotBytes;
  const size_t auxOff = roundUp(ctlBytes + llBytes, 4096);
  arenaBegin_ = roundUp(auxOff + kAuxFlagBytes, 1u << 20);
  if (arenaBegin_ >= bytes_) throw Error("symmetric heap too small for its control block and LL scratch", ErrorCode::InvalidUsage);
  freeBlocks_.clear();
  usedBlocks_.clear();
  freeBlocks_[arenaBegin_] = bytes_ - arenaBegin_;

  // The error block lives in DEVICE memory: every bounded wait polls its `poisoned` word, and a word in
  // host-mapped memory would turn each poll into a PCIe round trip in the middle of the kernels' hot
  // spin loops. The host reads it with a copy after synchronising.
  statusDev_ = static_cast<DeviceStatus*>(detail::gpuCalloc(sizeof(DeviceStatus)));
  status_ = new DeviceStatus();
  std::memset(status_, 0, sizeof(DeviceStatus));
  std::memset(&comm_, 0, sizeof(comm_));
  for (int r = 0; r < world_; r++) comm_.peerBase[r] = peerBase_[r];
  comm_.mcBase = mcBase_;
  comm_.heapBytes = bytes_;
  comm_.llScratchOff = ctlBytes;
  comm_.llSlotBytes = options.llSlotBytes;
  comm_.auxFlagsOff = auxOff;
  comm_.status = statusDev_;
  int64_t ms = options.timeoutMs >= 0 ? options.timeoutMs : env()->deviceTimeoutMs;
  comm_.timeoutNs = static_cast<uint64_t>(ms) * 1000000ull;
  comm_.rank = emulated_ ? 0 : rank_;
  comm_.world = world_;
}

std::shared_ptr<SymmetricHeap> SymmetricHeap::createEmulated(int world, const Options& options) {
  if (world < 1 || world > kMaxRanks) throw Error("emulated world size out of range", ErrorCode::InvalidUsage);
  std::shared_ptr<SymmetricHeap> h(new SymmetricHeap());
  h->emulated_ = true;
  h->world_ = world;
  h->rank_ = 0;
  MSCCLPP_CUDATHROW(cudaGetDevice(&h->deviceId_));
  size_t bytes = options.bytes ? options.bytes : static_cast<size_t>(env()->heapBytes);
  h->bytes_ = roundUp(bytes, 2u << 20);
  h->emulatedAlloc_ = detail::gpuCalloc(h->bytes_ * world);
  h->vaBase_ = reinterpret_cast<uint64_t>(h->emulatedAlloc_);
  for (int r = 0; r < world; r++) h->peerBase_[r] = h->vaBase_ + static_cast<uint64_t>(r) * h->bytes_;
  h->mcBase_ = 0;
  h->initLayout(options);
  return h;
}

std::shared_ptr<SymmetricHeap> SymmetricHeap::create(std::shared_ptr<Bootstrap> bootstrap, const Options& options) {
  if (!bootstrap) throw Error("SymmetricHeap::create needs a bootstrap", ErrorCode::InvalidUsage);
  const CudaDriver& drv = CudaDriver::get();
  AvoidCudaGraphCaptureGuard guard;
  std::shared_ptr<SymmetricHeap> h(new SymmetricHeap());
  h->bootstrap_ = bootstrap;
  h->rank_ = bootstrap->getRank();
  h->world_ = bootstrap->getNranks();
  if (h->world_ > kMaxRanks) throw Error("SymmetricHeap supports at most 16 ranks", ErrorCode::InvalidUsage);
  if (bootstrap->getNranksPerIpcDomain() != h->world_) {
    throw Error("SymmetricHeap needs all ranks inside one NVLink domain", ErrorCode::InvalidUsage);
  }
  MSCCLPP_CUDATHROW(cudaGetDevice(&h->deviceId_));
  MSCCLPP_CUDATHROW(cudaFree(nullptr));
  const int rank = h->rank_, world = h->world_;

  // NVLS only if every rank supports and wants it
  std::vector<int> nvlsVotes(world, 0);
  nvlsVotes[rank] = (options.enableNvls && isNvlsSupported() && world > 1) ? 1 : 0;
  bootstrap->allGather(nvlsVotes.data(), sizeof(int));
  bool useNvls = true;
  for (int v : nvlsVotes) useNvls = useNvls && (v != 0);

  size_t gran = detail::physicalGranularity(useNvls);
  size_t bytes = options.bytes ? options.bytes : static_cast<size_t>(env()->heapBytes);
  h->bytes_ = roundUp(bytes, gran);

  // ---- local allocation, exported as a POSIX fd
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = h->deviceId_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle local;
  MSCCLPP_CUTHROW(drv.cuMemCreate(&local, h->bytes_, &prop, 0));
  h->localHandle_ = local;
  int localFd = -1;
  MSCCLPP_CUTHROW(drv.cuMemExportToShareableHandle(&localFd, local, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  UnixFdServer& server = UnixFdServer::instance();
  std::vector<FdAdvert> adverts(world);
  std::memset(adverts.data(), 0, sizeof(FdAdvert) * world);
  std::strncpy(adverts[rank].serverName, server.name().c_str(), sizeof(adverts[rank].serverName) - 1);
  adverts[rank].fdId = server.registerFd(localFd);
  adverts[rank].ok = 1;
  ::close(localFd);
  bootstrap->allGather(adverts.data(), sizeof(FdAdvert));

  // ---- one contiguous VA range, slot r = rank r
  CUdeviceptr va = 0;
  MSCCLPP_CUTHROW(drv.cuMemAddressReserve(&va, h->bytes_ * world, gran, 0, 0));
  h->vaBase_ = va;
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = h->deviceId_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int r = 0; r < world; r++) {
    CUmemGenericAllocationHandle handle = local;
    if (r != rank) {
      int fd = requestFdFromPeer(adverts[r].serverName, adverts[r].fdId);
      CUresult res = drv.cuMemImportFromShareableHandle(&handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      ::close(fd);
      MSCCLPP_CUTHROW(res);
      h->peerHandles_[r] = handle;
    }
    const CUdeviceptr slot = va + static_cast<uint64_t>(r) * h->bytes_;
    MSCCLPP_CUTHROW(drv.cuMemMap(slot, h->bytes_, 0, handle, 0));
    MSCCLPP_CUTHROW(drv.cuMemSetAccess(slot, h->bytes_, &access, 1));
    h->peerBase_[r] = slot;
  }
  // zero my heap before anybody can look at it
  MSCCLPP_CUDATHROW(cudaMemset(reinterpret_cast<void*>(h->peerBase_[rank]), 0, h->bytes_));
  MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
  bootstrap->barrier();  // every peer has imported my fd and zeroed its heap
  server.unregisterFd(adverts[rank].fdId);

  // ---- multicast alias
  if (useNvls) {
    CUmulticastObjectProp mp{};
    mp.numDevices = static_cast<unsigned>(world);
    mp.size = h->bytes_;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmemGenericAllocationHandle mc = 0;
    FdAdvert mcAd{};
    if (rank == 0) {
      CUresult res = drv.cuMulticastCreate(&mc, &mp);
      if (res == CUDA_SUCCESS) {
        int fd = -1;
        res = drv.cuMemExportToShareableHandle(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
        if (res == CUDA_SUCCESS) {
          std::strncpy(mcAd.serverName, server.name().c_str(), sizeof(mcAd.serverName) - 1);
          mcAd.fdId = server.registerFd(fd);
          mcAd.ok = 1;
          ::close(fd);
        }
      }
      if (!mcAd.ok) LOG_WARN(LogSubsys::GPU, "multicast object creation failed (CUresult ", static_cast<int>(res), "); NVLS disabled");
    }
    std::vector<FdAdvert> mcAll(world);
    mcAll[rank] = mcAd;
    bootstrap->allGather(mcAll.data(), sizeof(FdAdvert));
    mcAd = mcAll[0];
    int okLocal = mcAd.ok;
    if (okLocal && rank != 0) {
      int fd = requestFdFromPeer(mcAd.serverName, mcAd.fdId);
      CUresult res = drv.cuMemImportFromShareableHandle(&mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      ::close(fd);
      if (res != CUDA_SUCCESS) okLocal = 0;
    }
    if (okLocal) {
      CUdevice cuDev;
      MSCCLPP_CUTHROW(drv.cuDeviceGet(&cuDev, h->deviceId_));
      if (drv.cuMulticastAddDevice(mc, cuDev) != CUDA_SUCCESS) okLocal = 0;
    }
    // binding is only legal once every device has been added; agree on success first
    std::vector<int> oks(world, 0);
    oks[rank] = okLocal;
    bootstrap->allGather(oks.data(), sizeof(int));
    bool allOk = true;
    for (int v : oks) allOk = allOk && (v != 0);
    if (rank == 0 && mcAd.ok) server.unregisterFd(mcAd.fdId);
    if (allOk) {
      MSCCLPP_CUTHROW(drv.cuMulticastBindMem(mc, 0, local, 0, h->bytes_, 0));
      bootstrap->barrier();
      CUdeviceptr mcVa = 0;
      MSCCLPP_CUTHROW(drv.cuMemAddressReserve(&mcVa, h->bytes_, gran, 0, 0));
      MSCCLPP_CUTHROW(drv.cuMemMap(mcVa, h->bytes_, 0, mc, 0));
      MSCCLPP_CUTHROW(drv.cuMemSetAccess(mcVa, h->bytes_, &access, 1));
      h->mcBase_ = mcVa;
      h->mcHandle_ = mc;
      bootstrap->barrier();
    } else if (mc != 0) {
      (void)drv.cuMemRelease(mc);
    }
  }
  h->initLayout(options);
  LOG_INFO(LogSubsys::GPU, "symmetric heap: rank ", rank, "/", world, " ", h->bytes_ >> 20, " MiB per rank, NVLS ",
           h->mcBase_ ? "on" : "off");
  return h;
}

SymmetricHeap::~SymmetricHeap() {
  try {
    destroy();
  } catch (...) {
  }
}

void SymmetricHeap::destroy() {
  if (destroyed_) return;
  destroyed_ = true;
  (void)cudaDeviceSynchronize();
  if (emulated_) {
    detail::gpuFree(emulatedAlloc_);
    emulatedAlloc_ = nullptr;
  } else {
    const CudaDriver* drv = CudaDriver::tryGet();
    if (drv) {
      // nobody may still be issuing multimem or peer accesses when the mappings go away
      if (bootstrap_) {
        try {
          bootstrap_->barrier();
        } catch (...) {
        }
      }
      if (mcBase_) {
        (void)drv->cuMemUnmap(mcBase_, bytes_);
        (void)drv->cuMemAddressFree(mcBase_, bytes_);
        CUdevice cuDev;
        if (drv->cuDeviceGet(&cuDev, deviceId_) == CUDA_SUCCESS) (void)drv->cuMulticastUnbind(mcHandle_, cuDev, 0, bytes_);
        (void)drv->cuMemRelease(mcHandle_);
        mcBase_ = 0;
      }
      if (bootstrap_) {
        try {
          bootstrap_->barrier();
        } catch (...) {
        }
      }
      for (int r = 0; r < world_; r++) {
        if (peerBase_[r]) (void)drv->cuMemUnmap(peerBase_[r], bytes_);
        if (r != rank_ && peerHandles_[r]) (void)drv->cuMemRelease(peerHandles_[r]);
      }
      if (vaBase_) (void)drv->cuMemAddressFree(vaBase_, bytes_ * world_);
      if (localHandle_) (void)drv->cuMemRelease(localHandle_);
    }
  }
  if (statusDev_) detail::gpuFree(statusDev_);
  statusDev_ = nullptr;
  delete status_;
  status_ = nullptr;
}

void* SymmetricHeap::alloc(size_t bytes, size_t alignment) {
  if (bytes == 0) bytes = 1;
  if (alignment < 256) alignment = 256;
  std::lock_guard<std::mutex> lock(allocMutex_);
  for (auto it = freeBlocks_.begin(); it != freeBlocks_.end(); ++it) {
    const size_t off = it->first, size = it->second;
    const size_t aligned = roundUp(off, alignment);
    const size_t need = (aligned - off) + roundUp(bytes, 256);
    if (need > size) continue;
    freeBlocks_.erase(it);
    if (aligned > off) freeBlocks_[off] = aligned - off;
    const size_t end = aligned + roundUp(bytes, 256);
    if (off + size > end) freeBlocks_[end] = off + size - end;
    usedBlocks_[aligned] = end - aligned;
    return reinterpret_cast<void*>(peerBase_[rank_] + aligned);
  }
  throw Error("symmetric heap exhausted (" + std::to_string(bytes) + " bytes requested); raise MSCCLPP_HEAP_BYTES",
              ErrorCode::InvalidUsage);
}

void SymmetricHeap::free(void* ptr) {
  if (ptr == nullptr) return;
  std::lock_guard<std::mutex> lock(allocMutex_);
  const size_t off = reinterpret_cast<uint64_t>(ptr) - peerBase_[rank_];
  auto it = usedBlocks_.find(off);
  if (it == usedBlocks_.end()) throw Error("SymmetricHeap::free of an unknown pointer", ErrorCode::InvalidUsage);
  size_t begin = off, size = it->second;
  usedBlocks_.erase(it);
  // agreements about buffers inside the freed block are void: the range may be handed out differently next time
  {
    const uint64_t lo = peerBase_[rank_] + off, hi = lo + size;
    for (auto c = symmetricCache_.lower_bound({lo, 0}); c != symmetricCache_.end() && c->first.first < hi;) c = symmetricCache_.erase(c);
  }
  // coalesce with neighbours
  auto next = freeBlocks_.lower_bound(begin);
  if (next != freeBlocks_.end() && next->first == begin + size) {
    size += next->second;
    next = freeBlocks_.erase(next);
  }
  if (next != freeBlocks_.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == begin) {
      begin = prev->first;
      size += prev->second;
      freeBlocks_.erase(prev);
    }
  }
  freeBlocks_[begin] = size;
}

size_t SymmetricHeap::bytesFree() const {
  std::lock_guard<std::mutex> lock(allocMutex_);
  size_t total = 0;
  for (auto& kv : freeBlocks_) total += kv.second;
  return total;
}

bool SymmetricHeap::contains(const void* ptr, size_t bytes) const {
  const uint64_t p = reinterpret_cast<uint64_t>(ptr);
  return p >= peerBase_[rank_] && p + bytes <= peerBase_[rank_] + bytes_;
}

bool SymmetricHeap::symmetricOnAllRanks(const void* ptr, size_t bytes) {
  const bool mine = contains(ptr, bytes);
  if (emulated_ || world_ == 1 || !bootstrap_) return mine;
  // A buffer outside the local heap settles the answer without talking to anybody: addresses of ordinary allocations
  // repeat in a rank-dependent way (caching allocators), so "first time seen" would not line up across ranks for them.
  // Heap buffers come from the symmetric allocator, whose call order is the same everywhere by contract. Should a peer
  // pass an ordinary buffer where this rank passes a heap one, the exchange below runs into the bootstrap's timeout and
  // the peer's kernel into its device-side one: a loud failure, never a kernel that addresses peers at a wrong offset.
  if (!mine) return false;
  const std::pair<uint64_t, size_t> key{reinterpret_cast<uint64_t>(ptr), bytes};
  {
    std::lock_guard<std::mutex> lock(allocMutex_);
    auto it = symmetricCache_.find(key);
    if (it != symmetricCache_.end()) return it->second;
  }
  // one word per rank: the buffer's heap offset
  std::vector<uint64_t> all(world_, 0);
  all[rank_] = reinterpret_cast<uint64_t>(ptr) - peerBase_[rank_];
  bootstrap_->allGather(all.data(), sizeof(uint64_t));
  bool same = mine;
  for (int r = 0; r < world_ && same; r++) same = all[r] == all[rank_];
  std::lock_guard<std::mutex> lock(allocMutex_);
  symmetricCache_[key] = same;
  return same;
}

void* SymmetricHeap::emulatedPtr(void* ptr, int r) const {
  return reinterpret_cast<void*>(peerBase_[r] + (reinterpret_cast<uint64_t>(ptr) - peerBase_[rank_]));
}

void SymmetricHeap::checkStatus() {
  if (statusDev_ == nullptr) return;
  refreshStatus();
  if (status_->code == kDevOk) return;
  DeviceStatus s = *status_;
  if (s.code == kDevErrorCapacity) {
    throw Error("receive buffer too small on rank " + std::to_string(s.rank) + ": capacity " + std::to_string(s.expected) +
                    " rows (nothing was sent; call resetStatus() and retry with a larger buffer)",
                ErrorCode::InvalidUsage);
  }
  std::string what = "device-side wait gave up: code " + std::to_string(s.code) + " rank " + std::to_string(s.rank) +
                     " block " + std::to_string(s.block) + " site " + std::to_string(s.where) + " peer " +
                     std::to_string(s.peer) + " expected " + std::to_string(s.expected) + " observed " +
                     std::to_string(s.observed) + " (" + std::to_string(s.count) + " waiters)";
  throw Error(what, ErrorCode::Timeout);
}

void SymmetricHeap::refreshStatus() {
  if (statusDev_ && status_) gpuMemcpy(status_, statusDev_, sizeof(DeviceStatus), cudaMemcpyDeviceToHost);
}

void SymmetricHeap::resetStatus() {
  if (status_) std::memset(status_, 0, sizeof(DeviceStatus));
  if (statusDev_) MSCCLPP_CUDATHROW(cudaMemset(statusDev_, 0, sizeof(DeviceStatus)));
}

void SymmetricHeap::setTimeoutMs(int64_t ms) { comm_.timeoutNs = static_cast<uint64_t>(ms) * 1000000ull; }

}  // namespace mscclpp
