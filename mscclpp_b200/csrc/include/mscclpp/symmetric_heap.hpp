// SymmetricHeap: the data plane this library is built around on NVSwitch machines.
//
// Each rank creates ONE VMM allocation of the same size, exports it as a POSIX file descriptor,
// and maps every rank's allocation into one contiguous virtual range (slot r = rank r). When the
// GPUs support multicast, all allocations are also bound to one multicast object, which gives every
// heap address a third alias through which the NVSwitch reduces (multimem.ld_reduce) or replicates
// (multimem.st). Collective scratch, flags and user tensors are carved out of this heap, so kernels
// reach any peer buffer with pointer arithmetic and nothing is registered on the hot path. (The
// reference registers and exchanges memory per buffer: src/core/registered_memory.cc:35-187,
// src/core/switch_channel.cc:174-191; its API is kept in core.hpp for code that wants it.)
//
// An "emulated" heap places `world` heaps of one process on ONE device, for running multi-rank
// kernels as a single cooperative launch when fewer GPUs than ranks are available.
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <utility>

#include "core.hpp"
#include "device/symm.cuh"

namespace mscclpp {

class SymmetricHeap {
 public:
  struct Options {
    size_t bytes = 0;            // per-rank heap size, 0 = MSCCLPP_HEAP_BYTES (default 2 GiB)
    size_t llSlotBytes = 4u << 20;  // LL packet scratch per source rank and buffer (payload = half)
    bool enableNvls = true;      // bind to a multicast object when the hardware allows it
    int64_t timeoutMs = -1;      // device wait budget, -1 = MSCCLPP_DEVICE_TIMEOUT_MS
  };

  // Collective over `bootstrap`: every rank of it must call create() with equal options.
  static std::shared_ptr<SymmetricHeap> create(std::shared_ptr<Bootstrap> bootstrap, const Options& options);
  // Single process, `world` heaps on the current device.
  static std::shared_ptr<SymmetricHeap> createEmulated(int world, const Options& options);
  ~SymmetricHeap();

  // Collective teardown (unmap multicast, unbind, unmap peers). Called by the destructor if needed;
  // calling it explicitly on every rank before exit keeps the order deterministic.
  void destroy();

  int rank() const { return rank_; }
  int world() const { return world_; }
  bool emulated() const { return emulated_; }
  bool nvls() const { return mcBase_ != 0; }
  size_t bytes() const { return bytes_; }
  void* localBase() const { return reinterpret_cast<void*>(peerBase_[rank_]); }
  void* peerBase(int r) const { return reinterpret_cast<void*>(peerBase_[r]); }
  void* mcBase() const { return reinterpret_cast<void*>(mcBase_); }

  // Carve `bytes` out of the local heap. Symmetric as long as every rank performs the same sequence
  // of alloc/free calls. Returned memory is NOT zeroed. Throws Error(InvalidUsage) when full.
  void* alloc(size_t bytes, size_t alignment = 256);
  void free(void* ptr);
  size_t bytesFree() const;
  bool contains(const void* ptr, size_t bytes = 1) const;
  // True when, on every rank, the buffer lies inside the heap at the same offset - the condition under which kernels may
  // address the peers' copies by offset. contains() is a rank-local fact; code that chooses between a zero-copy kernel
  // and a staged one must choose from this answer, or the ranks can end up in different kernels. For a buffer inside
  // the local heap the first call per (ptr, bytes) is COLLECTIVE (offsets are compared over the bootstrap; ranks must
  // present their heap buffers in the same order, as with any registration) and later calls are cache lookups; a
  // buffer outside the local heap answers false at once. Entries are dropped when the heap block that holds them is
  // freed. Emulated heaps answer from contains().
  bool symmetricOnAllRanks(const void* ptr, size_t bytes);
  // Emulated heaps: address of `ptr` (a rank-0 heap address) in emulated rank r's heap.
  void* emulatedPtr(void* ptr, int r) const;

  // Parameter block for kernels. `rank` is 0 for emulated heaps (kernels add blockIdx.y).
  DeviceComm deviceComm() const { return comm_; }

  // Host view of the device error block. checkStatus() throws Error(Timeout) if a device wait gave up.
  // Copy of the device error block as of the last checkStatus()/refreshStatus() (call after a synchronize).
  const DeviceStatus& status() const { return *status_; }
  void refreshStatus();
  void checkStatus();
  void resetStatus();
  void setTimeoutMs(int64_t ms);

  std::shared_ptr<Bootstrap> bootstrap() const { return bootstrap_; }

 private:
  SymmetricHeap() = default;
  void initLayout(const Options& options);

  std::shared_ptr<Bootstrap> bootstrap_;
  int rank_ = 0;
  int world_ = 1;
  int deviceId_ = 0;
  bool emulated_ = false;
  bool destroyed_ = false;
  size_t bytes_ = 0;
  uint64_t vaBase_ = 0;
  uint64_t peerBase_[kMaxRanks] = {};
  uint64_t mcBase_ = 0;
  uint64_t localHandle_ = 0;
  uint64_t peerHandles_[kMaxRanks] = {};
  uint64_t mcHandle_ = 0;
  void* emulatedAlloc_ = nullptr;
  DeviceStatus* status_ = nullptr;     // host copy
  DeviceStatus* statusDev_ = nullptr;  // device memory, what kernels see
  DeviceComm comm_{};

  // host-side first-fit allocator over [arenaBegin_, bytes_)
  mutable std::mutex allocMutex_;
  size_t arenaBegin_ = 0;
  std::map<size_t, size_t> freeBlocks_;   // offset -> size
  std::map<size_t, size_t> usedBlocks_;   // offset -> size
  std::map<std::pair<uint64_t, size_t>, bool> symmetricCache_;  // (address, bytes) -> agreed answer
};

}  // namespace mscclpp
