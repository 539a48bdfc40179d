// Internal layouts behind RegisteredMemory / Endpoint / Connection.
#pragma once

#include <cuda_runtime.h>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <mscclpp/core.hpp>

#include "ib.hpp"
#include "socket.hpp"

namespace mscclpp {

// Everything needed to reach one GPU (or host) allocation from another process of the same host.
// Import order: same process -> raw pointer; VMM allocation on another host of the same NVLink fabric -> fabric
// handle; VMM allocation on this host -> POSIX fd through the fd server; cudaMalloc allocation -> legacy CUDA IPC
// handle. Fabric handles are produced only with MSCCLPP_FABRIC_HANDLES=1 (they need the IMEX service of a multi-node
// NVLink system); the reference tries Fabric -> PosixFd -> RuntimeIpc in the same spirit (src/core/gpu_ipc_mem.cc:386-432).
struct GpuIpcMemHandle {
  enum Kind : uint32_t { kNone = 0, kRuntimeIpc = 1, kPosixFd = 2, kHost = 4, kFabric = 8 };
  uint32_t kinds = kNone;
  cudaIpcMemHandle_t runtimeIpc{};
  char fdServer[96] = {0};
  uint32_t fdId = 0;
  unsigned char fabric[64] = {0};  // CUmemFabricHandle
  uint64_t baseAddr = 0;   // base of the allocation in the owner
  uint64_t allocSize = 0;  // size of the whole allocation
  uint64_t offset = 0;     // offset of the registered range inside the allocation
  int deviceId = -1;

  static GpuIpcMemHandle create(void* ptr, size_t size);
};

// A mapping of somebody else's allocation into this process.
class GpuIpcMapping {
 public:
  // One mapping per remote allocation and process: registrations of different ranges of the same
  // allocation (semaphore tokens of one pool, slices of one buffer) share it.
  static std::shared_ptr<GpuIpcMapping> acquire(const GpuIpcMemHandle& handle);
  explicit GpuIpcMapping(const GpuIpcMemHandle& handle);
  ~GpuIpcMapping();
  void* base() const { return base_; }

 private:
  void* base_ = nullptr;
  size_t size_ = 0;
  bool vmm_ = false;
  uint64_t vmmHandle_ = 0;
};

struct RegisteredMemory::Impl {
  void* data = nullptr;          // usable pointer in this process
  void* originalDataPtr = nullptr;
  size_t size = 0;
  uint64_t hostHash = 0;
  uint64_t pidHash = 0;
  TransportFlags transports;
  bool isLocal = true;
  bool isHostMemory = false;
  int deviceId = -1;
  GpuIpcMemHandle ipc;
  std::shared_ptr<GpuIpcMapping> mapping;   // imported memory only
  uint32_t registeredFdId = 0;              // local VMM memory only (fd parked in the fd server)
  // InfiniBand: one memory region per IB transport the memory was registered for. The owner holds the region, everybody
  // else the address and remote key that came with the serialised form.
  struct IbEntry {
    Transport transport = Transport::Unknown;
    std::shared_ptr<const IbMr> mr;
    IbMrInfo info;
  };
  std::vector<IbEntry> ib;
  const IbEntry& ibEntry(Transport t) const;

  ~Impl();
  std::vector<char> serialize() const;
  static std::shared_ptr<Impl> deserialize(const std::vector<char>& data);
};

struct Endpoint::Impl {
  EndpointConfig config;
  uint64_t hostHash = 0;
  uint64_t pidHash = 0;
  SocketAddress ethAddress;                  // Ethernet: where this endpoint accepts its peer
  std::shared_ptr<Socket> ethListener;       // local side only
  std::shared_ptr<IbQp> ibQp;                // InfiniBand, local side only
  IbQpInfo ibQpInfo;                         // InfiniBand: what the peer needs to reach the queue pair
  bool ibNoAtomic = false;                   // tokens travel as immediate data instead of RDMA atomics
  std::vector<char> serialize() const;
  static std::shared_ptr<Impl> deserialize(const std::vector<char>& data);
};

class BaseConnection {
 public:
  BaseConnection(std::shared_ptr<Context> context, const Endpoint& local, const Endpoint& remote)
      : context_(context), local_(local), remote_(remote) {}
  virtual ~BaseConnection() = default;
  virtual void write(RegisteredMemory dst, uint64_t dstOffset, RegisteredMemory src, uint64_t srcOffset, uint64_t size) = 0;
  virtual void updateAndSync(RegisteredMemory dst, uint64_t dstOffset, uint64_t* src, uint64_t newValue) = 0;
  virtual void flush(int64_t timeoutUsec) = 0;
  virtual Transport transport() const = 0;
  virtual Transport remoteTransport() const = 0;
  // Transports whose tokens arrive at the CPU (InfiniBand without RDMA atomics) forward them to the semaphore's inbound
  // token: the semaphore names the token when it is built. One semaphore per such connection.
  virtual void startSignalForwarding(void* /*token*/, bool /*isHostMemory*/, int /*deviceId*/) {}
  std::shared_ptr<Context> context() const { return context_; }
  const Device& localDevice() const { return local_.device(); }
  int maxWriteQueueSize() const { return local_.maxWriteQueueSize(); }
  const Endpoint& localEndpoint() const { return local_; }
  const Endpoint& remoteEndpoint() const { return remote_; }

 protected:
  std::shared_ptr<Context> context_;
  Endpoint local_;
  Endpoint remote_;
};

void validateTransport(const RegisteredMemory& mem, Transport transport, uint64_t offset, uint64_t size);

}  // namespace mscclpp
