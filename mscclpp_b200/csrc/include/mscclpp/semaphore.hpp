// Host-side semaphore objects built on Semaphore (core.hpp): who signals and who waits decides the
// type (reference: include/mscclpp/semaphore.hpp, src/core/semaphore.cc:118-236).
#pragma once

#include <memory>

#include "core.hpp"
#include "semaphore_device.hpp"

namespace mscclpp {

// Host signals (through the connection), device waits.
class Host2DeviceSemaphore {
 public:
  explicit Host2DeviceSemaphore(const Semaphore& semaphore);
  Host2DeviceSemaphore(Communicator& communicator, const Connection& connection);
  Connection& connection();
  void signal();
  using DeviceHandle = Host2DeviceSemaphoreDeviceHandle;
  DeviceHandle deviceHandle() const;

 private:
  Semaphore semaphore_;
  std::shared_ptr<uint64_t> expectedInbound_;   // device memory
  std::shared_ptr<uint64_t> outbound_;          // host memory
};

// Host signals, host waits.
class Host2HostSemaphore {
 public:
  explicit Host2HostSemaphore(const Semaphore& semaphore);
  Host2HostSemaphore(Communicator& communicator, const Connection& connection);
  Connection& connection();
  void signal();
  bool poll();
  // Spins at most maxSpinCount times (-1 = forever); throws Error(Timeout) when it runs out.
  void wait(int64_t maxSpinCount = 10000000);

 private:
  Semaphore semaphore_;
  std::shared_ptr<uint64_t> expectedInbound_;   // host
  std::shared_ptr<uint64_t> outbound_;          // host
};

// Device signals the peer device directly through peer-mapped memory.
class MemoryDevice2DeviceSemaphore {
 public:
  explicit MemoryDevice2DeviceSemaphore(const Semaphore& semaphore);
  MemoryDevice2DeviceSemaphore(Communicator& communicator, const Connection& connection);
  Connection& connection();
  using DeviceHandle = MemoryDevice2DeviceSemaphoreDeviceHandle;
  DeviceHandle deviceHandle() const;

 private:
  Semaphore semaphore_;
  std::shared_ptr<uint64_t> expectedInbound_;   // device
  std::shared_ptr<uint64_t> outbound_;          // device
};

}  // namespace mscclpp
