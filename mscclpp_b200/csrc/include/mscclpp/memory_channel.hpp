// MemoryChannel: peer-mapped memory + device-to-device semaphore
// (reference: include/mscclpp/memory_channel.hpp:15-82, src/core/memory_channel.cc:11-35).
#pragma once

#include <memory>

#include "core.hpp"
#include "memory_channel_device.hpp"
#include "semaphore.hpp"

namespace mscclpp {

struct BaseMemoryChannel {
  BaseMemoryChannel() = default;
  explicit BaseMemoryChannel(std::shared_ptr<MemoryDevice2DeviceSemaphore> semaphore) : semaphore_(std::move(semaphore)) {}
  explicit BaseMemoryChannel(const Semaphore& semaphore)
      : semaphore_(std::make_shared<MemoryDevice2DeviceSemaphore>(semaphore)) {}
  using DeviceHandle = BaseMemoryChannelDeviceHandle;
  DeviceHandle deviceHandle() const;

 protected:
  std::shared_ptr<MemoryDevice2DeviceSemaphore> semaphore_;
};

struct MemoryChannel : public BaseMemoryChannel {
  MemoryChannel() = default;
  // dst: the peer's memory (received through Communicator::recvMemory); src: local memory.
  MemoryChannel(std::shared_ptr<MemoryDevice2DeviceSemaphore> semaphore, RegisteredMemory dst, RegisteredMemory src,
                void* packetBuffer = nullptr);
  MemoryChannel(const Semaphore& semaphore, RegisteredMemory dst, RegisteredMemory src, void* packetBuffer = nullptr);
  MemoryChannel(std::shared_ptr<MemoryDevice2DeviceSemaphore> semaphore, RegisteredMemory dst, void* src,
                void* packetBuffer = nullptr);
  using DeviceHandle = MemoryChannelDeviceHandle;
  DeviceHandle deviceHandle() const;

 private:
  RegisteredMemory dst_;
  void* src_ = nullptr;
  void* packetBuffer_ = nullptr;
};

}  // namespace mscclpp
