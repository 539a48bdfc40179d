// PortChannel and the ProxyService that executes its requests on a host thread
// (reference: include/mscclpp/port_channel.hpp:18-181, src/core/port_channel.cc:32-178).
#pragma once

#include <memory>
#include <unordered_map>
#include <vector>

#include "core.hpp"
#include "port_channel_device.hpp"
#include "proxy.hpp"
#include "semaphore.hpp"

namespace mscclpp {

class BaseProxyService {
 public:
  virtual ~BaseProxyService() = default;
  virtual void startProxy(bool blocking = false) = 0;
  virtual void stopProxy() = 0;
};

struct BasePortChannel {
  BasePortChannel() = default;
  BasePortChannel(SemaphoreId semaphoreId, std::shared_ptr<Host2DeviceSemaphore> semaphore, std::shared_ptr<Proxy> proxy)
      : semaphoreId_(semaphoreId), semaphore_(std::move(semaphore)), proxy_(std::move(proxy)) {}
  using DeviceHandle = BasePortChannelDeviceHandle;
  DeviceHandle deviceHandle() const;

 protected:
  SemaphoreId semaphoreId_ = 0;
  std::shared_ptr<Host2DeviceSemaphore> semaphore_;
  std::shared_ptr<Proxy> proxy_;
};

struct PortChannel : public BasePortChannel {
  PortChannel() = default;
  PortChannel(SemaphoreId semaphoreId, std::shared_ptr<Host2DeviceSemaphore> semaphore, std::shared_ptr<Proxy> proxy,
              MemoryId dst, MemoryId src)
      : BasePortChannel(semaphoreId, std::move(semaphore), std::move(proxy)), dst_(dst), src_(src) {}
  using DeviceHandle = PortChannelDeviceHandle;
  DeviceHandle deviceHandle() const;

 private:
  MemoryId dst_ = 0;
  MemoryId src_ = 0;
};

class ProxyService : public BaseProxyService {
 public:
  explicit ProxyService(int fifoSize = DEFAULT_FIFO_SIZE);
  ~ProxyService() override;
  SemaphoreId buildAndAddSemaphore(Communicator& communicator, const Connection& connection);
  SemaphoreId addSemaphore(const Semaphore& semaphore);
  SemaphoreId addSemaphore(std::shared_ptr<Host2DeviceSemaphore> semaphore);
  MemoryId addMemory(RegisteredMemory memory);
  // Next id addMemory() will return (ids are dense, starting at 0).
  MemoryId nextMemoryId(uint32_t count = 1) const;
  std::shared_ptr<Host2DeviceSemaphore> semaphore(SemaphoreId id) const;
  BasePortChannel basePortChannel(SemaphoreId id);
  PortChannel portChannel(SemaphoreId id, MemoryId dst, MemoryId src);
  void startProxy(bool blocking = false) override;
  void stopProxy() override;

 private:
  ProxyHandlerResult handleTrigger(ProxyTrigger trigger);
  std::vector<std::shared_ptr<Host2DeviceSemaphore>> semaphores_;
  std::vector<RegisteredMemory> memories_;
  std::shared_ptr<Proxy> proxy_;
  int deviceId_ = -1;
  std::unordered_map<const void*, int> inflight_;  // per-connection count of writes since the last flush
};

}  // namespace mscclpp
