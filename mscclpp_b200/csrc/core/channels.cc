// Host objects of MemoryChannel and PortChannel, and the ProxyService.
#include <mscclpp/memory_channel.hpp>
#include <mscclpp/numa.hpp>
#include <mscclpp/port_channel.hpp>

#include <mscclpp/gpu_utils.hpp>

#include "logger.hpp"
#include "registered_memory.hpp"

namespace mscclpp {

// ------------------------------------------------------------------------------------------ MemoryChannel
BaseMemoryChannel::DeviceHandle BaseMemoryChannel::deviceHandle() const {
  DeviceHandle h;
  h.semaphore_ = semaphore_->deviceHandle();
  return h;
}

MemoryChannel::MemoryChannel(std::shared_ptr<MemoryDevice2DeviceSemaphore> semaphore, RegisteredMemory dst, RegisteredMemory src,
                             void* packetBuffer)
    : BaseMemoryChannel(std::move(semaphore)), dst_(dst), src_(src.data()), packetBuffer_(packetBuffer) {
  if (!dst.transports().has(Transport::CudaIpc)) {
    throw Error("MemoryChannel: the peer's memory must be registered for CudaIpc", ErrorCode::InvalidUsage);
  }
  if (dst.data() == nullptr) throw Error("MemoryChannel: the peer's memory is not mapped in this process", ErrorCode::InvalidUsage);
}
MemoryChannel::MemoryChannel(const Semaphore& semaphore, RegisteredMemory dst, RegisteredMemory src, void* packetBuffer)
    : MemoryChannel(std::make_shared<MemoryDevice2DeviceSemaphore>(semaphore), dst, src, packetBuffer) {}
MemoryChannel::MemoryChannel(std::shared_ptr<MemoryDevice2DeviceSemaphore> semaphore, RegisteredMemory dst, void* src,
                             void* packetBuffer)
    : BaseMemoryChannel(std::move(semaphore)), dst_(dst), src_(src), packetBuffer_(packetBuffer) {
  if (dst.data() == nullptr) throw Error("MemoryChannel: the peer's memory is not mapped in this process", ErrorCode::InvalidUsage);
}

MemoryChannel::DeviceHandle MemoryChannel::deviceHandle() const {
  DeviceHandle h;
  h.semaphore_ = semaphore_->deviceHandle();
  h.dst_ = dst_.data();
  h.src_ = src_;
  h.packetBuffer_ = packetBuffer_;
  return h;
}

// ------------------------------------------------------------------------------------------ PortChannel
BasePortChannel::DeviceHandle BasePortChannel::deviceHandle() const {
  DeviceHandle h;
  h.semaphoreId_ = semaphoreId_;
  h.semaphore_ = semaphore_->deviceHandle();
  h.fifo_ = proxy_->fifo()->deviceHandle();
  return h;
}

PortChannel::DeviceHandle PortChannel::deviceHandle() const {
  DeviceHandle h;
  h.semaphoreId_ = semaphoreId_;
  h.semaphore_ = semaphore_->deviceHandle();
  h.fifo_ = proxy_->fifo()->deviceHandle();
  h.dst_ = dst_;
  h.src_ = src_;
  return h;
}

// ------------------------------------------------------------------------------------------ ProxyService
ProxyService::ProxyService(int fifoSize) {
  if (cudaGetDevice(&deviceId_) != cudaSuccess) {
    (void)cudaGetLastError();
    deviceId_ = -1;
  }
  const int dev = deviceId_;
  proxy_ = std::make_shared<Proxy>([this](ProxyTrigger t) { return handleTrigger(t); },
                                   [dev] {
                                     if (dev < 0) return;
                                     (void)cudaSetDevice(dev);
                                     // run next to the GPU: CPUs and memory of its NUMA node (best effort)
                                     try {
                                       numaBind(getDeviceNumaNode(dev));
                                     } catch (const std::exception&) {
                                     }
                                   },
                                   fifoSize);
}
ProxyService::~ProxyService() { stopProxy(); }

SemaphoreId ProxyService::buildAndAddSemaphore(Communicator& communicator, const Connection& connection) {
  semaphores_.push_back(std::make_shared<Host2DeviceSemaphore>(communicator, connection));
  return static_cast<SemaphoreId>(semaphores_.size() - 1);
}
SemaphoreId ProxyService::addSemaphore(const Semaphore& semaphore) {
  semaphores_.push_back(std::make_shared<Host2DeviceSemaphore>(semaphore));
  return static_cast<SemaphoreId>(semaphores_.size() - 1);
}
SemaphoreId ProxyService::addSemaphore(std::shared_ptr<Host2DeviceSemaphore> semaphore) {
  semaphores_.push_back(std::move(semaphore));
  return static_cast<SemaphoreId>(semaphores_.size() - 1);
}
MemoryId ProxyService::addMemory(RegisteredMemory memory) {
  if (memories_.size() >= (1u << kTriggerMemIdBits)) throw Error("too many memories for one ProxyService", ErrorCode::InvalidUsage);
  memories_.push_back(memory);
  return static_cast<MemoryId>(memories_.size() - 1);
}
MemoryId ProxyService::nextMemoryId(uint32_t count) const {
  if (count == 0) throw Error("count must be positive", ErrorCode::InvalidUsage);
  return static_cast<MemoryId>(memories_.size());
}
std::shared_ptr<Host2DeviceSemaphore> ProxyService::semaphore(SemaphoreId id) const { return semaphores_.at(id); }
BasePortChannel ProxyService::basePortChannel(SemaphoreId id) { return BasePortChannel(id, semaphores_.at(id), proxy_); }
PortChannel ProxyService::portChannel(SemaphoreId id, MemoryId dst, MemoryId src) {
  return PortChannel(id, semaphores_.at(id), proxy_, dst, src);
}
void ProxyService::startProxy(bool blocking) { proxy_->start(blocking); }
void ProxyService::stopProxy() { proxy_->stop(); }

ProxyHandlerResult ProxyService::handleTrigger(ProxyTrigger trigger) {
  const TriggerFields f = decodeTrigger(trigger);
  if (f.semaphoreId >= semaphores_.size()) {
    LOG_ERROR(LogSubsys::CONN, "proxy: request names unknown semaphore ", f.semaphoreId);
    return ProxyHandlerResult::Continue;
  }
  auto& sem = semaphores_[f.semaphoreId];
  Connection& conn = sem->connection();
  const void* key = conn.impl_.get();
  int& pending = inflight_[key];
  try {
    if (f.type & TriggerData) {
      if (f.dstMemoryId >= memories_.size() || f.srcMemoryId >= memories_.size()) {
        LOG_ERROR(LogSubsys::CONN, "proxy: request names an unknown memory id");
        return ProxyHandlerResult::Continue;
      }
      conn.write(memories_[f.dstMemoryId], f.dstOffset, memories_[f.srcMemoryId], f.srcOffset, f.size);
      pending++;
    }
    if (f.type & TriggerFlag) {
      sem->signal();
      pending++;
    }
    const int maxQueue = conn.getMaxWriteQueueSize();
    if ((f.type & TriggerSync) || (maxQueue > 0 && pending >= maxQueue)) {
      conn.flush();
      pending = 0;
    }
  } catch (const std::exception& e) {
    // A write or signal that did not happen must not look like one that did: the request stays unconsumed, so the
    // device-side flush() / putWithSignalAndFlush() that waits for it gives up with an error after its time limit.
    LOG_ERROR(LogSubsys::CONN, "proxy: request failed: ", e.what());
    return ProxyHandlerResult::Abort;
  }
  return ProxyHandlerResult::Continue;
}

}  // namespace mscclpp
