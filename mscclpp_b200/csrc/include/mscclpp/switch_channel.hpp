// NvlsConnection: one CUDA multicast object shared by a group of ranks; SwitchChannel: a user buffer
// bound into it (reference: include/mscclpp/switch_channel.hpp:13-78, src/core/switch_channel.cc:53-317).
#pragma once

#include <memory>
#include <vector>

#include "core.hpp"
#include "switch_channel_device.hpp"

namespace mscclpp {

class NvlsConnection;

class SwitchChannel {
 public:
  SwitchChannel() = default;
  SwitchChannel(void* devicePtr, void* mcPtr, size_t bufferSize, std::shared_ptr<NvlsConnection> connection,
                std::shared_ptr<void> binding = nullptr)
      : devicePtr_(devicePtr), mcPtr_(mcPtr), bufferSize_(bufferSize), connection_(std::move(connection)), binding_(std::move(binding)) {}
  using DeviceHandle = SwitchChannelDeviceHandle;
  DeviceHandle deviceHandle() const;
  void* getDevicePtr() const { return devicePtr_; }
  void* getMcPtr() const { return mcPtr_; }
  size_t bufferSize() const { return bufferSize_; }

 private:
  void* devicePtr_ = nullptr;
  void* mcPtr_ = nullptr;
  size_t bufferSize_ = 0;
  std::shared_ptr<NvlsConnection> connection_;
  std::shared_ptr<void> binding_;  // shared by the copies of the channel; the last one to go returns the range of the object
};

class NvlsConnection : public std::enable_shared_from_this<NvlsConnection> {
 public:
  ~NvlsConnection();
  // Minimum size and alignment of what bindAllocatedMemory accepts.
  static size_t getMultiCastMinGranularity();
  // Bind [devicePtr, +size) - memory from the VMM path (GpuBuffer, gpuCallocPhysical, SymmetricHeap) -
  // into the lowest free range of the multicast object that fits. Collective: every member must bind ranges of
  // the same size in the same order (and drop the returned channels in the same order: a range is unbound and
  // reused once the last copy of its channel is destroyed).
  SwitchChannel bindAllocatedMemory(void* devicePtr, size_t size);
  size_t capacity() const;
  int groupSize() const;

  struct Impl;
  explicit NvlsConnection(std::unique_ptr<Impl> impl);
  Impl* impl() { return pimpl_.get(); }

 private:
  std::unique_ptr<Impl> pimpl_;
};

// Collective over `allRanks` (every listed rank calls it with the same list and size; the first listed
// rank creates the multicast object). `bufferSize` bytes can be bound later.
std::shared_ptr<NvlsConnection> connectNvlsCollective(std::shared_ptr<Communicator> communicator, std::vector<int> allRanks,
                                                      size_t bufferSize);

}  // namespace mscclpp
