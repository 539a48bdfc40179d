// Host side of the GPU -> CPU FIFO.
#pragma once

#include <memory>

#include "fifo_device.hpp"

namespace mscclpp {

constexpr int DEFAULT_FIFO_SIZE = 512;

class Fifo {
 public:
  // `size` must be a power of two (slots).
  explicit Fifo(int size = DEFAULT_FIFO_SIZE);
  ~Fifo();
  // The oldest unconsumed trigger, or a trigger with fst == 0 && snd == 0 when there is none.
  // The parity bit is cleared in the returned copy.
  ProxyTrigger poll();
  // Mark the trigger returned by the last successful poll() as consumed.
  void pop();
  int size() const;
  uint64_t consumed() const;
  FifoDeviceHandle deviceHandle() const;
  // Host-side producer with the device's protocol (tests and host-driven use): returns the ticket.
  uint64_t pushFromHost(ProxyTrigger trigger);

 private:
  struct Impl;
  std::unique_ptr<Impl> pimpl_;
};

}  // namespace mscclpp
