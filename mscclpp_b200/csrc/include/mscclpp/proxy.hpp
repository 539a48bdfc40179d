// Proxy: a host thread that drains a Fifo and hands every trigger to a handler
// (reference: include/mscclpp/proxy.hpp, src/core/proxy.cc:42-100).
#pragma once

#include <functional>
#include <memory>

#include "fifo.hpp"

namespace mscclpp {

enum class ProxyHandlerResult {
  Continue,  // keep polling
  Stop,      // leave the loop after this trigger
  Abort,     // the request could not be carried out: leave the loop WITHOUT marking it consumed, so that a device-side
             // sync on it (or on anything queued behind it) runs into its time limit instead of reporting success
};

class Proxy;
using ProxyHandler = std::function<ProxyHandlerResult(ProxyTrigger)>;

class Proxy {
 public:
  // `threadInit` runs first on the proxy thread (set the CUDA device, bind to a NUMA node, ...).
  Proxy(ProxyHandler handler, std::function<void()> threadInit = {}, int fifoSize = DEFAULT_FIFO_SIZE);
  ~Proxy();
  void start(bool blocking = false);
  void stop();
  bool running() const;
  // True once a handler answered Abort: the thread has stopped and the FIFO is no longer drained.
  bool failed() const;
  std::shared_ptr<Fifo> fifo();
  // Called on the proxy thread between polls (progress of asynchronous work such as flushes).
  void setProgressHook(std::function<void()> hook);

 private:
  struct Impl;
  std::unique_ptr<Impl> pimpl_;
};

}  // namespace mscclpp
