#include <mscclpp/proxy.hpp>

#include <atomic>
#include <thread>

#include <mscclpp/errors.hpp>
#include <mscclpp/gpu_utils.hpp>

#include "logger.hpp"

namespace mscclpp {

struct Proxy::Impl {
  ProxyHandler handler;
  std::function<void()> threadInit;
  std::function<void()> progress;
  std::shared_ptr<Fifo> fifo;
  std::thread thread;
  std::atomic<bool> running{false};
  std::atomic<bool> stopRequested{false};
  std::atomic<bool> failed{false};
};

Proxy::Proxy(ProxyHandler handler, std::function<void()> threadInit, int fifoSize) : pimpl_(std::make_unique<Impl>()) {
  pimpl_->handler = std::move(handler);
  pimpl_->threadInit = std::move(threadInit);
  pimpl_->fifo = std::make_shared<Fifo>(fifoSize);
}

Proxy::~Proxy() { stop(); }

std::shared_ptr<Fifo> Proxy::fifo() { return pimpl_->fifo; }
bool Proxy::running() const { return pimpl_->running.load(); }
bool Proxy::failed() const { return pimpl_->failed.load(); }
void Proxy::setProgressHook(std::function<void()> hook) { pimpl_->progress = std::move(hook); }

void Proxy::start(bool blocking) {
  if (pimpl_->running.exchange(true)) return;
  pimpl_->stopRequested.store(false);
  std::atomic<bool> ready{false};
  pimpl_->thread = std::thread([this, &ready] {
    // set-up calls made here must not break a CUDA graph capture running on another thread
    AvoidCudaGraphCaptureGuard guard;
    if (pimpl_->threadInit) pimpl_->threadInit();
    ready.store(true, std::memory_order_release);
    Fifo& fifo = *pimpl_->fifo;
    int idle = 0;
    while (true) {
      ProxyTrigger t = fifo.poll();
      if (t.fst == 0 && t.snd == 0) {
        if (pimpl_->progress) pimpl_->progress();
        // check for shutdown only now and then: the poll loop is the latency-critical path
        if (++idle >= 256) {
          idle = 0;
          if (pimpl_->stopRequested.load(std::memory_order_acquire)) break;
        }
        continue;
      }
      idle = 0;
      ProxyHandlerResult r = pimpl_->handler(t);
      if (r == ProxyHandlerResult::Abort) {
        pimpl_->failed.store(true);
        LOG_ERROR(LogSubsys::CONN, "proxy: a request failed; the proxy thread stops and leaves the request unconsumed");
        break;
      }
      fifo.pop();
      if (pimpl_->progress) pimpl_->progress();
      if (r == ProxyHandlerResult::Stop) break;
    }
    pimpl_->running.store(false);
  });
  if (blocking) {
    while (!ready.load(std::memory_order_acquire)) std::this_thread::yield();
  } else {
    // `ready` lives on this stack frame: wait for the thread to pass it either way
    while (!ready.load(std::memory_order_acquire)) std::this_thread::yield();
  }
}

void Proxy::stop() {
  pimpl_->stopRequested.store(true, std::memory_order_release);
  if (pimpl_->thread.joinable()) pimpl_->thread.join();
  pimpl_->running.store(false);
}

}  // namespace mscclpp
