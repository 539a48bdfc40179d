#include <mscclpp/fifo.hpp>

#include <atomic>
#include <cstdlib>
#include <cstring>

#include <mscclpp/errors.hpp>
#include <mscclpp/gpu_utils.hpp>

#include "logger.hpp"

namespace mscclpp {

namespace {
bool cudaUsable() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return n > 0;
}
}  // namespace

struct Fifo::Impl {
  int size;
  bool onGpu;
  ProxyTrigger* triggers = nullptr;  // host-pinned (or plain host memory without a GPU)
  uint64_t* tail = nullptr;          // host-pinned
  uint64_t* head = nullptr;          // device (or host) memory
  uint64_t* tailCache = nullptr;     // device (or host) memory
  uint64_t consumed = 0;
  std::atomic<uint64_t> hostHead{0};
};

Fifo::Fifo(int size) : pimpl_(std::make_unique<Impl>()) {
  if (size < 1 || (size & (size - 1)) != 0) throw Error("FIFO size must be a power of two", ErrorCode::InvalidUsage);
  pimpl_->size = size;
  pimpl_->onGpu = cudaUsable();
  if (pimpl_->onGpu) {
    pimpl_->triggers = static_cast<ProxyTrigger*>(detail::gpuCallocHost(sizeof(ProxyTrigger) * size, cudaHostAllocMapped));
    pimpl_->tail = static_cast<uint64_t*>(detail::gpuCallocHost(sizeof(uint64_t), cudaHostAllocMapped));
    pimpl_->head = static_cast<uint64_t*>(detail::gpuCalloc(sizeof(uint64_t)));
    pimpl_->tailCache = static_cast<uint64_t*>(detail::gpuCalloc(sizeof(uint64_t)));
  } else {
    // no GPU in this process: the queue still works for host-side producers (unit tests, CPU ranks)
    pimpl_->triggers = static_cast<ProxyTrigger*>(std::aligned_alloc(64, sizeof(ProxyTrigger) * size));
    std::memset(pimpl_->triggers, 0, sizeof(ProxyTrigger) * size);
    pimpl_->tail = new uint64_t(0);
    pimpl_->head = new uint64_t(0);
    pimpl_->tailCache = new uint64_t(0);
  }
}

Fifo::~Fifo() {
  if (pimpl_->onGpu) {
    detail::gpuFreeHost(pimpl_->triggers);
    detail::gpuFreeHost(pimpl_->tail);
    detail::gpuFree(pimpl_->head);
    detail::gpuFree(pimpl_->tailCache);
  } else {
    std::free(pimpl_->triggers);
    delete pimpl_->tail;
    delete pimpl_->head;
    delete pimpl_->tailCache;
  }
}

ProxyTrigger Fifo::poll() {
  ProxyTrigger* slot = &pimpl_->triggers[pimpl_->consumed % pimpl_->size];
  // snd is written last by the 16-byte release store; read it first with acquire semantics
  uint64_t snd = reinterpret_cast<std::atomic<uint64_t>*>(&slot->snd)->load(std::memory_order_acquire);
  const uint64_t lap = pimpl_->consumed / pimpl_->size;
  const uint64_t want = (lap & 1ull) ? 0ull : kTriggerParityBit;
  ProxyTrigger out{0, 0};
  if ((snd & kTriggerParityBit) != want) return out;
  // a zero-initialised ring has parity 0 == "odd lap": rule out the never-written slot on lap 1, 3, ...
  uint64_t fst = reinterpret_cast<std::atomic<uint64_t>*>(&slot->fst)->load(std::memory_order_relaxed);
  if (want == 0 && fst == 0 && snd == 0) return out;
  out.fst = fst;
  out.snd = snd & ~kTriggerParityBit;
  if (out.fst == 0 && out.snd == 0) out.snd = 0;  // callers treat all-zero as "empty": producers never send it
  return out;
}

void Fifo::pop() {
  pimpl_->consumed++;
  reinterpret_cast<std::atomic<uint64_t>*>(pimpl_->tail)->store(pimpl_->consumed, std::memory_order_release);
}

int Fifo::size() const { return pimpl_->size; }
uint64_t Fifo::consumed() const { return pimpl_->consumed; }

FifoDeviceHandle Fifo::deviceHandle() const {
  FifoDeviceHandle h;
  h.triggers = pimpl_->triggers;
  h.head = pimpl_->head;
  h.tail = pimpl_->tail;
  h.tailCache = pimpl_->tailCache;
  h.size = pimpl_->size;
  return h;
}

uint64_t Fifo::pushFromHost(ProxyTrigger trigger) {
  if (trigger.fst == 0 && (trigger.snd & ~kTriggerParityBit) == 0) {
    throw Error("an all-zero trigger cannot be queued (it reads as an empty slot)", ErrorCode::InvalidUsage);
  }
  const uint64_t ticket = pimpl_->hostHead.fetch_add(1);
  auto* tail = reinterpret_cast<std::atomic<uint64_t>*>(pimpl_->tail);
  while (ticket >= static_cast<uint64_t>(pimpl_->size) + tail->load(std::memory_order_acquire)) {
  }
  const uint64_t lap = ticket / pimpl_->size;
  trigger.snd = (trigger.snd & ~kTriggerParityBit) | ((lap & 1ull) ? 0ull : kTriggerParityBit);
  ProxyTrigger* slot = &pimpl_->triggers[ticket % pimpl_->size];
  reinterpret_cast<std::atomic<uint64_t>*>(&slot->fst)->store(trigger.fst, std::memory_order_relaxed);
  reinterpret_cast<std::atomic<uint64_t>*>(&slot->snd)->store(trigger.snd, std::memory_order_release);
  return ticket;
}

}  // namespace mscclpp
