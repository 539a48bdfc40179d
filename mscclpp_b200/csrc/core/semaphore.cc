#include <mscclpp/semaphore.hpp>

#include <atomic>
#include <cstring>

#include <mscclpp/gpu_utils.hpp>

#include "context.hpp"
#include "logger.hpp"
#include "registered_memory.hpp"

namespace mscclpp {

// ------------------------------------------------------------------------------------------ TokenPool
TokenPool::TokenPool(size_t nTokens) : nTokens_(nTokens) {
  if (isNvlsSupported()) {
    base_ = detail::gpuCallocPhysical(nTokens * sizeof(uint64_t));
    physical_ = true;
  } else {
    base_ = detail::gpuCalloc(nTokens * sizeof(uint64_t));
  }
  freeList_.reserve(nTokens);
  for (size_t i = nTokens; i > 0; i--) freeList_.push_back(static_cast<uint32_t>(i - 1));
}
TokenPool::~TokenPool() {
  if (physical_) detail::gpuFreePhysical(base_);
  else detail::gpuFree(base_);
}
std::shared_ptr<uint64_t> TokenPool::getToken() {
  std::lock_guard<std::mutex> lock(mutex_);
  if (freeList_.empty()) throw Error("semaphore token pool exhausted", ErrorCode::InternalError);
  uint32_t idx = freeList_.back();
  freeList_.pop_back();
  uint64_t* p = static_cast<uint64_t*>(base_) + idx;
  return std::shared_ptr<uint64_t>(p, [this, idx](uint64_t* q) {
    (void)cudaMemset(q, 0, sizeof(uint64_t));
    std::lock_guard<std::mutex> l(mutex_);
    freeList_.push_back(idx);
  });
}
std::shared_ptr<TokenPool> Context::Impl::tokens() {
  std::lock_guard<std::mutex> lock(mutex);
  int dev = 0;
  MSCCLPP_CUDATHROW(cudaGetDevice(&dev));
  auto& pool = tokenPools[dev];
  if (!pool) pool = std::make_shared<TokenPool>(32768);
  return pool;
}

// ------------------------------------------------------------------------------------------ SemaphoreStub / Semaphore
struct SemaphoreStub::Impl {
  Connection connection;
  std::shared_ptr<uint64_t> token;      // owner side only
  std::shared_ptr<TokenPool> pool;      // keeps the pool alive as long as the token
  RegisteredMemory memory;
  Device device;
};

SemaphoreStub::SemaphoreStub(const Connection& connection) : pimpl_(std::make_shared<Impl>()) {
  pimpl_->connection = connection;
  pimpl_->device = connection.localDevice();
  TransportFlags flags(connection.transport());
  if (pimpl_->device.type == DeviceType::GPU) {
    CudaDeviceGuard guard(pimpl_->device.id);
    pimpl_->pool = connection.context()->impl()->tokens();
    pimpl_->token = pimpl_->pool->getToken();
    // register the whole pool once per stub: the handle then covers this token at its offset
    pimpl_->memory = connection.context()->registerMemory(pimpl_->token.get(), sizeof(uint64_t), flags);
  } else {
    pimpl_->token = std::shared_ptr<uint64_t>(new uint64_t(0));
    pimpl_->memory = connection.context()->registerMemory(pimpl_->token.get(), sizeof(uint64_t), flags);
  }
}
SemaphoreStub::SemaphoreStub(std::shared_ptr<Impl> pimpl) : pimpl_(std::move(pimpl)) {}
const RegisteredMemory& SemaphoreStub::memory() const { return pimpl_->memory; }
std::vector<char> SemaphoreStub::serialize() const { return pimpl_->memory.serialize(); }
SemaphoreStub SemaphoreStub::deserialize(const std::vector<char>& data) {
  auto impl = std::make_shared<Impl>();
  impl->memory = RegisteredMemory::deserialize(data);
  return SemaphoreStub(impl);
}

struct Semaphore::Impl {
  SemaphoreStub local;
  SemaphoreStub remote;
  Impl(const SemaphoreStub& l, const SemaphoreStub& r) : local(l), remote(r) {}
};
Semaphore::Semaphore(const SemaphoreStub& localStub, const SemaphoreStub& remoteStub)
    : pimpl_(std::make_shared<Impl>(localStub, remoteStub)) {
  // Both stubs made in this process for different GPUs (no serialisation in between, so nothing has mapped the remote
  // token for the local GPU yet): give the local GPU access to the remote token. Tokens are VMM allocations, which
  // peer access does not cover; other memory goes through cudaDeviceEnablePeerAccess.
  const auto& l = *localStub.pimpl_;
  const auto& r = *remoteStub.pimpl_;
  // transports that deliver tokens to the CPU learn here where this semaphore's inbound token lives
  if (l.connection.valid() && l.token) {
    l.connection.impl_->startSignalForwarding(l.token.get(), l.device.type != DeviceType::GPU, l.device.id);
  }
  if (r.token && l.device.type == DeviceType::GPU && r.device.type == DeviceType::GPU && l.device.id != r.device.id && l.device.id >= 0) {
    CudaDeviceGuard guard(l.device.id);
    if (!detail::gpuGrantAccessPhysical(r.token.get(), l.device.id)) {
      cudaError_t e = cudaDeviceEnablePeerAccess(r.device.id, 0);
      if (e != cudaSuccess) (void)cudaGetLastError();
    }
  }
}
Connection& Semaphore::connection() { return pimpl_->local.pimpl_->connection; }
const RegisteredMemory& Semaphore::localMemory() const { return pimpl_->local.memory(); }
const RegisteredMemory& Semaphore::remoteMemory() const { return pimpl_->remote.memory(); }

// ------------------------------------------------------------------------------------------ typed wrappers
namespace {
Semaphore buildNow(Communicator& comm, const Connection& conn) {
  return comm.buildSemaphore(conn, comm.remoteRankOf(conn), comm.tagOf(conn)).get();
}
std::shared_ptr<uint64_t> hostWord() { return std::shared_ptr<uint64_t>(new uint64_t(0)); }
}  // namespace

Host2DeviceSemaphore::Host2DeviceSemaphore(const Semaphore& semaphore)
    : semaphore_(semaphore), expectedInbound_(gpuCallocShared<uint64_t>()), outbound_(hostWord()) {
  if (semaphore_.connection().localDevice().type != DeviceType::GPU) {
    throw Error("Host2DeviceSemaphore needs a GPU endpoint on the waiting side", ErrorCode::InvalidUsage);
  }
}
Host2DeviceSemaphore::Host2DeviceSemaphore(Communicator& communicator, const Connection& connection)
    : Host2DeviceSemaphore(buildNow(communicator, connection)) {}
Connection& Host2DeviceSemaphore::connection() { return semaphore_.connection(); }
void Host2DeviceSemaphore::signal() {
  semaphore_.connection().updateAndSync(semaphore_.remoteMemory(), 0, outbound_.get(), *outbound_ + 1);
}
Host2DeviceSemaphore::DeviceHandle Host2DeviceSemaphore::deviceHandle() const {
  DeviceHandle h;
  h.inboundToken = reinterpret_cast<uint64_t*>(semaphore_.localMemory().data());
  h.expectedInboundToken = expectedInbound_.get();
  return h;
}

Host2HostSemaphore::Host2HostSemaphore(const Semaphore& semaphore)
    : semaphore_(semaphore), expectedInbound_(hostWord()), outbound_(hostWord()) {
  if (semaphore_.connection().localDevice().type != DeviceType::CPU) {
    throw Error("Host2HostSemaphore needs CPU endpoints", ErrorCode::InvalidUsage);
  }
}
Host2HostSemaphore::Host2HostSemaphore(Communicator& communicator, const Connection& connection)
    : Host2HostSemaphore(buildNow(communicator, connection)) {}
Connection& Host2HostSemaphore::connection() { return semaphore_.connection(); }
void Host2HostSemaphore::signal() {
  semaphore_.connection().updateAndSync(semaphore_.remoteMemory(), 0, outbound_.get(), *outbound_ + 1);
}
bool Host2HostSemaphore::poll() {
  auto* token = reinterpret_cast<std::atomic<uint64_t>*>(semaphore_.localMemory().data());
  if (token->load(std::memory_order_acquire) > *expectedInbound_) {
    (*expectedInbound_)++;
    return true;
  }
  return false;
}
void Host2HostSemaphore::wait(int64_t maxSpinCount) {
  (*expectedInbound_)++;
  auto* token = reinterpret_cast<std::atomic<uint64_t>*>(semaphore_.localMemory().data());
  int64_t spins = 0;
  while (token->load(std::memory_order_acquire) < *expectedInbound_) {
    if (maxSpinCount >= 0 && spins++ > maxSpinCount) {
      (*expectedInbound_)--;
      throw Error("Host2HostSemaphore::wait ran out of spins", ErrorCode::Timeout);
    }
  }
}

MemoryDevice2DeviceSemaphore::MemoryDevice2DeviceSemaphore(const Semaphore& semaphore)
    : semaphore_(semaphore), expectedInbound_(gpuCallocShared<uint64_t>()), outbound_(gpuCallocShared<uint64_t>()) {
  if (semaphore_.connection().localDevice().type != DeviceType::GPU) {
    throw Error("MemoryDevice2DeviceSemaphore needs GPU endpoints", ErrorCode::InvalidUsage);
  }
}
MemoryDevice2DeviceSemaphore::MemoryDevice2DeviceSemaphore(Communicator& communicator, const Connection& connection)
    : MemoryDevice2DeviceSemaphore(buildNow(communicator, connection)) {}
Connection& MemoryDevice2DeviceSemaphore::connection() { return semaphore_.connection(); }
MemoryDevice2DeviceSemaphore::DeviceHandle MemoryDevice2DeviceSemaphore::deviceHandle() const {
  DeviceHandle h;
  h.inboundToken = reinterpret_cast<uint64_t*>(semaphore_.localMemory().data());
  h.remoteInboundToken = reinterpret_cast<uint64_t*>(semaphore_.remoteMemory().data());
  h.expectedInboundToken = expectedInbound_.get();
  h.outboundToken = outbound_.get();
  if (h.remoteInboundToken == nullptr) {
    throw Error("the peer's semaphore token is not mapped here: MemoryDevice2DeviceSemaphore needs a CudaIpc connection",
                ErrorCode::InvalidUsage);
  }
  return h;
}

}  // namespace mscclpp
