// Communicator: exchange of endpoints, memories and semaphores over a Bootstrap.
// Ordering contract (reference: include/mscclpp/core.hpp:750-811, src/core/communicator.cc:12-181):
// futures are deferred; the receives belonging to one (peer, tag) execute in creation order no matter
// which future is waited on first. Implemented here as a per-(peer, tag) chain: each future first
// forces its predecessor.
#include <mscclpp/core.hpp>

#include <map>
#include <mutex>
#include <unordered_map>

#include "logger.hpp"
#include "registered_memory.hpp"

namespace mscclpp {

struct Communicator::Impl {
  std::shared_ptr<Bootstrap> bootstrap;
  std::shared_ptr<Context> context;
  std::mutex mutex;
  // last pending receive per (peer, tag); type-erased "make sure it has run"
  std::map<std::pair<int, int>, std::shared_future<void>> lastRecv;
  struct ConnInfo {
    int remoteRank;
    int tag;
  };
  std::unordered_map<const BaseConnection*, ConnInfo> connInfo;

  // Wraps `work` so that it runs after every earlier receive on (peer, tag), exactly once, lazily.
  template <typename T, typename Fn>
  std::shared_future<T> chain(int peer, int tag, Fn work) {
    std::lock_guard<std::mutex> lock(mutex);
    auto key = std::make_pair(peer, tag);
    std::shared_future<void> prev;
    auto it = lastRecv.find(key);
    if (it != lastRecv.end()) prev = it->second;
    std::shared_future<T> fut = std::async(std::launch::deferred, [prev, work]() -> T {
                                  if (prev.valid()) prev.get();
                                  return work();
                                }).share();
    lastRecv[key] = std::async(std::launch::deferred, [fut]() { (void)fut.get(); }).share();
    return fut;
  }
};

Communicator::Communicator(std::shared_ptr<Bootstrap> bootstrap, std::shared_ptr<Context> context)
    : pimpl_(std::make_unique<Impl>()) {
  pimpl_->bootstrap = std::move(bootstrap);
  pimpl_->context = context ? std::move(context) : Context::create();
}
Communicator::~Communicator() = default;

std::shared_ptr<Bootstrap> Communicator::bootstrap() { return pimpl_->bootstrap; }
std::shared_ptr<Context> Communicator::context() { return pimpl_->context; }

RegisteredMemory Communicator::registerMemory(void* ptr, size_t size, TransportFlags transports) {
  return pimpl_->context->registerMemory(ptr, size, transports);
}

void Communicator::sendMemory(RegisteredMemory memory, int remoteRank, int tag) {
  pimpl_->bootstrap->send(memory.serialize(), remoteRank, tag);
}

std::shared_future<RegisteredMemory> Communicator::recvMemory(int remoteRank, int tag) {
  auto bootstrap = pimpl_->bootstrap;
  return pimpl_->chain<RegisteredMemory>(remoteRank, tag, [bootstrap, remoteRank, tag]() {
    std::vector<char> data;
    bootstrap->recv(data, remoteRank, tag);
    return RegisteredMemory::deserialize(data);
  });
}

std::shared_future<Connection> Communicator::connect(const Endpoint& localEndpoint, int remoteRank, int tag) {
  pimpl_->bootstrap->send(localEndpoint.serialize(), remoteRank, tag);
  auto bootstrap = pimpl_->bootstrap;
  auto context = pimpl_->context;
  Impl* impl = pimpl_.get();
  return pimpl_->chain<Connection>(remoteRank, tag, [bootstrap, context, impl, localEndpoint, remoteRank, tag]() {
    std::vector<char> data;
    bootstrap->recv(data, remoteRank, tag);
    Endpoint remote = Endpoint::deserialize(data);
    Connection conn = context->connect(localEndpoint, remote);
    std::lock_guard<std::mutex> lock(impl->mutex);
    impl->connInfo[conn.impl_.get()] = Impl::ConnInfo{remoteRank, tag};
    return conn;
  });
}

std::shared_future<Connection> Communicator::connect(const EndpointConfig& localConfig, int remoteRank, int tag) {
  return connect(pimpl_->context->createEndpoint(localConfig), remoteRank, tag);
}

std::shared_future<Semaphore> Communicator::buildSemaphore(const Connection& connection, int remoteRank, int tag) {
  SemaphoreStub local(connection);
  pimpl_->bootstrap->send(local.serialize(), remoteRank, tag);
  auto bootstrap = pimpl_->bootstrap;
  return pimpl_->chain<Semaphore>(remoteRank, tag, [bootstrap, local, remoteRank, tag]() {
    std::vector<char> data;
    bootstrap->recv(data, remoteRank, tag);
    return Semaphore(local, SemaphoreStub::deserialize(data));
  });
}

int Communicator::remoteRankOf(const Connection& connection) {
  std::lock_guard<std::mutex> lock(pimpl_->mutex);
  auto it = pimpl_->connInfo.find(connection.impl_.get());
  if (it == pimpl_->connInfo.end()) throw Error("connection was not created by this communicator", ErrorCode::InvalidUsage);
  return it->second.remoteRank;
}

int Communicator::tagOf(const Connection& connection) {
  std::lock_guard<std::mutex> lock(pimpl_->mutex);
  auto it = pimpl_->connInfo.find(connection.impl_.get());
  if (it == pimpl_->connInfo.end()) throw Error("connection was not created by this communicator", ErrorCode::InvalidUsage);
  return it->second.tag;
}

}  // namespace mscclpp
