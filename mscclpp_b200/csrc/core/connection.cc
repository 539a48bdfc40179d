// Endpoint, Context and the three connection types (reference: src/core/endpoint.cc:20-72,
// src/core/context.cc:16-105, src/core/connection.cc:85-715).
//   CudaIpc   peer-mapped memory, copy engine via cudaMemcpyAsync on a private non-blocking stream
//   Ethernet  TCP: data staged through host memory; a receive thread applies writes at the destination
//   IBx       declared for API compatibility; this build has no verbs support and refuses to connect
#include <mscclpp/core.hpp>

#include <atomic>
#include <condition_variable>
#include <cstring>
#include <deque>

#include <mscclpp/env.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/npkit/npkit.hpp>

#include "context.hpp"
#include "logger.hpp"
#include "registered_memory.hpp"
#include "serialize.hpp"

namespace mscclpp {

std::string transportToString(Transport t) {
  switch (t) {
    case Transport::Unknown:
      return "Unknown";
    case Transport::CudaIpc:
      return "CudaIpc";
    case Transport::Ethernet:
      return "Ethernet";
    case Transport::NumTransports:
      return "NumTransports";
    default:
      return "IB" + std::to_string(static_cast<int>(t) - static_cast<int>(Transport::IB0));
  }
}

// ------------------------------------------------------------------------------------------ Endpoint
std::vector<char> Endpoint::Impl::serialize() const {
  Writer w;
  w.put<int32_t>(static_cast<int32_t>(config.transport));
  w.put<int32_t>(static_cast<int32_t>(config.device.type));
  w.put<int32_t>(config.device.id);
  w.put<int32_t>(config.maxWriteQueueSize);
  w.putRaw(&config.ib, sizeof(config.ib));
  w.put<uint64_t>(hostHash);
  w.put<uint64_t>(pidHash);
  w.putRaw(&ethAddress, sizeof(ethAddress));
  return w.bytes;
}

std::shared_ptr<Endpoint::Impl> Endpoint::Impl::deserialize(const std::vector<char>& data) {
  Reader r(data);
  auto impl = std::make_shared<Impl>();
  impl->config.transport = static_cast<Transport>(r.get<int32_t>());
  impl->config.device.type = static_cast<DeviceType>(r.get<int32_t>());
  impl->config.device.id = r.get<int32_t>();
  impl->config.maxWriteQueueSize = r.get<int32_t>();
  r.getRaw(&impl->config.ib, sizeof(impl->config.ib));
  impl->hostHash = r.get<uint64_t>();
  impl->pidHash = r.get<uint64_t>();
  r.getRaw(&impl->ethAddress, sizeof(impl->ethAddress));
  return impl;
}

Endpoint::Endpoint(std::shared_ptr<Impl> pimpl) : pimpl_(std::move(pimpl)) {}
const EndpointConfig& Endpoint::config() const { return pimpl_->config; }
Transport Endpoint::transport() const { return pimpl_->config.transport; }
const Device& Endpoint::device() const { return pimpl_->config.device; }
uint64_t Endpoint::hostHash() const { return pimpl_->hostHash; }
uint64_t Endpoint::pidHash() const { return pimpl_->pidHash; }
int Endpoint::maxWriteQueueSize() const { return pimpl_->config.maxWriteQueueSize; }
std::vector<char> Endpoint::serialize() const { return pimpl_->serialize(); }
Endpoint Endpoint::deserialize(const std::vector<char>& data) { return Endpoint(Impl::deserialize(data)); }

// ------------------------------------------------------------------------------------------ CudaIpc
namespace {

class CudaIpcConnection : public BaseConnection {
 public:
  CudaIpcConnection(std::shared_ptr<Context> ctx, const Endpoint& local, const Endpoint& remote)
      : BaseConnection(ctx, local, remote) {
    if (local.hostHash() != remote.hostHash()) {
      throw Error("CudaIpc connections need both endpoints on one host", ErrorCode::InvalidUsage);
    }
    stream_ = ctx->impl()->ipcStream();
  }
  Transport transport() const override { return Transport::CudaIpc; }
  Transport remoteTransport() const override { return Transport::CudaIpc; }

  void write(RegisteredMemory dst, uint64_t dstOffset, RegisteredMemory src, uint64_t srcOffset, uint64_t size) override {
    validateTransport(dst, Transport::CudaIpc, dstOffset, size);
    validateTransport(src, Transport::CudaIpc, srcOffset, size);
    char* d = static_cast<char*>(dst.data());
    char* s = static_cast<char*>(src.data());
    if (d == nullptr || s == nullptr) throw Error("CudaIpc write needs both memories mapped in this process", ErrorCode::InvalidUsage);
    MSCCLPP_CUDATHROW(cudaMemcpyAsync(d + dstOffset, s + srcOffset, size, cudaMemcpyDefault, stream_->stream()));
    stream_->markDirty();
  }

  void updateAndSync(RegisteredMemory dst, uint64_t dstOffset, uint64_t* src, uint64_t newValue) override {
    validateTransport(dst, Transport::CudaIpc, dstOffset, sizeof(uint64_t));
    *src = newValue;
    char* d = static_cast<char*>(dst.data());
    if (d == nullptr) throw Error("CudaIpc updateAndSync needs the destination mapped in this process", ErrorCode::InvalidUsage);
    // stream order puts the token after every earlier write of this connection
    MSCCLPP_CUDATHROW(cudaMemcpyAsync(d + dstOffset, src, sizeof(uint64_t), cudaMemcpyDefault, stream_->stream()));
    stream_->markDirty();
  }

  void flush(int64_t timeoutUsec) override {
    if (timeoutUsec >= 0) LOG_DEBUG(LogSubsys::CONN, "CudaIpc flush ignores the timeout: stream synchronisation is not cancellable");
    stream_->sync();
  }

 private:
  std::shared_ptr<IpcStream> stream_;
};

// ------------------------------------------------------------------------------------------ Ethernet
struct EthHeader {
  uint64_t dstPtr;
  uint64_t size;
  uint32_t kind;  // 0 = data, 1 = flush request, 2 = flush reply
  uint32_t dstIsHost;
};

class EthernetConnection : public BaseConnection {
 public:
  EthernetConnection(std::shared_ptr<Context> ctx, const Endpoint& local, const Endpoint& remote)
      : BaseConnection(ctx, local, remote) {
    // Both sides connect to each other's listener: the outbound socket carries my writes, the inbound
    // one carries the peer's. Self-connections work the same way.
    send_.connect(remote.pimpl_->ethAddress, 30000, &abort_);
    if (!local.pimpl_->ethListener) throw Error("Ethernet endpoint has no listener", ErrorCode::InternalError);
    recv_ = local.pimpl_->ethListener->accept(30000, &abort_);
    recvThread_ = std::thread([this] { recvLoop(); });
  }
  ~EthernetConnection() override {
    abort_.store(1);
    send_.close();
    if (recvThread_.joinable()) recvThread_.join();
  }
  Transport transport() const override { return Transport::Ethernet; }
  Transport remoteTransport() const override { return Transport::Ethernet; }

  void write(RegisteredMemory dst, uint64_t dstOffset, RegisteredMemory src, uint64_t srcOffset, uint64_t size) override {
    validateTransport(dst, Transport::Ethernet, dstOffset, size);
    validateTransport(src, Transport::Ethernet, srcOffset, size);
    staging_.resize(size);
    const char* s = static_cast<const char*>(src.data()) + srcOffset;
    if (src.pimpl_->isHostMemory) std::memcpy(staging_.data(), s, size);
    else gpuMemcpy(staging_.data(), s, size, cudaMemcpyDeviceToHost);
    EthHeader h{reinterpret_cast<uint64_t>(dst.originalDataPtr()) + dstOffset, size, 0, dst.pimpl_->isHostMemory ? 1u : 0u};
    std::lock_guard<std::mutex> lock(sendMutex_);
    send_.sendAll(&h, sizeof(h), -1, &abort_);
    send_.sendAll(staging_.data(), size, -1, &abort_);
  }

  void updateAndSync(RegisteredMemory dst, uint64_t dstOffset, uint64_t* src, uint64_t newValue) override {
    validateTransport(dst, Transport::Ethernet, dstOffset, sizeof(uint64_t));
    *src = newValue;
    EthHeader h{reinterpret_cast<uint64_t>(dst.originalDataPtr()) + dstOffset, sizeof(uint64_t), 0,
                dst.pimpl_->isHostMemory ? 1u : 0u};
    std::lock_guard<std::mutex> lock(sendMutex_);
    send_.sendAll(&h, sizeof(h), -1, &abort_);
    send_.sendAll(&newValue, sizeof(newValue), -1, &abort_);
  }

  void flush(int64_t timeoutUsec) override {
    // round trip: the peer's receive thread answers after it has applied everything sent before
    uint64_t want;
    {
      std::lock_guard<std::mutex> lock(sendMutex_);
      EthHeader h{0, 0, 1, 0};
      send_.sendAll(&h, sizeof(h), -1, &abort_);
      want = ++flushesSent_;
    }
    std::unique_lock<std::mutex> lock(flushMutex_);
    auto pred = [&] { return flushesAcked_ >= want || recvFailed_; };
    if (timeoutUsec < 0) {
      flushCv_.wait(lock, pred);
    } else if (!flushCv_.wait_for(lock, std::chrono::microseconds(timeoutUsec), pred)) {
      throw Error("Ethernet flush timed out", ErrorCode::Timeout);
    }
    if (recvFailed_) throw Error("Ethernet connection lost: " + recvError_, ErrorCode::RemoteError);
  }

 private:
  void recvLoop() {
    std::vector<char> buf;
    try {
      while (!abort_.load()) {
        EthHeader h{};
        recv_.recvAll(&h, sizeof(h), -1, &abort_);
        if (h.kind == 1) {
          EthHeader reply{0, 0, 2, 0};
          std::lock_guard<std::mutex> lock(sendMutex_);
          send_.sendAll(&reply, sizeof(reply), -1, &abort_);
          continue;
        }
        if (h.kind == 2) {
          std::lock_guard<std::mutex> lock(flushMutex_);
          flushesAcked_++;
          flushCv_.notify_all();
          continue;
        }
        buf.resize(h.size);
        recv_.recvAll(buf.data(), h.size, -1, &abort_);
        void* dst = reinterpret_cast<void*>(h.dstPtr);
        if (h.dstIsHost) {
          if (h.size == sizeof(uint64_t)) {
            // tokens are read by spinning CPUs/GPUs: publish with release semantics
            uint64_t v;
            std::memcpy(&v, buf.data(), sizeof(v));
            reinterpret_cast<std::atomic<uint64_t>*>(dst)->store(v, std::memory_order_release);
          } else {
            std::memcpy(dst, buf.data(), h.size);
          }
        } else {
          gpuMemcpy(dst, buf.data(), h.size, cudaMemcpyHostToDevice);
        }
      }
    } catch (const std::exception& e) {
      std::lock_guard<std::mutex> lock(flushMutex_);
      if (!abort_.load()) {
        recvFailed_ = true;
        recvError_ = e.what();
      }
      flushCv_.notify_all();
    }
  }

  Socket send_;
  Socket recv_;
  std::thread recvThread_;
  std::atomic<uint32_t> abort_{0};
  std::mutex sendMutex_;
  std::vector<char> staging_;
  std::mutex flushMutex_;
  std::condition_variable flushCv_;
  uint64_t flushesSent_ = 0;
  uint64_t flushesAcked_ = 0;
  bool recvFailed_ = false;
  std::string recvError_;
};

}  // namespace

// ------------------------------------------------------------------------------------------ Context
IpcStream::IpcStream(int deviceId) : deviceId_(deviceId) {}
IpcStream::~IpcStream() {
  if (stream_) (void)cudaStreamDestroy(stream_);
}
cudaStream_t IpcStream::stream() {
  if (stream_ == nullptr && !env()->cudaIpcUseDefaultStream) {
    CudaDeviceGuard guard(deviceId_);
    MSCCLPP_CUDATHROW(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  }
  return stream_;  // nullptr = default stream when MSCCLPP_CUDAIPC_USE_DEFAULT_STREAM is set
}
void IpcStream::sync() {
  if (!dirty_) return;
  CudaDeviceGuard guard(deviceId_);
  MSCCLPP_CUDATHROW(cudaStreamSynchronize(stream()));
  dirty_ = false;
}

std::shared_ptr<IpcStream> Context::Impl::ipcStream() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    dev = -1;
  }
  std::lock_guard<std::mutex> lock(mutex);
  // one stream per connection keeps unrelated peers from serialising behind each other
  auto s = std::make_shared<IpcStream>(dev);
  streams.push_back(s);
  return s;
}

Context::Context() : pimpl_(std::make_unique<Impl>()) {}
Context::~Context() = default;

RegisteredMemory Context::registerMemory(void* ptr, size_t size, TransportFlags transports) {
  auto impl = std::make_shared<RegisteredMemory::Impl>();
  impl->data = ptr;
  impl->originalDataPtr = ptr;
  impl->size = size;
  impl->hostHash = getHostHash();
  impl->pidHash = getPidHash();
  impl->transports = transports;
  impl->isLocal = true;
  if ((transports & AllIBTransports).any()) {
    throw Error("this build has no InfiniBand support: register with CudaIpc and/or Ethernet", ErrorCode::InvalidUsage);
  }
  if (transports.has(Transport::CudaIpc)) {
    impl->ipc = GpuIpcMemHandle::create(ptr, size);
    impl->isHostMemory = (impl->ipc.kinds & GpuIpcMemHandle::kHost) != 0;
    impl->deviceId = impl->ipc.deviceId;
    if (impl->ipc.kinds & GpuIpcMemHandle::kPosixFd) impl->registeredFdId = impl->ipc.fdId;
  } else {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess || attr.type == cudaMemoryTypeUnregistered ||
        attr.type == cudaMemoryTypeHost) {
      (void)cudaGetLastError();
      impl->isHostMemory = true;
    } else {
      impl->deviceId = attr.device;
    }
  }
  return RegisteredMemory(impl);
}

Endpoint Context::createEndpoint(EndpointConfig config) {
  auto impl = std::make_shared<Endpoint::Impl>();
  impl->config = config;
  impl->hostHash = getHostHash();
  impl->pidHash = getPidHash();
  if (config.device.type == DeviceType::GPU && config.device.id < 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) impl->config.device.id = dev;
    else (void)cudaGetLastError();
  }
  if (config.transport == Transport::Ethernet) {
    int family = AF_UNSPEC;
    if (env()->socketFamily == "AF_INET") family = AF_INET;
    if (env()->socketFamily == "AF_INET6") family = AF_INET6;
    auto ifs = findInterfaces(env()->socketIfname, family, 1);
    if (ifs.empty()) throw Error("no network interface for an Ethernet endpoint", ErrorCode::SystemError);
    SocketAddress a = ifs[0].address;
    a.setPort(0);
    impl->ethListener = std::make_shared<Socket>();
    impl->ethAddress = impl->ethListener->listen(a);
  } else if (config.transport != Transport::CudaIpc) {
    if (config.transport == Transport::Unknown || config.transport == Transport::NumTransports) {
      throw Error("endpoint needs a transport", ErrorCode::InvalidUsage);
    }
    throw Error("transport " + transportToString(config.transport) + " is not available: this build has no InfiniBand support",
                ErrorCode::InvalidUsage);
  }
  return Endpoint(impl);
}

Connection Context::connect(const Endpoint& localEndpoint, const Endpoint& remoteEndpoint) {
  if (localEndpoint.transport() != remoteEndpoint.transport()) {
    throw Error("endpoints of one connection must use the same transport", ErrorCode::InvalidUsage);
  }
  std::shared_ptr<BaseConnection> conn;
  switch (localEndpoint.transport()) {
    case Transport::CudaIpc:
      conn = std::make_shared<CudaIpcConnection>(shared_from_this(), localEndpoint, remoteEndpoint);
      break;
    case Transport::Ethernet:
      conn = std::make_shared<EthernetConnection>(shared_from_this(), localEndpoint, remoteEndpoint);
      break;
    default:
      throw Error("transport " + transportToString(localEndpoint.transport()) + " is not available in this build",
                  ErrorCode::InvalidUsage);
  }
  return Connection(conn);
}

// ------------------------------------------------------------------------------------------ Connection facade
Connection::Connection(std::shared_ptr<BaseConnection> impl) : impl_(std::move(impl)) {}
namespace {
// Host-side trace events around a connection call; channel 0 collects them (one proxy thread drives them).
struct TraceScope {
  TraceScope(Transport t, int cudaEntry, int ethEntry, uint32_t size)
      : on_(NpKit::Enabled()), type_(t == Transport::Ethernet ? ethEntry : cudaEntry), size_(size) {
    if (on_) NpKit::CollectCpuEvent(static_cast<uint8_t>(type_), size_, 0, NpKit::GetCpuTimestamp(), 0);
  }
  ~TraceScope() {
    if (on_) NpKit::CollectCpuEvent(static_cast<uint8_t>(type_ + 1), size_, 0, NpKit::GetCpuTimestamp(), 0);
  }
  bool on_;
  int type_;
  uint32_t size_;
};
}  // namespace

void Connection::write(RegisteredMemory dst, uint64_t dstOffset, RegisteredMemory src, uint64_t srcOffset, uint64_t size) {
  TraceScope trace(impl_->transport(), NPKIT_EVENT_CONN_CUDA_IPC_WRITE_ENTRY, NPKIT_EVENT_CONN_ETH_WRITE_ENTRY, static_cast<uint32_t>(size));
  impl_->write(dst, dstOffset, src, srcOffset, size);
}
void Connection::updateAndSync(RegisteredMemory dst, uint64_t dstOffset, uint64_t* src, uint64_t newValue) {
  TraceScope trace(impl_->transport(), NPKIT_EVENT_CONN_CUDA_IPC_UPDATE_AND_SYNC_ENTRY, NPKIT_EVENT_CONN_ETH_UPDATE_AND_SYNC_ENTRY, 8);
  impl_->updateAndSync(dst, dstOffset, src, newValue);
}
void Connection::flush(int64_t timeoutUsec) {
  TraceScope trace(impl_->transport(), NPKIT_EVENT_CONN_CUDA_IPC_FLUSH_ENTRY, NPKIT_EVENT_CONN_ETH_FLUSH_ENTRY, 0);
  impl_->flush(timeoutUsec);
}
Transport Connection::transport() const { return impl_->transport(); }
Transport Connection::remoteTransport() const { return impl_->remoteTransport(); }
std::shared_ptr<Context> Connection::context() const { return impl_->context(); }
const Device& Connection::localDevice() const { return impl_->localDevice(); }
int Connection::getMaxWriteQueueSize() const { return impl_->maxWriteQueueSize(); }

}  // namespace mscclpp
