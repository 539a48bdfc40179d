// Endpoint, Context and the three connection types (reference: src/core/endpoint.cc:20-72,
// src/core/context.cc:16-105, src/core/connection.cc:85-715).
//   CudaIpc   peer-mapped memory, copy engine via cudaMemcpyAsync on a private non-blocking stream
//   Ethernet  TCP: data staged through host memory; a receive thread applies writes at the destination
//   IBx       RDMA writes over a reliable-connection queue pair of a run-time loaded verbs library; tokens by RDMA
//             fetch-and-add, or (mode HostNoAtomic) as the immediate value of an empty write that the receiver's CPU
//             thread forwards into the semaphore's token
#include <mscclpp/core.hpp>

#include <atomic>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <thread>

#include <arpa/inet.h>

#include <mscclpp/env.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/npkit/npkit.hpp>
#include <mscclpp/utils.hpp>

#include "context.hpp"
#include "gdr.hpp"
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
  w.putRaw(&ibQpInfo, sizeof(ibQpInfo));
  w.put<uint8_t>(ibNoAtomic ? 1 : 0);
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
  r.getRaw(&impl->ibQpInfo, sizeof(impl->ibQpInfo));
  impl->ibNoAtomic = r.get<uint8_t>() != 0;
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
    // one host, or (with fabric handles switched on) the hosts of one multi-node NVLink domain
    if (local.hostHash() != remote.hostHash() && !detail::fabricHandlesWanted()) {
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

// ------------------------------------------------------------------------------------------ InfiniBand
bool isIb(Transport t) { return AllIBTransports.has(t); }

class IBConnection : public BaseConnection {
 public:
  IBConnection(std::shared_ptr<Context> ctx, const Endpoint& local, const Endpoint& remote)
      : BaseConnection(ctx, local, remote),
        transport_(local.transport()),
        remoteTransport_(remote.transport()),
        qp_(local.pimpl_->ibQp),
        noAtomic_(local.pimpl_->ibNoAtomic),
        maxSendWr_(local.config().ib.maxSendWr) {
    if (!qp_) throw Error("the local endpoint of an InfiniBand connection must have been created by this context", ErrorCode::InvalidUsage);
    if (noAtomic_ != remote.pimpl_->ibNoAtomic) {
      throw Error("both endpoints of an InfiniBand connection must use the same mode (RDMA atomics, or immediate data)",
                  ErrorCode::InvalidUsage);
    }
    qp_->rtr(remote.pimpl_->ibQpInfo);
    qp_->rts();
    // where the old value of a fetch-and-add lands; nobody reads it
    landingMr_ = ctx->impl()->ibContext(transport_).registerMr(&landing_, sizeof(landing_));
    if (noAtomic_) {
      // every token of the peer consumes one receive; the receive thread re-posts them
      const int n = std::max(local.config().ib.maxRecvWr, 1);
      for (int i = 0; i < n; i++) qp_->stageRecv(0);
      qp_->postRecv();
    }
    LOG_INFO(LogSubsys::CONN, "InfiniBand connection via ", ctx->impl()->ibContext(transport_).deviceName(),
             noAtomic_ ? " (tokens as immediate data)" : " (tokens by RDMA atomics)");
  }

  ~IBConnection() override {
    stop_.store(true);
    if (recvThread_.joinable()) recvThread_.join();
    if (sinkStream_ != nullptr) (void)cudaStreamDestroy(sinkStream_);
    if (sinkStaging_ != nullptr) (void)cudaFreeHost(sinkStaging_);
  }

  Transport transport() const override { return transport_; }
  Transport remoteTransport() const override { return remoteTransport_; }

  void write(RegisteredMemory dst, uint64_t dstOffset, RegisteredMemory src, uint64_t srcOffset, uint64_t size) override {
    validateTransport(dst, remoteTransport_, dstOffset, size);
    validateTransport(src, transport_, srcOffset, size);
    checkBroken();
    const auto& local = src.pimpl_->ibEntry(transport_);
    if (!local.mr) throw Error("the source of an InfiniBand write must be memory registered by this process", ErrorCode::InvalidUsage);
    const IbMrInfo remote = dst.pimpl_->ibEntry(remoteTransport_).info;
    constexpr uint64_t kMaxMessage = 1ull << 30;  // the verbs limit is 2 GiB per work request
    for (uint64_t done = 0; done < size;) {
      const uint32_t piece = static_cast<uint32_t>(std::min<uint64_t>(size - done, kMaxMessage));
      makeRoom();
      qp_->stageWrite(*local.mr, remote, piece, nextWrId_++, srcOffset + done, dstOffset + done, true);
      qp_->postSend();
      done += piece;
    }
  }

  void updateAndSync(RegisteredMemory dst, uint64_t dstOffset, uint64_t* src, uint64_t newValue) override {
    validateTransport(dst, remoteTransport_, dstOffset, sizeof(uint64_t));
    checkBroken();
    const IbMrInfo remote = dst.pimpl_->ibEntry(remoteTransport_).info;
    const uint64_t oldValue = *src;
    *src = newValue;
    makeRoom();
    if (noAtomic_) {
      // an empty write with the token's low half as immediate data: it completes at the peer after every earlier write of
      // this queue pair, and the peer's receive thread rebuilds the 64-bit value from the increasing sequence
      qp_->stageWriteWithImm(nullptr, remote, 0, nextWrId_++, 0, dstOffset, true, htonl(static_cast<uint32_t>(newValue)));
    } else {
      qp_->stageAtomicAdd(*landingMr_, remote, nextWrId_++, dstOffset, newValue - oldValue, true);
    }
    qp_->postSend();
  }

  void flush(int64_t timeoutUsec) override {
    checkBroken();
    const auto t0 = std::chrono::steady_clock::now();
    while (qp_->outstandingSignaled() > 0) {
      pollOnce();
      if (timeoutUsec >= 0 && qp_->outstandingSignaled() > 0 &&
          std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count() > timeoutUsec) {
        throw Error("InfiniBand flush timed out with " + std::to_string(qp_->outstandingSignaled()) + " work requests outstanding",
                    ErrorCode::Timeout);
      }
    }
    checkReceiver();
  }

  void startSignalForwarding(void* token, bool isHostMemory, int deviceId) override {
    if (!noAtomic_) return;
    std::lock_guard<std::mutex> lock(sinkMutex_);
    if (sinkAddr_ != nullptr) {
      if (sinkAddr_ == token) return;
      throw Error("an InfiniBand connection that carries tokens as immediate data serves one semaphore", ErrorCode::InvalidUsage);
    }
    sinkAddr_ = token;
    sinkIsHost_ = isHostMemory;
    sinkDevice_ = deviceId;
    if (!isHostMemory) {
      gdrWindow_ = GdrWindow::open(token, deviceId);
      if (!gdrWindow_) {
        LOG_WARN(LogSubsys::CONN, "tokens of this InfiniBand connection reach GPU memory through cudaMemcpy: ", gdrAvailability().reason);
      }
    }
    recvThread_ = std::thread([this] { recvLoop(); });
  }

 private:
  // keeps the number of unpolled signalled work requests below the send queue's depth
  void makeRoom() {
    while (qp_->outstandingSignaled() >= maxSendWr_ - 1) pollOnce();
  }

  void pollOnce() {
    checkBroken();
    const int n = qp_->pollSendCq();
    if (n < 0) throw IbError("polling the send completion queue failed", errno);
    for (int i = 0; i < n; i++) {
      const ibv_wc& wc = qp_->sendWc(i);
      if (wc.status != IBV_WC_SUCCESS) {
        // The queue pair is in its error state now: whatever else was posted is flushed by the device and nothing
        // further can be sent. Remember it, so that later calls fail at once instead of waiting for completions.
        broken_ = "work request " + std::to_string(wc.wr_id) + " failed: " + qp_->wcStatusString(wc.status);
        checkBroken();
      }
    }
  }

  void checkBroken() const {
    if (!broken_.empty()) throw Error("InfiniBand connection is broken: " + broken_, ErrorCode::RemoteError);
  }

  void checkReceiver() {
    if (recvFailed_.load(std::memory_order_acquire)) {
      std::lock_guard<std::mutex> lock(sinkMutex_);
      throw Error("the receive thread of this InfiniBand connection stopped: " + recvError_, ErrorCode::RemoteError);
    }
  }

  void failReceiver(const std::string& why) {
    {
      std::lock_guard<std::mutex> lock(sinkMutex_);
      recvError_ = why;
    }
    recvFailed_.store(true, std::memory_order_release);
    LOG_WARN(LogSubsys::CONN, "InfiniBand receive thread: ", why);
  }

  void deliver(uint64_t value) {
    if (sinkIsHost_) {
      reinterpret_cast<std::atomic<uint64_t>*>(sinkAddr_)->store(value, std::memory_order_release);
    } else if (gdrWindow_) {
      gdrWindow_->store(value);
    } else {
      if (sinkStream_ == nullptr) {
        MSCCLPP_CUDATHROW(cudaStreamCreateWithFlags(&sinkStream_, cudaStreamNonBlocking));
        MSCCLPP_CUDATHROW(cudaHostAlloc(reinterpret_cast<void**>(&sinkStaging_), sizeof(uint64_t), cudaHostAllocDefault));
      }
      *sinkStaging_ = value;
      MSCCLPP_CUDATHROW(cudaMemcpyAsync(sinkAddr_, sinkStaging_, sizeof(uint64_t), cudaMemcpyHostToDevice, sinkStream_));
      MSCCLPP_CUDATHROW(cudaStreamSynchronize(sinkStream_));
    }
  }

  void recvLoop() {
    try {
      if (!sinkIsHost_ && sinkDevice_ >= 0) MSCCLPP_CUDATHROW(cudaSetDevice(sinkDevice_));
      uint32_t lastLow = 0;
      uint64_t high = 0;
      while (!stop_.load(std::memory_order_relaxed)) {
        const int n = qp_->pollRecvCq();
        if (n < 0) return failReceiver("polling the receive completion queue failed");
        if (n == 0) {
          std::this_thread::yield();
          continue;
        }
        for (int i = 0; i < n; i++) {
          const ibv_wc& wc = qp_->recvWc(i);
          if (wc.status != IBV_WC_SUCCESS) return failReceiver("a receive failed: " + qp_->wcStatusString(wc.status));
          // tokens only grow: a low half below the previous one means the high half moved on
          const uint32_t low = ntohl(wc.imm_data);
          if (low < lastLow) high += 1ull << 32;
          lastLow = low;
          deliver(high | low);
          qp_->stageRecv(0);
        }
        qp_->postRecv();
      }
    } catch (const std::exception& e) {
      failReceiver(e.what());
    }
  }

  Transport transport_;
  Transport remoteTransport_;
  std::shared_ptr<IbQp> qp_;
  bool noAtomic_;
  int maxSendWr_;
  uint64_t landing_ = 0;
  std::shared_ptr<const IbMr> landingMr_;
  uint64_t nextWrId_ = 1;
  std::string broken_;  // why the queue pair stopped working (empty: it works)
  // token forwarding (immediate-data mode)
  std::mutex sinkMutex_;
  void* sinkAddr_ = nullptr;
  bool sinkIsHost_ = true;
  int sinkDevice_ = -1;
  std::unique_ptr<GdrWindow> gdrWindow_;
  cudaStream_t sinkStream_ = nullptr;
  uint64_t* sinkStaging_ = nullptr;
  std::thread recvThread_;
  std::atomic<bool> stop_{false};
  std::atomic<bool> recvFailed_{false};
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

IbCtx& Context::Impl::ibContext(Transport ibTransport) {
  std::lock_guard<std::mutex> lock(mutex);
  auto& slot = ibContexts[ibTransport];
  if (!slot) slot = std::make_shared<IbCtx>(getIBDeviceName(ibTransport));
  return *slot;
}

const RegisteredMemory::Impl::IbEntry& RegisteredMemory::Impl::ibEntry(Transport t) const {
  for (const auto& e : ib) {
    if (e.transport == t) return e;
  }
  throw Error("RegisteredMemory carries no InfiniBand registration for " + transportToString(t), ErrorCode::InvalidUsage);
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
  for (int t = static_cast<int>(Transport::IB0); t <= static_cast<int>(Transport::IB7); t++) {
    const Transport ibT = static_cast<Transport>(t);
    if (!transports.has(ibT)) continue;
    RegisteredMemory::Impl::IbEntry e;
    e.transport = ibT;
    e.mr = pimpl_->ibContext(ibT).registerMr(ptr, size);
    e.info = e.mr->info();
    impl->ib.push_back(std::move(e));
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
  } else if (isIb(config.transport)) {
    IbCtx& ib = pimpl_->ibContext(config.transport);
    EndpointConfig::Ib::Mode mode = config.ib.mode;
    if (mode == EndpointConfig::Ib::Mode::Default) {
      mode = env()->ibvMode == "host-no-atomic" ? EndpointConfig::Ib::Mode::HostNoAtomic : EndpointConfig::Ib::Mode::Host;
    }
    if (mode == EndpointConfig::Ib::Mode::Host && !ib.supportsRdmaAtomics()) {
      LOG_WARN(LogSubsys::CONN, ib.deviceName(), " has no RDMA atomics: tokens travel as immediate data");
      mode = EndpointConfig::Ib::Mode::HostNoAtomic;
    }
    impl->ibNoAtomic = mode == EndpointConfig::Ib::Mode::HostNoAtomic;
    const IbQp::Limits limits{config.ib.maxCqSize, config.ib.maxCqPollNum, config.ib.maxSendWr, config.ib.maxRecvWr,
                              config.ib.maxWrPerSend};
    impl->ibQp = ib.createQp(config.ib.port, config.ib.gidIndex, limits);
    impl->ibQpInfo = impl->ibQp->info();
  } else if (config.transport != Transport::CudaIpc) {
    throw Error("endpoint needs a transport", ErrorCode::InvalidUsage);
  }
  return Endpoint(impl);
}

Connection Context::connect(const Endpoint& localEndpoint, const Endpoint& remoteEndpoint) {
  const bool bothIb = isIb(localEndpoint.transport()) && isIb(remoteEndpoint.transport());  // IB0 may face the peer's IB3
  if (localEndpoint.transport() != remoteEndpoint.transport() && !bothIb) {
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
      if (!bothIb) throw Error("transport " + transportToString(localEndpoint.transport()) + " cannot connect", ErrorCode::InvalidUsage);
      conn = std::make_shared<IBConnection>(shared_from_this(), localEndpoint, remoteEndpoint);
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
