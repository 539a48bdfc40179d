// Host-side core API: bootstrap, transports, endpoints, connections, registered memory,
// semaphores and the Communicator. Public names and call signatures follow the reference
// (include/mscclpp/core.hpp:29-952) so code written against it compiles here; the implementation
// is independent and B200/NVSwitch-first (see symmetric_heap.hpp for the data-plane this library
// actually prefers: one VMM heap per rank, mapped everywhere once).
#pragma once

#include <array>
#include <bitset>
#include <cstdint>
#include <future>
#include <memory>
#include <string>
#include <vector>

#include "errors.hpp"

namespace mscclpp {

constexpr unsigned int UniqueIdBytes = 128;
using UniqueId = std::array<uint8_t, UniqueIdBytes>;

std::string version();

// ------------------------------------------------------------------------------------------ Bootstrap
// Control plane between ranks. Ordering contract: messages between one (sender, receiver, tag)
// triple arrive in send order; different tags are independent streams.
class Bootstrap {
 public:
  Bootstrap() = default;
  virtual ~Bootstrap() = default;
  virtual int getRank() const = 0;
  virtual int getNranks() const = 0;
  virtual int getNranksPerNode() const = 0;
  // Ranks that can map each other's GPU memory (one NVLink/NVSwitch domain). Defaults to the node.
  virtual int getNranksPerIpcDomain() const { return getNranksPerNode(); }
  virtual void send(void* data, int size, int peer, int tag) = 0;
  virtual void recv(void* data, int size, int peer, int tag) = 0;
  // allData holds nranks * size bytes; slot r is rank r's contribution (slot getRank() is the input).
  virtual void allGather(void* allData, int size) = 0;
  virtual void barrier() = 0;

  // Barrier among a subset (every listed rank must call it with the same list).
  void groupBarrier(const std::vector<int>& ranks);
  // Length-prefixed convenience wrappers.
  void send(const std::vector<char>& data, int peer, int tag);
  void recv(std::vector<char>& data, int peer, int tag);
};

// TCP implementation. Rank 0 hosts a short-lived rendezvous thread that collects every rank's
// listen address and publishes the full table; after that ranks talk directly (one lazily opened
// socket per (peer, tag, direction)), and allGather runs on a ring.
class TcpBootstrap : public Bootstrap {
 public:
  static UniqueId createUniqueId();

  TcpBootstrap(int rank, int nRanks);
  ~TcpBootstrap() override;

  // Unique id created by this object (rank 0 calls it, then ships the bytes out of band).
  UniqueId getUniqueId() const;
  void initialize(UniqueId uniqueId, int64_t timeoutSec = 30);
  // "ip:port" or "interface:ip:port": rank 0 listens there, everybody else connects there.
  void initialize(const std::string& ifIpPortTrio, int64_t timeoutSec = 30);
  // Unblocks and fails every pending or future socket operation of this bootstrap.
  void abort();

  int getRank() const override;
  int getNranks() const override;
  int getNranksPerNode() const override;
  int getNranksPerIpcDomain() const override;
  void send(void* data, int size, int peer, int tag) override;
  void recv(void* data, int size, int peer, int tag) override;
  void allGather(void* allData, int size) override;
  void barrier() override;
  // Ring broadcast from `root` (not in the abstract interface; used by NVLS set-up).
  void broadcast(void* data, int size, int root);

  using Bootstrap::recv;
  using Bootstrap::send;

 private:
  class Impl;
  std::unique_ptr<Impl> pimpl_;
};

// ------------------------------------------------------------------------------------------ Transports
enum class Transport {
  Unknown,
  CudaIpc,   // peer-mapped GPU memory inside one NVLink/NVSwitch domain
  IB0,
  IB1,
  IB2,
  IB3,
  IB4,
  IB5,
  IB6,
  IB7,
  Ethernet,  // TCP sockets, data staged through host memory
  NumTransports,
};

namespace detail {
constexpr size_t TransportFlagsSize = 11;
static_assert(TransportFlagsSize == static_cast<size_t>(Transport::NumTransports), "flag width mismatch");
using TransportFlagsBase = std::bitset<TransportFlagsSize>;
}  // namespace detail

class TransportFlags : private detail::TransportFlagsBase {
 public:
  TransportFlags() = default;
  TransportFlags(Transport transport) { set(static_cast<size_t>(transport)); }
  bool has(Transport transport) const { return test(static_cast<size_t>(transport)); }
  bool none() const { return detail::TransportFlagsBase::none(); }
  bool any() const { return detail::TransportFlagsBase::any(); }
  bool all() const { return detail::TransportFlagsBase::all(); }
  size_t count() const { return detail::TransportFlagsBase::count(); }
  TransportFlags& operator|=(TransportFlags other) {
    detail::TransportFlagsBase::operator|=(other);
    return *this;
  }
  TransportFlags operator|(TransportFlags other) const { return TransportFlags(*this) |= other; }
  TransportFlags operator|(Transport transport) const { return *this | TransportFlags(transport); }
  TransportFlags& operator&=(TransportFlags other) {
    detail::TransportFlagsBase::operator&=(other);
    return *this;
  }
  TransportFlags operator&(TransportFlags other) const { return TransportFlags(*this) &= other; }
  TransportFlags operator&(Transport transport) const { return *this & TransportFlags(transport); }
  TransportFlags& operator^=(TransportFlags other) {
    detail::TransportFlagsBase::operator^=(other);
    return *this;
  }
  TransportFlags operator^(TransportFlags other) const { return TransportFlags(*this) ^= other; }
  TransportFlags operator~() const {
    TransportFlags r(*this);
    r.flip();
    return r;
  }
  bool operator==(TransportFlags other) const {
    return static_cast<const detail::TransportFlagsBase&>(*this) == static_cast<const detail::TransportFlagsBase&>(other);
  }
  bool operator!=(TransportFlags other) const { return !(*this == other); }
  detail::TransportFlagsBase toBitset() const { return *this; }
  unsigned long toUlong() const { return to_ulong(); }
  static TransportFlags fromUlong(unsigned long v) {
    TransportFlags f;
    static_cast<detail::TransportFlagsBase&>(f) = detail::TransportFlagsBase(v);
    return f;
  }
};
inline TransportFlags operator|(Transport a, Transport b) { return TransportFlags(a) | b; }
inline TransportFlags operator&(Transport a, Transport b) { return TransportFlags(a) & b; }

const TransportFlags NoTransports = TransportFlags();
const TransportFlags AllIBTransports = Transport::IB0 | Transport::IB1 | Transport::IB2 | Transport::IB3 |
                                       Transport::IB4 | Transport::IB5 | Transport::IB6 | Transport::IB7;
const TransportFlags AllTransports = AllIBTransports | Transport::CudaIpc | Transport::Ethernet;

std::string transportToString(Transport t);

enum class DeviceType { Unknown, CPU, GPU };

struct Device {
  Device() = default;
  Device(DeviceType type, int id = -1) : type(type), id(id) {}
  DeviceType type = DeviceType::Unknown;
  int id = -1;  // -1 = the current CUDA device at endpoint creation
};

struct EndpointConfig {
  struct Ib {
    enum class Mode { Default, Host, HostNoAtomic };
    static constexpr int DefaultPort = -1;
    static constexpr int DefaultGidIndex = -1;
    static constexpr int DefaultMaxCqSize = 1024;
    static constexpr int DefaultMaxCqPollNum = 256;
    static constexpr int DefaultMaxSendWr = 8192;
    static constexpr int DefaultMaxRecvWr = 16;
    static constexpr int DefaultMaxWrPerSend = 64;
    int deviceIndex;
    int port;
    int gidIndex;
    int maxCqSize;
    int maxCqPollNum;
    int maxSendWr;
    int maxRecvWr;
    int maxWrPerSend;
    Mode mode;
    Ib(int deviceIndex = -1, int port = DefaultPort, int gidIndex = DefaultGidIndex, int maxCqSize = DefaultMaxCqSize,
       int maxCqPollNum = DefaultMaxCqPollNum, int maxSendWr = DefaultMaxSendWr, int maxRecvWr = DefaultMaxRecvWr,
       int maxWrPerSend = DefaultMaxWrPerSend, Mode mode = Mode::Default)
        : deviceIndex(deviceIndex),
          port(port),
          gidIndex(gidIndex),
          maxCqSize(maxCqSize),
          maxCqPollNum(maxCqPollNum),
          maxSendWr(maxSendWr),
          maxRecvWr(maxRecvWr),
          maxWrPerSend(maxWrPerSend),
          mode(mode) {}
  };

  Transport transport;
  Device device;
  int maxWriteQueueSize;  // -1 = transport default
  Ib ib;

  EndpointConfig(Transport transport = Transport::Unknown, Device device = DeviceType::GPU, int maxWriteQueueSize = -1,
                 Ib ib = {})
      : transport(transport), device(device), maxWriteQueueSize(maxWriteQueueSize), ib(ib) {}
};

class Context;
class Connection;
class BaseConnection;
class RegisteredMemory;
class SemaphoreStub;
class Semaphore;

// One side of a connection; serialisable so that the other side can connect to it.
class Endpoint {
 public:
  Endpoint() = default;
  const EndpointConfig& config() const;
  Transport transport() const;
  const Device& device() const;
  uint64_t hostHash() const;
  uint64_t pidHash() const;
  int maxWriteQueueSize() const;
  std::vector<char> serialize() const;
  static Endpoint deserialize(const std::vector<char>& data);

  struct Impl;
  explicit Endpoint(std::shared_ptr<Impl> pimpl);
  std::shared_ptr<Impl> pimpl_;
};

// Owns per-process transport resources (copy streams, the semaphore token pool, Ethernet listeners).
class Context : public std::enable_shared_from_this<Context> {
 public:
  static std::shared_ptr<Context> create() { return std::shared_ptr<Context>(new Context()); }
  ~Context();
  RegisteredMemory registerMemory(void* ptr, size_t size, TransportFlags transports);
  Endpoint createEndpoint(EndpointConfig config);
  Connection connect(const Endpoint& localEndpoint, const Endpoint& remoteEndpoint);

  struct Impl;
  Impl* impl() { return pimpl_.get(); }

 private:
  Context();
  std::unique_ptr<Impl> pimpl_;
};

// Non-owning description of a buffer plus what each transport needs to reach it remotely.
class RegisteredMemory {
 public:
  RegisteredMemory() = default;
  ~RegisteredMemory();
  void* data() const;             // usable address in THIS process (mapped peer memory for imported handles)
  void* originalDataPtr() const;  // address in the owning process
  size_t size() const;
  TransportFlags transports() const;
  std::vector<char> serialize() const;
  static RegisteredMemory deserialize(const std::vector<char>& data);
  bool isLocal() const;

  struct Impl;
  explicit RegisteredMemory(std::shared_ptr<Impl> pimpl);
  std::shared_ptr<Impl> pimpl_;
};

// Host-driven one-sided operations toward the peer of a connection.
class Connection {
 public:
  Connection() = default;
  void write(RegisteredMemory dst, uint64_t dstOffset, RegisteredMemory src, uint64_t srcOffset, uint64_t size);
  // *src = newValue locally, and the same 8 bytes are written to dst + dstOffset, ordered after earlier writes.
  void updateAndSync(RegisteredMemory dst, uint64_t dstOffset, uint64_t* src, uint64_t newValue);
  // Returns when everything issued so far is complete at the destination; throws Timeout otherwise.
  void flush(int64_t timeoutUsec = -1);
  Transport transport() const;
  Transport remoteTransport() const;
  std::shared_ptr<Context> context() const;
  const Device& localDevice() const;
  int getMaxWriteQueueSize() const;
  bool valid() const { return impl_ != nullptr; }

  explicit Connection(std::shared_ptr<BaseConnection> impl);
  std::shared_ptr<BaseConnection> impl_;
};

// Half of a semaphore: an 8-byte token in memory reachable through `connection`'s transport.
class SemaphoreStub {
 public:
  explicit SemaphoreStub(const Connection& connection);
  const RegisteredMemory& memory() const;
  std::vector<char> serialize() const;
  static SemaphoreStub deserialize(const std::vector<char>& data);

  struct Impl;
  explicit SemaphoreStub(std::shared_ptr<Impl> pimpl);
  std::shared_ptr<Impl> pimpl_;
};

class Semaphore {
 public:
  Semaphore() = default;
  Semaphore(const SemaphoreStub& localStub, const SemaphoreStub& remoteStub);
  Connection& connection();
  const RegisteredMemory& localMemory() const;
  const RegisteredMemory& remoteMemory() const;

  struct Impl;
  std::shared_ptr<Impl> pimpl_;
};

template <typename T>
using NonblockingFuture = std::shared_future<T>;

// Process-group facade. All exchange methods return *deferred* futures: the matching receive runs
// when get() is first called, and receives from one (peer, tag) run in the order the futures were
// created, regardless of the order in which get() is called.
class Communicator {
 public:
  explicit Communicator(std::shared_ptr<Bootstrap> bootstrap, std::shared_ptr<Context> context = nullptr);
  ~Communicator();
  std::shared_ptr<Bootstrap> bootstrap();
  std::shared_ptr<Context> context();
  RegisteredMemory registerMemory(void* ptr, size_t size, TransportFlags transports);
  void sendMemory(RegisteredMemory memory, int remoteRank, int tag = 0);
  std::shared_future<RegisteredMemory> recvMemory(int remoteRank, int tag = 0);
  std::shared_future<Connection> connect(const Endpoint& localEndpoint, int remoteRank, int tag = 0);
  std::shared_future<Connection> connect(const EndpointConfig& localConfig, int remoteRank, int tag = 0);
  std::shared_future<Semaphore> buildSemaphore(const Connection& connection, int remoteRank, int tag = 0);
  int remoteRankOf(const Connection& connection);
  int tagOf(const Connection& connection);

 private:
  struct Impl;
  std::unique_ptr<Impl> pimpl_;
};

// Maps a host object to the POD it hands to kernels.
template <class T>
using DeviceHandle = typename T::DeviceHandle;

template <typename T>
DeviceHandle<std::remove_reference_t<T>> deviceHandle(T&& t) {
  return t.deviceHandle();
}

template <class T>
using PacketPayload = typename T::Payload;

}  // namespace mscclpp
