// Blocking TCP sockets with deadline + abort-flag aware connect/accept/send/recv, a magic-number
// handshake, and network-interface discovery (MSCCLPP_SOCKET_IFNAME / MSCCLPP_SOCKET_FAMILY).
// Plays the role of the reference's non-blocking socket state machine
// (src/core/include/socket.h:60-111, src/core/bootstrap/socket.cc) with a simpler design: every
// operation is a poll() loop with a 50 ms tick that re-checks the deadline and the abort flag.
#pragma once

#include <atomic>
#include <cstdint>
#include <string>
#include <sys/socket.h>
#include <vector>

namespace mscclpp {

struct SocketAddress {
  sockaddr_storage storage{};
  socklen_t length = 0;

  int family() const { return storage.ss_family; }
  uint16_t port() const;
  void setPort(uint16_t port);
  std::string toString(bool withPort = true) const;  // "ip:port" / "[ip6]:port"
  // Parses "ip", "ip:port", "[ip6]:port" or "hostname:port".
  static SocketAddress parse(const std::string& text, uint16_t defaultPort = 0);
  bool sameHost(const SocketAddress& other) const;
};

struct NetInterface {
  std::string name;
  SocketAddress address;
};

// Interfaces that are up, filtered by MSCCLPP_SOCKET_IFNAME-style spec:
//   ""            first non-loopback, non-docker interface (loopback as last resort)
//   "eth,ib"      names starting with eth or ib     "=eth0" exact name     "^lo,docker" everything but these
// `family`: AF_UNSPEC, AF_INET or AF_INET6.
std::vector<NetInterface> findInterfaces(const std::string& spec, int family, int maxCount = 16);
// The interface whose subnet contains `remote` (used when only the root's address is known).
bool findInterfaceMatchingSubnet(const SocketAddress& remote, NetInterface* out);

constexpr uint64_t kSocketMagic = 0x6d7363636c703230ull;  // handshake word sent by every connector

class Socket {
 public:
  Socket() = default;
  explicit Socket(int fd) : fd_(fd) {}
  ~Socket();
  Socket(Socket&& o) noexcept;
  Socket& operator=(Socket&& o) noexcept;
  Socket(const Socket&) = delete;
  Socket& operator=(const Socket&) = delete;

  // Bind + listen on `addr` (port 0 = ephemeral). The bound address (with the real port) is returned.
  SocketAddress listen(const SocketAddress& addr, int backlog = 16384);
  // Accept one connection and verify its magic word. Throws Timeout / Aborted.
  Socket accept(int64_t timeoutMs, const std::atomic<uint32_t>* abortFlag = nullptr);
  // Connect with retries (ECONNREFUSED / ETIMEDOUT are retried until the deadline) and send the magic word.
  void connect(const SocketAddress& addr, int64_t timeoutMs, const std::atomic<uint32_t>* abortFlag = nullptr);

  void sendAll(const void* data, size_t bytes, int64_t timeoutMs = -1, const std::atomic<uint32_t>* abortFlag = nullptr);
  void recvAll(void* data, size_t bytes, int64_t timeoutMs = -1, const std::atomic<uint32_t>* abortFlag = nullptr);
  // Non-throwing probe: true when at least one byte (or EOF) can be read without blocking.
  bool readable(int timeoutMs);

  void close();
  bool valid() const { return fd_ >= 0; }
  int fd() const { return fd_; }
  int release() {
    int f = fd_;
    fd_ = -1;
    return f;
  }

 private:
  int fd_ = -1;
};

uint64_t getHostHash();          // hash of MSCCLPP_HOSTID or hostname + boot id
// Hash of the domain inside which GPU memory can be shared between processes: the NVLink fabric's cluster id and clique
// (multi-node NVLink, from NVML) when the current GPU is part of one, else the host. MSCCLPP_IPC_DOMAIN overrides it.
uint64_t getIpcDomainHash();
uint64_t getPidHash();           // hash of pid + mount namespace

}  // namespace mscclpp
