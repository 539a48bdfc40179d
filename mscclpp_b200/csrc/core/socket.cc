#include "socket.hpp"

#include <algorithm>
#include <arpa/inet.h>
#include <cerrno>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <fstream>
#include <ifaddrs.h>
#include <net/if.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <unistd.h>

#include <cuda_runtime.h>
#include <nvml.h>

#include <mscclpp/env.hpp>
#include <mscclpp/errors.hpp>

#include "logger.hpp"

namespace mscclpp {

namespace {

int64_t nowMs() {
  using namespace std::chrono;
  return duration_cast<milliseconds>(steady_clock::now().time_since_epoch()).count();
}

void checkAbort(const std::atomic<uint32_t>* abortFlag, const char* what) {
  if (abortFlag && abortFlag->load(std::memory_order_acquire) != 0) {
    throw Error(std::string(what) + " aborted", ErrorCode::Aborted);
  }
}

uint64_t fnv1a(const std::string& s) {
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : s) {
    h ^= c;
    h *= 1099511628211ull;
  }
  return h;
}

bool matchIfSpec(const std::string& name, const std::string& spec) {
  // spec without the leading ^ ; "=name" exact, otherwise prefix; comma separated
  size_t pos = 0;
  while (pos <= spec.size()) {
    size_t comma = spec.find(',', pos);
    if (comma == std::string::npos) comma = spec.size();
    std::string tok = spec.substr(pos, comma - pos);
    if (!tok.empty()) {
      if (tok[0] == '=') {
        if (name == tok.substr(1)) return true;
      } else if (name.compare(0, tok.size(), tok) == 0) {
        return true;
      }
    }
    pos = comma + 1;
  }
  return false;
}

}  // namespace

uint16_t SocketAddress::port() const {
  if (storage.ss_family == AF_INET) return ntohs(reinterpret_cast<const sockaddr_in*>(&storage)->sin_port);
  if (storage.ss_family == AF_INET6) return ntohs(reinterpret_cast<const sockaddr_in6*>(&storage)->sin6_port);
  return 0;
}

void SocketAddress::setPort(uint16_t port) {
  if (storage.ss_family == AF_INET) reinterpret_cast<sockaddr_in*>(&storage)->sin_port = htons(port);
  if (storage.ss_family == AF_INET6) reinterpret_cast<sockaddr_in6*>(&storage)->sin6_port = htons(port);
}

std::string SocketAddress::toString(bool withPort) const {
  char buf[INET6_ADDRSTRLEN] = {0};
  std::string out;
  if (storage.ss_family == AF_INET) {
    inet_ntop(AF_INET, &reinterpret_cast<const sockaddr_in*>(&storage)->sin_addr, buf, sizeof(buf));
    out = buf;
  } else if (storage.ss_family == AF_INET6) {
    inet_ntop(AF_INET6, &reinterpret_cast<const sockaddr_in6*>(&storage)->sin6_addr, buf, sizeof(buf));
    out = std::string("[") + buf + "]";
  } else {
    return "<unspecified>";
  }
  if (withPort) out += ":" + std::to_string(port());
  return out;
}

SocketAddress SocketAddress::parse(const std::string& text, uint16_t defaultPort) {
  std::string host = text, portStr;
  if (!text.empty() && text[0] == '[') {
    size_t close = text.find(']');
    if (close == std::string::npos) throw Error("bad address: " + text, ErrorCode::InvalidUsage);
    host = text.substr(1, close - 1);
    if (close + 1 < text.size() && text[close + 1] == ':') portStr = text.substr(close + 2);
  } else {
    size_t colon = text.rfind(':');
    if (colon != std::string::npos && text.find(':') == colon) {
      host = text.substr(0, colon);
      portStr = text.substr(colon + 1);
    }
  }
  addrinfo hints{};
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  addrinfo* res = nullptr;
  int rc = getaddrinfo(host.c_str(), nullptr, &hints, &res);
  if (rc != 0 || res == nullptr) throw Error("cannot resolve address: " + text, ErrorCode::InvalidUsage);
  SocketAddress out;
  std::memcpy(&out.storage, res->ai_addr, res->ai_addrlen);
  out.length = res->ai_addrlen;
  freeaddrinfo(res);
  out.setPort(portStr.empty() ? defaultPort : static_cast<uint16_t>(std::stoi(portStr)));
  return out;
}

bool SocketAddress::sameHost(const SocketAddress& other) const {
  if (storage.ss_family != other.storage.ss_family) return false;
  if (storage.ss_family == AF_INET) {
    return reinterpret_cast<const sockaddr_in*>(&storage)->sin_addr.s_addr ==
           reinterpret_cast<const sockaddr_in*>(&other.storage)->sin_addr.s_addr;
  }
  if (storage.ss_family == AF_INET6) {
    return std::memcmp(&reinterpret_cast<const sockaddr_in6*>(&storage)->sin6_addr,
                       &reinterpret_cast<const sockaddr_in6*>(&other.storage)->sin6_addr, sizeof(in6_addr)) == 0;
  }
  return false;
}

std::vector<NetInterface> findInterfaces(const std::string& specIn, int family, int maxCount) {
  std::vector<NetInterface> preferred, loopbacks;
  ifaddrs* list = nullptr;
  if (getifaddrs(&list) != 0) return preferred;
  std::string spec = specIn;
  bool exclude = false;
  if (!spec.empty() && spec[0] == '^') {
    exclude = true;
    spec = spec.substr(1);
  }
  for (ifaddrs* it = list; it != nullptr; it = it->ifa_next) {
    if (it->ifa_addr == nullptr) continue;
    int fam = it->ifa_addr->sa_family;
    if (fam != AF_INET && fam != AF_INET6) continue;
    if (family != AF_UNSPEC && fam != family) continue;
    if (!(it->ifa_flags & IFF_UP)) continue;
    std::string name(it->ifa_name);
    if (fam == AF_INET6) {
      auto* a6 = reinterpret_cast<sockaddr_in6*>(it->ifa_addr);
      if (IN6_IS_ADDR_LINKLOCAL(&a6->sin6_addr)) continue;
    }
    NetInterface ni;
    ni.name = name;
    ni.address.length = fam == AF_INET ? sizeof(sockaddr_in) : sizeof(sockaddr_in6);
    std::memcpy(&ni.address.storage, it->ifa_addr, ni.address.length);
    if (!spec.empty()) {
      bool m = matchIfSpec(name, spec);
      if (m == exclude) continue;
      preferred.push_back(ni);
    } else {
      const bool isLoop = (it->ifa_flags & IFF_LOOPBACK) != 0;
      const bool isDocker = name.compare(0, 6, "docker") == 0;
      if (isLoop || isDocker) loopbacks.push_back(ni);
      else preferred.push_back(ni);
    }
  }
  freeifaddrs(list);
  // IPv4 first: it is what "ip:port" strings usually carry
  std::stable_sort(preferred.begin(), preferred.end(),
                   [](const NetInterface& a, const NetInterface& b) { return a.address.family() == AF_INET && b.address.family() != AF_INET; });
  if (preferred.empty()) preferred = loopbacks;
  if (static_cast<int>(preferred.size()) > maxCount) preferred.resize(maxCount);
  return preferred;
}

bool findInterfaceMatchingSubnet(const SocketAddress& remote, NetInterface* out) {
  ifaddrs* list = nullptr;
  if (getifaddrs(&list) != 0) return false;
  bool found = false;
  for (ifaddrs* it = list; it != nullptr && !found; it = it->ifa_next) {
    if (it->ifa_addr == nullptr || it->ifa_netmask == nullptr) continue;
    if (it->ifa_addr->sa_family != remote.family() || !(it->ifa_flags & IFF_UP)) continue;
    if (remote.family() == AF_INET) {
      uint32_t a = reinterpret_cast<sockaddr_in*>(it->ifa_addr)->sin_addr.s_addr;
      uint32_t m = reinterpret_cast<sockaddr_in*>(it->ifa_netmask)->sin_addr.s_addr;
      uint32_t r = reinterpret_cast<const sockaddr_in*>(&remote.storage)->sin_addr.s_addr;
      if ((a & m) == (r & m)) found = true;
    } else if (remote.family() == AF_INET6) {
      auto* a = reinterpret_cast<sockaddr_in6*>(it->ifa_addr)->sin6_addr.s6_addr;
      auto* m = reinterpret_cast<sockaddr_in6*>(it->ifa_netmask)->sin6_addr.s6_addr;
      auto* r = reinterpret_cast<const sockaddr_in6*>(&remote.storage)->sin6_addr.s6_addr;
      found = true;
      for (int i = 0; i < 16; i++)
        if ((a[i] & m[i]) != (r[i] & m[i])) found = false;
    }
    if (found && out) {
      out->name = it->ifa_name;
      out->address.length = remote.family() == AF_INET ? sizeof(sockaddr_in) : sizeof(sockaddr_in6);
      std::memcpy(&out->address.storage, it->ifa_addr, out->address.length);
    }
  }
  freeifaddrs(list);
  return found;
}

Socket::~Socket() { close(); }
Socket::Socket(Socket&& o) noexcept : fd_(o.fd_) { o.fd_ = -1; }
Socket& Socket::operator=(Socket&& o) noexcept {
  if (this != &o) {
    close();
    fd_ = o.fd_;
    o.fd_ = -1;
  }
  return *this;
}

void Socket::close() {
  if (fd_ >= 0) {
    ::close(fd_);
    fd_ = -1;
  }
}

SocketAddress Socket::listen(const SocketAddress& addr, int backlog) {
  close();
  fd_ = ::socket(addr.family(), SOCK_STREAM, 0);
  if (fd_ < 0) throw SysError("socket() failed", errno);
  int one = 1;
  setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  if (::bind(fd_, reinterpret_cast<const sockaddr*>(&addr.storage), addr.length) != 0) {
    int e = errno;
    close();
    throw SysError("bind(" + addr.toString() + ") failed", e);
  }
  if (::listen(fd_, backlog) != 0) {
    int e = errno;
    close();
    throw SysError("listen() failed", e);
  }
  SocketAddress bound;
  bound.length = sizeof(bound.storage);
  if (getsockname(fd_, reinterpret_cast<sockaddr*>(&bound.storage), &bound.length) != 0) {
    throw SysError("getsockname() failed", errno);
  }
  return bound;
}

Socket Socket::accept(int64_t timeoutMs, const std::atomic<uint32_t>* abortFlag) {
  const int64_t deadline = timeoutMs < 0 ? -1 : nowMs() + timeoutMs;
  while (true) {
    checkAbort(abortFlag, "accept");
    pollfd p{fd_, POLLIN, 0};
    int rc = ::poll(&p, 1, 50);
    if (rc < 0 && errno != EINTR) throw SysError("poll() failed in accept", errno);
    if (rc > 0 && (p.revents & POLLIN)) {
      int cfd = ::accept(fd_, nullptr, nullptr);
      if (cfd < 0) {
        if (errno == EINTR || errno == EAGAIN || errno == ECONNABORTED) continue;
        throw SysError("accept() failed", errno);
      }
      Socket s(cfd);
      int one = 1;
      setsockopt(cfd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      uint64_t magic = 0;
      try {
        s.recvAll(&magic, sizeof(magic), 5000, abortFlag);
      } catch (const BaseError&) {
        continue;  // port scanner or a peer that died right after connecting
      }
      if (magic != kSocketMagic) {
        LOG_WARN(LogSubsys::NET, "dropping a connection with a wrong magic word");
        continue;
      }
      return s;
    }
    if (deadline >= 0 && nowMs() > deadline) throw Error("accept timed out", ErrorCode::Timeout);
  }
}

void Socket::connect(const SocketAddress& addr, int64_t timeoutMs, const std::atomic<uint32_t>* abortFlag) {
  const int64_t deadline = timeoutMs < 0 ? -1 : nowMs() + timeoutMs;
  int backoffMs = 1;
  while (true) {
    checkAbort(abortFlag, "connect");
    close();
    fd_ = ::socket(addr.family(), SOCK_STREAM, 0);
    if (fd_ < 0) throw SysError("socket() failed", errno);
    int rc = ::connect(fd_, reinterpret_cast<const sockaddr*>(&addr.storage), addr.length);
    if (rc == 0) break;
    int e = errno;
    if (e != ECONNREFUSED && e != ETIMEDOUT && e != EINTR && e != EAGAIN && e != ENETUNREACH && e != EHOSTUNREACH) {
      close();
      throw SysError("connect(" + addr.toString() + ") failed", e);
    }
    if (deadline >= 0 && nowMs() > deadline) {
      close();
      throw Error("connect(" + addr.toString() + ") timed out", ErrorCode::Timeout);
    }
    usleep(backoffMs * 1000);
    if (backoffMs < 64) backoffMs *= 2;
  }
  int one = 1;
  setsockopt(fd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  uint64_t magic = kSocketMagic;
  sendAll(&magic, sizeof(magic), timeoutMs, abortFlag);
}

void Socket::sendAll(const void* data, size_t bytes, int64_t timeoutMs, const std::atomic<uint32_t>* abortFlag) {
  const int64_t deadline = timeoutMs < 0 ? -1 : nowMs() + timeoutMs;
  const char* p = static_cast<const char*>(data);
  size_t done = 0;
  while (done < bytes) {
    checkAbort(abortFlag, "send");
    pollfd pf{fd_, POLLOUT, 0};
    int rc = ::poll(&pf, 1, 50);
    if (rc < 0 && errno != EINTR) throw SysError("poll() failed in send", errno);
    if (rc > 0) {
      ssize_t n = ::send(fd_, p + done, bytes - done, MSG_NOSIGNAL | MSG_DONTWAIT);
      if (n < 0) {
        if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
        throw SysError("send() failed", errno);
      }
      done += static_cast<size_t>(n);
      continue;
    }
    if (deadline >= 0 && nowMs() > deadline) throw Error("send timed out", ErrorCode::Timeout);
  }
}

void Socket::recvAll(void* data, size_t bytes, int64_t timeoutMs, const std::atomic<uint32_t>* abortFlag) {
  const int64_t deadline = timeoutMs < 0 ? -1 : nowMs() + timeoutMs;
  char* p = static_cast<char*>(data);
  size_t done = 0;
  while (done < bytes) {
    checkAbort(abortFlag, "recv");
    pollfd pf{fd_, POLLIN, 0};
    int rc = ::poll(&pf, 1, 50);
    if (rc < 0 && errno != EINTR) throw SysError("poll() failed in recv", errno);
    if (rc > 0) {
      ssize_t n = ::recv(fd_, p + done, bytes - done, MSG_DONTWAIT);
      if (n == 0) throw Error("peer closed the connection", ErrorCode::RemoteError);
      if (n < 0) {
        if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
        throw SysError("recv() failed", errno);
      }
      done += static_cast<size_t>(n);
      continue;
    }
    if (deadline >= 0 && nowMs() > deadline) throw Error("recv timed out", ErrorCode::Timeout);
  }
}

bool Socket::readable(int timeoutMs) {
  pollfd pf{fd_, POLLIN, 0};
  return ::poll(&pf, 1, timeoutMs) > 0;
}

uint64_t getHostHash() {
  std::string id = env()->hostid;
  if (id.empty()) {
    char host[256] = {0};
    gethostname(host, sizeof(host) - 1);
    id = host;
    std::ifstream boot("/proc/sys/kernel/random/boot_id");
    std::string bootId;
    if (boot && std::getline(boot, bootId)) id += bootId;
  }
  return fnv1a(id);
}

namespace {
// NVML is loaded on demand (it is part of the driver, absent on machines without one). True when the current CUDA device
// reports a completed, healthy fabric registration; then `hash` covers cluster id + clique.
bool fabricDomainHash(uint64_t& hash) {
  int dev = 0;
  char busId[32] = {0};
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetPCIBusId(busId, sizeof(busId), dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  void* lib = ::dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
  if (lib == nullptr) return false;
  using InitFn = nvmlReturn_t (*)();
  using HandleFn = nvmlReturn_t (*)(const char*, nvmlDevice_t*);
  using FabricFn = nvmlReturn_t (*)(nvmlDevice_t, nvmlGpuFabricInfoV_t*);
  auto init = reinterpret_cast<InitFn>(::dlsym(lib, "nvmlInit_v2"));
  auto shutdown = reinterpret_cast<InitFn>(::dlsym(lib, "nvmlShutdown"));
  auto byBusId = reinterpret_cast<HandleFn>(::dlsym(lib, "nvmlDeviceGetHandleByPciBusId_v2"));
  auto fabric = reinterpret_cast<FabricFn>(::dlsym(lib, "nvmlDeviceGetGpuFabricInfoV"));
  bool ok = false;
  if (init != nullptr && shutdown != nullptr && byBusId != nullptr && fabric != nullptr && init() == NVML_SUCCESS) {
    nvmlDevice_t handle;
    nvmlGpuFabricInfoV_t info{};
    info.version = nvmlGpuFabricInfo_v2;
    if (byBusId(busId, &handle) == NVML_SUCCESS && fabric(handle, &info) == NVML_SUCCESS &&
        info.state == NVML_GPU_FABRIC_STATE_COMPLETED && info.status == NVML_SUCCESS) {
      std::string id(reinterpret_cast<const char*>(info.clusterUuid), sizeof(info.clusterUuid));
      bool allZero = true;
      for (char c : id) allZero = allZero && c == 0;
      if (!allZero) {
        id += ":" + std::to_string(info.cliqueId);
        hash = fnv1a(id);
        ok = true;
      }
    }
    (void)shutdown();
  }
  ::dlclose(lib);
  return ok;
}
}  // namespace

uint64_t getIpcDomainHash() {
  if (const char* forced = std::getenv("MSCCLPP_IPC_DOMAIN")) {
    if (forced[0] != '\0') return fnv1a(std::string("domain:") + forced);
  }
  uint64_t h = 0;
  if (fabricDomainHash(h)) return h;
  return getHostHash();
}

uint64_t getPidHash() {
  std::string id = std::to_string(getpid());
  char link[256] = {0};
  ssize_t n = readlink("/proc/self/ns/pid", link, sizeof(link) - 1);
  if (n > 0) id += std::string(link, static_cast<size_t>(n));
  return fnv1a(id);
}

}  // namespace mscclpp
