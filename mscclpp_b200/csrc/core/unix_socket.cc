#include "unix_socket.hpp"

#include <cerrno>
#include <chrono>
#include <cstring>
#include <poll.h>
#include <random>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <mscclpp/errors.hpp>

#include "logger.hpp"

namespace mscclpp {

namespace {

struct FdRequest {
  uint32_t magic;
  uint32_t id;
};
struct FdReply {
  uint32_t magic;
  int32_t status;  // 0 = fd attached, otherwise an errno-like code
};
constexpr uint32_t kFdMagic = 0xfd5e12b2u;

sockaddr_un abstractAddress(const std::string& name, socklen_t* len) {
  sockaddr_un addr{};
  addr.sun_family = AF_UNIX;
  // abstract namespace: sun_path[0] == '\0', no file system entry, vanishes with the process
  const size_t n = std::min(name.size(), sizeof(addr.sun_path) - 2);
  std::memcpy(addr.sun_path + 1, name.data(), n);
  *len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
  return addr;
}

void sendReply(int sock, int32_t status, int fd) {
  FdReply reply{kFdMagic, status};
  iovec iov{&reply, sizeof(reply)};
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  if (status == 0 && fd >= 0) {
    std::memset(control, 0, sizeof(control));
    msg.msg_control = control;
    msg.msg_controllen = sizeof(control);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  if (::sendmsg(sock, &msg, MSG_NOSIGNAL) < 0) {
    LOG_WARN(LogSubsys::NET, "fd server: sendmsg failed: ", std::strerror(errno));
  }
}

}  // namespace

UnixFdServer& UnixFdServer::instance() {
  static UnixFdServer server;
  return server;
}

UnixFdServer::UnixFdServer() {
  std::random_device rd;
  name_ = "mscclpp_b200_fd_" + std::to_string(getpid()) + "_" + std::to_string(rd());
  listenFd_ = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (listenFd_ < 0) throw SysError("socket(AF_UNIX) failed", errno);
  socklen_t len = 0;
  sockaddr_un addr = abstractAddress(name_, &len);
  if (::bind(listenFd_, reinterpret_cast<sockaddr*>(&addr), len) != 0) throw SysError("bind(AF_UNIX) failed", errno);
  if (::listen(listenFd_, 128) != 0) throw SysError("listen(AF_UNIX) failed", errno);
  thread_ = std::thread([this] { serve(); });
}

UnixFdServer::~UnixFdServer() { stop(); }

void UnixFdServer::stop() {
  if (stop_.exchange(true)) return;
  if (thread_.joinable()) thread_.join();
  if (listenFd_ >= 0) ::close(listenFd_);
  listenFd_ = -1;
  std::lock_guard<std::mutex> lock(mutex_);
  for (auto& kv : fds_) ::close(kv.second);
  fds_.clear();
}

uint32_t UnixFdServer::registerFd(int fd) {
  int copy = ::dup(fd);
  if (copy < 0) throw SysError("dup() failed", errno);
  std::lock_guard<std::mutex> lock(mutex_);
  uint32_t id = nextId_++;
  fds_[id] = copy;
  return id;
}

void UnixFdServer::unregisterFd(uint32_t id) {
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = fds_.find(id);
  if (it != fds_.end()) {
    ::close(it->second);
    fds_.erase(it);
  }
}

void UnixFdServer::serve() {
  while (!stop_.load()) {
    pollfd p{listenFd_, POLLIN, 0};
    int rc = ::poll(&p, 1, 100);
    if (rc <= 0) continue;
    int conn = ::accept4(listenFd_, nullptr, nullptr, SOCK_CLOEXEC);
    if (conn < 0) continue;
    // a connection may carry several requests; it ends when the peer closes it
    while (!stop_.load()) {
      pollfd cp{conn, POLLIN, 0};
      if (::poll(&cp, 1, 2000) <= 0) break;
      FdRequest req{};
      ssize_t n = ::recv(conn, &req, sizeof(req), MSG_WAITALL);
      if (n != static_cast<ssize_t>(sizeof(req)) || req.magic != kFdMagic) break;
      int fd = -1;
      {
        std::lock_guard<std::mutex> lock(mutex_);
        auto it = fds_.find(req.id);
        if (it != fds_.end()) fd = it->second;
      }
      sendReply(conn, fd >= 0 ? 0 : ENOENT, fd);
    }
    ::close(conn);
  }
}

int requestFdFromPeer(const std::string& serverName, uint32_t id, int timeoutMs) {
  using namespace std::chrono;
  const auto deadline = steady_clock::now() + milliseconds(timeoutMs);
  int sock = -1;
  while (true) {
    sock = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (sock < 0) throw SysError("socket(AF_UNIX) failed", errno);
    socklen_t len = 0;
    sockaddr_un addr = abstractAddress(serverName, &len);
    if (::connect(sock, reinterpret_cast<sockaddr*>(&addr), len) == 0) break;
    int e = errno;
    ::close(sock);
    if (steady_clock::now() > deadline) {
      if (e == ECONNREFUSED || e == ENOENT) throw Error("fd server '" + serverName + "' is not reachable", ErrorCode::Timeout);
      throw SysError("connect(AF_UNIX) failed", e);
    }
    usleep(2000);
  }
  FdRequest req{kFdMagic, id};
  if (::send(sock, &req, sizeof(req), MSG_NOSIGNAL) != static_cast<ssize_t>(sizeof(req))) {
    int e = errno;
    ::close(sock);
    throw SysError("send to fd server failed", e);
  }
  pollfd p{sock, POLLIN, 0};
  if (::poll(&p, 1, timeoutMs) <= 0) {
    ::close(sock);
    throw Error("fd server '" + serverName + "' did not answer", ErrorCode::Timeout);
  }
  FdReply reply{};
  iovec iov{&reply, sizeof(reply)};
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  std::memset(control, 0, sizeof(control));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = control;
  msg.msg_controllen = sizeof(control);
  ssize_t n = ::recvmsg(sock, &msg, MSG_CMSG_CLOEXEC);
  ::close(sock);
  if (n != static_cast<ssize_t>(sizeof(reply)) || reply.magic != kFdMagic) {
    throw Error("malformed reply from fd server", ErrorCode::RemoteError);
  }
  if (reply.status != 0) throw Error("fd server does not know descriptor id " + std::to_string(id), ErrorCode::RemoteError);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (c == nullptr || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) {
    throw Error("fd server reply carries no descriptor", ErrorCode::RemoteError);
  }
  int fd = -1;
  std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
  return fd;
}

}  // namespace mscclpp
