// File-descriptor hand-over between processes of one host (SCM_RIGHTS over an abstract AF_UNIX
// socket). A process runs one UnixFdServer thread; peers ask it for descriptors it registered.
// This is how POSIX-fd handles of CUDA VMM allocations and multicast objects travel between ranks
// (role of the reference's UnixSocketServer/Client, src/core/unix_socket.cc:51-272).
#pragma once

#include <atomic>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <thread>

namespace mscclpp {

class UnixFdServer {
 public:
  // Process-wide instance, started on first use.
  static UnixFdServer& instance();
  ~UnixFdServer();

  // Name peers connect to (abstract namespace, unique per process).
  const std::string& name() const { return name_; }
  // Makes `fd` available to peers under the returned id. The server keeps its own dup of the fd.
  uint32_t registerFd(int fd);
  void unregisterFd(uint32_t id);
  void stop();

 private:
  UnixFdServer();
  void serve();
  std::string name_;
  int listenFd_ = -1;
  std::thread thread_;
  std::atomic<bool> stop_{false};
  std::mutex mutex_;
  std::map<uint32_t, int> fds_;
  uint32_t nextId_ = 1;
};

// Fetches descriptor `id` from the server called `serverName`. The caller owns the returned fd.
// Throws Error(Timeout / RemoteError) when the server does not answer or does not know the id.
int requestFdFromPeer(const std::string& serverName, uint32_t id, int timeoutMs = 10000);

}  // namespace mscclpp
