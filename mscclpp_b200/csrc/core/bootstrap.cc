// TcpBootstrap: rendezvous through a hub thread on rank 0, then direct peer sockets.
//
// Reference behaviour covered (src/core/bootstrap/bootstrap.cc:135-611): 128-byte UniqueId carrying the
// root address, "ip:port" initialisation, per-(peer, tag) ordered send/recv, allGather, barrier,
// broadcast, ranks-per-node discovery, connect/accept timeouts surfacing as ErrorCode::Timeout and an
// abort flag. The topology differs on purpose: instead of wiring a ring through the root, the root
// publishes the full address table once, so any pair can open a socket lazily without a third party.
#include <mscclpp/core.hpp>

#include <cstdlib>
#include <functional>
#include <sstream>

#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <thread>
#include <netinet/in.h>
#include <random>

#include <mscclpp/env.hpp>

#include "logger.hpp"
#include "socket.hpp"

namespace mscclpp {

// ------------------------------------------------------------------------------------------ Bootstrap helpers
void Bootstrap::groupBarrier(const std::vector<int>& ranks) {
  // dissemination barrier over the listed ranks, using a tag nobody else uses
  const int tag = 0x7ffe0000;
  int me = -1;
  const int n = static_cast<int>(ranks.size());
  for (int i = 0; i < n; i++)
    if (ranks[i] == getRank()) me = i;
  if (me < 0) throw Error("groupBarrier: calling rank is not in the group", ErrorCode::InvalidUsage);
  for (int dist = 1; dist < n; dist <<= 1) {
    int token = dist;
    int to = ranks[(me + dist) % n], from = ranks[(me - dist + n) % n];
    send(&token, sizeof(token), to, tag);
    recv(&token, sizeof(token), from, tag);
  }
}

void Bootstrap::send(const std::vector<char>& data, int peer, int tag) {
  uint64_t size = data.size();
  send(&size, sizeof(size), peer, tag);
  if (size > 0) send(const_cast<char*>(data.data()), static_cast<int>(size), peer, tag);
}

void Bootstrap::recv(std::vector<char>& data, int peer, int tag) {
  uint64_t size = 0;
  recv(&size, sizeof(size), peer, tag);
  data.resize(size);
  if (size > 0) recv(data.data(), static_cast<int>(size), peer, tag);
}

// ------------------------------------------------------------------------------------------ TcpBootstrap
namespace {

constexpr uint64_t kIdMagic = 0xb200c0117ec7ed01ull;
constexpr int kRingTag = 0x7fff0001;
constexpr int kBcastTag = 0x7fff0002;

// sockaddr_storage alone is 128 bytes; the id carries the root address in a compact form instead.
struct CompactAddress {
  uint16_t family;
  uint16_t port;
  uint32_t scope;
  uint8_t bytes[16];

  static CompactAddress from(const SocketAddress& a) {
    CompactAddress c{};
    c.family = static_cast<uint16_t>(a.family());
    c.port = a.port();
    if (a.family() == AF_INET) {
      std::memcpy(c.bytes, &reinterpret_cast<const sockaddr_in*>(&a.storage)->sin_addr, 4);
    } else if (a.family() == AF_INET6) {
      auto* s6 = reinterpret_cast<const sockaddr_in6*>(&a.storage);
      std::memcpy(c.bytes, &s6->sin6_addr, 16);
      c.scope = s6->sin6_scope_id;
    }
    return c;
  }
  SocketAddress expand() const {
    SocketAddress a;
    if (family == AF_INET) {
      auto* s4 = reinterpret_cast<sockaddr_in*>(&a.storage);
      s4->sin_family = AF_INET;
      std::memcpy(&s4->sin_addr, bytes, 4);
      a.length = sizeof(sockaddr_in);
    } else {
      auto* s6 = reinterpret_cast<sockaddr_in6*>(&a.storage);
      s6->sin6_family = AF_INET6;
      std::memcpy(&s6->sin6_addr, bytes, 16);
      s6->sin6_scope_id = scope;
      a.length = sizeof(sockaddr_in6);
    }
    a.setPort(port);
    return a;
  }
};

struct IdPayload {
  uint64_t magic;
  CompactAddress rootCompact;
  uint64_t nonce;
};
static_assert(sizeof(IdPayload) <= UniqueIdBytes, "UniqueId too small for a socket address");

struct RankInfo {
  int rank;
  int nRanks;
  uint64_t hostHash;
  SocketAddress listen;
};

struct PeerHello {
  int srcRank;
  int tag;
};

SocketAddress pickLocalAddress(const SocketAddress* towards) {
  const std::string spec = env()->socketIfname;
  int family = AF_UNSPEC;
  if (env()->socketFamily == "AF_INET") family = AF_INET;
  if (env()->socketFamily == "AF_INET6") family = AF_INET6;
  if (spec.empty() && towards != nullptr) {
    NetInterface ni;
    if (findInterfaceMatchingSubnet(*towards, &ni)) {
      ni.address.setPort(0);
      return ni.address;
    }
  }
  auto ifs = findInterfaces(spec, family, 1);
  if (ifs.empty()) throw Error("no usable network interface (MSCCLPP_SOCKET_IFNAME=" + spec + ")", ErrorCode::SystemError);
  SocketAddress a = ifs[0].address;
  a.setPort(0);
  return a;
}

}  // namespace

class TcpBootstrap::Impl {
 public:
  int rank;
  int nRanks;
  bool initialized = false;
  std::atomic<uint32_t> abortFlag{0};
  int64_t timeoutMs = 30000;

  UniqueId uniqueId{};
  bool haveId = false;
  Socket rootListen;  // rank 0 only
  std::thread rootThread;
  std::string rootError;
  ErrorCode rootErrorCode = ErrorCode::InternalError;

  Socket peerListen;
  std::vector<RankInfo> table;
  int nRanksPerNode = 1;
  int nRanksPerIpcDomain = 0;  // 0 = not determined yet

  std::mutex mutex;
  std::map<std::pair<int, int>, Socket> sendSocks;
  std::map<std::pair<int, int>, Socket> recvSocks;

  Impl(int r, int n) : rank(r), nRanks(n) {
    if (n <= 0 || r < 0 || r >= n) throw Error("TcpBootstrap: bad rank/nRanks", ErrorCode::InvalidUsage);
  }

  ~Impl() {
    abortFlag.store(1);
    if (rootThread.joinable()) rootThread.join();
  }

  IdPayload idPayload() const {
    IdPayload p;
    std::memcpy(&p, uniqueId.data(), sizeof(p));
    return p;
  }

  void makeId() {
    SocketAddress local = pickLocalAddress(nullptr);
    SocketAddress bound = rootListen.listen(local);
    IdPayload p{};
    p.magic = kIdMagic;
    p.rootCompact = CompactAddress::from(bound);
    p.nonce = std::random_device{}();
    uniqueId.fill(0);
    std::memcpy(uniqueId.data(), &p, sizeof(p));
    haveId = true;
  }

  void runRoot() {
    // collect one RankInfo per rank, then hand the whole table to everybody
    try {
      std::vector<Socket> conns(nRanks);
      std::vector<RankInfo> infos(nRanks);
      std::vector<bool> seen(nRanks, false);
      for (int i = 0; i < nRanks; i++) {
        Socket s = rootListen.accept(timeoutMs, &abortFlag);
        RankInfo info{};
        s.recvAll(&info, sizeof(info), timeoutMs, &abortFlag);
        if (info.nRanks != nRanks) throw Error("rank " + std::to_string(info.rank) + " reports a different world size", ErrorCode::InvalidUsage);
        if (info.rank < 0 || info.rank >= nRanks || seen[info.rank]) throw Error("duplicate or invalid rank " + std::to_string(info.rank) + " at rendezvous", ErrorCode::InvalidUsage);
        seen[info.rank] = true;
        infos[info.rank] = info;
        conns[info.rank] = std::move(s);
      }
      for (int r = 0; r < nRanks; r++) conns[r].sendAll(infos.data(), sizeof(RankInfo) * nRanks, timeoutMs, &abortFlag);
    } catch (const Error& e) {
      rootError = e.what();
      rootErrorCode = e.getErrorCode();
      LOG_WARN(LogSubsys::NET, "bootstrap root failed: ", rootError);
    } catch (const std::exception& e) {
      rootError = e.what();
      LOG_WARN(LogSubsys::NET, "bootstrap root failed: ", rootError);
    }
    rootListen.close();
  }

  void establish(int64_t timeoutSec) {
    timeoutMs = timeoutSec < 0 ? -1 : timeoutSec * 1000;
    IdPayload id = idPayload();
    if (id.magic != kIdMagic) throw Error("invalid UniqueId", ErrorCode::InvalidUsage);
    const SocketAddress rootAddr = id.rootCompact.expand();
    if (rank == 0) {
      if (!rootListen.valid()) {
        // id came from the static createUniqueId(): claim the advertised port now
        rootListen.listen(rootAddr);
      }
      rootThread = std::thread([this] { runRoot(); });
    }
    SocketAddress local = pickLocalAddress(&rootAddr);
    SocketAddress myListen = peerListen.listen(local);
    RankInfo mine{};
    mine.rank = rank;
    mine.nRanks = nRanks;
    mine.hostHash = getHostHash();
    mine.listen = myListen;
    Socket toRoot;
    toRoot.connect(rootAddr, timeoutMs, &abortFlag);
    toRoot.sendAll(&mine, sizeof(mine), timeoutMs, &abortFlag);
    table.resize(nRanks);
    try {
      toRoot.recvAll(table.data(), sizeof(RankInfo) * nRanks, timeoutMs, &abortFlag);
    } catch (const BaseError&) {
      // Rank 0 talks to its own root thread. When that thread gave up (a rank never joined) it dropped every
      // connection, which this side sees as "peer closed": report the root's reason (Timeout) instead.
      if (rank == 0 && rootThread.joinable()) {
        rootThread.join();
        if (!rootError.empty()) throw Error(rootError, rootErrorCode);
      }
      throw;
    }
    if (rank == 0 && rootThread.joinable()) rootThread.join();
    nRanksPerNode = 0;
    for (int r = 0; r < nRanks; r++)
      if (table[r].hostHash == table[rank].hostHash) nRanksPerNode++;
    initialized = true;
    LOG_INFO(LogSubsys::NET, "bootstrap rank ", rank, "/", nRanks, " listening on ", myListen.toString(), ", ",
             nRanksPerNode, " ranks on this node");
  }

  Socket& sendSocket(int peer, int tag) {
    auto key = std::make_pair(peer, tag);
    auto it = sendSocks.find(key);
    if (it != sendSocks.end()) return it->second;
    Socket s;
    s.connect(table[peer].listen, timeoutMs, &abortFlag);
    PeerHello hello{rank, tag};
    s.sendAll(&hello, sizeof(hello), timeoutMs, &abortFlag);
    return sendSocks.emplace(key, std::move(s)).first->second;
  }

  Socket& recvSocket(int peer, int tag) {
    auto key = std::make_pair(peer, tag);
    while (true) {
      auto it = recvSocks.find(key);
      if (it != recvSocks.end()) return it->second;
      // accept connections (from anybody) until the wanted one shows up; park the others
      Socket s = peerListen.accept(timeoutMs, &abortFlag);
      PeerHello hello{};
      s.recvAll(&hello, sizeof(hello), timeoutMs, &abortFlag);
      recvSocks.emplace(std::make_pair(hello.srcRank, hello.tag), std::move(s));
    }
  }

  void checkInit() const {
    if (!initialized) throw Error("TcpBootstrap is not initialized", ErrorCode::InvalidUsage);
  }

  void sendTo(const void* data, int size, int peer, int tag) {
    checkInit();
    if (peer < 0 || peer >= nRanks) throw Error("send: bad peer", ErrorCode::InvalidUsage);
    if (peer == rank) {
      std::lock_guard<std::mutex> lock(mutex);
      auto& q = selfQueue[tag];
      q.emplace_back(static_cast<const char*>(data), static_cast<const char*>(data) + size);
      return;
    }
    std::unique_lock<std::mutex> lock(mutex);
    Socket& s = sendSocket(peer, tag);
    lock.unlock();
    s.sendAll(data, size, timeoutMs, &abortFlag);
  }

  void recvFrom(void* data, int size, int peer, int tag) {
    checkInit();
    if (peer < 0 || peer >= nRanks) throw Error("recv: bad peer", ErrorCode::InvalidUsage);
    if (peer == rank) {
      std::lock_guard<std::mutex> lock(mutex);
      auto& q = selfQueue[tag];
      if (q.empty() || static_cast<int>(q.front().size()) != size) throw Error("recv from self without a matching send", ErrorCode::InvalidUsage);
      std::memcpy(data, q.front().data(), size);
      q.erase(q.begin());
      return;
    }
    std::unique_lock<std::mutex> lock(mutex);
    Socket& s = recvSocket(peer, tag);
    lock.unlock();
    s.recvAll(data, size, timeoutMs, &abortFlag);
  }

  std::map<int, std::vector<std::vector<char>>> selfQueue;
};

UniqueId TcpBootstrap::createUniqueId() {
  // Reserve an ephemeral port, publish it, release it: rank 0 re-binds it in initialize().
  Socket probe;
  SocketAddress bound = probe.listen(pickLocalAddress(nullptr));
  probe.close();
  IdPayload p{};
  p.magic = kIdMagic;
  p.rootCompact = CompactAddress::from(bound);
  p.nonce = std::random_device{}();
  UniqueId id{};
  std::memcpy(id.data(), &p, sizeof(p));
  return id;
}

TcpBootstrap::TcpBootstrap(int rank, int nRanks) : pimpl_(std::make_unique<Impl>(rank, nRanks)) {}
TcpBootstrap::~TcpBootstrap() = default;

UniqueId TcpBootstrap::getUniqueId() const {
  if (!pimpl_->haveId) pimpl_->makeId();
  return pimpl_->uniqueId;
}

void TcpBootstrap::initialize(UniqueId uniqueId, int64_t timeoutSec) {
  if (!(pimpl_->haveId && pimpl_->uniqueId == uniqueId)) {
    pimpl_->uniqueId = uniqueId;
    pimpl_->haveId = true;
  }
  pimpl_->establish(timeoutSec);
}

void TcpBootstrap::initialize(const std::string& ifIpPortTrio, int64_t timeoutSec) {
  // "ip:port" or "ifname:ip:port" ([ip6]:port also accepted)
  std::string spec = ifIpPortTrio;
  size_t first = spec.find(':');
  if (first != std::string::npos && spec[0] != '[') {
    std::string head = spec.substr(0, first);
    bool looksLikeIp = !head.empty() && (std::isdigit(static_cast<unsigned char>(head[0])) != 0);
    size_t colons = 0;
    for (char c : spec) colons += (c == ':');
    if (!looksLikeIp && colons >= 2) spec = spec.substr(first + 1);  // drop the interface name
  }
  IdPayload p{};
  p.magic = kIdMagic;
  p.rootCompact = CompactAddress::from(SocketAddress::parse(spec));
  if (p.rootCompact.port == 0) throw Error("initialize: a port is required in '" + ifIpPortTrio + "'", ErrorCode::InvalidUsage);
  pimpl_->uniqueId.fill(0);
  std::memcpy(pimpl_->uniqueId.data(), &p, sizeof(p));
  pimpl_->haveId = true;
  pimpl_->establish(timeoutSec);
}

void TcpBootstrap::abort() { pimpl_->abortFlag.store(1, std::memory_order_release); }

int TcpBootstrap::getRank() const { return pimpl_->rank; }
int TcpBootstrap::getNranks() const { return pimpl_->nRanks; }
int TcpBootstrap::getNranksPerNode() const { return pimpl_->nRanksPerNode; }
// Ranks that can map one another's GPU memory: the ranks of this host, widened to this NVLink fabric clique when the
// GPUs are part of one (reference: src/core/bootstrap/bootstrap.cc:459-493). Collective on first use (an allGather of
// host and fabric hashes). Domains must have equal sizes and hold consecutive ranks, which the channel and plan code
// relies on: an explicit layout (MSCCLPP_IPC_DOMAIN="a,a,b,b", one name per rank) that breaks the rule is refused; a
// detected fabric layout that breaks it is ignored with a warning and the hosts are the domains.
int TcpBootstrap::getNranksPerIpcDomain() const {
  Impl& impl = *pimpl_;
  impl.checkInit();
  if (impl.nRanksPerIpcDomain > 0) return impl.nRanksPerIpcDomain;
  struct Entry {
    uint64_t host, domain;
    uint32_t forced;
  };
  std::vector<Entry> all(impl.nRanks, Entry{0, 0, 0});
  Entry& me = all[impl.rank];
  me.host = getHostHash();
  me.domain = getIpcDomainHash();
  if (const char* forced = std::getenv("MSCCLPP_IPC_DOMAIN")) {
    std::vector<std::string> names;
    std::stringstream ss(forced);
    for (std::string item; std::getline(ss, item, ',');) names.push_back(item);
    if (!names.empty() && forced[0] != '\0') me.forced = 1;
    if (names.size() > 1) me.domain = std::hash<std::string>{}("domain:" + names[impl.rank % names.size()]);
  }
  const_cast<TcpBootstrap*>(this)->allGather(all.data(), sizeof(Entry));
  bool forced = false;
  for (const Entry& e : all) forced = forced || e.forced != 0;

  // size of this rank's domain under `key`, or a description of why the layout cannot be used
  auto layout = [&](auto key, std::string& problem) {
    int mine = 0;
    for (const Entry& e : all) mine += key(e) == key(all[impl.rank]) ? 1 : 0;
    if (impl.nRanks % mine != 0) {
      problem = std::to_string(impl.nRanks) + " ranks do not divide into domains of " + std::to_string(mine);
      return 0;
    }
    for (int r = 0; r < impl.nRanks; r++) {
      const int first = r - r % mine;
      if (key(all[r]) != key(all[first])) {
        problem = "rank " + std::to_string(r) + " is not in the domain of rank " + std::to_string(first);
        return 0;
      }
      if (r % mine == 0 && r > 0 && key(all[r]) == key(all[r - mine])) {
        problem = "the domain of rank " + std::to_string(r) + " is larger than that of rank " + std::to_string(impl.rank);
        return 0;
      }
    }
    return mine;
  };
  const std::string rule = "IPC domains must have equal sizes and hold consecutive ranks: ";
  std::string problem;
  int mine = layout([](const Entry& e) { return e.domain; }, problem);
  if (forced) {
    if (mine == 0) throw Error(rule + problem, ErrorCode::InvalidUsage);
  } else {
    std::string hostProblem;
    const int perHost = layout([](const Entry& e) { return e.host; }, hostProblem);
    if (mine == 0 || (perHost > 0 && mine < perHost)) {
      // a fabric layout that cannot be used, or one that would split a host: processes of one host can always share memory
      if (mine == 0) LOG_WARN(LogSubsys::NET, "ignoring the detected NVLink fabric layout (", problem, "): hosts are the IPC domains");
      mine = perHost > 0 ? perHost : impl.nRanksPerNode;
    }
  }
  LOG_INFO(LogSubsys::NET, "rank ", impl.rank, ": ", mine, " ranks per IPC domain");
  impl.nRanksPerIpcDomain = mine;
  return mine;
}

void TcpBootstrap::send(void* data, int size, int peer, int tag) { pimpl_->sendTo(data, size, peer, tag); }
void TcpBootstrap::recv(void* data, int size, int peer, int tag) { pimpl_->recvFrom(data, size, peer, tag); }

void TcpBootstrap::allGather(void* allData, int size) {
  pimpl_->checkInit();
  const int n = pimpl_->nRanks, r = pimpl_->rank;
  if (n == 1) return;
  char* base = static_cast<char*>(allData);
  const int next = (r + 1) % n, prev = (r - 1 + n) % n;
  // ring: in step i forward the slot received in step i-1
  for (int i = 0; i < n - 1; i++) {
    const int sendSlot = (r - i + n) % n, recvSlot = (r - i - 1 + n) % n;
    pimpl_->sendTo(base + static_cast<size_t>(sendSlot) * size, size, next, kRingTag);
    pimpl_->recvFrom(base + static_cast<size_t>(recvSlot) * size, size, prev, kRingTag);
  }
}

void TcpBootstrap::broadcast(void* data, int size, int root) {
  pimpl_->checkInit();
  const int n = pimpl_->nRanks, r = pimpl_->rank;
  if (n == 1) return;
  // binomial tree rooted at `root`
  const int rel = (r - root + n) % n;
  int mask = 1;
  while (mask < n) {
    if (rel & mask) {
      pimpl_->recvFrom(data, size, ((rel - mask) + root) % n, kBcastTag);
      break;
    }
    mask <<= 1;
  }
  mask >>= 1;
  while (mask > 0) {
    if (rel + mask < n) pimpl_->sendTo(data, size, ((rel + mask) + root) % n, kBcastTag);
    mask >>= 1;
  }
}

void TcpBootstrap::barrier() {
  std::vector<int> tokens(pimpl_->nRanks, 0);
  allGather(tokens.data(), sizeof(int));
}

}  // namespace mscclpp
