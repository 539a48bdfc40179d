// Host-only unit tests of the C++ core: errors, transport flags, FIFO protocol, bootstrap (threads as ranks),
// Ethernet connection + host semaphores, execution-plan parsing errors. No GPU needed.
#include <thread>

#include <mscclpp/core.hpp>
#include <mscclpp/errors.hpp>
#include <mscclpp/executor.hpp>
#include <mscclpp/semaphore.hpp>

#include "framework.hpp"

using namespace mscclpp;

TEST(Errors, CodesAndMessages) {
  try {
    throw Error("bad call", ErrorCode::InvalidUsage);
  } catch (const Error& e) {
    EXPECT_EQ(static_cast<int>(e.getErrorCode()), static_cast<int>(ErrorCode::InvalidUsage));
    EXPECT_TRUE(std::string(e.what()).find("bad call") != std::string::npos);
  }
  EXPECT_THROW(throw SysError("x", 2), BaseError);
}

TEST(Transport, FlagsAlgebra) {
  TransportFlags f = TransportFlags(Transport::CudaIpc) | Transport::Ethernet;
  EXPECT_TRUE(f.has(Transport::CudaIpc));
  EXPECT_TRUE(f.has(Transport::Ethernet));
  EXPECT_TRUE(!f.has(Transport::IB0));
  EXPECT_EQ(f.count(), size_t(2));
  EXPECT_TRUE((f & TransportFlags(Transport::IB0)).none());
}

static void runRanks(int n, const std::function<void(int, std::shared_ptr<TcpBootstrap>)>& fn) {
  UniqueId id = TcpBootstrap::createUniqueId();
  std::vector<std::thread> threads;
  for (int r = 0; r < n; r++) {
    threads.emplace_back([&, r] {
      auto b = std::make_shared<TcpBootstrap>(r, n);
      b->initialize(id, 30);
      fn(r, b);
    });
  }
  for (auto& t : threads) t.join();
}

TEST(Bootstrap, AllGatherBarrierSendRecv) {
  const int n = 4;
  std::vector<int> sums(n, 0);
  testing::Timer timer;
  runRanks(n, [&](int r, std::shared_ptr<TcpBootstrap> b) {
    std::vector<int> all(n, -1);
    all[r] = r * 10;
    b->allGather(all.data(), sizeof(int));
    for (int v : all) sums[r] += v;
    b->barrier();
    std::vector<char> msg = {static_cast<char>('a' + r)};
    b->send(msg, (r + 1) % n, 7);
    std::vector<char> got;
    b->recv(got, (r + n - 1) % n, 7);
    if (got.size() != 1 || got[0] != static_cast<char>('a' + (r + n - 1) % n)) sums[r] = -1;
    b->barrier();
  });
  for (int r = 0; r < n; r++) EXPECT_EQ(sums[r], 60);
  testing::reportPerf("bootstrap_4_ranks_setup_and_exchange", timer.elapsedUs(), "us");
}

TEST(Bootstrap, IpcDomains) {
  const int n = 4;
  std::vector<int> perDomain(n, 0), perNode(n, 0);
  // one host, no NVLink fabric: the domain is the node
  runRanks(n, [&](int r, std::shared_ptr<TcpBootstrap> b) {
    perDomain[r] = b->getNranksPerIpcDomain();
    perNode[r] = b->getNranksPerNode();
  });
  for (int r = 0; r < n; r++) EXPECT_EQ(perDomain[r], perNode[r]);
  // two domains of two consecutive ranks
  ::setenv("MSCCLPP_IPC_DOMAIN", "a,a,b,b", 1);
  runRanks(n, [&](int r, std::shared_ptr<TcpBootstrap> b) { perDomain[r] = b->getNranksPerIpcDomain(); });
  for (int r = 0; r < n; r++) EXPECT_EQ(perDomain[r], 2);
  // interleaved domains and domains of different sizes are refused on every rank
  for (const char* layout : {"a,b,a,b", "a,a,a,b"}) {
    ::setenv("MSCCLPP_IPC_DOMAIN", layout, 1);
    std::vector<int> refused(n, 0);
    runRanks(n, [&](int r, std::shared_ptr<TcpBootstrap> b) {
      try {
        (void)b->getNranksPerIpcDomain();
      } catch (const Error& e) {
        refused[r] = e.getErrorCode() == ErrorCode::InvalidUsage;
      }
    });
    for (int r = 0; r < n; r++) EXPECT_EQ(refused[r], 1);
  }
  ::unsetenv("MSCCLPP_IPC_DOMAIN");
}

TEST(Ethernet, WriteAndHostSemaphore) {
  std::vector<uint64_t> received(2, 0);
  runRanks(2, [&](int r, std::shared_ptr<TcpBootstrap> b) {
    Communicator comm(b);
    const int peer = 1 - r;
    std::vector<uint64_t> buf(64, r == 0 ? 0x1111 : 0);
    Connection conn = comm.connect(EndpointConfig(Transport::Ethernet, Device(DeviceType::CPU)), peer).get();
    RegisteredMemory local = comm.registerMemory(buf.data(), buf.size() * 8, Transport::Ethernet);
    comm.sendMemory(local, peer);
    RegisteredMemory remote = comm.recvMemory(peer).get();
    Host2HostSemaphore sem(comm, conn);
    if (r == 0) {
      conn.write(remote, 0, local, 0, buf.size() * 8);
      conn.flush();
      sem.signal();
    } else {
      sem.wait();
      received[1] = buf[63];
    }
    b->barrier();
  });
  EXPECT_EQ(received[1], uint64_t(0x1111));
}

TEST(ExecutionPlan, MalformedJsonIsRejected) {
  EXPECT_THROW(ExecutionPlan::fromString("{\"name\": \"x\"", 0), BaseError);
  EXPECT_THROW(ExecutionPlan::fromString("{\"name\": \"x\", \"collective\": \"allreduce\"}", 0), BaseError);
}

int main(int argc, char** argv) { return testing::runAll(argc, argv); }
