// InfiniBand transport against the software verbs provider (tests/cpp/fake_ibverbs.cc) and the GDRCopy wrapper against
// tests/cpp/fake_gdrapi.cc: no HCA, no GPU. The launcher sets MSCCLPP_IBV_SO and MSCCLPP_GDRCOPY_SO to the two libraries.
// Both "ranks" of every test live in this process, each with a Context of its own, and talk through serialised
// endpoints and memories exactly as two processes would.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include <mscclpp/core.hpp>
#include <mscclpp/semaphore.hpp>
#include <mscclpp/utils.hpp>

#include "core/gdr.hpp"
#include "core/ib.hpp"
#include "framework.hpp"

using namespace mscclpp;
using Mode = EndpointConfig::Ib::Mode;

namespace {

struct Pair {
  std::shared_ptr<Context> ctxA = Context::create();
  std::shared_ptr<Context> ctxB = Context::create();
  Endpoint epA, epB;
  Connection ab, ba;

  explicit Pair(Mode mode, int maxSendWr = EndpointConfig::Ib::DefaultMaxSendWr, Mode modeB = Mode::Default) {
    EndpointConfig ca(Transport::IB0, Device(DeviceType::CPU));
    EndpointConfig cb(Transport::IB1, Device(DeviceType::CPU));
    ca.ib.mode = mode;
    cb.ib.mode = modeB == Mode::Default ? mode : modeB;
    ca.ib.maxSendWr = cb.ib.maxSendWr = maxSendWr;
    epA = ctxA->createEndpoint(ca);
    epB = ctxB->createEndpoint(cb);
    ab = ctxA->connect(epA, Endpoint::deserialize(epB.serialize()));
    ba = ctxB->connect(epB, Endpoint::deserialize(epA.serialize()));
  }
};

RegisteredMemory asSeenByPeer(const RegisteredMemory& m) { return RegisteredMemory::deserialize(m.serialize()); }

// Waits by the clock, not by a spin count: on a loaded machine with few cores the peer thread may not run for a while.
void waitFor(Host2HostSemaphore& sem, double seconds = 30.0) {
  testing::Timer t;
  while (!sem.poll()) {
    if (t.elapsedUs() > seconds * 1e6) throw Error("the peer's signal did not arrive", ErrorCode::Timeout);
    std::this_thread::yield();
  }
}

}  // namespace

TEST(IbvTable, LoadsTheProviderAndListsItsDevices) {
  ASSERT_TRUE(IbvApi::available());
  const std::vector<std::string> names = ibDeviceNamesFromLibrary();
  ASSERT_EQ(names.size(), size_t(2));
  EXPECT_EQ(names[0], std::string("fake0"));
  EXPECT_EQ(getIBDeviceCount(), 2);
  EXPECT_EQ(getIBDeviceName(Transport::IB1), std::string("fake1"));
  EXPECT_TRUE(getIBTransportByDeviceName("fake1") == Transport::IB1);
  EXPECT_THROW(getIBDeviceName(Transport::IB5), Error);
  EXPECT_THROW(IbCtx("mlx5_99"), IbError);
}

TEST(IbQp, StateMachineWritesAndAtomics) {
  IbCtx a("fake0"), b("fake1");
  EXPECT_TRUE(a.supportsRdmaAtomics());
  EXPECT_TRUE(a.isPortUsable(1, -1));
  EXPECT_TRUE(!a.isPortUsable(2, -1));
  EXPECT_EQ(a.anyUsablePort(-1), 1);
  EXPECT_EQ(a.anyUsablePort(9), -1);  // the port has four GIDs
  const IbQp::Limits limits{64, 16, 32, 4, 8};
  auto qa = a.createQp(-1, -1, limits);
  auto qb = b.createQp(1, -1, limits);
  EXPECT_TRUE(qa->info().qpn != qb->info().qpn);
  EXPECT_EQ(int(qa->info().useGrh), 0);
  EXPECT_THROW(b.createQp(2, -1, limits), Error);

  std::vector<uint64_t> src(1024), dst(1024, 0);
  for (size_t i = 0; i < src.size(); i++) src[i] = i * 3 + 1;
  auto mrSrc = a.registerMr(src.data(), src.size() * 8);
  auto mrDst = b.registerMr(dst.data(), dst.size() * 8);

  // posting before the pair is connected is refused by the device
  qa->stageWrite(*mrSrc, mrDst->info(), 64, 1, 0, 0, true);
  EXPECT_THROW(qa->postSend(), IbError);
  EXPECT_EQ(qa->numStaged(), 0);

  qa->rtr(qb->info());
  qa->rts();
  qb->rtr(qa->info());  // fake1's port runs at a smaller MTU: both sides must settle on it
  qb->rts();
  EXPECT_THROW(qa->rtr(qb->info()), IbError);  // not twice

  // eight requests in one chain, the last one signalled
  for (int i = 0; i < 8; i++) qa->stageWrite(*mrSrc, mrDst->info(), 1024, 10 + i, i * 1024, i * 1024, i == 7);
  EXPECT_THROW(qa->stageWrite(*mrSrc, mrDst->info(), 8, 99, 0, 0, false), Error);  // maxWrPerSend
  qa->postSend();
  EXPECT_EQ(qa->outstandingSignaled(), 1);
  int n = 0;
  while ((n = qa->pollSendCq()) == 0) {
  }
  ASSERT_EQ(n, 1);
  EXPECT_EQ(qa->sendWc(0).wr_id, uint64_t(17));
  EXPECT_EQ(int(qa->sendWc(0).status), int(IBV_WC_SUCCESS));
  EXPECT_EQ(qa->outstandingSignaled(), 0);
  EXPECT_TRUE(std::memcmp(src.data(), dst.data(), 8 * 1024) == 0);

  // fetch-and-add on word 5 of the destination; the old value lands locally
  uint64_t landing = 0;
  auto mrLanding = a.registerMr(&landing, 8);
  const uint64_t before = dst[5];
  qa->stageAtomicAdd(*mrLanding, mrDst->info(), 20, 5 * 8, 1000, true);
  qa->postSend();
  while (qa->pollSendCq() == 0) {
  }
  EXPECT_EQ(dst[5], before + 1000);
  EXPECT_EQ(landing, before);
}

TEST(IbConnection, WriteTokenAndFlushBetweenTwoContexts) {
  Pair p(Mode::Host);
  EXPECT_TRUE(p.ab.transport() == Transport::IB0);
  EXPECT_TRUE(p.ab.remoteTransport() == Transport::IB1);
  std::vector<char> src(1 << 20), dst(1 << 20, 0);
  for (size_t i = 0; i < src.size(); i++) src[i] = static_cast<char>(i * 7 + 3);
  RegisteredMemory memSrc = p.ctxA->registerMemory(src.data(), src.size(), Transport::IB0);
  RegisteredMemory memDst = p.ctxB->registerMemory(dst.data(), dst.size(), Transport::IB1);
  RegisteredMemory remoteDst = asSeenByPeer(memDst);
  EXPECT_TRUE(remoteDst.transports().has(Transport::IB1));

  p.ab.write(remoteDst, 4096, memSrc, 0, (1 << 20) - 4096);
  p.ab.flush(5000000);
  EXPECT_TRUE(std::memcmp(dst.data() + 4096, src.data(), (1 << 20) - 4096) == 0);
  EXPECT_EQ(int(dst[0]), 0);

  // token: the peer's word follows the local one
  alignas(8) uint64_t token = 0;
  uint64_t mine = 0;
  RegisteredMemory memToken = p.ctxB->registerMemory(&token, 8, Transport::IB1);
  RegisteredMemory remoteToken = asSeenByPeer(memToken);
  p.ab.updateAndSync(remoteToken, 0, &mine, 5);
  p.ab.updateAndSync(remoteToken, 0, &mine, 9);
  p.ab.flush();
  EXPECT_EQ(mine, uint64_t(9));
  EXPECT_EQ(token, uint64_t(9));

  // contract violations are caught before anything is posted
  EXPECT_THROW(p.ab.write(remoteDst, (1 << 20) - 8, memSrc, 0, 64), Error);
  RegisteredMemory wrongTransport = p.ctxA->registerMemory(src.data(), 64, Transport::IB1);
  EXPECT_THROW(p.ab.write(remoteDst, 0, wrongTransport, 0, 64), Error);
  EXPECT_THROW(p.ab.write(remoteDst, 0, asSeenByPeer(memSrc), 0, 64), Error);  // the source must be local
}

TEST(IbConnection, ManyWritesStayWithinTheSendQueue) {
  Pair p(Mode::Host, /*maxSendWr=*/8);
  std::vector<uint32_t> src(4096), dst(4096, 0);
  for (size_t i = 0; i < src.size(); i++) src[i] = static_cast<uint32_t>(i ^ 0x5a5a);
  RegisteredMemory memSrc = p.ctxA->registerMemory(src.data(), src.size() * 4, Transport::IB0);
  RegisteredMemory memDst = p.ctxB->registerMemory(dst.data(), dst.size() * 4, Transport::IB1);
  RegisteredMemory remoteDst = asSeenByPeer(memDst);
  for (int i = 0; i < 1024; i++) p.ab.write(remoteDst, i * 16, memSrc, i * 16, 16);  // far more than the queue holds
  p.ab.flush(5000000);
  EXPECT_TRUE(src == dst);
}

TEST(IbConnection, RemoteFaultSurfacesInFlush) {
  Pair p(Mode::Host);
  std::vector<char> src(4096, 1);
  auto dst = std::make_unique<std::vector<char>>(4096, 0);
  RegisteredMemory memSrc = p.ctxA->registerMemory(src.data(), src.size(), Transport::IB0);
  RegisteredMemory remoteDst;
  {
    RegisteredMemory memDst = p.ctxB->registerMemory(dst->data(), dst->size(), Transport::IB1);
    remoteDst = asSeenByPeer(memDst);
  }  // the owner drops its registration: the remote key is stale now
  p.ab.write(remoteDst, 0, memSrc, 0, 4096);
  bool remoteError = false;
  try {
    p.ab.flush(5000000);
  } catch (const Error& e) {
    remoteError = e.getErrorCode() == ErrorCode::RemoteError && std::string(e.what()).find("remote access") != std::string::npos;
  }
  EXPECT_TRUE(remoteError);
  EXPECT_EQ(int((*dst)[0]), 0);
  // the queue pair is gone for good: later calls say so at once instead of waiting for completions that cannot come
  EXPECT_THROW(p.ab.write(remoteDst, 0, memSrc, 0, 64), Error);
  EXPECT_THROW(p.ab.flush(), Error);
}

TEST(IbConnection, FlushGivesUpAfterItsTimeLimit) {
  Pair p(Mode::Host);
  std::vector<char> src(256, 1), dst(256, 0);
  RegisteredMemory memSrc = p.ctxA->registerMemory(src.data(), src.size(), Transport::IB0);
  RegisteredMemory memDst = p.ctxB->registerMemory(dst.data(), dst.size(), Transport::IB1);
  RegisteredMemory remoteDst = asSeenByPeer(memDst);
  ::setenv("FAKE_IBV_DROP_COMPLETIONS", "1", 1);
  p.ab.write(remoteDst, 0, memSrc, 0, 256);
  ::unsetenv("FAKE_IBV_DROP_COMPLETIONS");
  bool timedOut = false;
  testing::Timer t;
  try {
    p.ab.flush(20000);
  } catch (const Error& e) {
    timedOut = e.getErrorCode() == ErrorCode::Timeout;
  }
  EXPECT_TRUE(timedOut);
  EXPECT_TRUE(t.elapsedUs() >= 20000 && t.elapsedUs() < 2000000);
}

TEST(IbConnection, BothSidesMustAgreeOnTheTokenMode) {
  bool refused = false;
  try {
    Pair p(Mode::Host, EndpointConfig::Ib::DefaultMaxSendWr, Mode::HostNoAtomic);
  } catch (const Error& e) {
    refused = e.getErrorCode() == ErrorCode::InvalidUsage;
  }
  EXPECT_TRUE(refused);
}

TEST(IbConnection, DevicesWithoutAtomicsFallBackToImmediateData) {
  ::setenv("FAKE_IBV_NO_ATOMICS", "1", 1);
  {
    Pair p(Mode::Host);  // asked for atomics, the devices have none
    alignas(8) uint64_t token = 0;
    uint64_t mine = 0;
    RegisteredMemory memToken = p.ctxB->registerMemory(&token, 8, Transport::IB1);
    RegisteredMemory remoteToken = asSeenByPeer(memToken);
    p.ab.updateAndSync(remoteToken, 0, &mine, 1);
    p.ab.flush(5000000);
    EXPECT_EQ(token, uint64_t(0));  // nothing was added remotely: the value travelled as immediate data to a receive
  }
  ::unsetenv("FAKE_IBV_NO_ATOMICS");
}

static void pingPong(Mode mode, int rounds) {
  Pair p(mode);
  SemaphoreStub stubA(p.ab), stubB(p.ba);
  Semaphore semA(stubA, SemaphoreStub::deserialize(stubB.serialize()));
  Semaphore semB(stubB, SemaphoreStub::deserialize(stubA.serialize()));
  Host2HostSemaphore a(semA), b(semB);
  std::vector<uint64_t> payload(512, 0), landed(512, 0);
  RegisteredMemory memPayload = p.ctxA->registerMemory(payload.data(), payload.size() * 8, Transport::IB0);
  RegisteredMemory memLanded = p.ctxB->registerMemory(landed.data(), landed.size() * 8, Transport::IB1);
  RegisteredMemory remoteLanded = asSeenByPeer(memLanded);
  std::atomic<int> bad{0};
  std::thread peer([&] {
    for (int r = 1; r <= rounds; r++) {
      waitFor(b);
      // the token is ordered after the write that preceded it
      for (uint64_t v : landed) bad += (v != uint64_t(r));
      b.signal();
    }
    b.connection().flush(5000000);
  });
  for (int r = 1; r <= rounds; r++) {
    for (auto& v : payload) v = r;
    p.ab.write(remoteLanded, 0, memPayload, 0, payload.size() * 8);
    a.signal();
    waitFor(a);
  }
  p.ab.flush(5000000);
  peer.join();
  EXPECT_EQ(bad.load(), 0);
}

TEST(IbSemaphore, HostToHostPingPongWithRdmaAtomics) { pingPong(Mode::Host, 200); }
TEST(IbSemaphore, HostToHostPingPongWithImmediateData) { pingPong(Mode::HostNoAtomic, 200); }

TEST(IbSemaphore, RoceNeedsGlobalRouting) {
  ::setenv("FAKE_IBV_ROCE", "1", 1);
  {
    IbCtx a("fake0");
    auto q = a.createQp(-1, -1, IbQp::Limits{16, 8, 8, 2, 4});
    EXPECT_EQ(int(q->info().useGrh), 1);
    EXPECT_TRUE(q->info().interfaceId != 0);
  }
  pingPong(Mode::Host, 5);  // the device refuses an address vector without a GID here
  ::unsetenv("FAKE_IBV_ROCE");
}

TEST(IbCommunicator, TwoRanksOverTheBootstrap) {
  // the whole path a program takes: bootstrap, Communicator::connect with an InfiniBand endpoint per rank (IB0 faces IB1),
  // memory exchange, semaphore construction, write + signal in both directions
  UniqueId id = TcpBootstrap::createUniqueId();
  std::vector<uint64_t> seen(2, 0);
  std::vector<std::string> errors(2);
  std::vector<std::thread> ranks;
  for (int r = 0; r < 2; r++) {
    ranks.emplace_back([&, r] {
      try {
        auto bootstrap = std::make_shared<TcpBootstrap>(r, 2);
        bootstrap->initialize(id, 30);
        Communicator comm(bootstrap);
        const int peer = 1 - r;
        const Transport mine = r == 0 ? Transport::IB0 : Transport::IB1;
        std::vector<uint64_t> buf(256, r == 0 ? 0xabcd0000ull : 0);
        Connection conn = comm.connect(EndpointConfig(mine, Device(DeviceType::CPU)), peer).get();
        RegisteredMemory local = comm.registerMemory(buf.data(), buf.size() * 8, mine);
        comm.sendMemory(local, peer);
        RegisteredMemory remote = comm.recvMemory(peer).get();
        Host2HostSemaphore sem(comm, conn);
        if (r == 0) {
          for (size_t i = 0; i < buf.size(); i++) buf[i] += i;
          conn.write(remote, 0, local, 0, buf.size() * 8);
          sem.signal();
          conn.flush(5000000);
          waitFor(sem);  // the peer's answer
          seen[0] = buf[0];
        } else {
          waitFor(sem);
          seen[1] = buf[255];
          buf[0] = 0x600d;
          conn.write(remote, 0, local, 0, 8);
          sem.signal();
          conn.flush(5000000);
        }
        bootstrap->barrier();
      } catch (const std::exception& e) {
        errors[r] = e.what();
      }
    });
  }
  for (auto& t : ranks) t.join();
  EXPECT_EQ(errors[0], std::string());
  EXPECT_EQ(errors[1], std::string());
  EXPECT_EQ(seen[1], uint64_t(0xabcd0000ull + 255));
  EXPECT_EQ(seen[0], uint64_t(0x600d));
}

TEST(Gdr, MapsThePageAroundAnAddress) {
  ASSERT_TRUE(gdrAvailability().usable);
  EXPECT_EQ(gdrAvailability().reason, std::string("GDRCopy is available"));
  char* block = static_cast<char*>(std::aligned_alloc(65536, 3 * 65536));
  std::memset(block, 0, 3 * 65536);
  uint64_t* word = reinterpret_cast<uint64_t*>(block + 65536 + 4096 + 24);
  {
    auto window = GdrWindow::open(word, -1);
    ASSERT_TRUE(window != nullptr);
    EXPECT_TRUE(window->word() == word);
    window->store(0x1122334455667788ull);
    EXPECT_EQ(*word, 0x1122334455667788ull);
    EXPECT_EQ(window->load(), 0x1122334455667788ull);
  }
  EXPECT_TRUE(GdrWindow::open(nullptr, -1) == nullptr);
  std::free(block);
}

int main(int argc, char** argv) { return testing::runAll(argc, argv); }
