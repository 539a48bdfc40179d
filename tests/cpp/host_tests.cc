// Host-only unit tests of the pieces below the Communicator: sockets (addresses, loopback transfer, deadlines),
// descriptor passing over AF_UNIX, the JSON reader, the algorithm registry and its selectors, the environment singleton
// and the execution-plan loader on a plan produced by the DSL (path in MSCCLPP_TEST_PLAN). No GPU needed.
#include <unistd.h>

#include <sched.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

#include <mscclpp/algorithm.hpp>
#include <mscclpp/core.hpp>
#include <mscclpp/env.hpp>
#include <mscclpp/errors.hpp>
#include <mscclpp/executor.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/numa.hpp>
#include <mscclpp/proxy.hpp>
#include <mscclpp/utils.hpp>
#include <mscclpp/version.hpp>
#include <mscclpp/device.hpp>

#include "core/json.hpp"
#include "core/range_allocator.hpp"
#include "core/socket.hpp"
#include "core/unix_socket.hpp"
#include <mscclpp/ext/collectives/algorithm_collection_builder.hpp>

#include "framework.hpp"

using namespace mscclpp;

TEST(SocketAddress, ParseAndPrint) {
  SocketAddress a = SocketAddress::parse("127.0.0.1:4321");
  EXPECT_EQ(a.family(), AF_INET);
  EXPECT_EQ(a.port(), uint16_t(4321));
  EXPECT_EQ(a.toString(), std::string("127.0.0.1:4321"));
  EXPECT_EQ(a.toString(false), std::string("127.0.0.1"));
  SocketAddress b = SocketAddress::parse("[::1]:80");
  EXPECT_EQ(b.family(), AF_INET6);
  EXPECT_EQ(b.port(), uint16_t(80));
  SocketAddress c = SocketAddress::parse("127.0.0.1", 99);
  EXPECT_EQ(c.port(), uint16_t(99));
  c.setPort(100);
  EXPECT_EQ(c.port(), uint16_t(100));
  EXPECT_TRUE(a.sameHost(c));
  EXPECT_TRUE(!a.sameHost(b));
}

TEST(Socket, LoopbackTransferOfOneMegabyte) {
  Socket listener;
  SocketAddress bound = listener.listen(SocketAddress::parse("127.0.0.1:0"));
  EXPECT_TRUE(bound.port() != 0);
  const size_t n = 1 << 20;
  std::vector<uint8_t> sent(n), got(n, 0);
  for (size_t i = 0; i < n; i++) sent[i] = static_cast<uint8_t>(i * 131 + 7);
  testing::Timer timer;
  std::thread client([&] {
    Socket s;
    s.connect(bound, 5000);
    s.sendAll(sent.data(), n, 5000);
    uint32_t ack = 0;
    s.recvAll(&ack, sizeof(ack), 5000);
    if (ack != 0xabcd) sent[0] ^= 0xff;  // makes the comparison below fail
  });
  Socket peer = listener.accept(5000);
  EXPECT_TRUE(peer.valid());
  peer.recvAll(got.data(), n, 5000);
  uint32_t ack = 0xabcd;
  peer.sendAll(&ack, sizeof(ack), 5000);
  client.join();
  EXPECT_TRUE(std::memcmp(sent.data(), got.data(), n) == 0);
  testing::reportPerf("socket_loopback_1MB", timer.elapsedUs(), "us");
}

TEST(Socket, DeadlinesAndAbortFlag) {
  Socket listener;
  SocketAddress bound = listener.listen(SocketAddress::parse("127.0.0.1:0"));
  // nobody connects: accept gives up at its deadline
  auto t0 = std::chrono::steady_clock::now();
  EXPECT_THROW(listener.accept(200), BaseError);
  auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
  EXPECT_TRUE(ms >= 150 && ms < 3000);
  // an abort flag raised by another thread ends a long wait early
  std::atomic<uint32_t> abortFlag{0};
  std::thread raiser([&] {
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
    abortFlag.store(1);
  });
  t0 = std::chrono::steady_clock::now();
  EXPECT_THROW(listener.accept(20000, &abortFlag), BaseError);
  ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
  raiser.join();
  EXPECT_TRUE(ms < 5000);
  // a peer that connects but sends nothing: recvAll gives up, readable() says no
  std::thread client([&] {
    Socket s;
    s.connect(bound, 5000);
    std::this_thread::sleep_for(std::chrono::milliseconds(600));
  });
  Socket peer = listener.accept(5000);
  EXPECT_TRUE(!peer.readable(50));
  char byte;
  EXPECT_THROW(peer.recvAll(&byte, 1, 200), BaseError);
  client.join();
}

TEST(Socket, InterfaceDiscovery) {
  auto all = findInterfaces("^nonexistent", AF_UNSPEC);
  EXPECT_TRUE(!all.empty());  // at least loopback
  auto lo = findInterfaces("=lo", AF_INET);
  for (const auto& itf : lo) EXPECT_EQ(itf.name, std::string("lo"));
  EXPECT_TRUE(getHostHash() == getHostHash());
  EXPECT_TRUE(getPidHash() == getPidHash());
}

TEST(UnixFd, DescriptorTravelsThroughTheServer) {
  int fds[2];
  ASSERT_TRUE(::pipe(fds) == 0);
  UnixFdServer& server = UnixFdServer::instance();
  const uint32_t id = server.registerFd(fds[1]);
  int received = -1;
  std::thread peer([&] { received = requestFdFromPeer(server.name(), id, 5000); });
  peer.join();
  ASSERT_TRUE(received >= 0);
  EXPECT_TRUE(received != fds[1]);  // a new descriptor for the same pipe
  const char msg[] = "through the duplicate";
  ASSERT_TRUE(::write(received, msg, sizeof(msg)) == static_cast<ssize_t>(sizeof(msg)));
  char back[64] = {0};
  ASSERT_TRUE(::read(fds[0], back, sizeof(back)) == static_cast<ssize_t>(sizeof(msg)));
  EXPECT_EQ(std::string(back), std::string(msg));
  EXPECT_THROW(requestFdFromPeer(server.name(), id + 1000, 1000), BaseError);  // unknown id
  server.unregisterFd(id);
  EXPECT_THROW(requestFdFromPeer(server.name(), id, 1000), BaseError);
  ::close(received);
  ::close(fds[0]);
  ::close(fds[1]);
}

TEST(Json, ValuesNestingAndErrors) {
  json::Value v = json::parse(R"({"name": "plan \"a\"\n", "n": 42, "neg": -7, "x": 1.5e2, "ok": true, "none": null,
                                  "list": [1, [2, 3], {"k": "v"}], "big": 18446744073709551615})");
  EXPECT_EQ(v.at("name").asString(), std::string("plan \"a\"\n"));
  EXPECT_EQ(v.at("n").asInt(), int64_t(42));
  EXPECT_EQ(v.at("neg").asInt(), int64_t(-7));
  EXPECT_EQ(v.at("x").asInt(), int64_t(150));
  EXPECT_TRUE(v.at("ok").asBool());
  EXPECT_TRUE(v.contains("none") && !v.contains("missing"));
  EXPECT_EQ(v.at("list").size(), size_t(3));
  EXPECT_EQ(v.at("list").at(1).at(1).asInt(), int64_t(3));
  EXPECT_EQ(v.at("list").at(2).at("k").asString(), std::string("v"));
  EXPECT_EQ(v.at("big").asUInt(), UINT64_MAX);
  EXPECT_EQ(v.intOr("missing", 5), int64_t(5));
  EXPECT_THROW(v.at("missing"), BaseError);
  EXPECT_THROW(v.at("n").asString(), BaseError);
  EXPECT_THROW(v.at("neg").asUInt(), BaseError);
  EXPECT_THROW(json::parse("{\"a\": [1, 2"), BaseError);
  EXPECT_THROW(json::parse("{\"a\" 1}"), BaseError);
  EXPECT_THROW(json::parse(""), BaseError);
}

static std::shared_ptr<Algorithm> dummyAlgo(const std::string& name, const std::string& collective, size_t lo, size_t hi, int* calls) {
  return std::make_shared<NativeAlgorithm>(
      name, collective, [](std::shared_ptr<Communicator>) {},
      [calls](const void*, void*, size_t, size_t, DataType, ReduceOp, cudaStream_t, int, int, bool,
              const std::unordered_map<std::string, uintptr_t>&) {
        (*calls)++;
        return CommResult::Success;
      },
      lo, hi);
}

TEST(DefaultSelector, SizesWorldsAndBufferPlacement) {
  // the registered names with stand-in kernels; ranges as buildDefaultAlgorithms gives them on eight and on two ranks
  using Map = std::unordered_map<std::string, std::unordered_map<std::string, std::shared_ptr<Algorithm>>>;
  int calls = 0;
  auto build = [&](int world) {
    Map m;
    auto add = [&](const char* coll, const char* name, uint64_t lo, uint64_t hi) { m[coll][name] = dummyAlgo(name, coll, lo, hi, &calls); };
    add("allreduce", "default_allreduce_packet", 0, 8u << 20);
    add("allreduce", "default_allreduce_nvls_packet", 0, 8u << 20);
    add("allreduce", "default_allreduce_packet_ll128", 0, world <= 2 ? (4u << 20) : (world <= 4 ? (512u << 10) : (256u << 10)));
    add("allreduce", "default_allreduce_nvls_zero_copy", 0, UINT64_MAX);
    add("allreduce", "default_allreduce_rsag_zero_copy", 0, UINT64_MAX);
    add("allreduce", "default_allreduce_nvls_warp_pipeline", 0, UINT64_MAX);
    add("allreduce", "default_allreduce_nvls_block_pipeline", 0, UINT64_MAX);
    add("allreduce", "default_allreduce_rsag", 0, 64u << 20);
    add("allreduce", "default_allreduce_rsag_pipeline", 0, UINT64_MAX);
    add("allgather", "default_allgather_fullmesh2", 0, UINT64_MAX);
    add("reducescatter", "default_reducescatter_zero_copy", 0, UINT64_MAX);
    add("alltoall", "default_alltoall", 0, UINT64_MAX);
    add("broadcast", "default_broadcast", 0, UINT64_MAX);
    return m;
  };
  auto pick = [&](const Map& m, const char* coll, int world, size_t bytes, bool symmetric) -> std::string {
    CollectiveRequest req;
    req.collective = coll;
    req.worldSize = world;
    req.messageSize = bytes;
    req.symmetricMemory = symmetric;
    auto a = collective::selectDefaultAlgorithm(m, req);
    return a ? a->name() : std::string("(none)");
  };
  const Map m8 = build(8), m2 = build(2);
  EXPECT_EQ(pick(m8, "allreduce", 8, 1u << 10, true), std::string("default_allreduce_nvls_packet"));
  EXPECT_EQ(pick(m8, "allreduce", 8, 64u << 10, true), std::string("default_allreduce_nvls_packet"));
  EXPECT_EQ(pick(m8, "allreduce", 8, 128u << 10, true), std::string("default_allreduce_packet_ll128"));
  EXPECT_EQ(pick(m8, "allreduce", 8, 256u << 10, true), std::string("default_allreduce_packet_ll128"));
  EXPECT_EQ(pick(m8, "allreduce", 8, 512u << 10, true), std::string("default_allreduce_nvls_zero_copy"));
  EXPECT_EQ(pick(m8, "allreduce", 8, 256u << 20, true), std::string("default_allreduce_nvls_zero_copy"));
  // two ranks: lines up to 4 MB, then plain peer loads and stores (the switch has nothing to combine)
  EXPECT_EQ(pick(m2, "allreduce", 2, 2u << 20, true), std::string("default_allreduce_packet_ll128"));
  EXPECT_EQ(pick(m2, "allreduce", 2, 8u << 20, true), std::string("default_allreduce_rsag_zero_copy"));
  // buffers outside the heap: the pipelined kernels
  EXPECT_EQ(pick(m8, "allreduce", 8, 2u << 20, false), std::string("default_allreduce_nvls_warp_pipeline"));
  EXPECT_EQ(pick(m8, "allreduce", 8, 64u << 20, false), std::string("default_allreduce_nvls_block_pipeline"));
  EXPECT_EQ(pick(m2, "allreduce", 2, 64u << 20, false), std::string("default_allreduce_rsag_pipeline"));
  // a size that is not a whole number of 16-byte words cannot take the zero-copy kernels
  EXPECT_EQ(pick(m8, "allreduce", 8, (64u << 20) + 2, true), std::string("default_allreduce_nvls_block_pipeline"));
  // the other collectives: divisibility by 16 bytes per rank, else nothing (the caller falls back)
  EXPECT_EQ(pick(m8, "allgather", 8, 1u << 20, true), std::string("default_allgather_fullmesh2"));
  EXPECT_EQ(pick(m8, "reducescatter", 8, 1u << 20, true), std::string("default_reducescatter_zero_copy"));
  EXPECT_EQ(pick(m8, "reducescatter", 8, (1u << 20) + 16, true), std::string("(none)"));
  EXPECT_EQ(pick(m8, "alltoall", 8, 1u << 20, true), std::string("default_alltoall"));
  EXPECT_EQ(pick(m8, "broadcast", 8, 12345, true), std::string("default_broadcast"));
  EXPECT_EQ(pick(m8, "scan", 8, 1024, true), std::string("(none)"));
  // without a multicast mapping the switch algorithms are not registered: packets and peer loads take over
  Map plain = build(8);
  plain["allreduce"].erase("default_allreduce_nvls_packet");
  plain["allreduce"].erase("default_allreduce_nvls_zero_copy");
  plain["allreduce"].erase("default_allreduce_nvls_warp_pipeline");
  plain["allreduce"].erase("default_allreduce_nvls_block_pipeline");
  EXPECT_EQ(pick(plain, "allreduce", 8, 1u << 10, true), std::string("default_allreduce_packet"));
  EXPECT_EQ(pick(plain, "allreduce", 8, 64u << 20, true), std::string("default_allreduce_rsag_zero_copy"));
  EXPECT_EQ(pick(plain, "allreduce", 8, 2u << 20, false), std::string("default_allreduce_rsag"));
  EXPECT_EQ(pick(plain, "allreduce", 8, 64u << 20, false), std::string("default_allreduce_rsag_pipeline"));
}

TEST(AlgorithmCollection, RegistrySelectorsAndExtend) {
  int smallCalls = 0, largeCalls = 0, otherCalls = 0;
  AlgorithmCollection coll;
  coll.registerAlgorithm("allreduce", "small", dummyAlgo("small", "allreduce", 0, 4096, &smallCalls));
  coll.registerAlgorithm("allreduce", "large", dummyAlgo("large", "allreduce", 4097, UINT64_MAX, &largeCalls));
  EXPECT_EQ(coll.getAlgorithmsByCollective("allreduce").size(), size_t(2));
  EXPECT_EQ(coll.getAlgorithmsByCollective("allgather").size(), size_t(0));
  EXPECT_EQ(coll.getAllAlgorithms().size(), size_t(2));

  CollectiveRequest req;
  req.collective = "allreduce";
  req.messageSize = 1024;
  EXPECT_TRUE(coll.selectAlgorithm(req) == nullptr);  // no selector installed yet

  // fallback: first algorithm whose message range holds the request; user selector: only answers for >= 1 MB
  auto byRange = [](const auto& map, const CollectiveRequest& r) -> std::shared_ptr<Algorithm> {
    auto it = map.find(r.collective);
    if (it == map.end()) return nullptr;
    for (const auto& kv : it->second) {
      auto range = kv.second->messageRange();
      if (r.messageSize >= range.first && r.messageSize <= range.second) return kv.second;
    }
    return nullptr;
  };
  auto userSel = [](const auto& map, const CollectiveRequest& r) -> std::shared_ptr<Algorithm> {
    if (r.messageSize < (1u << 20)) return nullptr;
    return map.at(r.collective).at("small");  // deliberately odd, to see that the user selector wins
  };
  coll.setSelectors(userSel, byRange);
  EXPECT_EQ(coll.selectAlgorithm(req)->name(), std::string("small"));
  req.messageSize = 65536;
  EXPECT_EQ(coll.selectAlgorithm(req)->name(), std::string("large"));
  req.messageSize = 4u << 20;
  EXPECT_EQ(coll.selectAlgorithm(req)->name(), std::string("small"));
  req.collective = "broadcast";
  req.messageSize = 8;
  EXPECT_TRUE(coll.selectAlgorithm(req) == nullptr);

  // ranges can be retuned after registration
  auto large = coll.getAlgorithmsByCollective("allreduce").at("large");
  large->setMessageSizeRange(100, 200);
  EXPECT_EQ(large->messageRange().first, size_t(100));
  EXPECT_EQ(large->messageRange().second, size_t(200));
  EXPECT_TRUE(large->type() == AlgorithmType::Native);
  EXPECT_TRUE(large->bufferMode() == CollectiveBufferMode::Any);

  AlgorithmCollection other;
  other.registerAlgorithm("allgather", "other", dummyAlgo("other", "allgather", 0, UINT64_MAX, &otherCalls));
  coll.extend(other);
  EXPECT_EQ(coll.getAllAlgorithms().size(), size_t(3));
  EXPECT_EQ(coll.getAlgorithmsByCollective("allgather").count("other"), size_t(1));

  // execute reaches the closure (no communicator or executor needed by a native algorithm that ignores them)
  auto algo = coll.getAlgorithmsByCollective("allgather").at("other");
  CommResult res = algo->execute(nullptr, nullptr, nullptr, 0, 0, DataType::FLOAT32, SUM, nullptr, nullptr, 0, 0, false, {}, DataType::AUTO);
  EXPECT_TRUE(res == CommResult::Success);
  EXPECT_EQ(otherCalls, 1);
  EXPECT_EQ(smallCalls + largeCalls, 0);
}

TEST(CollectiveRequest, BufferMode) {
  CollectiveRequest req;
  int a = 0, b = 0;
  req.inputBuffer = &a;
  req.outputBuffer = &a;
  EXPECT_TRUE(req.bufferMode() == CollectiveBufferMode::InPlace);
  req.outputBuffer = &b;
  EXPECT_TRUE(req.bufferMode() == CollectiveBufferMode::OutOfPlace);
}

TEST(Env, SingletonAndDefaults) {
  auto e1 = env();
  auto e2 = env();
  EXPECT_TRUE(e1.get() == e2.get());
  const char* timeout = std::getenv("MSCCLPP_DEVICE_TIMEOUT_MS");
  if (timeout == nullptr) EXPECT_EQ(e1->deviceTimeoutMs, 10000L);
  else EXPECT_EQ(e1->deviceTimeoutMs, std::atol(timeout));
  if (std::getenv("MSCCLPP_HEAP_BYTES") == nullptr) EXPECT_EQ(e1->heapBytes, 2L << 30);
  if (std::getenv("MSCCLPP_IB_GID_INDEX") == nullptr) EXPECT_EQ(e1->ibGidIndex, -1);
  EXPECT_TRUE(!e1->cacheDir.empty());
}

TEST(Utils, HostNameIbDevicesVersion) {
  const std::string full = getHostName(1024, '\0');
  EXPECT_TRUE(!full.empty());
  EXPECT_TRUE(getHostName(3, '\0').size() <= 3);
  EXPECT_TRUE(getHostName(1024, full[0]).empty());  // cut at the first occurrence of the delimiter
  const int n = getIBDeviceCount();
  EXPECT_TRUE(n >= 0);
  if (n == 0) {
    EXPECT_THROW(getIBDeviceName(Transport::IB0), BaseError);
  } else {
    EXPECT_TRUE(getIBTransportByDeviceName(getIBDeviceName(Transport::IB0)) == Transport::IB0);
  }
  EXPECT_THROW(getIBDeviceName(Transport::CudaIpc), BaseError);
  EXPECT_THROW(getIBTransportByDeviceName("no_such_device"), BaseError);
  EXPECT_EQ(MSCCLPP_VERSION, MSCCLPP_MAJOR * 10000 + MSCCLPP_MINOR * 100 + MSCCLPP_PATCH);
  EXPECT_TRUE(version().rfind(std::to_string(MSCCLPP_MAJOR) + "." + std::to_string(MSCCLPP_MINOR) + "." + std::to_string(MSCCLPP_PATCH), 0) == 0);
  std::size_t seed = 0;
  detail::hashCombine(seed, std::string("a"));
  const std::size_t one = seed;
  detail::hashCombine(seed, 7);
  EXPECT_TRUE(one != 0 && seed != one);
#ifndef MSCCLPP_HOST_COMPILE
  EXPECT_TRUE(false);  // a plain host compiler must see MSCCLPP_HOST_COMPILE
#endif
}

TEST(GpuUtils, AllocationFamilyInstantiates) {
  // no GPU here: only check that every member of the family exists with the expected types
  std::shared_ptr<int> (*a)(size_t) = &gpuCallocUncachedShared<int>;
  UniqueGpuPtr<int> (*b)(size_t) = &gpuCallocUncachedUnique<int>;
  UniqueGpuHostPtr<int> (*c)(size_t, unsigned) = &gpuCallocHostUnique<int>;
  UniqueGpuPhysicalPtr<int> (*d)(size_t, size_t) = &gpuCallocPhysicalUnique<int>;
  void (*e)(void*, int, size_t) = &gpuMemset;
  EXPECT_TRUE(a != nullptr && b != nullptr && c != nullptr && d != nullptr && e != nullptr);
  EXPECT_TRUE(static_cast<int>(GpuBufferGranularity::MultiCastMinimum) != static_cast<int>(GpuBufferGranularity::MultiCastRecommended));
}

TEST(Proxy, AFailedRequestStaysUnconsumed) {
  // a handler that cannot carry out a request answers Abort: the proxy stops and the request is NOT marked consumed, so a
  // device-side sync on it times out instead of reporting a transfer that never happened
  std::atomic<int> handled{0};
  Proxy proxy([&](ProxyTrigger t) {
    handled++;
    return t.fst == 13 ? ProxyHandlerResult::Abort : ProxyHandlerResult::Continue;
  });
  proxy.start();
  auto fifo = proxy.fifo();
  ProxyTrigger good{1, 1}, bad{13, 1};
  fifo->pushFromHost(good);
  fifo->pushFromHost(bad);
  fifo->pushFromHost(good);
  for (int i = 0; i < 2000 && !proxy.failed(); i++) usleep(1000);
  EXPECT_TRUE(proxy.failed());
  EXPECT_EQ(handled.load(), 2);             // the request behind the failed one is never looked at
  EXPECT_EQ(fifo->consumed(), uint64_t(1));  // only the first one counts as done
  proxy.stop();
}

TEST(RangeAllocator, FirstFitReleaseAndCoalescing) {
  // offsets of a multicast object: ranges come back when channels go away and are reused, lowest address first
  RangeAllocator r(10 * 4096 + 100, 4096);
  EXPECT_EQ(r.capacity(), size_t(10 * 4096));
  const size_t a = r.allocate(4096), b = r.allocate(5000), c = r.allocate(3 * 4096);
  EXPECT_EQ(a, size_t(0));
  EXPECT_EQ(b, size_t(4096));       // 5000 bytes take two granules
  EXPECT_EQ(c, size_t(3 * 4096));
  EXPECT_EQ(r.bytesFree(), size_t(4 * 4096));
  EXPECT_EQ(r.allocate(5 * 4096), RangeAllocator::npos);
  r.release(b);
  EXPECT_EQ(r.largestFree(), size_t(4 * 4096));  // the tail, not the two-granule hole
  EXPECT_EQ(r.allocate(2 * 4096), size_t(4096));  // the hole is taken first
  r.release(a);
  r.release(4096);
  r.release(c);
  EXPECT_EQ(r.largestFree(), r.capacity());  // everything merged back into one range
  EXPECT_EQ(r.rangesInUse(), size_t(0));
  // many rounds of bind / unbind never exhaust the object (a pointer that only advances would after ten)
  for (int round = 0; round < 1000; round++) {
    const size_t x = r.allocate(6 * 4096), y = r.allocate(4 * 4096);
    EXPECT_TRUE(x != RangeAllocator::npos && y != RangeAllocator::npos);
    r.release(round % 2 ? x : y);
    r.release(round % 2 ? y : x);
  }
  EXPECT_THROW(r.release(12345), std::invalid_argument);
  EXPECT_EQ(r.allocate(0), RangeAllocator::npos);
}

TEST(Numa, CpuListsAndBinding) {
  std::vector<int> cpus = parseCpuList("0-2,5, 7-8\n");
  EXPECT_EQ(cpus.size(), size_t(6));
  EXPECT_EQ(cpus.back(), 8);
  EXPECT_THROW(parseCpuList("4-2"), BaseError);
  EXPECT_THROW(parseCpuList("x"), BaseError);
  EXPECT_THROW(getNumaNodeCpus(4096), BaseError);
  numaBind(-1);  // unknown node: no-op
  std::thread worker([] {  // bind a thread of its own, the test runner keeps its affinity
    try {
      std::vector<int> node0 = getNumaNodeCpus(0);
      numaBind(0);
      cpu_set_t now;
      CPU_ZERO(&now);
      sched_getaffinity(0, sizeof(now), &now);
      for (int c = 0; c < CPU_SETSIZE; c++) {
        if (CPU_ISSET(c, &now)) EXPECT_TRUE(std::find(node0.begin(), node0.end(), c) != node0.end());
      }
    } catch (const BaseError&) {
      // machines without NUMA information in sysfs, or a cpuset that excludes node 0
    }
  });
  worker.join();
}

TEST(ExecutionPlan, LoadsAPlanWrittenByTheDsl) {
  const char* path = std::getenv("MSCCLPP_TEST_PLAN");
  if (path == nullptr) {
    std::printf("[  SKIPPED ] MSCCLPP_TEST_PLAN is not set\n");
    return;
  }
  ExecutionPlan plan(path, 0);
  EXPECT_EQ(plan.collective(), std::string("allreduce"));
  EXPECT_TRUE(!plan.name().empty());
  EXPECT_EQ(plan.nRanks(), 8);
  EXPECT_TRUE(plan.nThreadsPerBlock() > 0);
  EXPECT_TRUE(plan.minMessageSize() <= plan.maxMessageSize());
  ExecutionPlan lastRank(path, 7);
  EXPECT_EQ(lastRank.name(), plan.name());
  EXPECT_THROW(ExecutionPlan(path, 8), BaseError);  // rank outside the plan
  EXPECT_THROW(ExecutionPlan("/nonexistent/plan.json", 0), BaseError);
}

int main(int argc, char** argv) { return testing::runAll(argc, argv); }
