// NCCL-API shim: libmscclpp_b200_nccl.so exports the NCCL C ABI on top of this library so that
// unmodified NCCL applications (PyTorch `backend="nccl"`, nccl-tests) run on it under LD_PRELOAD.
// Behaviour follows the reference shim (src/ext/nccl/nccl.cc:83-905): world size 1 is a memcpy; a
// forced-fallback list (MSCCLPP_FORCE_NCCL_FALLBACK_OPERATION) sends named collectives to the real
// NCCL; otherwise the algorithm collection picks a native or DSL algorithm; what nothing here handles
// goes to the real NCCL when MSCCLPP_NCCL_LIB_PATH names one, else it is an error.
#include <mscclpp/ext/nccl/nccl.h>

#include <algorithm>
#include <cstring>
#include <dlfcn.h>
#include <map>
#include <mutex>
#include <sstream>
#include <vector>

#include <mscclpp/core.hpp>
#include <mscclpp/env.hpp>
#include <mscclpp/executor.hpp>
#include <mscclpp/ext/collectives/algorithm_collection_builder.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/symmetric_heap.hpp>

#include "../core/logger.hpp"

using namespace mscclpp;

// ------------------------------------------------------------------------------------------ real NCCL (optional)
namespace {

struct RealNccl {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Reduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  ncclResult_t (*AlltoAll)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  bool ok = false;
};

RealNccl& realNccl() {
  static RealNccl r;
  static std::once_flag once;
  std::call_once(once, [] {
    const std::string path = env()->ncclLibPath;
    if (path.empty()) return;
    r.lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL | RTLD_DEEPBIND);
    if (!r.lib) {
      LOG_WARN(LogSubsys::NCCL, "cannot dlopen ", path, ": ", dlerror());
      return;
    }
#define LOAD(field, sym) r.field = reinterpret_cast<decltype(r.field)>(dlsym(r.lib, sym))
    LOAD(GetUniqueId, "ncclGetUniqueId");
    LOAD(CommInitRank, "ncclCommInitRank");
    LOAD(CommDestroy, "ncclCommDestroy");
    LOAD(CommAbort, "ncclCommAbort");
    LOAD(AllReduce, "ncclAllReduce");
    LOAD(AllGather, "ncclAllGather");
    LOAD(ReduceScatter, "ncclReduceScatter");
    LOAD(Broadcast, "ncclBroadcast");
    LOAD(Reduce, "ncclReduce");
    LOAD(Send, "ncclSend");
    LOAD(Recv, "ncclRecv");
    LOAD(GroupStart, "ncclGroupStart");
    LOAD(GroupEnd, "ncclGroupEnd");
    LOAD(AlltoAll, "ncclAlltoAll");
#undef LOAD
    r.ok = r.GetUniqueId && r.CommInitRank && r.AllReduce && r.AllGather && r.ReduceScatter && r.Broadcast && r.Send && r.Recv &&
           r.GroupStart && r.GroupEnd;
    if (!r.ok) LOG_WARN(LogSubsys::NCCL, path, " lacks required NCCL symbols; fallback disabled");
  });
  return r;
}

thread_local std::string lastError;

// execution plans loaded through mscclLoadAlgo, by handle
std::mutex loadedAlgoMutex;
std::map<int, std::shared_ptr<DslAlgorithm>> loadedAlgos;
int nextAlgoHandle = 1;

ncclResult_t fail(ncclResult_t code, const std::string& msg) {
  lastError = msg;
  LOG_WARN(LogSubsys::NCCL, msg);
  return code;
}

bool toDataType(ncclDataType_t t, DataType& out) {
  switch (t) {
    case ncclInt32: out = DataType::INT32; return true;
    case ncclUint32: out = DataType::UINT32; return true;
    case ncclFloat16: out = DataType::FLOAT16; return true;
    case ncclFloat32: out = DataType::FLOAT32; return true;
    case ncclBfloat16: out = DataType::BFLOAT16; return true;
    case ncclUint8: out = DataType::UINT8; return true;
    case ncclFloat8e4m3: out = DataType::FLOAT8_E4M3; return true;
    case ncclFloat8e5m2: out = DataType::FLOAT8_E5M2; return true;
    default: return false;
  }
}

size_t typeSize(ncclDataType_t t) { return ncclTypeSize(t); }

bool forcedFallback(const char* op) {
  static std::vector<std::string> list = [] {
    std::vector<std::string> v;
    std::stringstream ss(env()->forceNcclFallbackOperation);
    std::string tok;
    while (std::getline(ss, tok, ',')) {
      tok.erase(std::remove_if(tok.begin(), tok.end(), [](unsigned char c) { return std::isspace(c); }), tok.end());
      std::transform(tok.begin(), tok.end(), tok.begin(), [](unsigned char c) { return std::tolower(c); });
      if (!tok.empty()) v.push_back(tok);
    }
    return v;
  }();
  for (auto& s : list)
    if (s == "all" || s == op) return true;
  return false;
}

ncclResult_t toNccl(CommResult r) {
  switch (r) {
    case CommResult::Success: return ncclSuccess;
    case CommResult::UnhandledCudaError: return ncclUnhandledCudaError;
    case CommResult::SystemError: return ncclSystemError;
    case CommResult::InvalidArgument: return ncclInvalidArgument;
    case CommResult::InvalidUsage: return ncclInvalidUsage;
    case CommResult::RemoteError: return ncclRemoteError;
    case CommResult::InProgress: return ncclInProgress;
    default: return ncclInternalError;
  }
}

std::mutex g_heapMutex;
std::weak_ptr<SymmetricHeap> g_lastHeap;   // ncclMemAlloc has no communicator argument
struct MemAlloc {
  std::weak_ptr<SymmetricHeap> heap;
  bool physical = false;  // allocated before any communicator existed: plain VMM memory
};
std::map<void*, MemAlloc> g_memAllocs;

}  // namespace

struct ncclComm {
  std::shared_ptr<TcpBootstrap> bootstrap;
  std::shared_ptr<Communicator> comm;
  std::shared_ptr<SymmetricHeap> heap;
  std::shared_ptr<Executor> executor;
  AlgorithmCollection algos;
  int rank = 0, nranks = 1, cudaDev = 0;
  ncclComm_t real = nullptr;
  bool destroyed = false;
  // asynchronous error reporting: the device status block is copied to pinned host memory on a stream of its own
  DeviceStatus* hostStatus = nullptr;
  cudaStream_t statusStream = nullptr;
  cudaEvent_t statusEvent = nullptr;
  bool statusPending = false;
  ncclResult_t asyncError = ncclSuccess;
};

namespace {

ncclResult_t initComm(ncclComm_t* out, int nranks, const UniqueId& id, int rank) {
  try {
    auto c = new ncclComm();
    c->rank = rank;
    c->nranks = nranks;
    MSCCLPP_CUDATHROW(cudaGetDevice(&c->cudaDev));
    c->bootstrap = std::make_shared<TcpBootstrap>(rank, nranks);
    c->bootstrap->initialize(id, 120);
    c->comm = std::make_shared<Communicator>(c->bootstrap);
    SymmetricHeap::Options opt;
    opt.enableNvls = !env()->forceDisableNvls;
    c->heap = SymmetricHeap::create(c->bootstrap, opt);
    c->executor = std::make_shared<Executor>(c->heap);
    c->algos = collective::AlgorithmCollectionBuilder::getInstance()->buildDefaultAlgorithms(c->heap);
    {
      std::lock_guard<std::mutex> lock(g_heapMutex);
      g_lastHeap = c->heap;
    }
    MSCCLPP_CUDATHROW(cudaHostAlloc(reinterpret_cast<void**>(&c->hostStatus), sizeof(DeviceStatus), cudaHostAllocDefault));
    std::memset(c->hostStatus, 0, sizeof(DeviceStatus));
    MSCCLPP_CUDATHROW(cudaStreamCreateWithFlags(&c->statusStream, cudaStreamNonBlocking));
    MSCCLPP_CUDATHROW(cudaEventCreateWithFlags(&c->statusEvent, cudaEventDisableTiming));
    RealNccl& real = realNccl();
    if (real.ok) {
      ncclUniqueId realId{};
      if (rank == 0 && real.GetUniqueId(&realId) != ncclSuccess) throw Error("real ncclGetUniqueId failed", ErrorCode::InternalError);
      c->bootstrap->broadcast(&realId, sizeof(realId), 0);
      if (real.CommInitRank(&c->real, nranks, realId, rank) != ncclSuccess) {
        LOG_WARN(LogSubsys::NCCL, "real ncclCommInitRank failed; fallback disabled for this communicator");
        c->real = nullptr;
      }
    }
    *out = c;
    return ncclSuccess;
  } catch (const std::exception& e) {
    return fail(ncclInternalError, std::string("ncclCommInitRank: ") + e.what());
  }
}

template <typename Fn>
ncclResult_t runCollective(ncclComm_t comm, const char* opName, const char* collective, const void* sendbuff, void* recvbuff,
                           size_t inBytes, size_t outBytes, size_t messageSize, ncclDataType_t datatype, ncclRedOp_t op,
                           cudaStream_t stream, Fn fallback) {
  if (comm == nullptr || comm->destroyed) return fail(ncclInvalidArgument, std::string(opName) + ": invalid communicator");
  if (sendbuff == nullptr || recvbuff == nullptr) return fail(ncclInvalidArgument, std::string(opName) + ": null buffer");
  if (inBytes == 0 || outBytes == 0) return ncclSuccess;
  DataType dtype;
  const bool typeOk = toDataType(datatype, dtype);
  const bool opOk = op == ncclSum || op == ncclMin || std::strcmp(collective, "allgather") == 0;
  if (!forcedFallback(opName) && typeOk && opOk) {
    CollectiveRequest req;
    req.worldSize = comm->nranks;
    req.nRanksPerNode = comm->bootstrap->getNranksPerNode();
    req.rank = comm->rank;
    req.inputBuffer = sendbuff;
    req.outputBuffer = recvbuff;
    req.messageSize = messageSize;
    req.stream = stream;
    req.collective = collective;
    req.dtype = dtype;
    req.op = op == ncclMin ? MIN : SUM;
    // agreed among all ranks (a rank-local test could send the ranks into different kernels)
    req.symmetricMemory = comm->heap->symmetricOnAllRanks(sendbuff, inBytes) && comm->heap->symmetricOnAllRanks(recvbuff, outBytes);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess) req.inCapture = cap != cudaStreamCaptureStatusNone;
    else (void)cudaGetLastError();
    auto algo = comm->algos.selectAlgorithm(req);
    if (algo) {
      CommResult r = algo->execute(comm->comm, sendbuff, recvbuff, inBytes, outBytes, dtype, req.op, stream, comm->executor, 0, 0,
                                   req.symmetricMemory, {}, DataType::AUTO);
      if (r == CommResult::Success) return ncclSuccess;
      if (r != CommResult::InvalidUsage && r != CommResult::InvalidArgument) return fail(toNccl(r), std::string(opName) + ": " + algo->name() + " failed");
      // the chosen algorithm refused these arguments: try the real NCCL below
    }
  }
  if (comm->real != nullptr) return fallback();
  return fail(ncclInvalidUsage, std::string(opName) + ": no algorithm handles this call and no fallback NCCL is loaded "
                                                       "(set MSCCLPP_NCCL_LIB_PATH)");
}

}  // namespace

extern "C" {

ncclResult_t ncclGetVersion(int* version) {
  if (version == nullptr) return ncclInvalidArgument;
  *version = NCCL_VERSION_CODE;
  return ncclSuccess;
}

ncclResult_t ncclGetUniqueId(ncclUniqueId* uniqueId) {
  if (uniqueId == nullptr) return ncclInvalidArgument;
  try {
    UniqueId id = TcpBootstrap::createUniqueId();
    static_assert(sizeof(ncclUniqueId) == UniqueIdBytes, "id size mismatch");
    std::memcpy(uniqueId->internal, id.data(), UniqueIdBytes);
    return ncclSuccess;
  } catch (const std::exception& e) {
    return fail(ncclSystemError, std::string("ncclGetUniqueId: ") + e.what());
  }
}

ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank) {
  if (comm == nullptr || nranks < 1 || rank < 0 || rank >= nranks) return fail(ncclInvalidArgument, "ncclCommInitRank: bad arguments");
  UniqueId id;
  std::memcpy(id.data(), commId.internal, UniqueIdBytes);
  return initComm(comm, nranks, id, rank);
}

ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank, ncclConfig_t*) {
  return ncclCommInitRank(comm, nranks, commId, rank);
}

ncclResult_t ncclCommInitRankScalable(ncclComm_t* newcomm, int nranks, int myrank, int nId, ncclUniqueId* commIds, ncclConfig_t*) {
  if (nId < 1 || commIds == nullptr) return fail(ncclInvalidArgument, "ncclCommInitRankScalable: no ids");
  return ncclCommInitRank(newcomm, nranks, commIds[0], myrank);
}

ncclResult_t ncclCommInitAll(ncclComm_t* comm, int ndev, const int*) {
  if (ndev != 1) return fail(ncclInvalidUsage, "ncclCommInitAll: one process drives one GPU in this library (ndev must be 1)");
  ncclUniqueId id;
  ncclResult_t r = ncclGetUniqueId(&id);
  if (r != ncclSuccess) return r;
  return ncclCommInitRank(comm, 1, id, 0);
}

ncclResult_t ncclCommFinalize(ncclComm_t comm) {
  if (comm == nullptr) return ncclInvalidArgument;
  (void)cudaDeviceSynchronize();
  return ncclSuccess;
}

ncclResult_t ncclCommDestroy(ncclComm_t comm) {
  if (comm == nullptr) return ncclSuccess;
  if (comm->destroyed) return fail(ncclInvalidArgument, "ncclCommDestroy: communicator destroyed twice");
  comm->destroyed = true;
  try {
    (void)cudaDeviceSynchronize();
    if (comm->real && realNccl().CommDestroy) realNccl().CommDestroy(comm->real);
    if (comm->statusStream) (void)cudaStreamDestroy(comm->statusStream);
    if (comm->statusEvent) (void)cudaEventDestroy(comm->statusEvent);
    if (comm->hostStatus) (void)cudaFreeHost(comm->hostStatus);
    comm->executor.reset();
    comm->algos = AlgorithmCollection();
    if (comm->heap) comm->heap->destroy();
    delete comm;
  } catch (const std::exception& e) {
    return fail(ncclInternalError, std::string("ncclCommDestroy: ") + e.what());
  }
  return ncclSuccess;
}

ncclResult_t ncclCommAbort(ncclComm_t comm) {
  if (comm == nullptr) return ncclSuccess;
  if (comm->bootstrap) comm->bootstrap->abort();
  if (comm->real && realNccl().CommAbort) realNccl().CommAbort(comm->real);
  comm->real = nullptr;
  // no collective teardown is possible once peers may be gone: local resources only
  comm->destroyed = true;
  return ncclSuccess;
}

ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t*) {
  if (comm == nullptr || newcomm == nullptr) return ncclInvalidArgument;
  try {
    struct Entry {
      int color, key, rank;
    };
    std::vector<Entry> all(comm->nranks);
    all[comm->rank] = Entry{color, key, comm->rank};
    comm->bootstrap->allGather(all.data(), sizeof(Entry));
    if (color == NCCL_SPLIT_NOCOLOR) {
      *newcomm = nullptr;
      return ncclSuccess;
    }
    std::vector<Entry> mine;
    for (auto& e : all)
      if (e.color == color) mine.push_back(e);
    std::stable_sort(mine.begin(), mine.end(), [](const Entry& a, const Entry& b) { return a.key != b.key ? a.key < b.key : a.rank < b.rank; });
    int newRank = -1;
    for (size_t i = 0; i < mine.size(); i++)
      if (mine[i].rank == comm->rank) newRank = static_cast<int>(i);
    // the group's new rank 0 creates the id and sends it to the others over the parent's bootstrap
    UniqueId id;
    const int tag = 0x7ffc0000 + (color & 0xffff);
    if (newRank == 0) {
      id = TcpBootstrap::createUniqueId();
      for (size_t i = 1; i < mine.size(); i++) comm->bootstrap->send(id.data(), UniqueIdBytes, mine[i].rank, tag);
    } else {
      comm->bootstrap->recv(id.data(), UniqueIdBytes, mine[0].rank, tag);
    }
    return initComm(newcomm, static_cast<int>(mine.size()), id, newRank);
  } catch (const std::exception& e) {
    return fail(ncclInternalError, std::string("ncclCommSplit: ") + e.what());
  }
}

ncclResult_t ncclCommShrink(ncclComm_t, int*, int, ncclComm_t*, ncclConfig_t*, int) {
  return fail(ncclInvalidUsage, "ncclCommShrink is not supported");
}

const char* ncclGetErrorString(ncclResult_t result) {
  switch (result) {
    case ncclSuccess: return "no error";
    case ncclUnhandledCudaError: return "unhandled cuda error";
    case ncclSystemError: return "unhandled system error";
    case ncclInternalError: return "internal error";
    case ncclInvalidArgument: return "invalid argument";
    case ncclInvalidUsage: return "invalid usage";
    case ncclRemoteError: return "remote process exited or there was a network error";
    case ncclInProgress: return "NCCL operation in progress";
    default: return "unknown result code";
  }
}

const char* ncclGetLastError(ncclComm_t) { return lastError.c_str(); }

ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError) {
  if (comm == nullptr || asyncError == nullptr) return ncclInvalidArgument;
  // A device-side wait that ran out is this library's asynchronous error. The status block lives in device memory;
  // it is copied to pinned host memory on a non-blocking stream of its own, so this call never waits for the
  // application's kernels: it reports what the previous copy found and starts the next one.
  DeviceStatus* dev = comm->heap ? comm->heap->deviceComm().status : nullptr;
  if (dev != nullptr && comm->hostStatus != nullptr && !comm->destroyed) {
    if (comm->statusPending && cudaEventQuery(comm->statusEvent) == cudaSuccess) {
      comm->statusPending = false;
      if (comm->hostStatus->code != kDevOk && comm->asyncError == ncclSuccess) {
        comm->asyncError = comm->hostStatus->code == kDevErrorCapacity ? ncclInvalidUsage : ncclRemoteError;
        lastError = "device-side wait gave up (code " + std::to_string(comm->hostStatus->code) + ", site " +
                    std::to_string(comm->hostStatus->where) + ", peer " + std::to_string(comm->hostStatus->peer) + ")";
      }
    }
    if (!comm->statusPending) {
      if (cudaMemcpyAsync(comm->hostStatus, dev, sizeof(DeviceStatus), cudaMemcpyDeviceToHost, comm->statusStream) == cudaSuccess &&
          cudaEventRecord(comm->statusEvent, comm->statusStream) == cudaSuccess) {
        comm->statusPending = true;
      } else {
        (void)cudaGetLastError();
      }
    }
  }
  *asyncError = comm->asyncError;
  return ncclSuccess;
}

ncclResult_t ncclCommCount(const ncclComm_t comm, int* count) {
  if (comm == nullptr || count == nullptr) return ncclInvalidArgument;
  *count = comm->nranks;
  return ncclSuccess;
}
ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int* device) {
  if (comm == nullptr || device == nullptr) return ncclInvalidArgument;
  *device = comm->cudaDev;
  return ncclSuccess;
}
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank) {
  if (comm == nullptr || rank == nullptr) return ncclInvalidArgument;
  *rank = comm->rank;
  return ncclSuccess;
}

ncclResult_t ncclCommRegister(const ncclComm_t, void*, size_t, void** handle) {
  if (handle) *handle = nullptr;
  return ncclSuccess;  // heap memory needs no registration; other memory is staged
}
ncclResult_t ncclCommDeregister(const ncclComm_t, void*) { return ncclSuccess; }
ncclResult_t ncclCommWindowRegister(ncclComm_t, void*, size_t, ncclWindow_t* win, int) {
  if (win) *win = nullptr;
  return ncclSuccess;
}
ncclResult_t ncclCommWindowDeregister(ncclComm_t, ncclWindow_t) { return ncclSuccess; }

ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t*, void*, ncclDataType_t, ncclScalarResidence_t, ncclComm_t) {
  return fail(ncclInvalidUsage, "ncclRedOpCreatePreMulSum is not supported");
}
ncclResult_t ncclRedOpDestroy(ncclRedOp_t, ncclComm_t) { return ncclSuccess; }

ncclResult_t ncclMemAlloc(void** ptr, size_t size) {
  if (ptr == nullptr || size == 0) return ncclInvalidArgument;
  try {
    std::lock_guard<std::mutex> lock(g_heapMutex);
    if (auto heap = g_lastHeap.lock()) {
      // symmetric-heap memory: zero-copy for every algorithm, as long as all ranks allocate in the same order
      *ptr = heap->alloc(size, 256);
      g_memAllocs[*ptr] = MemAlloc{heap, false};
    } else {
      *ptr = detail::gpuCallocPhysical(size);
      g_memAllocs[*ptr] = MemAlloc{{}, true};
    }
    return ncclSuccess;
  } catch (const std::exception& e) {
    return fail(ncclUnhandledCudaError, std::string("ncclMemAlloc: ") + e.what());
  }
}

ncclResult_t ncclMemFree(void* ptr) {
  if (ptr == nullptr) return ncclSuccess;
  std::lock_guard<std::mutex> lock(g_heapMutex);
  auto it = g_memAllocs.find(ptr);
  if (it == g_memAllocs.end()) return fail(ncclInvalidArgument, "ncclMemFree: pointer was not allocated by ncclMemAlloc");
  try {
    if (it->second.physical) detail::gpuFreePhysical(ptr);
    else if (auto heap = it->second.heap.lock()) heap->free(ptr);
  } catch (const std::exception&) {
  }
  g_memAllocs.erase(it);
  return ncclSuccess;
}

ncclResult_t ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm,
                           cudaStream_t stream) {
  const size_t bytes = count * typeSize(datatype);
  if (comm != nullptr && comm->nranks == 1) {
    if (sendbuff != recvbuff && cudaMemcpyAsync(recvbuff, sendbuff, bytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return ncclUnhandledCudaError;
    return ncclSuccess;
  }
  return runCollective(comm, "allreduce", "allreduce", sendbuff, recvbuff, bytes, bytes, bytes, datatype, op, stream,
                       [&] { return realNccl().AllReduce(sendbuff, recvbuff, count, datatype, op, comm->real, stream); });
}

ncclResult_t ncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm,
                           cudaStream_t stream) {
  const size_t bytes = sendcount * typeSize(datatype);
  if (comm != nullptr && comm->nranks == 1) {
    if (sendbuff != recvbuff && cudaMemcpyAsync(recvbuff, sendbuff, bytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return ncclUnhandledCudaError;
    return ncclSuccess;
  }
  const size_t total = comm ? bytes * comm->nranks : 0;
  // in-place allgather (sendbuff == recvbuff + rank * bytes) works: the kernel copies the slice onto itself
  return runCollective(comm, "allgather", "allgather", sendbuff, recvbuff, bytes, total, bytes, datatype, ncclSum, stream,
                       [&] { return realNccl().AllGather(sendbuff, recvbuff, sendcount, datatype, comm->real, stream); });
}

ncclResult_t ncclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op,
                               ncclComm_t comm, cudaStream_t stream) {
  const size_t bytes = recvcount * typeSize(datatype);
  if (comm != nullptr && comm->nranks == 1) {
    if (sendbuff != recvbuff && cudaMemcpyAsync(recvbuff, sendbuff, bytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return ncclUnhandledCudaError;
    return ncclSuccess;
  }
  const size_t total = comm ? bytes * comm->nranks : 0;
  return runCollective(comm, "reducescatter", "reducescatter", sendbuff, recvbuff, total, bytes, total, datatype, op, stream,
                       [&] { return realNccl().ReduceScatter(sendbuff, recvbuff, recvcount, datatype, op, comm->real, stream); });
}

ncclResult_t ncclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm,
                           cudaStream_t stream) {
  if (comm == nullptr) return ncclInvalidArgument;
  const size_t bytes = count * typeSize(datatype);
  if (comm->nranks == 1) {
    if (sendbuff != recvbuff && cudaMemcpyAsync(recvbuff, sendbuff, bytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return ncclUnhandledCudaError;
    return ncclSuccess;
  }
  if (root < 0 || root >= comm->nranks) return fail(ncclInvalidArgument, "broadcast: bad root");
  if (!forcedFallback("broadcast") && bytes > 0) {
    CollectiveRequest req;
    req.worldSize = comm->nranks;
    req.nRanksPerNode = comm->bootstrap->getNranksPerNode();
    req.rank = comm->rank;
    req.inputBuffer = sendbuff;
    req.outputBuffer = recvbuff;
    req.messageSize = bytes;
    req.stream = stream;
    req.collective = "broadcast";
    req.dtype = DataType::UINT8;
    auto algo = comm->algos.selectAlgorithm(req);
    if (algo) {
      // the root may pass a null / unrelated recvbuff semantics-wise equal to sendbuff: NCCL requires recvbuff everywhere
      CommResult r = algo->execute(comm->comm, sendbuff != nullptr ? sendbuff : recvbuff, recvbuff, bytes, bytes, DataType::UINT8, NOP, stream,
                                   comm->executor, 0, 0, false, {{"root", static_cast<uintptr_t>(root)}}, DataType::AUTO);
      if (r == CommResult::Success) return ncclSuccess;
      if (r != CommResult::InvalidUsage && r != CommResult::InvalidArgument) return fail(toNccl(r), "broadcast: default_broadcast failed");
    }
  }
  if (bytes == 0) return ncclSuccess;
  if (comm->real != nullptr) return realNccl().Broadcast(sendbuff, recvbuff, count, datatype, root, comm->real, stream);
  return fail(ncclInvalidUsage, "broadcast: no algorithm handles this call and no fallback NCCL is loaded (set MSCCLPP_NCCL_LIB_PATH)");
}

ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
  return ncclBroadcast(buff, buff, count, datatype, root, comm, stream);
}

ncclResult_t ncclReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root,
                        ncclComm_t comm, cudaStream_t stream) {
  if (comm == nullptr) return ncclInvalidArgument;
  if (comm->real != nullptr && realNccl().Reduce) return realNccl().Reduce(sendbuff, recvbuff, count, datatype, op, root, comm->real, stream);
  return fail(ncclInvalidUsage, "reduce: handled by the fallback NCCL only (set MSCCLPP_NCCL_LIB_PATH)");
}

ncclResult_t ncclAlltoAll(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclComm_t comm,
                          cudaStream_t stream) {
  // `count` elements go to (and come from) every rank
  if (comm == nullptr) return ncclInvalidArgument;
  const size_t total = count * typeSize(datatype) * static_cast<size_t>(comm->nranks);
  if (comm->nranks == 1) {
    if (sendbuff != recvbuff && cudaMemcpyAsync(recvbuff, sendbuff, total, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return ncclUnhandledCudaError;
    return ncclSuccess;
  }
  if (sendbuff == recvbuff) return fail(ncclInvalidUsage, "alltoall: in-place operation is not supported");
  return runCollective(comm, "alltoall", "alltoall", sendbuff, recvbuff, total, total, total, ncclUint8, ncclSum, stream, [&] {
    if (realNccl().AlltoAll) return realNccl().AlltoAll(sendbuff, recvbuff, count, datatype, comm->real, stream);
    return fail(ncclInvalidUsage, "alltoall: the fallback NCCL has no ncclAlltoAll");
  });
}

ncclResult_t ncclAllToAll(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclComm_t comm,
                          cudaStream_t stream) {
  return ncclAlltoAll(sendbuff, recvbuff, count, datatype, comm, stream);  // the spelling of the MSCCL++ header
}

ncclResult_t ncclAllToAllv(const void* sendbuff, const size_t sendcounts[], const size_t sdispls[], void* recvbuff,
                           const size_t recvcounts[], const size_t rdispls[], ncclDataType_t datatype, ncclComm_t comm,
                           cudaStream_t stream) {
  if (comm == nullptr || comm->destroyed) return fail(ncclInvalidArgument, "alltoallv: invalid communicator");
  if (sendcounts == nullptr || sdispls == nullptr || recvcounts == nullptr || rdispls == nullptr) return ncclInvalidArgument;
  const int n = comm->nranks;
  // Whether the layout is uniform is a property of THIS rank's arguments; a peer's row may be ragged. Choosing the native
  // all-to-all kernel from it could put some ranks into that kernel and others into send/recv, so with a fallback NCCL
  // loaded every alltoallv takes the grouped point-to-point path, whatever the counts look like here.
  if (comm->real == nullptr) {
    // No fallback library: only the uniform case can run at all (the native kernel), and only if it is uniform on every
    // rank - which the caller has to guarantee; a ragged call is refused.
    bool uniform = true;
    for (int r = 0; r < n && uniform; r++) {
      uniform = sendcounts[r] == sendcounts[0] && recvcounts[r] == sendcounts[0] && sdispls[r] == static_cast<size_t>(r) * sendcounts[0] &&
                rdispls[r] == static_cast<size_t>(r) * sendcounts[0];
    }
    if (uniform) return ncclAlltoAll(sendbuff, recvbuff, sendcounts[0], datatype, comm, stream);
    return fail(ncclInvalidUsage, "alltoallv with ragged counts needs the fallback NCCL (set MSCCLPP_NCCL_LIB_PATH)");
  }
  RealNccl& r = realNccl();
  const size_t ts = typeSize(datatype);
  ncclResult_t rc = r.GroupStart();
  for (int peer = 0; peer < n && rc == ncclSuccess; peer++) {
    if (sendcounts[peer] > 0) rc = r.Send(static_cast<const char*>(sendbuff) + sdispls[peer] * ts, sendcounts[peer], datatype, peer, comm->real, stream);
    if (rc == ncclSuccess && recvcounts[peer] > 0) rc = r.Recv(static_cast<char*>(recvbuff) + rdispls[peer] * ts, recvcounts[peer], datatype, peer, comm->real, stream);
  }
  const ncclResult_t end = r.GroupEnd();
  return rc != ncclSuccess ? rc : end;
}

ncclResult_t mscclLoadAlgo(const char* mscclAlgoFilePath, mscclAlgoHandle_t* mscclAlgoHandle, int rank) {
  if (mscclAlgoFilePath == nullptr || mscclAlgoHandle == nullptr) return ncclInvalidArgument;
  try {
    ExecutionPlan plan(mscclAlgoFilePath, rank);
    auto algo = std::make_shared<DslAlgorithm>(mscclAlgoFilePath, plan);
    std::lock_guard<std::mutex> lock(loadedAlgoMutex);
    *mscclAlgoHandle = nextAlgoHandle++;
    loadedAlgos[*mscclAlgoHandle] = algo;
    return ncclSuccess;
  } catch (const std::exception& e) {
    return fail(ncclInvalidUsage, std::string("mscclLoadAlgo: ") + e.what());
  }
}

ncclResult_t mscclRunAlgo(const void* sendBuff, const size_t[] /*sendCounts*/, const size_t[] /*sDisPls*/, void* recvBuff,
                          const size_t[] /*recvCounts*/, const size_t[] /*rDisPls*/, size_t count, ncclDataType_t dataType, int /*root*/,
                          int /*peer*/, ncclRedOp_t op, mscclAlgoHandle_t mscclAlgoHandle, ncclComm_t comm, cudaStream_t stream) {
  if (comm == nullptr || comm->destroyed) return fail(ncclInvalidArgument, "mscclRunAlgo: invalid communicator");
  std::shared_ptr<DslAlgorithm> algo;
  {
    std::lock_guard<std::mutex> lock(loadedAlgoMutex);
    auto it = loadedAlgos.find(mscclAlgoHandle);
    if (it == loadedAlgos.end()) return fail(ncclInvalidArgument, "mscclRunAlgo: unknown algorithm handle");
    algo = it->second;
  }
  DataType dtype;
  if (!toDataType(dataType, dtype)) return fail(ncclInvalidArgument, "mscclRunAlgo: unsupported data type");
  if (op != ncclSum && op != ncclMin) return fail(ncclInvalidArgument, "mscclRunAlgo: sum and min are supported");
  // `count` follows the NCCL convention of the plan's collective
  const size_t unit = count * typeSize(dataType), all = unit * static_cast<size_t>(comm->nranks);
  const std::string& coll = algo->collective();
  const size_t inBytes = (coll == "reducescatter" || coll == "alltoall") ? all : unit;
  const size_t outBytes = (coll == "allgather" || coll == "alltoall") ? all : unit;
  if (sendBuff == nullptr || recvBuff == nullptr) return ncclInvalidArgument;
  if (count == 0) return ncclSuccess;
  const CommResult r = algo->execute(comm->comm, sendBuff, recvBuff, inBytes, outBytes, dtype, op == ncclMin ? MIN : SUM, stream,
                                     comm->executor, 0, 0, false, {}, DataType::AUTO);
  return r == CommResult::Success ? ncclSuccess : fail(toNccl(r), "mscclRunAlgo: " + algo->name() + " failed");
}

ncclResult_t mscclUnloadAlgo(mscclAlgoHandle_t mscclAlgoHandle) {
  std::lock_guard<std::mutex> lock(loadedAlgoMutex);
  return loadedAlgos.erase(mscclAlgoHandle) == 1 ? ncclSuccess : ncclInvalidArgument;
}

ncclResult_t ncclSend(const void* sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream) {
  if (comm == nullptr) return ncclInvalidArgument;
  if (comm->real != nullptr) return realNccl().Send(sendbuff, count, datatype, peer, comm->real, stream);
  return fail(ncclInvalidUsage, "send: pipeline point-to-point stays on NCCL (set MSCCLPP_NCCL_LIB_PATH)");
}

ncclResult_t ncclRecv(void* recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream) {
  if (comm == nullptr) return ncclInvalidArgument;
  if (comm->real != nullptr) return realNccl().Recv(recvbuff, count, datatype, peer, comm->real, stream);
  return fail(ncclInvalidUsage, "recv: pipeline point-to-point stays on NCCL (set MSCCLPP_NCCL_LIB_PATH)");
}

ncclResult_t ncclGroupStart(void) {
  RealNccl& r = realNccl();
  return r.ok ? r.GroupStart() : ncclSuccess;
}
ncclResult_t ncclGroupEnd(void) {
  RealNccl& r = realNccl();
  return r.ok ? r.GroupEnd() : ncclSuccess;
}
ncclResult_t ncclGroupSimulateEnd(ncclSimInfo_t*) { return fail(ncclInvalidUsage, "ncclGroupSimulateEnd is not supported"); }

}  // extern "C"
