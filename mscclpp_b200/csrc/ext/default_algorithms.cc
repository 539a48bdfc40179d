// Default native algorithms on a symmetric heap, registered under the reference's names
// (src/ext/collectives/algorithm_collection_builder.cc:64-104), and the B200 selector.
//
// How the names map onto this library's kernels:
//   default_allreduce_packet                        one-shot LL16 over peer stores (any local buffers)
//   default_allreduce_allpair_packet                one-shot LL8 over peer stores (8-byte packets: lowest latency, tiny messages)
//   default_allreduce_nvls_packet                   one-shot LL16, one multimem.st per packet
//   default_allreduce_nvls_zero_copy                two-shot multimem.ld_reduce + multimem.st (heap buffers)
//   default_allreduce_rsag_zero_copy                two-shot peer loads + stores (heap buffers)
//   for user buffers outside the heap, ONE kernel that copies in, reduces through heap scratch and copies out, slice by
//   slice (collectives_pipeline.cu):
//   default_allreduce_nvls_block_pipeline           switch reduction, 64 KB slices
//   default_allreduce_nvls_warp_pipeline            switch reduction, 16 KB slices (finer grain for mid sizes)
//   default_allreduce_rsag_pipeline                 peer loads/stores, 64 KB slices
//   default_allreduce_rsag / _fullmesh              peer loads/stores, the whole message in one round (<= scratch / 4)
//   default_allgather_fullmesh / _fullmesh2, default_reducescatter_zero_copy     two-shot kernel in AG / RS mode
#include <mscclpp/ext/collectives/algorithm_collection_builder.hpp>

#include <algorithm>
#include <cstdlib>
#include <dirent.h>
#include <mutex>

#include <mscclpp/env.hpp>
#include <mscclpp/gpu_utils.hpp>

#include "../core/logger.hpp"
#include "../kernels/collectives.cuh"

namespace mscclpp {
namespace collective {

namespace {

struct Staging {
  std::shared_ptr<SymmetricHeap> heap;
  void* in = nullptr;
  void* out = nullptr;
  size_t inBytes = 0, outBytes = 0;
  void* ensure(void*& slot, size_t& have, size_t bytes) {
    if (have >= bytes) return slot;
    AvoidCudaGraphCaptureGuard guard;
    if (slot) {
      (void)cudaDeviceSynchronize();
      heap->free(slot);
    }
    size_t rounded = 256;
    while (rounded < bytes) rounded <<= 1;  // every rank rounds the same way -> symmetric offsets
    slot = heap->alloc(rounded, 256);
    have = rounded;
    return slot;
  }
};

CommResult toResult(cudaError_t e) { return e == cudaSuccess ? CommResult::Success : (e == cudaErrorInvalidValue ? CommResult::InvalidArgument : CommResult::UnhandledCudaError); }

CollArgs baseArgs(SymmetricHeap& heap, const void* in, void* out, size_t bytes, int mode, bool nvls) {
  CollArgs a{};
  a.comm = heap.deviceComm();
  a.in = in;
  a.out = out;
  a.bytes = bytes;
  a.emuRanks = 1;
  a.mode = mode;
  a.nvls = nvls ? 1 : 0;
  return a;
}

void gridFor(size_t bytes, bool nvls, int& blocks, int& threads) {
  threads = 512;
  if (nvls) blocks = bytes < (8u << 20) ? 16 : (bytes < (64u << 20) ? 32 : 64);
  // peer loads are bound by what one SM keeps in flight over NVLink: from 1 MB on one block per SM, 128 of them
  else blocks = bytes < (1u << 20) ? 32 : 128;
}

std::shared_ptr<Algorithm> makeLL(const std::string& name, std::shared_ptr<SymmetricHeap> heap, bool nvls, bool ll8 = false) {
  const size_t cap = heap->deviceComm().llSlotBytes / 2;
  return std::make_shared<NativeAlgorithm>(
      name, "allreduce", nullptr,
      [heap, nvls, ll8](const void* in, void* out, size_t inBytes, size_t, DataType dtype, ReduceOp op, cudaStream_t stream, int nBlocks,
                        int nThreads, bool, const std::unordered_map<std::string, uintptr_t>&) {
        CollArgs a = baseArgs(*heap, in, out, inBytes, kAllReduce, nvls);
        a.ll8 = ll8 ? 1 : 0;
        const size_t units = (inBytes + 15) / 16;
        if (nThreads <= 0) nThreads = 512;
        if (nBlocks <= 0) nBlocks = static_cast<int>(std::max<size_t>(1, std::min<size_t>(56, (units + nThreads - 1) / nThreads)));
        return toResult(launchAllreduceLL(a, dtype, op, nBlocks, nThreads, stream));
      },
      0, cap, CollectiveBufferMode::Any);
}

std::shared_ptr<Algorithm> makeTwoShot(const std::string& name, const std::string& collective, std::shared_ptr<SymmetricHeap> heap,
                                       int mode, bool nvls, bool staged, std::shared_ptr<Staging> staging) {
  return std::make_shared<NativeAlgorithm>(
      name, collective, nullptr,
      [heap, mode, nvls, staged, staging](const void* in, void* out, size_t inBytes, size_t outBytes, DataType dtype, ReduceOp op,
                                          cudaStream_t stream, int nBlocks, int nThreads, bool,
                                          const std::unordered_map<std::string, uintptr_t>&) {
        const size_t big = std::max(inBytes, outBytes);
        if (nBlocks <= 0 || nThreads <= 0) gridFor(big, nvls, nBlocks, nThreads);
        const void* kin = in;
        void* kout = out;
        // Peers read `in` (allreduce, reducescatter) and write `out` (allreduce, allgather): only those sides
        // must live in the heap. An allreduce whose size is not a multiple of 16 bytes is padded in staging.
        const bool padded = mode == kAllReduce && inBytes % 16 != 0;
        // The choice between the caller's buffers and staging is the same on every rank: it rests on sizes, on the mode
        // and on symmetricOnAllRanks(), never on where THIS rank's buffer happens to be. (all-to-all reads `in` locally
        // only, like all-gather.)
        const bool needIn = mode != kAllGather && mode != kAllToAll && (padded || !heap->symmetricOnAllRanks(in, inBytes));
        const bool needOut = mode != kReduceScatter && (padded || !heap->symmetricOnAllRanks(out, outBytes));
        if (needIn || needOut) {
          if (!staged) return CommResult::InvalidUsage;
          if (needIn) {
            kin = staging->ensure(staging->in, staging->inBytes, inBytes);
            if (cudaMemcpyAsync(const_cast<void*>(kin), in, inBytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return CommResult::UnhandledCudaError;
          }
          if (needOut) kout = (mode == kAllReduce && needIn) ? const_cast<void*>(kin) : staging->ensure(staging->out, staging->outBytes, outBytes);
        }
        if (padded) inBytes = (inBytes + 15) / 16 * 16;
        CollArgs a = baseArgs(*heap, kin, kout, mode == kAllGather ? outBytes : inBytes, mode, nvls);
        cudaError_t e = launchTwoShot(a, dtype, op, nBlocks, nThreads, stream);
        if (e != cudaSuccess) return toResult(e);
        if (kout != out && cudaMemcpyAsync(out, kout, outBytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return CommResult::UnhandledCudaError;
        return CommResult::Success;
      },
      0, UINT64_MAX, CollectiveBufferMode::Any);
}

// Pipeline scratch of one heap: carved out when the default algorithms are built (a collective moment, so the offset is the
// same on every rank) and shared by the pipeline algorithms, which run one at a time on a heap anyway.
struct PipeScratch {
  std::shared_ptr<SymmetricHeap> heap;
  void* base = nullptr;
  size_t bytes = 0;
  ~PipeScratch() {
    try {
      if (base) heap->free(base);
    } catch (...) {
    }
  }
};

// Largest message of the LL128 allreduce: every rank receives the whole message from every peer, so the useful range (and
// the scratch, 2 x world x 1.07 x this) shrinks as the world grows.
size_t ll128MaxBytes(int world) { return world <= 2 ? (4u << 20) : (world <= 4 ? (512u << 10) : (256u << 10)); }

// One-shot allreduce with 128-byte lines (120 bytes of payload + flag), in a zeroed heap scratch of its own.
std::shared_ptr<Algorithm> makeLL128(const std::string& name, std::shared_ptr<SymmetricHeap> heap, std::shared_ptr<PipeScratch> scratch,
                                     size_t slotBytes) {
  return std::make_shared<NativeAlgorithm>(
      name, "allreduce", nullptr,
      [heap, scratch, slotBytes](const void* in, void* out, size_t inBytes, size_t, DataType dtype, ReduceOp op, cudaStream_t stream, int nBlocks,
                                 int nThreads, bool, const std::unordered_map<std::string, uintptr_t>&) {
        CollArgs a = baseArgs(*heap, in, out, inBytes, kAllReduce, false);
        a.ll128Scratch = scratch->base;
        a.ll128SlotBytes = slotBytes;
        const size_t lines = (inBytes + 119) / 120;
        if (nThreads <= 0) nThreads = 512;
        if (nBlocks <= 0) nBlocks = static_cast<int>(std::max<size_t>(1, std::min<size_t>(64, (lines * 8 + nThreads - 1) / nThreads)));
        return toResult(launchAllreduceLL128(a, dtype, op, nBlocks, nThreads, stream));
      },
      0, ll128MaxBytes(heap->world()), CollectiveBufferMode::Any);
}

// Allreduce of buffers outside the heap in one kernel. sliceBytes == 0: one round covers the whole message.
std::shared_ptr<Algorithm> makePipeline(const std::string& name, std::shared_ptr<SymmetricHeap> heap, bool nvls, size_t sliceBytes,
                                        std::shared_ptr<PipeScratch> scratch) {
  const int world = heap->world();
  const size_t maxBytes = sliceBytes == 0 ? scratch->bytes / 4 : UINT64_MAX;
  return std::make_shared<NativeAlgorithm>(
      name, "allreduce", nullptr,
      [heap, nvls, sliceBytes, scratch, world](const void* in, void* out, size_t inBytes, size_t, DataType dtype, ReduceOp op, cudaStream_t stream,
                                                int nBlocks, int nThreads, bool, const std::unordered_map<std::string, uintptr_t>&) {
        const size_t unit = 16 * static_cast<size_t>(world);
        size_t slice = sliceBytes;
        int maxBlocks = 128;
        if (slice == 0) {
          // one round: as many blocks as give each at least 16 KB, each block's slice a multiple of 16 * world bytes
          int blocks = static_cast<int>(std::min<size_t>(maxBlocks, std::max<size_t>(1, inBytes / (16u << 10))));
          if (nBlocks > 0) blocks = std::min(nBlocks, kBarrierSlots);
          slice = ((inBytes + blocks - 1) / blocks + unit - 1) / unit * unit;
          if (pipelineScratchBytes(blocks, slice) > scratch->bytes) return CommResult::InvalidUsage;
          nBlocks = blocks;
        } else {
          slice = (slice + unit - 1) / unit * unit;
          maxBlocks = static_cast<int>(std::min<size_t>(kBarrierSlots, scratch->bytes / (4 * slice)));
          if (maxBlocks < 1) return CommResult::InvalidUsage;
          const int want = static_cast<int>(std::min<size_t>(maxBlocks, (inBytes + slice - 1) / slice));
          nBlocks = nBlocks > 0 ? std::min(nBlocks, maxBlocks) : std::min(want, 128);
        }
        if (nThreads <= 0) nThreads = 512;
        PipeArgs a{};
        a.comm = heap->deviceComm();
        a.in = in;
        a.out = out;
        a.bytes = inBytes;
        a.scratch = scratch->base;
        a.sliceBytes = slice;
        a.emuRanks = 1;
        a.nvls = nvls ? 1 : 0;
        return toResult(launchPipelineAllreduce(a, dtype, op, nBlocks, nThreads, stream));
      },
      0, maxBytes, CollectiveBufferMode::Any);
}

// Broadcast: the root's `in` goes to every rank's `out` (staged through the heap when `out` is an ordinary buffer).
// The root travels in extras["root"].
std::shared_ptr<Algorithm> makeBroadcast(std::shared_ptr<SymmetricHeap> heap, bool nvls, std::shared_ptr<Staging> staging) {
  return std::make_shared<NativeAlgorithm>(
      "default_broadcast", "broadcast", nullptr,
      [heap, nvls, staging](const void* in, void* out, size_t inBytes, size_t outBytes, DataType, ReduceOp, cudaStream_t stream, int nBlocks,
                            int nThreads, bool, const std::unordered_map<std::string, uintptr_t>& extras) {
        auto it = extras.find("root");
        if (it == extras.end() || inBytes != outBytes) return CommResult::InvalidArgument;
        const int root = static_cast<int>(it->second);
        const size_t padded = (inBytes + 15) / 16 * 16;
        if (nBlocks <= 0 || nThreads <= 0) gridFor(padded, nvls, nBlocks, nThreads);
        // every rank writes into / receives in a heap buffer at the same offset; the root's source may be anywhere
        const bool direct = padded == inBytes && heap->contains(out, outBytes);
        void* kout = direct ? out : staging->ensure(staging->out, staging->outBytes, padded);
        const void* kin = in;
        if (heap->rank() == root && padded != inBytes) {
          // pad the source through the staging buffer so that the kernel moves whole 16-byte words
          kin = staging->ensure(staging->in, staging->inBytes, padded);
          if (cudaMemcpyAsync(const_cast<void*>(kin), in, inBytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return CommResult::UnhandledCudaError;
        } else if (padded != inBytes) {
          (void)staging->ensure(staging->in, staging->inBytes, padded);  // keep the allocation sequence equal on all ranks
        }
        CollArgs a = baseArgs(*heap, kin, kout, padded, kBroadcast, nvls);
        a.root = root;
        cudaError_t e = launchTwoShot(a, DataType::UINT32, SUM, nBlocks, nThreads, stream);
        if (e != cudaSuccess) return toResult(e);
        if (kout != out && cudaMemcpyAsync(out, kout, outBytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) return CommResult::UnhandledCudaError;
        return CommResult::Success;
      },
      0, UINT64_MAX, CollectiveBufferMode::Any);
}

}  // namespace

std::shared_ptr<AlgorithmCollectionBuilder> AlgorithmCollectionBuilder::getInstance() {
  static std::shared_ptr<AlgorithmCollectionBuilder> instance;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  if (!instance) instance = std::shared_ptr<AlgorithmCollectionBuilder>(new AlgorithmCollectionBuilder());
  return instance;
}

void AlgorithmCollectionBuilder::reset() {
  auto self = getInstance();
  self->builders_.clear();
  self->selector_ = nullptr;
  self->fallbackSelector_ = nullptr;
}

void AlgorithmCollectionBuilder::addAlgorithmBuilder(std::shared_ptr<AlgorithmBuilder> builder) { builders_.push_back(std::move(builder)); }
void AlgorithmCollectionBuilder::setAlgorithmSelector(AlgoSelectFunc selector) { selector_ = std::move(selector); }
void AlgorithmCollectionBuilder::setFallbackAlgorithmSelector(AlgoSelectFunc selector) { fallbackSelector_ = std::move(selector); }

AlgorithmCollection AlgorithmCollectionBuilder::build() {
  AlgorithmCollection c;
  for (auto& b : builders_) {
    auto algo = b->build();
    c.registerAlgorithm(algo->collective(), algo->name(), algo);
  }
  c.setSelectors(selector_, fallbackSelector_ ? fallbackSelector_ : selectDefaultAlgorithm);
  return c;
}

AlgorithmCollection AlgorithmCollectionBuilder::buildDefaultAlgorithms(std::shared_ptr<SymmetricHeap> heap) {
  AlgorithmCollection c = build();
  const bool nvls = heap->nvls();
  auto staging = std::make_shared<Staging>();
  staging->heap = heap;
  auto add = [&c](std::shared_ptr<Algorithm> a) { c.registerAlgorithm(a->collective(), a->name(), a); };
  add(makeLL("default_allreduce_packet", heap, false));
  add(makeLL("default_allreduce_allpair_packet", heap, false, true));
  if (nvls) add(makeLL("default_allreduce_nvls_packet", heap, true));
  if (nvls) add(makeTwoShot("default_allreduce_nvls_zero_copy", "allreduce", heap, kAllReduce, true, false, staging));
  add(makeTwoShot("default_allreduce_rsag_zero_copy", "allreduce", heap, kAllReduce, false, false, staging));
  // LL128 lines for the mid-size range: a scratch of their own (see collectives.cu), zeroed before anybody may write into it
  {
    auto llScratch = std::make_shared<PipeScratch>();
    llScratch->heap = heap;
    const size_t slot = (ll128MaxBytes(heap->world()) + 119) / 120 * 128;
    const size_t want = ll128ScratchBytes(heap->world(), slot);
    if (heap->bytesFree() >= want + (64u << 20)) {
      try {
        llScratch->base = heap->alloc(want, 256);
        llScratch->bytes = want;
      } catch (const BaseError&) {
        llScratch->base = nullptr;
      }
    }
    if (llScratch->base != nullptr) {
      if (cudaMemset(llScratch->base, 0, want) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        (void)cudaGetLastError();
        heap->free(llScratch->base);
        llScratch->base = nullptr;
      }
    }
    // every rank must agree on whether the algorithm exists, and nobody may send lines before everybody has zeroed
    int mine = llScratch->base != nullptr ? 1 : 0;
    std::vector<int> all(heap->world(), 0);
    all[heap->rank()] = mine;
    if (heap->bootstrap()) {
      heap->bootstrap()->allGather(all.data(), sizeof(int));
    }
    bool everybody = true;
    for (int v : all) everybody = everybody && v != 0;
    if (everybody) {
      add(makeLL128("default_allreduce_packet_ll128", heap, llScratch, slot));
    } else if (llScratch->base != nullptr) {
      heap->free(llScratch->base);
      llScratch->base = nullptr;
    }
  }
  // Buffers outside the heap: one pipelined kernel through heap scratch. The scratch is carved out here, where every
  // rank is (building the collection is collective), never on a code path that only some ranks may take.
  auto pipeScratch = std::make_shared<PipeScratch>();
  pipeScratch->heap = heap;
  {
    size_t want = 32u << 20;  // 128 blocks x 64 KB slices, double buffered, in + out
    if (const char* e = std::getenv("MSCCLPP_PIPELINE_SCRATCH_MB")) want = static_cast<size_t>(std::max(1, std::atoi(e))) << 20;
    if (heap->bytesFree() >= want + (64u << 20)) {
      try {
        pipeScratch->base = heap->alloc(want, 256);
        pipeScratch->bytes = want;
      } catch (const BaseError&) {
        pipeScratch->base = nullptr;
      }
    }
  }
  if (pipeScratch->base != nullptr) {
    if (nvls) {
      add(makePipeline("default_allreduce_nvls_warp_pipeline", heap, true, 16u << 10, pipeScratch));
      add(makePipeline("default_allreduce_nvls_block_pipeline", heap, true, 64u << 10, pipeScratch));
    }
    add(makePipeline("default_allreduce_rsag", heap, false, 0, pipeScratch));
    add(makePipeline("default_allreduce_rsag_pipeline", heap, false, 64u << 10, pipeScratch));
    add(makePipeline("default_allreduce_fullmesh", heap, false, 0, pipeScratch));
  } else {
    // a heap too small for the scratch: copy in, two-shot kernel, copy out (three operations on the caller's stream)
    LOG_WARN(LogSubsys::ALGO, "symmetric heap too small for the pipeline scratch: buffers outside the heap take staged copies");
    if (nvls) add(makeTwoShot("default_allreduce_nvls_block_pipeline", "allreduce", heap, kAllReduce, true, true, staging));
    add(makeTwoShot("default_allreduce_rsag_pipeline", "allreduce", heap, kAllReduce, false, true, staging));
  }
  add(makeTwoShot("default_allgather_fullmesh", "allgather", heap, kAllGather, false, true, staging));
  add(makeTwoShot("default_allgather_fullmesh2", "allgather", heap, kAllGather, nvls, true, staging));
  add(makeTwoShot("default_reducescatter_zero_copy", "reducescatter", heap, kReduceScatter, nvls, true, staging));
  add(makeBroadcast(heap, nvls, staging));
  add(makeTwoShot("default_alltoall", "alltoall", heap, kAllToAll, false, true, staging));

  // DSL plans installed under <cache>/default/*.json
  const std::string dir = env()->cacheDir + "/default";
  if (DIR* d = opendir(dir.c_str())) {
    while (dirent* ent = readdir(d)) {
      std::string file = ent->d_name;
      if (file.size() < 6 || file.substr(file.size() - 5) != ".json") continue;
      try {
        ExecutionPlan plan(dir + "/" + file, heap->rank());
        if (plan.nRanks() != heap->world()) continue;
        auto algo = std::make_shared<DslAlgorithm>(file.substr(0, file.size() - 5), plan);
        c.registerAlgorithm(algo->collective(), algo->name(), algo);
      } catch (const BaseError& e) {
        LOG_WARN(LogSubsys::ALGO, "skipping plan ", file, ": ", e.what());
      }
    }
    closedir(d);
  }
  return c;
}

std::shared_ptr<Algorithm> selectDefaultAlgorithm(
    const std::unordered_map<std::string, std::unordered_map<std::string, std::shared_ptr<Algorithm>>>& algoMapByCollective,
    const CollectiveRequest& request) {
  auto it = algoMapByCollective.find(request.collective);
  if (it == algoMapByCollective.end()) return nullptr;
  const auto& algos = it->second;
  auto get = [&](const char* name) -> std::shared_ptr<Algorithm> {
    auto a = algos.find(name);
    return a == algos.end() ? nullptr : a->second;
  };
  // DSL plans that match the size and buffer mode take precedence, like in the reference
  for (auto& kv : algos) {
    if (kv.second->type() != AlgorithmType::DSL) continue;
    auto range = kv.second->messageRange();
    const bool modeOk = kv.second->bufferMode() == CollectiveBufferMode::Any || kv.second->bufferMode() == request.bufferMode();
    if (request.messageSize >= range.first && request.messageSize <= range.second && modeOk) return kv.second;
  }
  const size_t n = request.messageSize;
  const int world = request.worldSize;
  if (request.collective == "allreduce") {
    // Thresholds measured on 2, 4 and 8 B200s (eager launches, bf16). Every rank sends its whole buffer to every peer in
    // the one-shot packet algorithms, so their range shrinks as the world grows.
    auto pkt = get("default_allreduce_packet");
    auto nvlsPkt = get("default_allreduce_nvls_packet");
    const size_t llCap = pkt ? pkt->messageRange().second : 0;
    if (n <= (64u << 10) && nvlsPkt) return nvlsPkt;  // one multimem.st per packet: flat latency floor
    size_t pktMax = world <= 2 ? (1u << 20) : (world <= 4 ? (256u << 10) : (128u << 10));
    // buffers outside the heap pay the scratch detour on the large-message path, so packets stay ahead a little longer
    if (!request.symmetricMemory) pktMax *= 2;
    // 128-byte lines carry 15/16 payload instead of 1/2: ahead of the 16-byte packets from 64 KB on and of the two-shot
    // kernels (two cross-rank barriers, ~20 us before the first byte) up to a few MB (measured on two B200s in graph
    // replay: 1 MB 7.1 vs 10.4 us with LL16, 2 MB 11.0 vs 23.7 us two-shot, 4 MB 18.6 vs 27.2 us)
    auto pkt128 = get("default_allreduce_packet_ll128");
    if (pkt128 && n > (64u << 10) && n <= pkt128->messageRange().second) return pkt128;
    if (n <= pktMax && n <= llCap && pkt) return pkt;
    if (request.symmetricMemory && n % 16 == 0) {
      // with two ranks the switch has nothing to combine: plain peer loads and stores on 128 SMs win from 4 MB on
      // (measured on two B200s: 2 MB 24.6 vs 23.6 us through the switch, 4 MB 26.8 vs 28.5, 16 MB 52.0 vs 59.7)
      const bool preferSwitch = world > 2 || n < (4u << 20);
      if (preferSwitch) {
        if (auto a = get("default_allreduce_nvls_zero_copy")) return a;
      }
      return get("default_allreduce_rsag_zero_copy");
    }
    if (world > 2 || n < (16u << 20)) {
      if (auto a = get(n >= (4u << 20) ? "default_allreduce_nvls_block_pipeline" : "default_allreduce_nvls_warp_pipeline")) return a;
    }
    auto rsag = get("default_allreduce_rsag");
    if (rsag && n < (4u << 20) && n <= rsag->messageRange().second) return rsag;
    return get("default_allreduce_rsag_pipeline");
  }
  if (request.collective == "allgather") {
    if ((n * request.worldSize) % (16 * static_cast<size_t>(request.worldSize)) != 0) return nullptr;
    return get("default_allgather_fullmesh2");
  }
  if (request.collective == "broadcast") return get("default_broadcast");
  if (request.collective == "alltoall") {
    if (n % (16 * static_cast<size_t>(request.worldSize)) != 0) return nullptr;
    return get("default_alltoall");
  }
  if (request.collective == "reducescatter") {
    if (n % (16 * static_cast<size_t>(request.worldSize)) != 0) return nullptr;
    return get("default_reducescatter_zero_copy");
  }
  return nullptr;
}

}  // namespace collective
}  // namespace mscclpp
