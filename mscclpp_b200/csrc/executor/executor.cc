// ExecutionPlan (JSON -> per-rank op lists) and Executor (op lists -> DevPlan for a message size ->
// interpreter kernel launch). Chunk-to-byte arithmetic follows the plan format's rules
// (reference: src/core/executor/execution_plan.cc:191-216, 478-668; src/core/executor/executor.cc:158-563).
#include <mscclpp/executor.hpp>
#include <mscclpp/npkit/npkit.hpp>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <map>
#include <mutex>
#include <unordered_map>

#include <mscclpp/env.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/numa.hpp>
#include <mscclpp/proxy.hpp>

#include "../core/json.hpp"
#include "../core/logger.hpp"
#include "execution_common.hpp"
#include "execution_kernel.hpp"

namespace mscclpp {

namespace {

const std::unordered_map<std::string, OpType>& opNames() {
  static const std::unordered_map<std::string, OpType> table = {
      {"nop", OpType::NOP},
      {"barrier", OpType::BARRIER},
      {"signal", OpType::SIGNAL},
      {"rlxsignal", OpType::RELAXED_SIGNAL},
      {"wait", OpType::WAIT},
      {"rlxwait", OpType::RELAXED_WAIT},
      {"flush", OpType::FLUSH},
      {"put", OpType::PUT},
      {"pws", OpType::PUT_WITH_SIGNAL},
      {"pwsf", OpType::PUT_WITH_SIGNAL_AND_FLUSH},
      {"get", OpType::GET},
      {"copy", OpType::COPY},
      {"re", OpType::REDUCE},
      {"res", OpType::REDUCE_SEND},
      {"rre", OpType::READ_REDUCE},
      {"rres", OpType::READ_REDUCE_SEND},
      {"ppkt", OpType::PUT_PACKETS},
      {"rppkt", OpType::READ_PUT_PACKETS},
      {"cpkt", OpType::COPY_PACKETS},
      {"upkt", OpType::UNPACK_PACKETS},
      {"repkt", OpType::REDUCE_PACKETS},
      {"respkt", OpType::REDUCE_SEND_PACKETS},
      {"recpkt", OpType::REDUCE_COPY_PACKETS},
      {"recspkt", OpType::REDUCE_COPY_SEND_PACKETS},
      {"glres", OpType::GROUP_LOAD_REDUCE_STORE},
      {"gstore", OpType::GROUP_STORE},
      {"gstorepkt", OpType::GROUP_STORE_PACKETS},
      {"sem_acquire", OpType::SEM_ACQUIRE},
      {"sem_release", OpType::SEM_RELEASE},
  };
  return table;
}

uint64_t calcOffset(uint64_t sizeUnits, uint64_t index, uint64_t parts, uint64_t alignment) {
  const uint64_t q = sizeUnits / parts, r = sizeUnits % parts;
  return (index * q + std::min(index, r)) * alignment;
}

}  // namespace

// ------------------------------------------------------------------------------------------ ExecutionPlan
struct ExecutionPlan::Impl {
  json::Value root;
  int rank = 0;
  std::string name, collective, protocol;
  bool inplace = false;
  bool reuseResources = false;
  bool doubleScratch = false;
  uint64_t alignment = 16;
  uint64_t minSize = 0, maxSize = UINT64_MAX;
  int nThreadsPerBlock = 1024;
  int nRanks = 0;
  // mate[type][rank][channel] = (peer, peer's channel index)
  std::vector<std::vector<DevChannel>> mates[2];

  void load(json::Value&& v, int r) {
    root = std::move(v);
    rank = r;
    name = root.at("name").asString();
    collective = root.at("collective").asString();
    protocol = root.at("protocol").asString();
    if (protocol != "Simple" && protocol != "LL") throw Error("plan '" + name + "': unknown protocol " + protocol, ErrorCode::ExecutorError);
    inplace = root.boolOr("inplace", false);
    reuseResources = root.boolOr("reuse_resources", false);
    doubleScratch = root.boolOr("use_double_scratch_buffer", false);
    alignment = root.uintOr("buffer_alignment", 16);
    minSize = root.uintOr("min_message_size", 0);
    maxSize = root.uintOr("max_message_size", UINT64_MAX);
    nThreadsPerBlock = static_cast<int>(root.intOr("num_threads_per_block", 1024));
    const json::Value& gpus = root.at("gpus");
    nRanks = static_cast<int>(gpus.size());
    if (nRanks < 1 || nRanks > kMaxRanks) throw Error("plan '" + name + "': unsupported number of ranks", ErrorCode::ExecutorError);
    if (rank < 0 || rank >= nRanks) throw Error("plan '" + name + "' has no rank " + std::to_string(rank), ErrorCode::ExecutorError);
    pairChannels();
  }

  static int typeIndex(const std::string& t) {
    if (t == "memory") return 0;
    if (t == "port") return 1;
    return -1;
  }

  // The k-th channel from a to b pairs with the k-th channel from b to a (connections are made in per-peer order).
  void pairChannels() {
    const json::Value& gpus = root.at("gpus");
    for (int t = 0; t < 2; t++) {
      std::vector<std::vector<int>> peers(nRanks);
      for (int r = 0; r < nRanks; r++) {
        for (size_t c = 0; c < gpus.at(r).at("channels").size(); c++) {
          const json::Value& ch = gpus.at(r).at("channels").at(c);
          if (typeIndex(ch.at("channel_type").asString()) != t) continue;
          for (size_t i = 0; i < ch.at("connected_to").size(); i++) peers[r].push_back(static_cast<int>(ch.at("connected_to").at(i).asInt()));
        }
        if (peers[r].size() > static_cast<size_t>(kExecMaxChannels)) throw Error("plan '" + name + "': too many channels", ErrorCode::ExecutorError);
      }
      mates[t].assign(nRanks, {});
      for (int r = 0; r < nRanks; r++) {
        std::map<int, int> seen;
        for (size_t c = 0; c < peers[r].size(); c++) {
          const int p = peers[r][c];
          if (p < 0 || p >= nRanks) throw Error("plan '" + name + "': channel to invalid rank", ErrorCode::ExecutorError);
          const int k = seen[p]++;
          int mate = -1, count = 0;
          for (size_t i = 0; i < peers[p].size(); i++) {
            if (peers[p][i] == r) {
              if (count == k) {
                mate = static_cast<int>(i);
                break;
              }
              count++;
            }
          }
          mates[t][r].push_back(DevChannel{static_cast<int16_t>(p), static_cast<int16_t>(mate)});
        }
      }
    }
  }
};

ExecutionPlan::ExecutionPlan(const std::string& planPath, int rank) : impl_(std::make_shared<Impl>()) {
  impl_->load(json::parseFile(planPath), rank);
}
ExecutionPlan ExecutionPlan::fromString(const std::string& jsonText, int rank) {
  ExecutionPlan p;
  p.impl_ = std::make_shared<Impl>();
  p.impl_->load(json::parse(jsonText), rank);
  return p;
}
ExecutionPlan::~ExecutionPlan() = default;
ExecutionPlan::ExecutionPlan(const ExecutionPlan&) = default;
ExecutionPlan& ExecutionPlan::operator=(const ExecutionPlan&) = default;
std::string ExecutionPlan::name() const { return impl_->name; }
std::string ExecutionPlan::collective() const { return impl_->collective; }
std::string ExecutionPlan::protocol() const { return impl_->protocol; }
size_t ExecutionPlan::minMessageSize() const { return impl_->minSize; }
size_t ExecutionPlan::maxMessageSize() const { return impl_->maxSize; }
bool ExecutionPlan::isInPlace() const { return impl_->inplace; }
int ExecutionPlan::nRanks() const { return impl_->nRanks; }
int ExecutionPlan::nThreadsPerBlock() const { return impl_->nThreadsPerBlock; }

// ------------------------------------------------------------------------------------------ plan -> DevPlan
namespace {

struct Resolved {
  std::vector<DevOp> ops;
  DevPlan plan{};
  uint64_t scratchBytes = 0;  // one half
  bool usesPort = false;      // the plan has port-channel operations: its launches need the executor's host proxy
};

struct Layout {
  uint64_t S = 0, C = 0, A = 16;
  uint64_t chunkUpper = 0;
  uint64_t inOff = 0, outOff = 0, scratchOff = 0;  // heap offsets
  uint64_t inBytes = 0, outBytes = 0, scratchBytes = 0;  // extent of each buffer (scratch: one half, payload space)
  // Buffers OUTSIDE the heap that every rank has mapped (zero copy): delta[r] = address of rank r's buffer in this process
  // minus the base of rank r's heap, so that the interpreter's "heap base of the owner + offset" lands in the buffer
  // (unsigned arithmetic, the sum wraps to the right address). Heap-resident buffers have the same delta on every rank:
  // their heap offset.
  bool inMapped = false, outMapped = false;
  uint64_t inDelta[kMaxRanks] = {}, outDelta[kMaxRanks] = {};
};

class Resolver {
 public:
  Resolver(const ExecutionPlan::Impl& plan, int rank, const Layout& layout) : p_(plan), rank_(rank), l_(layout) {
    gpu_ = &p_.root.at("gpus").at(rank);
  }

  Resolved run() {
    Resolved out;
    const json::Value& tbs = gpu_->at("threadblocks");
    if (tbs.size() > static_cast<size_t>(kExecMaxThreadBlocks)) throw Error("plan '" + p_.name + "': too many thread blocks", ErrorCode::ExecutorError);
    out.plan.nThreadBlocks = static_cast<uint32_t>(tbs.size());
    collectGroups(out.plan);
    for (size_t t = 0; t < tbs.size(); t++) {
      tb_ = &tbs.at(t);
      out.plan.tbs[t].opBegin = static_cast<uint32_t>(out.ops.size());
      emitOps(tb_->at("ops"), out.ops, false);
      out.plan.tbs[t].opEnd = static_cast<uint32_t>(out.ops.size());
    }
    out.plan.nOps = static_cast<uint32_t>(out.ops.size());
    out.usesPort = usesPort_;
    for (int t = 0; t < 2; t++) {
      const auto& m = p_.mates[t][rank_];
      for (size_t c = 0; c < m.size(); c++) out.plan.channels[t][c] = m[c];
    }
    const json::Value& sems = gpu_->contains("semaphores") ? gpu_->at("semaphores") : emptyArray_;
    if (sems.size() > static_cast<size_t>(kExecMaxSemaphores)) throw Error("plan '" + p_.name + "': too many semaphores", ErrorCode::ExecutorError);
    out.plan.nSemaphores = static_cast<uint32_t>(sems.size());
    for (size_t i = 0; i < sems.size(); i++) out.plan.semInit[i] = static_cast<int32_t>(sems.at(i).at("init_value").asInt());
    return out;
  }

 private:
  void collectGroups(DevPlan& plan) {
    const json::Value& chans = gpu_->at("channels");
    int g = 0;
    for (size_t c = 0; c < chans.size(); c++) {
      const json::Value& ch = chans.at(c);
      if (ch.at("channel_type").asString() != "switch") continue;
      if (g >= 8) {
        // many switch channels usually repeat the same group (instances): share entries
      }
      const json::Value& ranks = ch.at("rank_groups").at(0).at("ranks");
      DevGroup grp{};
      grp.nRanks = static_cast<int16_t>(ranks.size());
      if (ranks.size() > static_cast<size_t>(kExecMaxRanksInGroup)) throw Error("switch group too large", ErrorCode::ExecutorError);
      for (size_t i = 0; i < ranks.size(); i++) grp.ranks[i] = static_cast<int16_t>(ranks.at(i).asInt());
      int found = -1;
      for (int i = 0; i < g; i++)
        if (std::memcmp(&plan.groups[i], &grp, sizeof(grp)) == 0) found = i;
      if (found < 0) {
        if (g >= 8) throw Error("plan '" + p_.name + "': more than 8 distinct switch groups", ErrorCode::ExecutorError);
        plan.groups[g] = grp;
        found = g++;
      }
      // older plan files name the buffer "buff"
      switchChannels_.push_back({ch.at(ch.contains("buffer_type") ? "buffer_type" : "buff").asString(), found});
    }
  }

  uint64_t baseOf(const std::string& type, int owner, bool viaSwitch) const {
    if (type == "s") return l_.scratchOff;
    if (type != "i" && type != "o") throw Error("plan '" + p_.name + "': unknown buffer type '" + type + "'", ErrorCode::ExecutorError);
    const bool mapped = type == "i" ? l_.inMapped : l_.outMapped;
    if (!mapped) return type == "i" ? l_.inOff : l_.outOff;
    if (viaSwitch) throw Error("plan '" + p_.name + "': switch channels need their buffers in the symmetric heap", ErrorCode::ExecutorError);
    return type == "i" ? l_.inDelta[owner] : l_.outDelta[owner];
  }

  DevOperand operand(const json::Value& o, const json::Value& op) const {
    const uint64_t units = l_.S / l_.A;
    uint64_t start = calcOffset(units, o.at("index").asUInt(), l_.C, l_.A);
    uint64_t end = calcOffset(units, o.at("index").asUInt() + o.at("size").asUInt(), l_.C, l_.A);
    if (op.contains("tbg_info")) {
      const uint64_t tb = op.at("tbg_info").at("tb_id").asUInt(), n = op.at("tbg_info").at("tbg_size").asUInt();
      const uint64_t spanUnits = (end - start) / l_.A;
      const uint64_t s2 = calcOffset(spanUnits, tb, n, l_.A), e2 = calcOffset(spanUnits, tb + 1, n, l_.A);
      end = start + e2;
      start = start + s2;
    }
    DevOperand d{};
    d.size = end - start;
    std::string type;
    if (o.contains("buffer_id")) {
      const std::string ctype = op.contains("channel_type") ? op.at("channel_type").asString() : "memory";
      const json::Value& refs = tb_->at("remote_buffer_refs");
      const json::Value* ids = nullptr;
      for (size_t i = 0; i < refs.size(); i++)
        if (refs.at(i).at("access_channel_type").asString() == ctype) ids = &refs.at(i).at("remote_buffer_ids");
      if (ids == nullptr) throw Error("plan '" + p_.name + "': thread block has no remote buffers for " + ctype, ErrorCode::ExecutorError);
      const json::Value& rb = gpu_->at("remote_buffers").at(ids->at(o.at("buffer_id").asUInt()).asUInt());
      d.rank = static_cast<int16_t>(rb.at("rank").asInt());
      type = rb.at("type").asString();
    } else if (o.contains("switch_channel_id")) {
      const json::Value& chans = tb_->at("channels");
      const json::Value* ids = nullptr;
      for (size_t i = 0; i < chans.size(); i++)
        if (chans.at(i).at("channel_type").asString() == "switch") ids = &chans.at(i).at("channel_ids");
      if (ids == nullptr) throw Error("plan '" + p_.name + "': thread block has no switch channels", ErrorCode::ExecutorError);
      const size_t gpuLevel = ids->at(o.at("switch_channel_id").asUInt()).asUInt();
      if (gpuLevel >= switchChannels_.size()) throw Error("plan '" + p_.name + "': switch channel index out of range", ErrorCode::ExecutorError);
      d.rank = static_cast<int16_t>(rank_);
      d.isSwitch = 1;
      d.switchGroup = static_cast<uint16_t>(switchChannels_[gpuLevel].second);
      type = switchChannels_[gpuLevel].first;
    } else {
      d.rank = static_cast<int16_t>(rank_);
      type = o.at("type").asString();
    }
    d.isScratch = type == "s" ? 1 : 0;
    d.offset = baseOf(type, d.rank, d.isSwitch != 0) + start;
    // Every range a plan names is checked against the buffer it names before anything is launched: a plan whose chunk
    // arithmetic runs past a buffer is reported here, with its name, instead of scribbling over the neighbours on the GPU
    // (the role a memory checker plays where one can be run). Packet ranges are checked in payload space; the packet
    // form spends exactly twice that inside the scratch half, which is sized for it.
    const uint64_t extent = type == "i" ? l_.inBytes : (type == "o" ? l_.outBytes : l_.scratchBytes);
    if (extent != 0 && start + d.size > extent) {
      throw Error("plan '" + p_.name + "': rank " + std::to_string(rank_) + " names bytes [" + std::to_string(start) + ", " +
                      std::to_string(start + d.size) + ") of a '" + type + "' buffer of " + std::to_string(extent) + " bytes",
                  ErrorCode::ExecutorError);
    }
    return d;
  }

  void emitOps(const json::Value& ops, std::vector<DevOp>& out, bool inPipeline) {
    for (size_t i = 0; i < ops.size(); i++) {
      const json::Value& op = ops.at(i);
      const std::string& name = op.at("name").asString();
      if (name == "pipeline") {
        if (inPipeline) throw Error("plan '" + p_.name + "': nested pipelines", ErrorCode::ExecutorError);
        const uint64_t unit = op.at("iter_context").at("unit_size").asUInt();
        const uint64_t chunks = op.at("iter_context").at("num_chunks").asUInt();
        if (unit == 0) throw Error("plan '" + p_.name + "': pipeline with unit size 0", ErrorCode::ExecutorError);
        DevOp begin{};
        begin.type = static_cast<uint8_t>(OpType::PIPELINE_BEGIN);
        begin.arg0 = static_cast<uint32_t>(std::max<uint64_t>(1, (chunks * l_.chunkUpper + unit - 1) / unit));
        begin.arg1 = static_cast<uint32_t>(unit);
        out.push_back(begin);
        emitOps(op.at("ops"), out, true);
        DevOp end{};
        end.type = static_cast<uint8_t>(OpType::PIPELINE_END);
        out.push_back(end);
        continue;
      }
      auto it = opNames().find(name);
      if (it == opNames().end()) throw Error("plan '" + p_.name + "': unknown op '" + name + "'", ErrorCode::ExecutorError);
      DevOp d{};
      d.type = static_cast<uint8_t>(it->second);
      d.inPipeline = inPipeline ? 1 : 0;
      const std::string ctype = op.contains("channel_type") ? op.at("channel_type").asString() : "";
      d.channelType = ctype == "port" ? 1 : 0;
      if (d.channelType == 1) usesPort_ = true;
      if (op.contains("src_buff")) {
        const json::Value& src = op.at("src_buff");
        if (src.size() > static_cast<size_t>(kExecMaxOperands)) throw Error("plan '" + p_.name + "': too many sources in one op", ErrorCode::ExecutorError);
        d.nSrc = static_cast<uint8_t>(src.size());
        for (size_t k = 0; k < src.size(); k++) d.src[k] = operand(src.at(k), op);
      }
      if (op.contains("dst_buff")) {
        const json::Value& dst = op.at("dst_buff");
        if (dst.size() > static_cast<size_t>(kExecMaxOperands)) throw Error("plan '" + p_.name + "': too many destinations in one op", ErrorCode::ExecutorError);
        d.nDst = static_cast<uint8_t>(dst.size());
        for (size_t k = 0; k < dst.size(); k++) d.dst[k] = operand(dst.at(k), op);
      }
      if (op.contains("channel_ids") && (ctype == "memory" || ctype == "port")) {
        const json::Value& ids = op.at("channel_ids");
        const json::Value& chans = tb_->at("channels");
        const json::Value* table = nullptr;
        for (size_t k = 0; k < chans.size(); k++)
          if (chans.at(k).at("channel_type").asString() == ctype) table = &chans.at(k).at("channel_ids");
        if (table == nullptr) throw Error("plan '" + p_.name + "': op uses " + ctype + " channels the thread block does not have", ErrorCode::ExecutorError);
        if (ids.size() > static_cast<size_t>(kExecMaxIds)) throw Error("plan '" + p_.name + "': too many channels in one op", ErrorCode::ExecutorError);
        d.nIds = static_cast<uint8_t>(ids.size());
        for (size_t k = 0; k < ids.size(); k++) d.ids[k] = static_cast<uint16_t>(table->at(ids.at(k).asUInt()).asUInt());
      }
      if (op.contains("semaphore_ids")) {
        const json::Value& ids = op.at("semaphore_ids");
        d.nIds = static_cast<uint8_t>(ids.size());
        for (size_t k = 0; k < ids.size(); k++) d.ids[k] = static_cast<uint16_t>(ids.at(k).asUInt());
      }
      if (it->second == OpType::BARRIER) {
        d.arg0 = static_cast<uint32_t>(op.at("num_threadblocks").asUInt());
        d.arg1 = static_cast<uint32_t>(op.at("barrier_id").asUInt());
        if (d.arg1 >= static_cast<uint32_t>(kExecMaxBarriers)) throw Error("plan '" + p_.name + "': barrier id too large", ErrorCode::ExecutorError);
      }
      out.push_back(d);
    }
  }

  const ExecutionPlan::Impl& p_;
  int rank_;
  bool usesPort_ = false;
  Layout l_;
  const json::Value* gpu_ = nullptr;
  const json::Value* tb_ = nullptr;
  json::Value emptyArray_ = [] {
    json::Value v;
    v.kind = json::Value::Kind::Array;
    return v;
  }();
  std::vector<std::pair<std::string, int>> switchChannels_;
};

}  // namespace

// ------------------------------------------------------------------------------------------ Executor
struct Executor::Impl {
  std::shared_ptr<SymmetricHeap> heap;
  std::shared_ptr<Communicator> comm;

  struct Context {
    void* state = nullptr;      // ExecState in the heap
    void* scratch = nullptr;    // heap
    uint64_t scratchHalf = 0;
    bool doubleScratch = false;
    void* stageIn = nullptr;    // heap staging for user buffers outside the heap
    void* stageOut = nullptr;
    size_t stageInBytes = 0, stageOutBytes = 0;
    uint64_t scratchBytesTotal = 0;
    // device plans for the last message size
    uint64_t S = 0;
    uint64_t placement = 0;   // hash of where the buffers were when the device plans were resolved
    int zeroCopyPlan = -1;    // 1: the plan may run on mapped user buffers (memory channels only), 0: not, -1: not looked at yet
    std::vector<DevOp*> devOps;
    std::vector<DevPlan*> devPlans;
    int maxThreadBlocks = 0;
    // port channels: what the host proxy needs to carry out a request of this context
    bool usesPort = false;
    int portIndex = -1;                                    // slot in Impl::portTable
    std::vector<std::vector<DevChannel>> portChannels;     // [local (emulated) rank][channel] -> peer, mate
    std::vector<std::vector<uint64_t>> portSignalsSent;    // [local rank][channel]: value last written to the peer's word
  };
  std::map<std::string, Context> contexts;

  // ---- zero copy on buffers outside the heap (the reference's executor registers whatever buffer it is given and
  // exchanges the handles, src/core/executor/executor.cc: setupRegisteredMemories): the buffer of every rank is mapped into
  // every other rank's address space once and found again by (address, size).
  struct MappedBuffer {
    RegisteredMemory local;
    std::vector<char> wire;                    // the local registration, serialised
    std::vector<RegisteredMemory> remote;      // [rank], imported
    std::vector<std::vector<char>> remoteWire; // what each rank sent last time (re-imported only when it changes)
    uint64_t address[kMaxRanks] = {};          // rank r's buffer as mapped here
    bool usable = false;
  };
  std::shared_ptr<mscclpp::Context> regContext;
  std::map<std::pair<uintptr_t, size_t>, MappedBuffer> mapped;
  uint64_t zeroCopyLaunches = 0;

  // ---- guard bands around the executor's own heap buffers (MSCCLPP_EXECUTOR_CANARY=1). The reference has no such
  // check; its plans are trusted. Here a plan's operands are range-checked when they are resolved, and the bands catch
  // what the checks cannot see: a kernel (this rank's or a peer's) that writes past the extent it was given.
  static constexpr size_t kGuardBytes = 256;
  static constexpr int kGuardByte = 0xA5;
  bool canaries = false;
  struct Guarded {
    std::string label;
    size_t bytes;
  };
  std::map<void*, Guarded> guarded;  // payload pointer -> what it is

  int localRanks() const { return heap->emulated() ? heap->world() : 1; }
  void* onRank(void* p, int r) const { return heap->emulated() ? heap->emulatedPtr(p, r) : p; }

  void* allocGuarded(size_t bytes, const std::string& label) {
    if (!canaries) return heap->alloc(bytes, 256);
    char* raw = static_cast<char*>(heap->alloc(bytes + 2 * kGuardBytes, 256));
    for (int r = 0; r < localRanks(); r++) {
      MSCCLPP_CUDATHROW(cudaMemset(onRank(raw, r), kGuardByte, kGuardBytes));
      MSCCLPP_CUDATHROW(cudaMemset(onRank(raw + kGuardBytes + bytes, r), kGuardByte, kGuardBytes));
    }
    MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
    guarded[raw + kGuardBytes] = Guarded{label, bytes};
    return raw + kGuardBytes;
  }

  void freeGuarded(void* p) {
    if (!canaries) {
      heap->free(p);
      return;
    }
    guarded.erase(p);
    heap->free(static_cast<char*>(p) - kGuardBytes);
  }

  std::vector<Executor::CanaryRegion> canaryRegions() const {
    std::vector<Executor::CanaryRegion> out;
    for (const auto& kv : guarded) {
      char* payload = static_cast<char*>(kv.first);
      for (int r = 0; r < localRanks(); r++) {
        const std::string who = heap->emulated() ? "/rank " + std::to_string(r) : std::string();
        out.push_back({kv.second.label + "/front" + who, reinterpret_cast<uint64_t>(onRank(payload - kGuardBytes, r)), kGuardBytes});
        out.push_back({kv.second.label + "/back" + who, reinterpret_cast<uint64_t>(onRank(payload + kv.second.bytes, r)), kGuardBytes});
      }
    }
    return out;
  }

  size_t checkCanaries() const {
    if (!canaries) return 0;
    MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
    const auto regions = canaryRegions();
    std::vector<unsigned char> host(kGuardBytes);
    for (const auto& reg : regions) {
      MSCCLPP_CUDATHROW(cudaMemcpy(host.data(), reinterpret_cast<const void*>(reg.address), reg.bytes, cudaMemcpyDeviceToHost));
      size_t first = reg.bytes, count = 0;
      for (size_t i = 0; i < reg.bytes; i++) {
        if (host[i] != kGuardByte) {
          if (first == reg.bytes) first = i;
          count++;
        }
      }
      if (count != 0)
        throw Error("executor guard band " + reg.label + ": " + std::to_string(count) + " of " + std::to_string(reg.bytes) +
                        " bytes were overwritten, the first at byte " + std::to_string(first) +
                        " of the band (a kernel wrote outside the buffer it was given)",
                    ErrorCode::ExecutorError);
    }
    return regions.size();
  }

  // The first execute() that names a buffer (address, size) exchanges its registration with every rank; later calls find
  // it in the cache. Like the reference's executor (its contexts are keyed by the buffers' addresses,
  // src/core/executor/executor.cc), this assumes that the ranks see new buffers on the same calls - true of programs that
  // allocate alike on every rank, and the only case in which an exchange could be entered by some ranks only.
  // MSCCLPP_EXECUTOR_ZERO_COPY=0 switches zero copy off for programs that cannot promise it. Returns null when some rank
  // could not export or import (then every rank stages, by the same answer, and remembers it).
  MappedBuffer* mapEverywhere(void* ptr, size_t bytes) {
    constexpr int kSlot = 1024;
    auto bs = heap->bootstrap();
    if (!bs) return nullptr;
    if (!regContext) regContext = mscclpp::Context::create();
    const int world = heap->world(), me = heap->rank();
    auto found = mapped.find({reinterpret_cast<uintptr_t>(ptr), bytes});
    if (found != mapped.end()) return found->second.usable ? &found->second : nullptr;
    MappedBuffer& mb = mapped[{reinterpret_cast<uintptr_t>(ptr), bytes}];
    if (mb.wire.empty()) {
      try {
        mb.local = regContext->registerMemory(ptr, bytes, TransportFlags(Transport::CudaIpc));
        mb.wire = mb.local.serialize();
        if (mb.wire.size() + 8 > kSlot) mb.wire.clear();
      } catch (const BaseError& e) {
        LOG_WARN(LogSubsys::EXEC, "buffer outside the heap cannot be exported (", e.what(), "): staged copies instead");
        mb.wire.clear();
      }
      mb.remote.assign(world, RegisteredMemory());
      mb.remoteWire.assign(world, {});
    }
    std::vector<char> all(static_cast<size_t>(world) * kSlot, 0);
    {
      char* mine = all.data() + static_cast<size_t>(me) * kSlot;
      const uint32_t len = static_cast<uint32_t>(mb.wire.size());
      std::memcpy(mine, &len, 4);
      if (len) std::memcpy(mine + 8, mb.wire.data(), len);
    }
    bs->allGather(all.data(), kSlot);
    int ok = 1;
    for (int r = 0; r < world && ok; r++) {
      const char* slot = all.data() + static_cast<size_t>(r) * kSlot;
      uint32_t len = 0;
      std::memcpy(&len, slot, 4);
      if (len == 0 || len + 8 > kSlot) {
        ok = 0;
        break;
      }
      if (r == me) {
        mb.address[r] = reinterpret_cast<uint64_t>(ptr);
        continue;
      }
      std::vector<char> wire(slot + 8, slot + 8 + len);
      if (wire != mb.remoteWire[r]) {
        try {
          mb.remote[r] = RegisteredMemory::deserialize(wire);
          mb.remoteWire[r] = wire;
        } catch (const BaseError& e) {
          LOG_WARN(LogSubsys::EXEC, "cannot import rank ", r, "'s buffer (", e.what(), "): staged copies instead");
          ok = 0;
          break;
        }
      }
      mb.address[r] = reinterpret_cast<uint64_t>(mb.remote[r].data());
      if (mb.address[r] == 0) ok = 0;
    }
    // a rank that failed to import says so; everybody takes the common answer
    std::vector<int> votes(world, 0);
    votes[me] = ok;
    bs->allGather(votes.data(), sizeof(int));
    for (int v : votes) ok = ok && v;
    mb.usable = ok != 0;
    return mb.usable ? &mb : nullptr;
  }

  // ---- host proxy for port-channel operations (the reference's executor owns a ProxyService the same way,
  // src/core/executor/executor.cc:145-155): one thread drains the FIFO the interpreter kernel pushes requests into.
  static constexpr int kPortContexts = 16;
  static constexpr int kSignalRing = 1024;
  std::unique_ptr<Proxy> proxy;
  cudaStream_t proxyStream = nullptr;
  uint64_t* signalRing = nullptr;  // pinned host words, one per signal in flight
  uint64_t signalsIssued = 0;
  Context* portTable[kPortContexts] = {};
  std::mutex portMutex;            // portTable is written by execute() and read by the proxy thread
  std::atomic<bool> proxyFailed{false};
  std::string proxyError;

  void failProxy(const std::string& what) {
    // Remember the failure for the next execute() and poison the device status, so that kernels waiting for a signal or a
    // flush that will never be honoured give up at once instead of running out their budget.
    {
      std::lock_guard<std::mutex> lock(portMutex);
      if (proxyError.empty()) proxyError = what;
    }
    proxyFailed.store(true);
    LOG_ERROR(LogSubsys::EXEC, "executor proxy: ", what);
    DeviceStatus* st = heap->deviceComm().status;
    if (st != nullptr) {
      static const uint32_t one = 1;
      (void)cudaMemcpy(&st->poisoned, &one, sizeof(one), cudaMemcpyHostToDevice);
    }
  }

  ProxyHandlerResult handlePortRequest(ProxyTrigger trigger) {
    const PortRequest r = decodePortRequest(trigger);
    Context* ctx = nullptr;
    {
      std::lock_guard<std::mutex> lock(portMutex);
      ctx = portTable[r.context % kPortContexts];
    }
    const int localRank = heap->emulated() ? static_cast<int>(r.rank) : 0;
    if (ctx == nullptr || localRank >= static_cast<int>(ctx->portChannels.size()) ||
        r.channel >= ctx->portChannels[localRank].size()) {
      failProxy("request names an unknown context or channel");
      return ProxyHandlerResult::Abort;
    }
    const DevChannel ch = ctx->portChannels[localRank][r.channel];
    const int srcRank = heap->emulated() ? static_cast<int>(r.rank) : heap->rank();
    char* srcBase = static_cast<char*>(heap->peerBase(srcRank));
    char* dstBase = static_cast<char*>(heap->peerBase(ch.peer));
    cudaError_t e = cudaSuccess;
    if ((r.kind & kPortData) && r.size != 0) {
      if (r.srcOff + r.size > heap->bytes() || r.dstOff + r.size > heap->bytes()) {
        failProxy("request reaches beyond the heap");
        return ProxyHandlerResult::Abort;
      }
      e = cudaMemcpyAsync(dstBase + r.dstOff, srcBase + r.srcOff, r.size, cudaMemcpyDeviceToDevice, proxyStream);
    }
    if (e == cudaSuccess && (r.kind & kPortSignal)) {
      // the peer's signal word receives the running count, stream-ordered behind the data
      if (signalsIssued != 0 && signalsIssued % kSignalRing == 0) e = cudaStreamSynchronize(proxyStream);  // ring slots are free again
      if (e == cudaSuccess) {
        uint64_t* slot = signalRing + signalsIssued % kSignalRing;
        signalsIssued++;
        *slot = ++ctx->portSignalsSent[localRank][r.channel];
        ExecState* peerState = reinterpret_cast<ExecState*>(dstBase + (reinterpret_cast<char*>(ctx->state) - static_cast<char*>(heap->localBase())));
        e = cudaMemcpyAsync(&peerState->inbound[1][ch.mate], slot, sizeof(uint64_t), cudaMemcpyHostToDevice, proxyStream);
      }
    }
    if (e == cudaSuccess && (r.kind & kPortSync)) e = cudaStreamSynchronize(proxyStream);
    if (e != cudaSuccess) {
      failProxy(std::string("CUDA call failed: ") + cudaGetErrorString(e));
      return ProxyHandlerResult::Abort;
    }
    return ProxyHandlerResult::Continue;
  }

  void ensureProxy() {
    if (proxy) return;
    AvoidCudaGraphCaptureGuard guard;
    int dev = 0;
    MSCCLPP_CUDATHROW(cudaGetDevice(&dev));
    MSCCLPP_CUDATHROW(cudaStreamCreateWithFlags(&proxyStream, cudaStreamNonBlocking));
    MSCCLPP_CUDATHROW(cudaHostAlloc(reinterpret_cast<void**>(&signalRing), kSignalRing * sizeof(uint64_t), cudaHostAllocDefault));
    proxy = std::make_unique<Proxy>([this](ProxyTrigger t) { return handlePortRequest(t); },
                                    [dev] {
                                      (void)cudaSetDevice(dev);
                                      try {
                                        numaBind(getDeviceNumaNode(dev));
                                      } catch (const BaseError&) {
                                        // best effort: the proxy works from any node
                                      }
                                    });
    proxy->start();
  }

  void stopProxy() {
    if (proxy) proxy->stop();
    proxy.reset();
    if (proxyStream) (void)cudaStreamDestroy(proxyStream);
    if (signalRing) (void)cudaFreeHost(signalRing);
    proxyStream = nullptr;
    signalRing = nullptr;
  }

  void freeDevPlans(Context& c) {
    for (auto p : c.devOps) detail::gpuFree(p);
    for (auto p : c.devPlans) detail::gpuFree(p);
    c.devOps.clear();
    c.devPlans.clear();
  }

  void freeContext(Context& c) {
    {
      std::lock_guard<std::mutex> lock(portMutex);
      for (auto& slot : portTable)
        if (slot == &c) slot = nullptr;
    }
    freeDevPlans(c);
    if (c.state) heap->free(c.state);
    if (c.scratch) freeGuarded(c.scratch);
    if (c.stageIn) freeGuarded(c.stageIn);
    if (c.stageOut) freeGuarded(c.stageOut);
    c = Context();
  }
};

namespace {
// MSCCLPP_NPKIT_DUMP_DIR switches the tracer on for the life time of the executor, like in the reference
// (src/core/executor/executor.cc: the constructor calls NpKit::Init, the destructor NpKit::Dump).
void startTracing(SymmetricHeap& heap) {
  if (!env()->npkitDumpDir.empty() && !NpKit::Enabled()) NpKit::Init(heap.rank());
}
bool canariesWanted() {
  const char* e = std::getenv("MSCCLPP_EXECUTOR_CANARY");
  return e != nullptr && e[0] != '\0' && e[0] != '0';
}
}  // namespace

Executor::Executor(std::shared_ptr<SymmetricHeap> heap) : impl_(std::make_unique<Impl>()) {
  impl_->heap = std::move(heap);
  impl_->canaries = canariesWanted();
  startTracing(*impl_->heap);
}

Executor::Executor(std::shared_ptr<Communicator> comm, std::shared_ptr<char>) : impl_(std::make_unique<Impl>()) {
  impl_->comm = comm;
  SymmetricHeap::Options opt;
  impl_->heap = SymmetricHeap::create(comm->bootstrap(), opt);
  impl_->canaries = canariesWanted();
  startTracing(*impl_->heap);
}

Executor::~Executor() {
  try {
    if (!env()->npkitDumpDir.empty() && NpKit::Enabled()) {
      NpKit::Dump(env()->npkitDumpDir);
      NpKit::Shutdown();
    }
    reset();
    impl_->stopProxy();
  } catch (...) {
  }
}

std::shared_ptr<SymmetricHeap> Executor::heap() const { return impl_->heap; }
uint64_t Executor::zeroCopyLaunches() const { return impl_->zeroCopyLaunches; }
std::vector<Executor::CanaryRegion> Executor::canaryRegions() const { return impl_->canaryRegions(); }
size_t Executor::checkCanaries() { return impl_->checkCanaries(); }

void Executor::reset() {
  (void)cudaDeviceSynchronize();
  std::exception_ptr overwritten;  // the buffers are returned either way; the finding is reported afterwards
  try {
    impl_->checkCanaries();
  } catch (...) {
    overwritten = std::current_exception();
  }
  for (auto& kv : impl_->contexts) impl_->freeContext(kv.second);
  impl_->contexts.clear();
  impl_->mapped.clear();  // imported mappings are released with their RegisteredMemory objects
  if (overwritten) std::rethrow_exception(overwritten);
}

void Executor::execute(int rank, void* sendbuff, void* recvbuff, size_t sendBuffSize, size_t recvBuffSize, DataType dataType,
                       const ExecutionPlan& plan, cudaStream_t stream, PacketType packetType) {
  SymmetricHeap& heap = *impl_->heap;
  const ExecutionPlan::Impl& p = *plan.impl_;
  if (impl_->proxyFailed.load()) {
    std::lock_guard<std::mutex> lock(impl_->portMutex);
    throw Error("the executor's host proxy failed earlier: " + impl_->proxyError, ErrorCode::ExecutorError);
  }
  if (!heap.emulated() && rank != heap.rank()) throw Error("Executor::execute: rank does not match the heap", ErrorCode::InvalidUsage);
  if (p.nRanks != heap.world()) throw Error("plan '" + p.name + "' is for " + std::to_string(p.nRanks) + " ranks, the heap has " + std::to_string(heap.world()), ErrorCode::ExecutorError);
  const json::Value& g0 = p.root.at("gpus").at(0);
  const uint64_t inChunks = g0.at("input_chunks").asUInt(), outChunks = g0.at("output_chunks").asUInt();
  Layout layout;
  layout.A = p.alignment;
  if (inChunks != 0) {
    layout.S = sendBuffSize;
    layout.C = inChunks;
  } else {
    layout.S = recvBuffSize;
    layout.C = outChunks;
  }
  if (layout.C == 0) throw Error("plan '" + p.name + "' has no chunks", ErrorCode::ExecutorError);
  if (layout.S % layout.A != 0) throw Error("message size must be a multiple of the plan's buffer alignment", ErrorCode::ExecutorError);
  if (layout.S < p.minSize || layout.S > p.maxSize) throw Error("message size outside the plan's range", ErrorCode::ExecutorError);
  layout.chunkUpper = std::max<uint64_t>(calcOffset(layout.S / layout.A, 1, layout.C, layout.A), (layout.S + layout.C - 1) / layout.C);

  Impl::Context& ctx = impl_->contexts[p.name];
  AvoidCudaGraphCaptureGuard guard;
  // ---- scratch sized for this message (collective: every rank takes the same decisions)
  uint64_t maxScratchChunks = 0;
  for (int r = 0; r < p.nRanks; r++) maxScratchChunks = std::max<uint64_t>(maxScratchChunks, p.root.at("gpus").at(r).at("scratch_chunks").asUInt());
  uint64_t half = maxScratchChunks * layout.chunkUpper * (p.protocol == "LL" ? 2 : 1);
  half = (half + 255) / 256 * 256;
  const uint64_t total = half * (p.doubleScratch ? 2 : 1);
  bool rebuild = ctx.devPlans.empty() || ctx.S != layout.S;
  if (ctx.state == nullptr) {
    ctx.state = heap.alloc(sizeof(ExecState), 256);
    for (int r = 0; r < (heap.emulated() ? heap.world() : 1); r++)
      MSCCLPP_CUDATHROW(cudaMemset(heap.emulated() ? heap.emulatedPtr(ctx.state, r) : ctx.state, 0, sizeof(ExecState)));
    MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
    if (heap.bootstrap()) heap.bootstrap()->barrier();  // nobody signals into a state block that is not zeroed yet
    rebuild = true;
  }
  if (total > ctx.scratchBytesTotal) {
    if (ctx.scratch) {
      MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
      impl_->freeGuarded(ctx.scratch);
    }
    ctx.scratch = total ? impl_->allocGuarded(total, p.name + "/scratch") : nullptr;
    if (ctx.scratch) {
      for (int r = 0; r < (heap.emulated() ? heap.world() : 1); r++)
        MSCCLPP_CUDATHROW(cudaMemset(heap.emulated() ? heap.emulatedPtr(ctx.scratch, r) : ctx.scratch, 0, total));
      MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
      if (heap.bootstrap()) heap.bootstrap()->barrier();
    }
    ctx.scratchBytesTotal = total;
    rebuild = true;
  }
  if (ctx.scratchHalf != half || ctx.doubleScratch != p.doubleScratch) rebuild = true;
  ctx.scratchHalf = half;
  ctx.doubleScratch = p.doubleScratch;

  // ---- buffers: in the heap -> in place; elsewhere -> mapped on every rank (zero copy) when the plan and the size allow
  // it, else staged through the heap
  const bool sameBuffer = p.inplace && recvbuff == sendbuff;
  auto symmetric = [&](void* user, size_t bytes) { return user == nullptr || bytes == 0 || heap.symmetricOnAllRanks(user, bytes); };
  const bool inSym = symmetric(sendbuff, sendBuffSize);
  const bool outSym = sameBuffer ? inSym : symmetric(recvbuff, recvBuffSize);
  if ((!inSym || !outSym) && heap.emulated()) throw Error("emulated ranks need buffers from the heap", ErrorCode::InvalidUsage);
  // Zero copy is decided from what every rank knows alike: the plan (memory channels only - the switch addresses heap
  // offsets, and the host proxy of the port channels copies inside the heap), the message size (small messages are staged: two
  // copies of less than a megabyte are not worth a mapping), the environment switch.
  Impl::MappedBuffer* inMap = nullptr;
  Impl::MappedBuffer* outMap = nullptr;
  if (!inSym || !outSym) {
    if (ctx.zeroCopyPlan < 0) {
      bool eligible = true;
      for (int r = 0; r < p.nRanks && eligible; r++) {
        const json::Value& chans = p.root.at("gpus").at(r).at("channels");
        for (size_t i = 0; i < chans.size() && eligible; i++) {
          const std::string type = chans.at(i).at("channel_type").asString();
          if (type == "port") eligible = false;
          if (type == "switch") {
            const std::string buf = chans.at(i).at(chans.at(i).contains("buffer_type") ? "buffer_type" : "buff").asString();
            if (buf != "s") eligible = false;
          }
        }
      }
      ctx.zeroCopyPlan = eligible ? 1 : 0;
    }
    const char* knob = std::getenv("MSCCLPP_EXECUTOR_ZERO_COPY");
    size_t minBytes = 1u << 20;
    if (const char* e = std::getenv("MSCCLPP_EXECUTOR_ZERO_COPY_MIN_BYTES")) minBytes = static_cast<size_t>(std::strtoull(e, nullptr, 10));
    const bool want = ctx.zeroCopyPlan == 1 && !(knob != nullptr && knob[0] == '0') && std::max(sendBuffSize, recvBuffSize) >= minBytes;
    if (want) {
      bool ok = true;
      if (!inSym) {
        inMap = impl_->mapEverywhere(sendbuff, sendBuffSize);
        ok = inMap != nullptr;
      }
      if (ok && !outSym && !sameBuffer) {
        outMap = impl_->mapEverywhere(recvbuff, recvBuffSize);
        ok = outMap != nullptr;
      }
      if (!ok) inMap = outMap = nullptr;  // (the same answer on every rank) -> staged
      if (sameBuffer) outMap = inMap;
    }
  }
  auto stage = [&](void* user, size_t bytes, bool isSym, void*& slot, size_t& slotBytes, const char* what) -> void* {
    if (user == nullptr || bytes == 0 || isSym) return user;
    if (slotBytes < bytes) {
      if (slot) {
        MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
        impl_->freeGuarded(slot);
      }
      slot = impl_->allocGuarded(bytes, p.name + what);
      slotBytes = bytes;
      rebuild = true;
    }
    return slot;
  };
  void* in = inMap ? sendbuff : stage(sendbuff, sendBuffSize, inSym, ctx.stageIn, ctx.stageInBytes, "/staged input");
  void* out = sameBuffer ? in : (outMap ? recvbuff : stage(recvbuff, recvBuffSize, outSym, ctx.stageOut, ctx.stageOutBytes, "/staged output"));
  if (in != sendbuff) MSCCLPP_CUDATHROW(cudaMemcpyAsync(in, sendbuff, sendBuffSize, cudaMemcpyDeviceToDevice, stream));
  const uint64_t base = reinterpret_cast<uint64_t>(heap.localBase());
  layout.inOff = in ? reinterpret_cast<uint64_t>(in) - base : 0;
  layout.outOff = out ? reinterpret_cast<uint64_t>(out) - base : layout.inOff;
  if (p.inplace && (in == nullptr || out == nullptr)) {
    if (in == nullptr) layout.inOff = layout.outOff;
    if (out == nullptr) layout.outOff = layout.inOff;
  }
  const DeviceComm dc = heap.deviceComm();
  uint64_t placement = 1469598103934665603ull;  // what the device plans were resolved against (offsets, or every rank's mapping)
  auto mix = [&](uint64_t v) { placement = (placement ^ v) * 1099511628211ull; };
  if (inMap) {
    layout.inMapped = true;
    for (int r = 0; r < p.nRanks; r++) {
      layout.inDelta[r] = inMap->address[r] - dc.peerBase[r];
      mix(layout.inDelta[r]);
    }
  } else {
    mix(layout.inOff);
  }
  if (outMap) {
    layout.outMapped = true;
    for (int r = 0; r < p.nRanks; r++) {
      layout.outDelta[r] = outMap->address[r] - dc.peerBase[r];
      mix(layout.outDelta[r] + 1);
    }
  } else {
    mix(layout.outOff + 1);
  }
  if (inMap || outMap) impl_->zeroCopyLaunches++;
  layout.scratchOff = ctx.scratch ? reinterpret_cast<uint64_t>(ctx.scratch) - base : 0;
  layout.inBytes = in ? sendBuffSize : recvBuffSize;
  layout.outBytes = out ? recvBuffSize : sendBuffSize;
  layout.scratchBytes = maxScratchChunks * layout.chunkUpper;
  if (ctx.placement != placement) rebuild = true;

  // ---- device plans (cached per message size and buffer placement)
  if (rebuild) {
    MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
    impl_->freeDevPlans(ctx);
    const int nPlans = heap.emulated() ? heap.world() : 1;
    ctx.maxThreadBlocks = 0;
    ctx.usesPort = false;
    ctx.portChannels.assign(nPlans, {});
    if (ctx.portSignalsSent.size() != static_cast<size_t>(nPlans)) ctx.portSignalsSent.assign(nPlans, std::vector<uint64_t>(kExecMaxChannels, 0));
    for (int e = 0; e < nPlans; e++) {
      const int r = heap.emulated() ? e : heap.rank();
      Resolved res = Resolver(p, r, layout).run();
      ctx.usesPort = ctx.usesPort || res.usesPort;
      ctx.portChannels[e].assign(res.plan.channels[1], res.plan.channels[1] + kExecMaxChannels);
      DevOp* dops = static_cast<DevOp*>(detail::gpuCalloc(std::max<size_t>(1, res.ops.size()) * sizeof(DevOp)));
      if (!res.ops.empty()) gpuMemcpy(dops, res.ops.data(), res.ops.size() * sizeof(DevOp), cudaMemcpyHostToDevice);
      res.plan.ops = dops;
      DevPlan* dplan = static_cast<DevPlan*>(detail::gpuCalloc(sizeof(DevPlan)));
      gpuMemcpy(dplan, &res.plan, sizeof(DevPlan), cudaMemcpyHostToDevice);
      ctx.devOps.push_back(dops);
      ctx.devPlans.push_back(dplan);
      ctx.maxThreadBlocks = std::max<int>(ctx.maxThreadBlocks, static_cast<int>(res.plan.nThreadBlocks));
    }
    ctx.S = layout.S;
    ctx.placement = placement;
  }

  ExecArgs args{};
  args.comm = heap.deviceComm();
  for (size_t e = 0; e < ctx.devPlans.size(); e++) args.plans[e] = ctx.devPlans[e];
  args.stateOff = reinterpret_cast<uint64_t>(ctx.state) - base;
  args.scratchOff = layout.scratchOff;
  args.scratchHalf = p.doubleScratch ? half : 0;
  args.emuRanks = heap.emulated() ? heap.world() : 1;
  args.packetLL8 = packetType == PacketType::LL8 ? 1 : 0;
  if (ctx.usesPort) {
    impl_->ensureProxy();
    std::lock_guard<std::mutex> lock(impl_->portMutex);
    if (ctx.portIndex < 0) {
      // a free slot, else the one of the least recently created context (sixteen plans with port channels at a time)
      int slot = -1;
      for (int i = 0; i < Impl::kPortContexts && slot < 0; i++)
        if (impl_->portTable[i] == nullptr) slot = i;
      if (slot < 0) throw Error("more than 16 plans with port channels are live on this executor: call reset()", ErrorCode::ExecutorError);
      ctx.portIndex = slot;
    }
    impl_->portTable[ctx.portIndex] = &ctx;
    args.portContext = ctx.portIndex;
    args.portFifo = impl_->proxy->fifo()->deviceHandle();
  }
  args.npkit = NpKit::GetGpuEventCollectContexts();
  if (ctx.maxThreadBlocks > 0) {
    cudaError_t e = launchExecutionKernel(args, dataType, ctx.maxThreadBlocks, p.nThreadsPerBlock, stream);
    if (e == cudaErrorCooperativeLaunchTooLarge) {
      (void)cudaGetLastError();
      throw Error("plan '" + p.name + "' needs " + std::to_string(ctx.maxThreadBlocks) + " thread blocks of " + std::to_string(p.nThreadsPerBlock) +
                      " threads" + (args.emuRanks > 1 ? " for each of " + std::to_string(args.emuRanks) + " emulated ranks" : std::string()) +
                      " resident at the same time (its blocks wait on one another); this GPU cannot hold that many - use fewer thread "
                      "blocks or fewer threads per block",
                  ErrorCode::ExecutorError);
    }
    if (e != cudaSuccess) throw CudaError("execution kernel launch failed for plan '" + p.name + "'", static_cast<int>(e));
  }
  if (out != recvbuff && recvbuff != nullptr) {
    MSCCLPP_CUDATHROW(cudaMemcpyAsync(recvbuff, out, recvBuffSize, cudaMemcpyDeviceToDevice, stream));
  }
}

}  // namespace mscclpp
