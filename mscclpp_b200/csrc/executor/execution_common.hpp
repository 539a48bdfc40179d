// Device-side representation of an execution plan: what the host resolves per (plan, message size)
// and the interpreter kernel consumes.
#pragma once

#include <cstdint>

#include <mscclpp/device/symm.cuh>
#include <mscclpp/fifo_device.hpp>

#include <mscclpp/npkit/npkit_struct.hpp>

namespace mscclpp {

enum class OpType : uint8_t {
  NOP = 0,
  BARRIER,
  SIGNAL,
  RELAXED_SIGNAL,
  WAIT,
  RELAXED_WAIT,
  FLUSH,
  PUT,
  PUT_WITH_SIGNAL,
  PUT_WITH_SIGNAL_AND_FLUSH,
  GET,
  COPY,
  REDUCE,
  REDUCE_SEND,
  READ_REDUCE,
  READ_REDUCE_SEND,
  PUT_PACKETS,
  READ_PUT_PACKETS,
  COPY_PACKETS,
  UNPACK_PACKETS,
  REDUCE_PACKETS,
  REDUCE_SEND_PACKETS,
  REDUCE_COPY_PACKETS,
  REDUCE_COPY_SEND_PACKETS,
  GROUP_LOAD_REDUCE_STORE,
  GROUP_STORE,
  GROUP_STORE_PACKETS,
  SEM_ACQUIRE,
  SEM_RELEASE,
  PIPELINE_BEGIN,
  PIPELINE_END,
};

constexpr int kExecMaxOperands = 16;
constexpr int kExecMaxIds = 16;
constexpr int kExecMaxThreadBlocks = 128;
constexpr int kExecMaxChannels = 256;     // per channel type and rank
constexpr int kExecMaxSemaphores = 64;
constexpr int kExecMaxBarriers = 32;
constexpr int kExecMaxRanksInGroup = 16;

// One buffer range. `offset` is a HEAP offset (payload space); packet-space operands are expanded by the
// kernel (scratch base + 2 x payload offset, for LL16 and LL8 alike).
struct DevOperand {
  uint64_t offset;      // heap offset of the first byte (payload space)
  uint64_t size;        // bytes (payload space)
  int16_t rank;         // owning rank (local operands: the executing rank)
  uint8_t isScratch;    // scratch buffer: packet ops address it in packet space
  uint8_t isSwitch;     // multimem operand: address through mcBase (group = all ranks of switchGroup)
  uint16_t switchGroup; // index into DevPlan::groups
  uint16_t pad;
};

struct DevOp {
  uint8_t type;         // OpType
  uint8_t nSrc;
  uint8_t nDst;
  uint8_t nIds;
  uint8_t channelType;  // 0 memory, 1 port
  uint8_t inPipeline;   // operands are sliced per pipeline iteration
  uint16_t pad;
  uint32_t arg0;        // BARRIER: number of thread blocks; PIPELINE_BEGIN: iterations
  uint32_t arg1;        // PIPELINE_BEGIN: unit size in bytes; BARRIER: barrier id
  uint16_t ids[kExecMaxIds];  // channel ids (rank-level) or semaphore ids
  DevOperand src[kExecMaxOperands];
  DevOperand dst[kExecMaxOperands];
};

struct DevChannel {
  int16_t peer;       // rank at the other end
  int16_t mate;       // index of the paired channel on the peer
};

struct DevGroup {
  int16_t nRanks;
  int16_t ranks[kExecMaxRanksInGroup];
};

struct DevThreadBlock {
  uint32_t opBegin;
  uint32_t opEnd;
};

// Per-rank state kept in the heap (same offset on every rank): channel semaphores are written by peers.
struct ExecState {
  uint64_t inbound[2][kExecMaxChannels];   // [memory/port][channel]: signals received
  uint64_t expected[2][kExecMaxChannels];  // private: signals consumed
  int32_t semaphores[kExecMaxSemaphores];  // device semaphores of the plan (reset to init values per launch by block 0)
  uint32_t barriers[kExecMaxBarriers];     // grid barrier counters (monotonic)
  uint32_t barrierGen[kExecMaxBarriers];   // completed barrier generations (written by the last launch's end)
  uint32_t semInit;                        // launch epoch for which `semaphores` has been initialised
};

struct DevPlan {
  uint32_t nThreadBlocks;
  uint32_t nOps;
  DevThreadBlock tbs[kExecMaxThreadBlocks];
  DevChannel channels[2][kExecMaxChannels];
  DevGroup groups[8];
  int32_t semInit[kExecMaxSemaphores];
  uint32_t nSemaphores;
  uint32_t pad;
  const DevOp* ops;       // device array
};

// Request of a port-channel operation to the executor's host proxy (one 16-byte FIFO trigger):
//   fst: source heap offset [0,40) | size low 20 bits [40,60) | issuing rank [60,64)
//   snd: destination heap offset [0,40) | size high 8 bits [40,48) | channel id [48,56) | kind [56,59) | context [59,63)
// (bit 63 of snd belongs to the FIFO). Sizes are bytes, at most kPortMaxBytes per request.
constexpr uint64_t kPortMaxBytes = (1ull << 28) - 16;
constexpr uint32_t kPortData = 1, kPortSignal = 2, kPortSync = 4;
struct PortRequest {
  uint64_t srcOff, dstOff, size;
  uint32_t rank, channel, kind, context;
};
MSCCLPP_HOST_DEVICE_INLINE ProxyTrigger encodePortRequest(const PortRequest& r) {
  ProxyTrigger t;
  t.fst = (r.srcOff & ((1ull << 40) - 1)) | ((r.size & 0xfffffull) << 40) | (static_cast<uint64_t>(r.rank & 15u) << 60);
  t.snd = (r.dstOff & ((1ull << 40) - 1)) | (((r.size >> 20) & 0xffull) << 40) | (static_cast<uint64_t>(r.channel & 255u) << 48) |
          (static_cast<uint64_t>(r.kind & 7u) << 56) | (static_cast<uint64_t>(r.context & 15u) << 59);
  return t;
}
MSCCLPP_HOST_DEVICE_INLINE PortRequest decodePortRequest(const ProxyTrigger& t) {
  PortRequest r;
  r.srcOff = t.fst & ((1ull << 40) - 1);
  r.size = ((t.fst >> 40) & 0xfffffull) | (((t.snd >> 40) & 0xffull) << 20);
  r.rank = static_cast<uint32_t>(t.fst >> 60) & 15u;
  r.dstOff = t.snd & ((1ull << 40) - 1);
  r.channel = static_cast<uint32_t>(t.snd >> 48) & 255u;
  r.kind = static_cast<uint32_t>(t.snd >> 56) & 7u;
  r.context = static_cast<uint32_t>(t.snd >> 59) & 15u;
  return r;
}

struct ExecArgs {
  DeviceComm comm;
  const DevPlan* plans[kMaxRanks];  // [emulated rank]; real mode uses entry 0
  uint64_t stateOff;     // heap offset of ExecState
  uint64_t scratchOff;   // heap offset of the scratch buffer (first half when double buffered)
  uint64_t scratchHalf;  // bytes of one scratch half (0 = no double buffering)
  int emuRanks;
  int packetLL8;         // packet ops use 8-byte LL8 packets instead of 16-byte LL16 ones
  int portContext;       // index of this plan context in the host proxy's table
  FifoDeviceHandle portFifo;  // request queue of the executor's host proxy (triggers == nullptr: the plan has no port ops)
  NpKitEventCollectContext* npkit;  // tracer buffers, nullptr = tracing off
};

}  // namespace mscclpp
