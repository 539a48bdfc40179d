// Plan interpreter for sm_100a: one CUDA block per plan thread block walks its op list. Semantics of
// the 30 opcodes follow the execution-plan contract (reference handlers:
// src/core/include/execution_kernel.hpp:75-685), re-implemented on the symmetric heap:
//   * operands are (rank, heap offset) pairs resolved by the host; peer memory is peerBase[rank] + offset;
//   * channel signals are counters in the peer's ExecState; waits are bounded;
//   * port-channel put / signal / flush are REQUESTS to the executor's host proxy (a trigger in its FIFO, like the
//     reference's port channels, src/core/include/execution_kernel.hpp:120-187): the proxy thread copies the bytes with
//     the copy engines, writes the peer's signal word behind them and answers a flush when its stream has drained;
//   * LL packets (16-byte LL16 or 8-byte LL8, chosen per launch like the reference's PacketType) carry the launch epoch as
//     flag, so scratch is never cleared;
//   * switch ops use multimem when the heap has a multicast mapping and fall back to a loop over the
//     group's ranks otherwise (which is also how emulated ranks on one GPU run them);
//   * float-like types reduce with an fp32 accumulator and round once per op; fp8 plans work (the
//     reference silently skips them on CUDA).
#include "execution_kernel.hpp"

#include <mscclpp/copy_device.hpp>
#include <mscclpp/npkit/npkit.hpp>
#include <mscclpp/packet_device.hpp>

namespace mscclpp {

namespace {

template <typename T, bool kFloat = IsFloatLike<T>::value>
struct ExecAccum;
template <typename T>
struct ExecAccum<T, true> {
  float acc[Vec16<T>::kElems];
  MSCCLPP_DEVICE_INLINE void init(uint4 v) { Vec16<T>::toFloat(v, acc); }
  MSCCLPP_DEVICE_INLINE void add(uint4 v) { accumulate16<T, SUM>(acc, v); }
  MSCCLPP_DEVICE_INLINE uint4 result() const { return Vec16<T>::fromFloat(acc); }
};
template <typename T>
struct ExecAccum<T, false> {
  uint4 acc;
  MSCCLPP_DEVICE_INLINE void init(uint4 v) { acc = v; }
  MSCCLPP_DEVICE_INLINE void add(uint4 v) { acc = reduce16<T, SUM>(acc, v); }
  MSCCLPP_DEVICE_INLINE uint4 result() const { return acc; }
};

struct Ctx {
  const DeviceComm* c;
  const ExecArgs* a;
  const DevPlan* plan;
  ExecState* state;
  int rank;
  uint32_t epoch;
  uint64_t half;      // byte offset of the active scratch half
  uint64_t pipeOff;   // byte offset of the current pipeline iteration inside each operand
  uint64_t pipeUnit;  // bytes per pipeline iteration (0 = not in a pipeline)
  uint32_t* barrierPasses;  // shared memory: grid barriers this block has passed in this launch, per barrier id
  bool healthy;
};

// Byte range of an operand after pipeline slicing: returns size, sets `skip` to the offset inside the operand.
MSCCLPP_DEVICE_INLINE uint64_t sliced(const Ctx& x, const DevOp& op, const DevOperand& o, uint64_t& skip) {
  if (!op.inPipeline || x.pipeUnit == 0) {
    skip = 0;
    return o.size;
  }
  skip = x.pipeOff < o.size ? x.pipeOff : o.size;
  const uint64_t left = o.size - skip;
  return left < x.pipeUnit ? left : x.pipeUnit;
}
MSCCLPP_DEVICE_INLINE char* plainAddr(const Ctx& x, const DevOperand& o, uint64_t skip) {
  return reinterpret_cast<char*>(x.c->peerBase[o.rank] + o.offset + (o.isScratch ? x.half : 0) + skip);
}
// Packet space: scratch base + 2 x payload offset (both packet formats spend twice the payload: 16 bytes for 8, 8 for 4).
template <typename Pkt>
MSCCLPP_DEVICE_INLINE Pkt* pktAddr(const Ctx& x, const DevOperand& o, uint64_t skip, int rank) {
  static_assert(sizeof(Pkt) == 2 * sizeof(typename Pkt::Payload), "packet space is twice the payload space");
  const uint64_t payloadOff = o.offset - x.a->scratchOff + skip;
  return reinterpret_cast<Pkt*>(x.c->peerBase[rank] + x.a->scratchOff + x.half + 2 * payloadOff);
}

// `count` payload words (4 bytes each) starting at packet `pk`, into / out of a zero-padded 16-byte vector.
template <typename Pkt>
MSCCLPP_DEVICE_INLINE bool readWords(const Pkt* pk, int words, uint32_t epoch, uint4& out, const Ctx& x, int src) {
  uint32_t w[4] = {0, 0, 0, 0};
  if constexpr (sizeof(typename Pkt::Payload) == 8) {
    for (int i = 0; i < words / 2; i++) {
      uint2 v;
      if (!pk[i].read(epoch, v, x.c->status, x.c->timeoutNs, x.rank, src)) return false;
      w[2 * i] = v.x;
      w[2 * i + 1] = v.y;
    }
  } else {
    for (int i = 0; i < words; i++) {
      if (!pk[i].read(epoch, w[i], x.c->status, x.c->timeoutNs, x.rank, src)) return false;
    }
  }
  out = make_uint4(w[0], w[1], w[2], w[3]);
  return true;
}
template <typename Pkt>
MSCCLPP_DEVICE_INLINE void writeWords(Pkt* pk, int words, uint4 v, uint32_t epoch) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if constexpr (sizeof(typename Pkt::Payload) == 8) {
    for (int i = 0; i < words / 2; i++) pk[i].write(w[2 * i], w[2 * i + 1], epoch);
  } else {
    for (int i = 0; i < words; i++) pk[i].write(w[i], epoch);
  }
}

MSCCLPP_DEVICE_INLINE void signalChannels(const Ctx& x, const DevOp& op, bool relaxed) {
  const int t = threadIdx.x;
  if (t < op.nIds) {
    const DevChannel ch = x.plan->channels[op.channelType][op.ids[t]];
    ExecState* peer = reinterpret_cast<ExecState*>(x.c->peerBase[ch.peer] + x.a->stateOff);
    if (relaxed) {
      ptx::red_relaxed_sys_add(&peer->inbound[op.channelType][ch.mate], 1);
    } else {
      ptx::fence_acq_rel_sys();
      ptx::red_release_sys_add(&peer->inbound[op.channelType][ch.mate], 1);
    }
  }
}

MSCCLPP_DEVICE_INLINE void waitChannels(Ctx& x, const DevOp& op, bool relaxed) {
  __shared__ int waitOk;
  if (threadIdx.x == 0) waitOk = 1;
  __syncthreads();
  const int t = threadIdx.x;
  if (t < op.nIds) {
    const int cid = op.ids[t];
    const uint64_t expect = ++x.state->expected[op.channelType][cid];
    if (!waitGreaterEqual(&x.state->inbound[op.channelType][cid], expect, x.c->status, x.c->timeoutNs, kDevTimeoutSemaphore,
                          x.rank, 500 + cid, x.plan->channels[op.channelType][cid].peer)) {
      waitOk = 0;
    }
    (void)relaxed;  // acquire is used in both cases: a relaxed wait is a pure optimisation hint
  }
  __syncthreads();
  if (!waitOk) x.healthy = false;
}

// Port-channel operations: thread 0 queues one request per destination for the host proxy. kind: data and/or signal
// and/or sync; with sync the thread also waits (bounded) until the proxy has consumed the request, which it does only
// after its copy stream has drained.
// packetSpace: both ends are packet-format scratch ranges (the bytes moved are the packets themselves, twice the payload).
MSCCLPP_DEVICE_INLINE void portRequests(Ctx& x, const DevOp& op, uint32_t kind, bool packetSpace = false) {
  __shared__ int portOk;
  __syncthreads();  // data this block produced for the put is complete
  if (threadIdx.x == 0) {
    portOk = 1;
    __threadfence_system();  // ... and visible to the copy engines
    FifoDeviceHandle fifo = x.a->portFifo;
    uint64_t last = UINT64_MAX;
    const int n = (kind & kPortData) ? op.nDst : op.nIds;
    for (int i = 0; i < n && portOk; i++) {
      PortRequest r{};
      r.rank = static_cast<uint32_t>(x.rank);
      r.channel = op.ids[i < op.nIds ? i : 0];
      r.context = static_cast<uint32_t>(x.a->portContext);
      uint64_t left = 0, skip = 0;
      if (kind & kPortData) {
        const DevOperand& so = i < op.nSrc ? op.src[i] : op.src[0];
        left = sliced(x, op, so, skip);
        if (packetSpace) {
          r.srcOff = x.a->scratchOff + x.half + 2 * (so.offset - x.a->scratchOff + skip);
          r.dstOff = x.a->scratchOff + x.half + 2 * (op.dst[i].offset - x.a->scratchOff + skip);
          left *= 2;
        } else {
          r.srcOff = so.offset + (so.isScratch ? x.half : 0) + skip;
          r.dstOff = op.dst[i].offset + (op.dst[i].isScratch ? x.half : 0) + skip;
        }
      }
      do {  // large puts go out in pieces; signal and sync ride on the last one
        r.size = left > kPortMaxBytes ? kPortMaxBytes : left;
        left -= r.size;
        r.kind = left == 0 ? kind : kPortData;
        if (r.size == 0) r.kind &= ~kPortData;
        if (r.kind != 0) {
          last = fifo.push(encodePortRequest(r), x.c->status, x.c->timeoutNs);
          if (last == UINT64_MAX) portOk = 0;
        }
        r.srcOff += r.size;
        r.dstOff += r.size;
      } while (left != 0 && portOk);
    }
    if ((kind & kPortSync) && portOk && last != UINT64_MAX) {
      if (!fifo.sync(last, x.c->status, x.c->timeoutNs)) portOk = 0;
    }
  }
  __syncthreads();
  if (!portOk) x.healthy = false;
}

// dst[k] (all of them) = sum over src[*]. Sizes are multiples of 16 bytes (plans align chunks to 16).
template <typename T>
MSCCLPP_DEVICE_INLINE void reduceOp(const Ctx& x, const DevOp& op) {
  uint64_t skip;
  const uint64_t bytes = sliced(x, op, op.src[0], skip);
  const uint64_t nvec = bytes / 16;
  for (uint64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
    ExecAccum<T> acc;
    acc.init(ptx::ld_nc_na_v4(plainAddr(x, op.src[0], skip) + i * 16));
    for (int s = 1; s < op.nSrc; s++) acc.add(ptx::ld_nc_na_v4(plainAddr(x, op.src[s], skip) + i * 16));
    const uint4 r = acc.result();
    for (int d = 0; d < op.nDst; d++) ptx::st_na_v4(plainAddr(x, op.dst[d], skip) + i * 16, r);
  }
  // tail shorter than one vector (only with alignment < 16): element-wise through a zero-padded word
  const uint64_t tail = bytes - nvec * 16;
  if (tail != 0 && threadIdx.x == 0) {
    auto load = [&](const DevOperand& o) {
      uint32_t w[4] = {0, 0, 0, 0};
      const char* p = plainAddr(x, o, skip) + nvec * 16;
      for (uint64_t b = 0; b < tail; b++) w[b >> 2] |= static_cast<uint32_t>(static_cast<uint8_t>(p[b])) << (8 * (b & 3));
      return make_uint4(w[0], w[1], w[2], w[3]);
    };
    ExecAccum<T> acc;
    acc.init(load(op.src[0]));
    for (int s = 1; s < op.nSrc; s++) acc.add(load(op.src[s]));
    const uint4 r = acc.result();
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    for (int d = 0; d < op.nDst; d++) {
      char* p = plainAddr(x, op.dst[d], skip) + nvec * 16;
      for (uint64_t b = 0; b < tail; b++) p[b] = static_cast<char>(w[b >> 2] >> (8 * (b & 3)));
    }
  }
}

// Packet flavours of reduce: plain src[0] (+) packets src[1..] -> plain dst[0]; optionally the result as a
// packet into local dst[1] (copy variants) and as packets into the remaining (remote) destinations.
template <typename T, typename Pkt>
MSCCLPP_DEVICE_INLINE void reducePacketsOp(Ctx& x, const DevOp& op, bool copyPacket) {
  uint64_t skip;
  const uint64_t bytes = sliced(x, op, op.src[0], skip);
  constexpr int kPktPer16 = 16 / static_cast<int>(sizeof(typename Pkt::Payload));
  const uint64_t nvec = bytes / 16;  // full 16-byte units: the reduction runs on whole vectors
  // what is left after them is a whole number of payloads (a trailing 8-byte packet with LL16, up to three 4-byte ones
  // with LL8): thread 0 takes it through a zero-padded vector
  const int tailWords = static_cast<int>((bytes - nvec * 16) / 4);
  bool ok = true;
  auto unit = [&](uint64_t i, int words) {
    ExecAccum<T> acc;
    const char* srcp = plainAddr(x, op.src[0], skip) + i * 16;
    uint4 own;
    if (words == 4) {
      own = *reinterpret_cast<const uint4*>(srcp);
    } else {
      uint32_t w[4] = {0, 0, 0, 0};
      for (int k = 0; k < words; k++) w[k] = reinterpret_cast<const uint32_t*>(srcp)[k];
      own = make_uint4(w[0], w[1], w[2], w[3]);
    }
    acc.init(own);
    for (int s = 1; s < op.nSrc && ok; s++) {
      uint4 v;
      ok = readWords<Pkt>(pktAddr<Pkt>(x, op.src[s], skip, x.rank) + kPktPer16 * i, words, x.epoch, v, x, s);
      if (ok) acc.add(v);
    }
    if (!ok) return;
    const uint4 r = acc.result();
    char* dstp = plainAddr(x, op.dst[0], skip) + i * 16;
    if (words == 4) {
      *reinterpret_cast<uint4*>(dstp) = r;
    } else {
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
      for (int k = 0; k < words; k++) reinterpret_cast<uint32_t*>(dstp)[k] = w[k];
    }
    int d = 1;
    if (copyPacket && op.nDst > 1) {
      writeWords<Pkt>(pktAddr<Pkt>(x, op.dst[1], skip, x.rank) + kPktPer16 * i, words, r, x.epoch);
      d = 2;
    }
    for (; d < op.nDst; d++) writeWords<Pkt>(pktAddr<Pkt>(x, op.dst[d], skip, op.dst[d].rank) + kPktPer16 * i, words, r, x.epoch);
  };
  for (uint64_t i = threadIdx.x; i < nvec && ok; i += blockDim.x) unit(i, 4);
  if (ok && tailWords != 0 && threadIdx.x == 0) unit(nvec, tailWords);
  if (!ok) x.healthy = false;
}

template <typename T>
MSCCLPP_DEVICE_INLINE uint4 switchLoadReduce(const Ctx& x, const DevOperand& o, uint64_t byteOff) {
  if (x.c->mcBase != 0) {
    const void* mc = reinterpret_cast<const void*>(x.c->mcBase + o.offset + (o.isScratch ? x.half : 0) + byteOff);
    if constexpr (__is_same(T, __half)) return ptx::multimem_ld_reduce_add_f16x2_acc32(mc);
    else if constexpr (__is_same(T, __nv_bfloat16)) return ptx::multimem_ld_reduce_add_bf16x2_acc32(mc);
    else if constexpr (__is_same(T, float)) return ptx::multimem_ld_reduce_add_f32(mc);
    else if constexpr (__is_same(T, f8e4m3)) return ptx::multimem_ld_reduce_add_e4m3x4(mc);
    else if constexpr (__is_same(T, f8e5m2)) return ptx::multimem_ld_reduce_add_e5m2x4(mc);
  }
  // software path: no multicast mapping, or a type the switch cannot add
  const DevGroup& g = x.plan->groups[o.switchGroup];
  ExecAccum<T> acc;
  for (int i = 0; i < g.nRanks; i++) {
    const uint4 v = ptx::ld_nc_na_v4(reinterpret_cast<const void*>(x.c->peerBase[g.ranks[i]] + o.offset + (o.isScratch ? x.half : 0) + byteOff));
    if (i == 0) acc.init(v);
    else acc.add(v);
  }
  return acc.result();
}

MSCCLPP_DEVICE_INLINE void switchStore(const Ctx& x, const DevOperand& o, uint64_t byteOff, uint4 v) {
  if (x.c->mcBase != 0) {
    ptx::multimem_st_v4(reinterpret_cast<void*>(x.c->mcBase + o.offset + (o.isScratch ? x.half : 0) + byteOff), v);
    return;
  }
  const DevGroup& g = x.plan->groups[o.switchGroup];
  for (int i = 0; i < g.nRanks; i++)
    ptx::st_na_v4(reinterpret_cast<void*>(x.c->peerBase[g.ranks[i]] + o.offset + (o.isScratch ? x.half : 0) + byteOff), v);
}

template <typename T, typename Pkt>
MSCCLPP_DEVICE_INLINE void execOp(Ctx& x, const DevOp& op) {
  using Payload = typename Pkt::Payload;
  const OpType type = static_cast<OpType>(op.type);
  uint64_t skip = 0;
  switch (type) {
    case OpType::NOP:
      __syncthreads();
      break;
    case OpType::BARRIER: {
      __shared__ int barOk;
      __syncthreads();
      if (threadIdx.x == 0) {
        barOk = 1;
        const uint32_t target = (++x.barrierPasses[op.arg1]) * op.arg0;
        uint32_t* counter = &x.state->barriers[op.arg1];
        ptx::fence_acq_rel_gpu();
        ptx::red_release_gpu_add(counter, 1u);
        SpinGuard g(x.c->status, x.c->timeoutNs);
        uint32_t v;
        while (static_cast<int32_t>((v = ptx::ld_acquire_gpu(counter)) - target) < 0) {
          if (!g.keepSpinning()) {
            g.report(kDevTimeoutBarrier, x.rank, 600 + op.arg1, 0, target, v);
            barOk = 0;
            break;
          }
        }
      }
      __syncthreads();
      if (!barOk) x.healthy = false;
      break;
    }
    case OpType::SIGNAL:
      if (op.channelType == 1 && x.a->portFifo.triggers != nullptr) portRequests(x, op, kPortSignal);
      else signalChannels(x, op, false);
      break;
    case OpType::RELAXED_SIGNAL:
      if (op.channelType == 1 && x.a->portFifo.triggers != nullptr) portRequests(x, op, kPortSignal);
      else signalChannels(x, op, true);
      break;
    case OpType::WAIT:
      waitChannels(x, op, false);
      break;
    case OpType::RELAXED_WAIT:
      waitChannels(x, op, true);
      break;
    case OpType::FLUSH:
      // everything this rank asked of the proxy so far has been carried out when this returns
      if (x.a->portFifo.triggers != nullptr) portRequests(x, op, kPortSync);
      break;
    case OpType::PUT:
    case OpType::PUT_WITH_SIGNAL:
    case OpType::PUT_WITH_SIGNAL_AND_FLUSH:
      if (op.channelType == 1 && x.a->portFifo.triggers != nullptr) {
        portRequests(x, op, kPortData | (type != OpType::PUT ? kPortSignal : 0u) | (type == OpType::PUT_WITH_SIGNAL_AND_FLUSH ? kPortSync : 0u));
        break;
      }
      for (int i = 0; i < op.nDst; i++) {
        const uint64_t n = sliced(x, op, op.src[i], skip);
        copyBytes(plainAddr(x, op.dst[i], skip), plainAddr(x, op.src[i], skip), n, threadIdx.x, blockDim.x);
      }
      if (type != OpType::PUT) {
        __syncthreads();
        signalChannels(x, op, false);
      }
      break;
    case OpType::GET:
    case OpType::COPY:
      for (int i = 0; i < op.nDst; i++) {
        const uint64_t n = sliced(x, op, op.src[i], skip);
        copyBytes(plainAddr(x, op.dst[i], skip), plainAddr(x, op.src[i], skip), n, threadIdx.x, blockDim.x);
      }
      break;
    case OpType::REDUCE:
    case OpType::REDUCE_SEND:
    case OpType::READ_REDUCE:
    case OpType::READ_REDUCE_SEND:
      reduceOp<T>(x, op);
      break;
    case OpType::PUT_PACKETS:
      // over a port channel the source is packet-format scratch that this block completed earlier: the proxy moves the
      // packets as they are (the reference makes the same assumption, src/core/include/execution_kernel.hpp:275-289)
      if (op.channelType == 1 && x.a->portFifo.triggers != nullptr && op.src[0].isScratch) {
        portRequests(x, op, kPortData, true);
        break;
      }
      for (int i = 0; i < op.nDst; i++) {
        const DevOperand& s = i < op.nSrc ? op.src[i] : op.src[0];
        const uint64_t n = sliced(x, op, s, skip);
        copyToPackets<Pkt>(pktAddr<Pkt>(x, op.dst[i], skip, op.dst[i].rank), plainAddr(x, s, skip), n, threadIdx.x, blockDim.x, x.epoch);
      }
      break;
    case OpType::READ_PUT_PACKETS: {
      const uint64_t n = sliced(x, op, op.src[0], skip) / sizeof(Payload);
      const Pkt* in = pktAddr<Pkt>(x, op.src[0], skip, x.rank);
      bool ok = true;
      if (op.channelType == 1 && x.a->portFifo.triggers != nullptr) {
        // wait until every local packet of the range has arrived, then let the proxy forward the packets unchanged
        for (uint64_t i = threadIdx.x; i < n && ok; i += blockDim.x) {
          Payload v;
          ok = in[i].read(x.epoch, v, x.c->status, x.c->timeoutNs, x.rank, 0);
        }
        if (!__syncthreads_and(ok ? 1 : 0)) {
          x.healthy = false;
          break;
        }
        portRequests(x, op, kPortData, true);
        break;
      }
      for (uint64_t i = threadIdx.x; i < n && ok; i += blockDim.x) {
        Payload v;
        ok = in[i].read(x.epoch, v, x.c->status, x.c->timeoutNs, x.rank, 0);
        if (!ok) break;
        for (int d = 0; d < op.nDst; d++) pktAddr<Pkt>(x, op.dst[d], skip, op.dst[d].rank)[i].write(v, x.epoch);
      }
      if (!ok) x.healthy = false;
      break;
    }
    case OpType::COPY_PACKETS: {
      const uint64_t n = sliced(x, op, op.src[0], skip);
      copyToPackets<Pkt>(pktAddr<Pkt>(x, op.dst[0], skip, x.rank), plainAddr(x, op.src[0], skip), n, threadIdx.x, blockDim.x, x.epoch);
      break;
    }
    case OpType::UNPACK_PACKETS: {
      const uint64_t n = sliced(x, op, op.src[0], skip);
      if (!copyFromPackets<Pkt>(plainAddr(x, op.dst[0], skip), pktAddr<Pkt>(x, op.src[0], skip, x.rank), n, threadIdx.x, blockDim.x,
                                       x.epoch, x.c->status, x.c->timeoutNs)) {
        x.healthy = false;
      }
      break;
    }
    case OpType::REDUCE_PACKETS:
    case OpType::REDUCE_SEND_PACKETS:
      reducePacketsOp<T, Pkt>(x, op, false);
      break;
    case OpType::REDUCE_COPY_PACKETS:
    case OpType::REDUCE_COPY_SEND_PACKETS:
      reducePacketsOp<T, Pkt>(x, op, true);
      break;
    case OpType::GROUP_LOAD_REDUCE_STORE: {
      const uint64_t n = sliced(x, op, op.src[0], skip) / 16;
      for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) {
        const uint4 v = switchLoadReduce<T>(x, op.src[0], skip + i * 16);
        switchStore(x, op.dst[0], skip + i * 16, v);
      }
      break;
    }
    case OpType::GROUP_STORE: {
      const uint64_t n = sliced(x, op, op.src[0], skip) / 16;
      for (uint64_t i = threadIdx.x; i < n; i += blockDim.x)
        switchStore(x, op.dst[0], skip + i * 16, *reinterpret_cast<const uint4*>(plainAddr(x, op.src[0], skip) + i * 16));
      break;
    }
    case OpType::GROUP_STORE_PACKETS: {
      const uint64_t n = sliced(x, op, op.src[0], skip) / sizeof(Payload);
      const Pkt* in = pktAddr<Pkt>(x, op.src[0], skip, x.rank);
      const DevGroup& g = x.plan->groups[op.dst[0].switchGroup];
      bool ok = true;
      for (uint64_t i = threadIdx.x; i < n && ok; i += blockDim.x) {
        Payload v;
        ok = in[i].read(x.epoch, v, x.c->status, x.c->timeoutNs, x.rank, 0);
        if (!ok) break;
        if (x.c->mcBase != 0) {
          const uint64_t payloadOff = op.dst[0].offset - x.a->scratchOff + skip;
          void* mc = reinterpret_cast<void*>(x.c->mcBase + x.a->scratchOff + x.half + 2 * payloadOff + i * sizeof(Pkt));
          if constexpr (sizeof(Payload) == 8) {
            ptx::multimem_st_v4(mc, make_uint4(v.x, x.epoch, v.y, x.epoch));
          } else {
            ptx::multimem_st_v2(mc, make_uint2(v, x.epoch));
          }
        } else {
          for (int r = 0; r < g.nRanks; r++) pktAddr<Pkt>(x, op.dst[0], skip, g.ranks[r])[i].write(v, x.epoch);
        }
      }
      if (!ok) x.healthy = false;
      break;
    }
    case OpType::SEM_ACQUIRE:
    case OpType::SEM_RELEASE: {
      __shared__ int semOk;
      if (threadIdx.x == 0) semOk = 1;
      __syncthreads();
      if (threadIdx.x < op.nIds) {
        // semaphores are re-armed by block 0 at the start of every launch: wait for that first
        if (!waitGreaterEqual(&x.state->semInit, x.epoch, x.c->status, x.c->timeoutNs, kDevTimeoutSemaphore, x.rank, 700, 0)) {
          semOk = 0;
        } else {
          int* sem = &x.state->semaphores[op.ids[threadIdx.x]];
          if (type == OpType::SEM_RELEASE) {
            __threadfence();
            atomicAdd(sem, 1);
          } else {
            SpinGuard g(x.c->status, x.c->timeoutNs);
            while (true) {
              const int cur = *reinterpret_cast<volatile int*>(sem);
              if (cur > 0 && atomicCAS(sem, cur, cur - 1) == cur) {
                __threadfence();
                break;
              }
              if (!g.keepSpinning()) {
                g.report(kDevTimeoutSemaphore, x.rank, 701, 0, 1, static_cast<uint64_t>(cur));
                semOk = 0;
                break;
              }
            }
          }
        }
      }
      __syncthreads();
      if (!semOk) x.healthy = false;
      break;
    }
    default:
      break;
  }
}

// One operation with its entry/exit trace events (thread 0; the cost is one predictable branch when tracing is off).
template <typename T, typename Pkt>
MSCCLPP_DEVICE_INLINE void tracedOp(Ctx& x, const DevOp& op) {
  NpKitEventCollectContext* trace = x.a->npkit;
  if (trace != nullptr && threadIdx.x == 0)
    npkitCollectGpuEvent(trace, NPKIT_EVENT_EXECUTOR_OP_BASE_ENTRY + op.type, static_cast<uint32_t>(op.nSrc ? op.src[0].size : 0), x.rank);
  execOp<T, Pkt>(x, op);
  if (trace != nullptr) {
    // the exit stamp is taken when the whole block is done with the operation; the vote also keeps the
    // health flag uniform, so that every thread leaves the operation loop at the same place
    x.healthy = __syncthreads_and(x.healthy ? 1 : 0) != 0;
    if (threadIdx.x == 0)
      npkitCollectGpuEvent(trace, NPKIT_EVENT_EXECUTOR_OP_BASE_EXIT + op.type, static_cast<uint32_t>(op.nSrc ? op.src[0].size : 0), x.rank);
  }
}

template <typename T, typename Pkt>
__global__ void __launch_bounds__(1024, 1) executionKernel(ExecArgs a) {
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const uint32_t epoch = launchEpoch(c, rank);
  const DevPlan* plan = a.plans[blockIdx.y];
  ExecState* state = reinterpret_cast<ExecState*>(c.peerBase[rank] + a.stateOff);

  __shared__ uint32_t barrierPasses[kExecMaxBarriers];
  if (threadIdx.x < kExecMaxBarriers) barrierPasses[threadIdx.x] = 0;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (uint32_t i = 0; i < plan->nSemaphores; i++) state->semaphores[i] = plan->semInit[i];
    __threadfence();
    ptx::st_release_sys(&state->semInit, epoch);
  }

  if (blockIdx.x < plan->nThreadBlocks) {
    Ctx x;
    x.c = &c;
    x.a = &a;
    x.plan = plan;
    x.state = state;
    x.rank = rank;
    x.epoch = epoch;
    x.half = a.scratchHalf ? static_cast<uint64_t>(epoch & 1u) * a.scratchHalf : 0;
    x.pipeOff = 0;
    x.pipeUnit = 0;
    x.barrierPasses = barrierPasses;
    x.healthy = true;
    const DevThreadBlock tb = plan->tbs[blockIdx.x];
    const DevOp* ops = plan->ops;
    uint32_t i = tb.opBegin;
    while (i < tb.opEnd && x.healthy) {
      const DevOp& op = ops[i];
      if (static_cast<OpType>(op.type) == OpType::PIPELINE_BEGIN) {
        uint32_t end = i + 1;
        while (end < tb.opEnd && static_cast<OpType>(ops[end].type) != OpType::PIPELINE_END) end++;
        x.pipeUnit = op.arg1;
        for (uint32_t it = 0; it < op.arg0 && x.healthy; it++) {
          x.pipeOff = static_cast<uint64_t>(it) * op.arg1;
          for (uint32_t k = i + 1; k < end && x.healthy; k++) tracedOp<T, Pkt>(x, ops[k]);
        }
        x.pipeUnit = 0;
        x.pipeOff = 0;
        i = end + 1;
        continue;
      }
      tracedOp<T, Pkt>(x, op);
      i++;
    }
  }

  // end of launch: the last block re-arms the grid-barrier counters for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    SymmControl* ctl = control(c, rank);
    __threadfence();
    const uint32_t prev = atomicAdd(&ctl->done, 1u);
    if (prev == gridDim.x - 1) {
      ctl->done = 0;
      for (int b = 0; b < kExecMaxBarriers; b++) state->barriers[b] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&ctl->epoch) = epoch;
    }
  }
}

template <typename T>
cudaError_t launchTyped(const ExecArgs& args, int nBlocks, int nThreads, cudaStream_t stream) {
  dim3 grid(nBlocks, args.emuRanks > 1 ? args.emuRanks : 1, 1);
  dim3 block(nThreads, 1, 1);
  // thread blocks of a plan wait on one another (barriers, semaphores) and on peers: co-residency is required
  ExecArgs copy = args;
  void* params[] = {&copy};
  const void* kernel = args.packetLL8 ? reinterpret_cast<const void*>(executionKernel<T, LL8Packet>)
                                      : reinterpret_cast<const void*>(executionKernel<T, LL16Packet>);
  // every block of the launch has to be resident at once: say so here, with numbers, instead of leaving it to the launch
  int perSm = 0, sms = 0, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kernel, nThreads, 0) == cudaSuccess) {
    if (static_cast<long long>(perSm) * sms < static_cast<long long>(grid.x) * grid.y) return cudaErrorCooperativeLaunchTooLarge;
  }
  return cudaLaunchCooperativeKernel(kernel, grid, block, params, 0, stream);
}

}  // namespace

cudaError_t launchExecutionKernel(const ExecArgs& args, DataType dtype, int nBlocks, int nThreads, cudaStream_t stream) {
  if (nBlocks < 1 || nThreads < 32 || nThreads > 1024) return cudaErrorInvalidValue;
  switch (dtype) {
    case DataType::FLOAT16:
      return launchTyped<__half>(args, nBlocks, nThreads, stream);
    case DataType::BFLOAT16:
      return launchTyped<__nv_bfloat16>(args, nBlocks, nThreads, stream);
    case DataType::FLOAT32:
      return launchTyped<float>(args, nBlocks, nThreads, stream);
    case DataType::INT32:
      return launchTyped<int32_t>(args, nBlocks, nThreads, stream);
    case DataType::UINT32:
      return launchTyped<uint32_t>(args, nBlocks, nThreads, stream);
    case DataType::UINT8:
      return launchTyped<uint8_t>(args, nBlocks, nThreads, stream);
    case DataType::FLOAT8_E4M3:
      return launchTyped<f8e4m3>(args, nBlocks, nThreads, stream);
    case DataType::FLOAT8_E5M2:
      return launchTyped<f8e5m2>(args, nBlocks, nThreads, stream);
    case DataType::FLOAT8_E4M3B15:
      return launchTyped<f8e4m3b15>(args, nBlocks, nThreads, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace mscclpp
