// Native sm_100a collective kernels on the symmetric heap.
//
//  * allreduceLLKernel   one-shot LL16: each rank stores its whole input as {data,flag} packets into
//                        every peer's scratch (plain peer stores, or ONE multimem.st that the NVSwitch
//                        replicates), then reduces the N packet streams locally. No barrier at all.
//                        Role of the reference's allreduce_packet / allpair_packet / nvls_packet
//                        (src/ext/collectives/allreduce/allreduce_packet.cu:15-151,
//                         allreduce_allpair_packet.cu:15-69, allreduce_nvls_packet.cu:14-56).
//                        With kLL8 the same exchange uses 8-byte {data, flag} packets (one 8-byte store each, the
//                        format of the reference's all-pairs kernel, allreduce_allpair_packet.cu:15-69): twice the
//                        stores per byte of payload, but each packet is a single naturally atomic access.
//  * twoShotKernel       zero-copy reduce-scatter + all-gather in one pass: a rank reduces its 1/N of
//                        the buffer straight out of all peers' inputs (peer loads or
//                        multimem.ld_reduce) and writes the result into all peers' outputs (peer
//                        stores or multimem.st). Role of allreduce_rsag_zero_copy.cu:41-113 and
//                        allreduce_nvls_zero_copy.cu:16-69. Also serves standalone reduce-scatter
//                        and allgather (allgather_fullmesh_2.cu:11-118).
//  Both take an optional fused epilogue that the reference does not have: add a residual stream and
//  apply RMSNorm on the reduced rows before they are written, so the TP layer's allreduce,
//  residual-add and norm are one kernel.
#include "collectives.cuh"

#include <type_traits>

#include <mscclpp/packet_device.hpp>

namespace mscclpp {

namespace {

template <typename T>
struct ElemOf {
  using type = T;
};

MSCCLPP_DEVICE_INLINE uint4 loadUnit(const char* base, uint64_t u, uint64_t bytes) {
  const uint64_t off = u * 16;
  if (off + 16 <= bytes) return *reinterpret_cast<const uint4*>(base + off);
  uint32_t w[4] = {0, 0, 0, 0};
  for (uint64_t i = off; i < bytes; i++) {
    w[(i - off) >> 2] |= static_cast<uint32_t>(static_cast<uint8_t>(base[i])) << (8 * ((i - off) & 3));
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
MSCCLPP_DEVICE_INLINE void storeUnit(char* base, uint64_t u, uint64_t bytes, uint4 v) {
  const uint64_t off = u * 16;
  if (off + 16 <= bytes) {
    *reinterpret_cast<uint4*>(base + off) = v;
    return;
  }
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  for (uint64_t i = off; i < bytes; i++) base[i] = static_cast<char>(w[(i - off) >> 2] >> (8 * ((i - off) & 3)));
}

// Running reduction over 16-byte words. Callers feed the contributions in rank order so that every
// rank computes bit-identical results. Float-like types accumulate in fp32 and round once.
template <typename T, ReduceOp Op, bool kFloat = IsFloatLike<T>::value>
struct Accum;
template <typename T, ReduceOp Op>
struct Accum<T, Op, true> {
  float acc[Vec16<T>::kElems];
  MSCCLPP_DEVICE_INLINE void init(uint4 v) { Vec16<T>::toFloat(v, acc); }
  MSCCLPP_DEVICE_INLINE void add(uint4 v) { accumulate16<T, Op>(acc, v); }
  MSCCLPP_DEVICE_INLINE uint4 result() const { return Vec16<T>::fromFloat(acc); }
};
template <typename T, ReduceOp Op>
struct Accum<T, Op, false> {
  uint4 acc;
  MSCCLPP_DEVICE_INLINE void init(uint4 v) { acc = v; }
  MSCCLPP_DEVICE_INLINE void add(uint4 v) { acc = reduce16<T, Op>(acc, v); }
  MSCCLPP_DEVICE_INLINE uint4 result() const { return acc; }
};

// Block-wide sum of one float per thread (blockDim.x <= 1024).
MSCCLPP_DEVICE_INLINE float blockSum(float v) {
  __shared__ float warpSums[32];
  __shared__ float total;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();  // protects warpSums/total against the previous call
  if (lane == 0) warpSums[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float s = (lane < (blockDim.x + 31) / 32) ? warpSums[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) total = s;
  }
  __syncthreads();
  return total;
}

// x = reduced + residual (rounded to T); returns sum of squares of the rounded values.
template <typename T>
MSCCLPP_DEVICE_INLINE float addResidual(uint4& x, uint4 residual, bool hasResidual) {
  float f[Vec16<T>::kElems];
  Vec16<T>::toFloat(x, f);
  if (hasResidual) {
    float r[Vec16<T>::kElems];
    Vec16<T>::toFloat(residual, r);
#pragma unroll
    for (int i = 0; i < Vec16<T>::kElems; i++) f[i] += r[i];
    x = Vec16<T>::fromFloat(f);
    Vec16<T>::toFloat(x, f);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < Vec16<T>::kElems; i++) ss += f[i] * f[i];
  return ss;
}

template <typename T>
MSCCLPP_DEVICE_INLINE uint4 scaleRow(uint4 x, float rinv, const char* gamma, uint64_t unitInRow) {
  float f[Vec16<T>::kElems];
  Vec16<T>::toFloat(x, f);
  if (gamma != nullptr) {
    float g[Vec16<T>::kElems];
    Vec16<T>::toFloat(*reinterpret_cast<const uint4*>(gamma + unitInRow * 16), g);
#pragma unroll
    for (int i = 0; i < Vec16<T>::kElems; i++) f[i] = f[i] * rinv * g[i];
  } else {
#pragma unroll
    for (int i = 0; i < Vec16<T>::kElems; i++) f[i] = f[i] * rinv;
  }
  return Vec16<T>::fromFloat(f);
}

// ============================================================================================
// One-shot LL16 allreduce
// ============================================================================================
template <typename T, ReduceOp Op, bool kNvls, bool kNorm, bool kLL8 = false>
__global__ void __launch_bounds__(kNorm ? 1024 : 512, 1) allreduceLLKernel(CollArgs a) {
  static_assert(!(kLL8 && (kNvls || kNorm)), "the 8-byte packet form is the plain peer-store exchange only");
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const int world = c.world;
  const uint64_t emu = static_cast<uint64_t>(blockIdx.y) * a.emuStride;
  const char* in = reinterpret_cast<const char*>(a.in) + emu;
  char* out = reinterpret_cast<char*>(a.out) + emu;
  const uint32_t flag = launchEpoch(c, rank);
  const uint64_t bufOff = c.llScratchOff + static_cast<uint64_t>(flag & 1u) * (static_cast<uint64_t>(world) * c.llSlotBytes);
  const uint64_t bytes = a.bytes;
  const uint64_t nunits = (bytes + 15) / 16;

  // ---- unit iteration space: flat (plain allreduce) or row-per-block (fused norm)
  const uint64_t unitsPerRow = kNorm ? (static_cast<uint64_t>(a.hidden) * sizeof(T)) / 16 : 0;

  // ---- send: my whole input to every peer
  {
    const uint64_t start = kNorm ? 0 : static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t step = kNorm ? 0 : static_cast<uint64_t>(gridDim.x) * blockDim.x;
    auto sendUnit = [&](uint64_t u) {
      const uint4 d = loadUnit(in, u, bytes);
      if constexpr (kNvls) {
        char* mc = reinterpret_cast<char*>(c.mcBase + bufOff + static_cast<uint64_t>(rank) * c.llSlotBytes + u * 32);
        ptx::multimem_st_v4(mc, make_uint4(d.x, flag, d.y, flag));
        ptx::multimem_st_v4(mc + 16, make_uint4(d.z, flag, d.w, flag));
      } else if constexpr (kLL8) {
        for (int i = 1; i < world; i++) {
          const int p = (rank + i) % world;
          LL8Packet* pk = reinterpret_cast<LL8Packet*>(c.peerBase[p] + bufOff + static_cast<uint64_t>(rank) * c.llSlotBytes + u * 32);
          pk[0].write(d.x, flag);
          pk[1].write(d.y, flag);
          pk[2].write(d.z, flag);
          pk[3].write(d.w, flag);
        }
      } else {
        for (int i = 1; i < world; i++) {
          const int p = (rank + i) % world;
          LL16Packet* pk = reinterpret_cast<LL16Packet*>(c.peerBase[p] + bufOff +
                                                         static_cast<uint64_t>(rank) * c.llSlotBytes + u * 32);
          pk[0].write(d.x, d.y, flag);
          pk[1].write(d.z, d.w, flag);
        }
      }
    };
    if constexpr (kNorm) {
      for (int row = blockIdx.x; row < a.rows; row += gridDim.x)
        for (uint64_t ru = threadIdx.x; ru < unitsPerRow; ru += blockDim.x) sendUnit(row * unitsPerRow + ru);
    } else {
      for (uint64_t u = start; u < nunits; u += step) sendUnit(u);
    }
  }
  // the packets are on their way: count this block out of the launch while they travel (instead of at the very end,
  // where the round trip of that atomic would be exposed)
  retireLaunchEarly(c, rank, flag);

  // ---- receive + reduce. The packets of ALL peers are requested before the first one is looked at: polled one after the
  // other they cost a dependent L2 round trip each (14 in a row with eight ranks).
  bool healthy = true;
  auto recvUnit = [&](uint64_t u, uint4& result) -> bool {
    const uint4 own = loadUnit(in, u, bytes);
    const uint64_t slotBase = c.peerBase[rank] + bufOff + u * 32;
    Accum<T, Op> acc;
    // Peers are taken in batches (eight at a time where the registers allow it, four in the variants with 64 registers per
    // thread). The packets of a batch are all requested before any flag is looked at, and polled TOGETHER until every one
    // carries this launch's flag: the wait for the slowest peer is paid once, and one round trip after it everything is
    // in registers. The contributions are added in rank order. (LL8 and LL16 share the layout: data words at even, flags
    // at odd 32-bit positions.)
    constexpr int kBatch = (kNorm || kLL8) ? 4 : 8;
    for (int p0 = 0; p0 < world; p0 += kBatch) {
      uint4 word[kBatch];
      SpinGuard guard(c.status, c.timeoutNs);
      for (;;) {
        bool allHere = true;
#pragma unroll
        for (int i = 0; i < kBatch; i++) {
          const int p = p0 + i;
          if (p < world && p != rank) {
            const char* pk = reinterpret_cast<const char*>(slotBase + static_cast<uint64_t>(p) * c.llSlotBytes);
            const uint4 a0 = ptx::ld_volatile_v4(pk), a1 = ptx::ld_volatile_v4(pk + 16);
            word[i] = make_uint4(a0.x, a0.z, a1.x, a1.z);
            allHere = allHere && a0.y == flag && a0.w == flag && a1.y == flag && a1.w == flag;
          }
        }
        if (allHere) break;
        if (!guard.keepSpinning()) {
          guard.report(kDevTimeoutPacket, rank, kLL8 ? 8 : 16, p0, flag, 0);
          return false;
        }
      }
#pragma unroll
      for (int i = 0; i < kBatch; i++) {
        const int p = p0 + i;
        if (p < world) {
          const uint4 v = p == rank ? own : word[i];
          if (p == 0) acc.init(v); else acc.add(v);
        }
      }
    }
    result = acc.result();
    return true;
  };

  if constexpr (!kNorm) {
    const uint64_t start = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t step = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t u = start; u < nunits && healthy; u += step) {
      uint4 r;
      healthy = recvUnit(u, r);
      if (healthy) storeUnit(out, u, bytes, r);
    }
  } else {
    const char* resIn = a.residualIn ? reinterpret_cast<const char*>(a.residualIn) + emu : nullptr;
    char* resOut = a.residualOut ? reinterpret_cast<char*>(a.residualOut) + emu : nullptr;
    const char* gamma = reinterpret_cast<const char*>(a.gamma);
    char* stash = resOut ? resOut : out;  // where the un-normalised row lives between the passes
    for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
      float ss = 0.f;
      for (uint64_t ru = threadIdx.x; ru < unitsPerRow; ru += blockDim.x) {
        const uint64_t u = row * unitsPerRow + ru;
        uint4 x = make_uint4(0, 0, 0, 0);
        if (healthy) healthy = recvUnit(u, x);
        uint4 res = resIn ? *reinterpret_cast<const uint4*>(resIn + u * 16) : make_uint4(0, 0, 0, 0);
        ss += addResidual<T>(x, res, resIn != nullptr);
        *reinterpret_cast<uint4*>(stash + u * 16) = x;
      }
      const float total = blockSum(ss);
      const float rinv = rsqrtf(total / static_cast<float>(a.hidden) + a.eps);
      for (uint64_t ru = threadIdx.x; ru < unitsPerRow; ru += blockDim.x) {
        const uint64_t u = row * unitsPerRow + ru;
        const uint4 x = *reinterpret_cast<const uint4*>(stash + u * 16);  // written by this same thread
        *reinterpret_cast<uint4*>(out + u * 16) = scaleRow<T>(x, rinv, gamma, ru);
      }
    }
  }
}

// ============================================================================================
// One-shot LL128 allreduce
// ============================================================================================
// The same exchange as allreduceLLKernel with 128-byte lines instead of 16-byte packets: a line carries 120 bytes of
// payload and one 8-byte flag (15/16 of the scratch traffic is payload, against 1/2 with LL16), and is written by eight
// consecutive lanes of a warp in ONE instruction, so that it leaves the SM as one 128-byte transaction; the receiver
// takes a line once the flag lane sees this launch's epoch (packet_device.hpp: ll128Write / ll128ReadFast, every wait
// bounded). Line L covers bytes [120 L, 120 L + 120) of the buffer: lane s < 7 of the line's group holds bytes
// [16 s, 16 s + 16) of them, lane 7 the last 8. Pieces start on 8-byte boundaries, so they move as two 8-byte words.
// Role of the reference's packet allreduce for mid-size messages (its LL protocol has the 8- and 16-byte packets only,
// include/mscclpp/packet_device.hpp); the line format follows the description in this library's own header.
MSCCLPP_DEVICE_INLINE uint4 loadPiece(const char* base, uint64_t off, uint64_t bytes, int pieceBytes, bool aligned8) {
  uint4 v = make_uint4(0, 0, 0, 0);
  if (aligned8 && off + pieceBytes <= bytes) {
    const uint2 lo = *reinterpret_cast<const uint2*>(base + off);
    v.x = lo.x;
    v.y = lo.y;
    if (pieceBytes == 16) {
      const uint2 hi = *reinterpret_cast<const uint2*>(base + off + 8);
      v.z = hi.x;
      v.w = hi.y;
    }
  } else if (off < bytes) {
    uint32_t w[4] = {0, 0, 0, 0};
    for (uint64_t i = off; i < bytes && i < off + pieceBytes; i++) {
      w[(i - off) >> 2] |= static_cast<uint32_t>(static_cast<uint8_t>(base[i])) << (8 * ((i - off) & 3));
    }
    v = make_uint4(w[0], w[1], w[2], w[3]);
  }
  return v;
}
MSCCLPP_DEVICE_INLINE void storePiece(char* base, uint64_t off, uint64_t bytes, int pieceBytes, uint4 v, bool aligned8) {
  if (aligned8 && off + pieceBytes <= bytes) {
    *reinterpret_cast<uint2*>(base + off) = make_uint2(v.x, v.y);
    if (pieceBytes == 16) *reinterpret_cast<uint2*>(base + off + 8) = make_uint2(v.z, v.w);
  } else if (off < bytes) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    for (uint64_t i = off; i < bytes && i < off + pieceBytes; i++) base[i] = static_cast<char>(w[(i - off) >> 2] >> (8 * ((i - off) & 3)));
  }
}

template <typename T, ReduceOp Op>
__global__ void __launch_bounds__(512, 1) allreduceLL128Kernel(CollArgs a) {
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const int world = c.world;
  const uint64_t emu = static_cast<uint64_t>(blockIdx.y) * a.emuStride;
  const char* in = reinterpret_cast<const char*>(a.in) + emu;
  char* out = reinterpret_cast<char*>(a.out) + emu;
  const uint32_t epoch = launchEpoch(c, rank);
  const uint64_t flag = (static_cast<uint64_t>(0x4c4c3132u) << 32) | epoch;  // never equal to payload left by the 16-byte formats
  // the lines have a scratch of their own ([2 buffers][world][slot]): in the scratch of the 8- and 16-byte packets every odd
  // 32-bit word is a flag, and payload of this format left there could pass for one
  const uint64_t slotBytes = a.ll128SlotBytes;
  const uint64_t bufOff = (reinterpret_cast<uint64_t>(a.ll128Scratch) - c.peerBase[c.rank]) +
                          static_cast<uint64_t>(epoch & 1u) * (static_cast<uint64_t>(world) * slotBytes);
  const uint64_t bytes = a.bytes;
  const uint64_t numLines = (bytes + kLL128PayloadBytes - 1) / kLL128PayloadBytes;
  const uint32_t sub = threadIdx.x & 7;
  const uint32_t groupMask = 0xffu << ((threadIdx.x & 31) & ~7u);
  const int pieceBytes = sub == 7 ? 8 : 16;
  // pieces move as 8-byte words when both buffers allow it, byte by byte otherwise (slow, but every rank may take the
  // decision for itself: it changes nothing on the wire)
  const bool aligned8 = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 7) == 0;
  const uint64_t firstLine = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
  const uint64_t lineStep = (static_cast<uint64_t>(gridDim.x) * blockDim.x) >> 3;

  // ---- send: my whole input to every peer
  for (uint64_t line = firstLine; line < numLines; line += lineStep) {
    const uint4 d = loadPiece(in, line * kLL128PayloadBytes + sub * 16, bytes, pieceBytes, aligned8);
    for (int i = 1; i < world; i++) {
      const int p = (rank + i) % world;
      LL128Line* dst = reinterpret_cast<LL128Line*>(c.peerBase[p] + bufOff + static_cast<uint64_t>(rank) * slotBytes) + line;
      ll128Write(dst, sub, d, flag);
    }
  }
  // the lines are on their way: count this block out of the launch while they travel
  retireLaunchEarly(c, rank, epoch);

  // ---- receive + reduce (contributions in rank order: every rank computes the same bits)
  bool healthy = true;
  for (uint64_t line = firstLine; line < numLines && healthy; line += lineStep) {
    const uint64_t off = line * kLL128PayloadBytes + sub * 16;
    const uint4 own = loadPiece(in, off, bytes, pieceBytes, aligned8);
    // every peer's line is requested before the first flag is looked at, and the lines are polled together until the flag
    // lane has seen this launch's flag on all of them (one wait for the slowest peer, one round trip after it)
    uint4 got[8];
    {
      SpinGuard guard(c.status, c.timeoutNs);
      bool alive = true;
      for (;;) {
        bool mine = true;
#pragma unroll
        for (int p = 0; p < 8; p++) {
          if (p < world && p != rank) {
            const LL128Line* src = reinterpret_cast<const LL128Line*>(c.peerBase[rank] + bufOff + static_cast<uint64_t>(p) * slotBytes) + line;
            got[p] = ptx::ld_volatile_v4(&src->w[sub]);
            if (sub == 7) mine = mine && got[p].z == static_cast<uint32_t>(flag) && got[p].w == static_cast<uint32_t>(flag >> 32);
          }
        }
        if ((__ballot_sync(groupMask, mine) & groupMask) == groupMask) break;
        if (alive && !guard.keepSpinning()) {
          guard.report(kDevTimeoutPacket, rank, 129, 0, flag, 0);
          alive = false;
        }
        if ((__ballot_sync(groupMask, alive) & groupMask) != groupMask) {
          healthy = false;
          break;
        }
      }
    }
    Accum<T, Op> acc;
    if (healthy) {
#pragma unroll
      for (int p = 0; p < 8; p++) {
        if (p < world) {
          uint4 v = own;
          if (p != rank) {
            v = got[p];
            if (sub == 7) v.z = v.w = 0;  // the flag is not data
          }
          if (p == 0) acc.init(v); else acc.add(v);
        }
      }
    }
    for (int p = 8; p < world && healthy; p++) {
      uint4 v = own;
      if (p != rank) {
        const LL128Line* src = reinterpret_cast<const LL128Line*>(c.peerBase[rank] + bufOff + static_cast<uint64_t>(p) * slotBytes) + line;
        if (!ll128ReadFast(src, sub, groupMask, flag, v, c.status, c.timeoutNs, rank, p)) healthy = false;
        if (sub == 7) v.z = v.w = 0;
      }
      acc.add(v);
    }
    // (a group leaves the loop together: ll128Read returns the same answer to its eight lanes)
    if (healthy) storePiece(out, off, bytes, pieceBytes, acc.result(), aligned8);
  }
}

// ============================================================================================
// Two-shot zero-copy (peer loads/stores or NVLS multimem)
// ============================================================================================
template <typename T, ReduceOp Op>
MSCCLPP_DEVICE_INLINE uint4 multimemLoadReduce(const void* mc) {
  if constexpr (__is_same(T, __half)) {
    if constexpr (Op == SUM) return ptx::multimem_ld_reduce_add_f16x2_acc32(mc);
    else return ptx::multimem_ld_reduce_min_f16x2(mc);
  } else if constexpr (__is_same(T, __nv_bfloat16)) {
    if constexpr (Op == SUM) return ptx::multimem_ld_reduce_add_bf16x2_acc32(mc);
    else return ptx::multimem_ld_reduce_min_bf16x2(mc);
  } else if constexpr (__is_same(T, float)) {
    return ptx::multimem_ld_reduce_add_f32(mc);
  } else if constexpr (__is_same(T, f8e4m3)) {
    return ptx::multimem_ld_reduce_add_e4m3x4(mc);
  } else if constexpr (__is_same(T, f8e5m2)) {
    return ptx::multimem_ld_reduce_add_e5m2x4(mc);
  } else if constexpr (__is_same(T, int32_t)) {
    uint4 v;
    const char* p = reinterpret_cast<const char*>(mc);
    v.x = ptx::multimem_ld_reduce_add_s32(p);
    v.y = ptx::multimem_ld_reduce_add_s32(p + 4);
    v.z = ptx::multimem_ld_reduce_add_s32(p + 8);
    v.w = ptx::multimem_ld_reduce_add_s32(p + 12);
    return v;
  } else {
    uint4 v;
    const char* p = reinterpret_cast<const char*>(mc);
    v.x = ptx::multimem_ld_reduce_add_u32(p);
    v.y = ptx::multimem_ld_reduce_add_u32(p + 4);
    v.z = ptx::multimem_ld_reduce_add_u32(p + 8);
    v.w = ptx::multimem_ld_reduce_add_u32(p + 12);
    return v;
  }
}

// Which (type, op) pairs the switch can reduce by itself.
template <typename T, ReduceOp Op>
constexpr bool nvlsReducible() {
  if (__is_same(T, __half) || __is_same(T, __nv_bfloat16)) return true;
  if (Op != SUM) return false;
  return __is_same(T, float) || __is_same(T, int32_t) || __is_same(T, uint32_t) || __is_same(T, f8e4m3) ||
         __is_same(T, f8e5m2);
}

// Gather the `world` contributions of 16-byte unit at byte offset `off` of the symmetric `in`.
template <typename T, ReduceOp Op, bool kNvls>
MSCCLPP_DEVICE_INLINE uint4 gatherReduce(const DeviceComm& c, int rank, uint64_t inOff, uint64_t off) {
  if constexpr (kNvls) {
    return multimemLoadReduce<T, Op>(reinterpret_cast<const void*>(c.mcBase + inOff + off));
  } else {
    Accum<T, Op> acc;
    if (c.world <= 8) {
      // issue every peer load before the first use so that all of them are in flight together
      uint4 v[8];
#pragma unroll
      for (int p = 0; p < 8; p++)
        if (p < c.world) v[p] = ptx::ld_nc_na_v4(reinterpret_cast<const void*>(c.peerBase[p] + inOff + off));
      acc.init(v[0]);
#pragma unroll
      for (int p = 1; p < 8; p++)
        if (p < c.world) acc.add(v[p]);
    } else {
      acc.init(ptx::ld_nc_na_v4(reinterpret_cast<const void*>(c.peerBase[0] + inOff + off)));
      for (int p = 1; p < c.world; p++)
        acc.add(ptx::ld_nc_na_v4(reinterpret_cast<const void*>(c.peerBase[p] + inOff + off)));
    }
    return acc.result();
  }
}

template <bool kNvls>
MSCCLPP_DEVICE_INLINE void scatterStore(const DeviceComm& c, int rank, uint64_t outOff, uint64_t off, uint4 v) {
  if constexpr (kNvls) {
    ptx::multimem_st_v4(reinterpret_cast<void*>(c.mcBase + outOff + off), v);
  } else {
    for (int i = 0; i < c.world; i++) {
      const int p = (rank + i) % c.world;
      ptx::st_na_v4(reinterpret_cast<void*>(c.peerBase[p] + outOff + off), v);
    }
  }
}

MSCCLPP_DEVICE_INLINE uint64_t splitStart(uint64_t total, int parts, int i) {
  const uint64_t q = total / parts, r = total % parts;
  return static_cast<uint64_t>(i) * q + (static_cast<uint64_t>(i) < r ? i : r);
}

template <typename T, ReduceOp Op, bool kNvls, bool kNorm>
__global__ void __launch_bounds__(512, 1) twoShotKernel(CollArgs a) {
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const int world = c.world;
  // `in`/`out` are given for rank comm.rank; emulated ranks sit at the same heap offset.
  const uint64_t inOff = reinterpret_cast<uint64_t>(a.in) - c.peerBase[c.rank];
  const uint64_t outOff = reinterpret_cast<uint64_t>(a.out) - c.peerBase[c.rank];
  const uint32_t epoch = launchEpoch(c, rank);
  const int slot = blockIdx.x;
  unsigned long long* tl = (a.stamps != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) ? a.stamps : nullptr;
  if (tl) tl[0] = ptx::globaltimer();

  // opening barrier: the peers only have to be IN this launch (what they will read of mine was written by earlier
  // launches, and what I will read of theirs likewise): a flag, no fence
  bool healthy = rankBarrier(c, rank, 0, slot, epoch, false);
  // no grid barrier in this kernel: the block counts itself out of the launch now, under the work, not at the end
  retireLaunchEarly(c, rank, epoch);
  if (tl) tl[1] = ptx::globaltimer();

  if (healthy) {
    if constexpr (kNorm) {
      // rows are split over ranks; a block owns whole rows so it can take the row norm
      const uint64_t unitsPerRow = (static_cast<uint64_t>(a.hidden) * sizeof(T)) / 16;
      const int rowBegin = static_cast<int>(splitStart(a.rows, world, rank));
      const int rowEnd = static_cast<int>(splitStart(a.rows, world, rank + 1));
      const uint64_t resInOff = a.residualIn ? reinterpret_cast<uint64_t>(a.residualIn) - c.peerBase[c.rank] : 0;
      const uint64_t resOutOff = a.residualOut ? reinterpret_cast<uint64_t>(a.residualOut) - c.peerBase[c.rank] : 0;
      const char* gamma = reinterpret_cast<const char*>(a.gamma);
      const uint64_t local = c.peerBase[rank];
      // un-normalised row is stashed in the local residualOut (or local out) between the two passes
      const uint64_t stashOff = a.residualOut ? resOutOff : outOff;
      for (int row = rowBegin + blockIdx.x; row < rowEnd; row += gridDim.x) {
        float ss = 0.f;
        for (uint64_t ru = threadIdx.x; ru < unitsPerRow; ru += blockDim.x) {
          const uint64_t off = (row * unitsPerRow + ru) * 16;
          uint4 x = gatherReduce<T, Op, kNvls>(c, rank, inOff, off);
          uint4 res = a.residualIn ? *reinterpret_cast<const uint4*>(local + resInOff + off) : make_uint4(0, 0, 0, 0);
          ss += addResidual<T>(x, res, a.residualIn != nullptr);
          if (a.residualOut && a.broadcastResidual) {
            scatterStore<kNvls>(c, rank, resOutOff, off, x);
            if constexpr (kNvls) *reinterpret_cast<uint4*>(local + stashOff + off) = x;  // keep a locally ordered copy
          } else {
            *reinterpret_cast<uint4*>(local + stashOff + off) = x;
          }
        }
        const float total = blockSum(ss);
        const float rinv = rsqrtf(total / static_cast<float>(a.hidden) + a.eps);
        for (uint64_t ru = threadIdx.x; ru < unitsPerRow; ru += blockDim.x) {
          const uint64_t off = (row * unitsPerRow + ru) * 16;
          const uint4 x = *reinterpret_cast<const uint4*>(local + stashOff + off);
          scatterStore<kNvls>(c, rank, outOff, off, scaleRow<T>(x, rinv, gamma, ru));
        }
      }
    } else if (a.mode == kAllToAll) {
      // chunk p of my `in` becomes chunk `rank` of rank p's `out`: plain peer stores, own chunk first
      const uint64_t chunkUnits = a.bytes / 16 / world;
      const uint64_t local = c.peerBase[rank];
      for (int i = 0; i < world; i++) {
        const int p = (rank + i) % world;
        const uint64_t dst = c.peerBase[p] + outOff + static_cast<uint64_t>(rank) * chunkUnits * 16;
        const uint64_t src = local + inOff + static_cast<uint64_t>(p) * chunkUnits * 16;
        for (uint64_t u = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < chunkUnits;
             u += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
          ptx::st_na_v4(reinterpret_cast<void*>(dst + u * 16), *reinterpret_cast<const uint4*>(src + u * 16));
        }
      }
    } else if (a.mode == kBroadcast) {
      // the root streams its buffer into every rank's `out` (one multimem.st or one peer store per rank and word)
      if (rank == a.root) {
        const uint64_t nunits = a.bytes / 16;
        const uint64_t local = c.peerBase[rank];
        for (uint64_t u = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < nunits;
             u += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
          const uint4 v = *reinterpret_cast<const uint4*>(local + inOff + u * 16);
          scatterStore<kNvls>(c, rank, outOff, u * 16, v);
        }
      }
    } else if (a.mode == kAllGather) {
      // `in` = my slice (bytes/world), `out` = whole buffer on every rank
      const uint64_t sliceUnits = a.bytes / 16 / world;
      const uint64_t dst0 = static_cast<uint64_t>(rank) * sliceUnits * 16;
      const uint64_t local = c.peerBase[rank];
      for (uint64_t u = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < sliceUnits;
           u += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint4 v = *reinterpret_cast<const uint4*>(local + inOff + u * 16);
        scatterStore<kNvls>(c, rank, outOff, dst0 + u * 16, v);
      }
    } else {
      const uint64_t nunits = a.bytes / 16;
      // One-shot form (allreduce, peer loads): every rank reduces the WHOLE buffer out of all peers' inputs and writes only
      // its own output - (world - 1) x the bytes come in over NVLink, nothing goes out, and no store has to land anywhere
      // before the closing barrier. With two ranks that is the same number of bytes per link direction as the two-shot
      // form, in one phase of loads.
      const bool oneShot = a.oneShot == 1 && a.mode == kAllReduce && !kNvls;
      const uint64_t begin = oneShot ? 0 : splitStart(nunits, world, rank);
      const uint64_t end = oneShot ? nunits : splitStart(nunits, world, rank + 1);
      const uint64_t local = c.peerBase[rank];
      const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
      const uint64_t nthreads = static_cast<uint64_t>(gridDim.x) * blockDim.x;
      // several independent 16-byte requests per thread and peer keep enough bytes in flight over NVLink: four words
      // (x world loads each), eight when there are only two ranks to load from
      auto sweep = [&](auto unrollTag) {
        constexpr int kUnroll = decltype(unrollTag)::value;
        for (uint64_t u0 = begin + tid; u0 < end; u0 += nthreads * kUnroll) {
          uint4 r[kUnroll];
#pragma unroll
          for (int k = 0; k < kUnroll; k++) {
            const uint64_t u = u0 + k * nthreads;
            if (u < end) r[k] = gatherReduce<T, Op, kNvls>(c, rank, inOff, u * 16);
          }
#pragma unroll
          for (int k = 0; k < kUnroll; k++) {
            const uint64_t u = u0 + k * nthreads;
            if (u < end) {
              if (a.mode == kReduceScatter)
                *reinterpret_cast<uint4*>(local + outOff + (u - begin) * 16) = r[k];
              else if (oneShot)
                *reinterpret_cast<uint4*>(local + outOff + u * 16) = r[k];
              else
                scatterStore<kNvls>(c, rank, outOff, u * 16, r[k]);
            }
          }
        }
      };
      if (!kNvls && world <= 2) sweep(std::integral_constant<int, 8>{});
      else sweep(std::integral_constant<int, 4>{});
    }
  }
  if (tl) tl[2] = ptx::globaltimer();
  // all my stores are issued; tell the peers, and learn that theirs into my buffers are done
  if (healthy) rankBarrier(c, rank, 1, slot, epoch);
  if (tl) tl[3] = tl[4] = ptx::globaltimer();
}

// --------------------------------------------------------------------------------------------
template <typename KernelT>
cudaError_t launchMaybeCooperative(KernelT kernel, const CollArgs& args, int nBlocks, int nThreads, cudaStream_t stream) {
  dim3 grid(nBlocks, args.emuRanks > 1 ? args.emuRanks : 1, 1);
  dim3 block(nThreads, 1, 1);
  if (args.emuRanks > 1) {
    // emulated ranks wait on one another inside one grid: it has to be co-resident
    CollArgs copy = args;
    void* params[] = {&copy};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, params, 0, stream);
  }
  kernel<<<grid, block, 0, stream>>>(args);
  return cudaGetLastError();
}

template <typename T, ReduceOp Op>
cudaError_t launchLLTyped(const CollArgs& a, int nBlocks, int nThreads, cudaStream_t s) {
  if (a.norm) {
    if (a.ll8) return cudaErrorInvalidValue;
    if constexpr (IsFloatLike<T>::value && Op == SUM && sizeof(T) >= 2) {
      return a.nvls ? launchMaybeCooperative(allreduceLLKernel<T, Op, true, true>, a, nBlocks, nThreads, s)
                    : launchMaybeCooperative(allreduceLLKernel<T, Op, false, true>, a, nBlocks, nThreads, s);
    } else {
      return cudaErrorInvalidValue;
    }
  }
  if (a.ll8) {
    if (a.nvls) return cudaErrorInvalidValue;
    return launchMaybeCooperative(allreduceLLKernel<T, Op, false, false, true>, a, nBlocks, nThreads, s);
  }
  return a.nvls ? launchMaybeCooperative(allreduceLLKernel<T, Op, true, false>, a, nBlocks, nThreads, s)
                : launchMaybeCooperative(allreduceLLKernel<T, Op, false, false>, a, nBlocks, nThreads, s);
}

template <typename T, ReduceOp Op>
cudaError_t launchTwoShotTyped(const CollArgs& a, int nBlocks, int nThreads, cudaStream_t s) {
  if (a.norm) {
    if constexpr (IsFloatLike<T>::value && Op == SUM && sizeof(T) >= 2) {
      if (a.nvls) return launchMaybeCooperative(twoShotKernel<T, Op, true, true>, a, nBlocks, nThreads, s);
      return launchMaybeCooperative(twoShotKernel<T, Op, false, true>, a, nBlocks, nThreads, s);
    } else {
      return cudaErrorInvalidValue;
    }
  }
  if (a.nvls && a.mode != kAllGather && a.mode != kBroadcast && a.mode != kAllToAll) {
    if constexpr (nvlsReducible<T, Op>()) {
      return launchMaybeCooperative(twoShotKernel<T, Op, true, false>, a, nBlocks, nThreads, s);
    } else {
      return cudaErrorInvalidValue;
    }
  }
  if (a.nvls) return launchMaybeCooperative(twoShotKernel<uint32_t, SUM, true, false>, a, nBlocks, nThreads, s);
  return launchMaybeCooperative(twoShotKernel<T, Op, false, false>, a, nBlocks, nThreads, s);
}

#define MSCCLPP_DISPATCH_TYPE_OP(FN, dtype, op, ...)                                               \
  do {                                                                                             \
    const bool isMin = (op) == MIN;                                                                \
    switch (dtype) {                                                                               \
      case DataType::FLOAT16:                                                                      \
        return isMin ? FN<__half, MIN>(__VA_ARGS__) : FN<__half, SUM>(__VA_ARGS__);                \
      case DataType::BFLOAT16:                                                                     \
        return isMin ? FN<__nv_bfloat16, MIN>(__VA_ARGS__) : FN<__nv_bfloat16, SUM>(__VA_ARGS__);  \
      case DataType::FLOAT32:                                                                      \
        return isMin ? FN<float, MIN>(__VA_ARGS__) : FN<float, SUM>(__VA_ARGS__);                  \
      case DataType::INT32:                                                                        \
        return isMin ? FN<int32_t, MIN>(__VA_ARGS__) : FN<int32_t, SUM>(__VA_ARGS__);              \
      case DataType::UINT32:                                                                       \
        return isMin ? FN<uint32_t, MIN>(__VA_ARGS__) : FN<uint32_t, SUM>(__VA_ARGS__);            \
      case DataType::UINT8:                                                                        \
        return isMin ? FN<uint8_t, MIN>(__VA_ARGS__) : FN<uint8_t, SUM>(__VA_ARGS__);              \
      case DataType::FLOAT8_E4M3:                                                                  \
        return isMin ? FN<f8e4m3, MIN>(__VA_ARGS__) : FN<f8e4m3, SUM>(__VA_ARGS__);                \
      case DataType::FLOAT8_E5M2:                                                                  \
        return isMin ? FN<f8e5m2, MIN>(__VA_ARGS__) : FN<f8e5m2, SUM>(__VA_ARGS__);                \
      case DataType::FLOAT8_E4M3B15:                                                               \
        return isMin ? FN<f8e4m3b15, MIN>(__VA_ARGS__) : FN<f8e4m3b15, SUM>(__VA_ARGS__);          \
      default:                                                                                     \
        return cudaErrorInvalidValue;                                                              \
    }                                                                                              \
  } while (0)

}  // namespace

cudaError_t launchAllreduceLL(const CollArgs& args, DataType dtype, ReduceOp op, int nBlocks, int nThreads,
                              cudaStream_t stream) {
  if (args.bytes * 2 > args.comm.llSlotBytes) return cudaErrorInvalidValue;
  if (nBlocks < 1 || nThreads < 32 || nThreads > (args.norm ? 1024 : 512)) return cudaErrorInvalidValue;
  if (args.norm && ((static_cast<uint64_t>(args.hidden) * dataTypeSize(dtype)) % 16 != 0)) return cudaErrorInvalidValue;
  MSCCLPP_DISPATCH_TYPE_OP(launchLLTyped, dtype, op, args, nBlocks, nThreads, stream);
}

template <typename T, ReduceOp Op>
cudaError_t launchLL128Typed(const CollArgs& a, int nBlocks, int nThreads, cudaStream_t s) {
  return launchMaybeCooperative(allreduceLL128Kernel<T, Op>, a, nBlocks, nThreads, s);
}

cudaError_t launchAllreduceLL128(const CollArgs& args, DataType dtype, ReduceOp op, int nBlocks, int nThreads, cudaStream_t stream) {
  const uint64_t lines = (args.bytes + kLL128PayloadBytes - 1) / kLL128PayloadBytes;
  if (args.ll128Scratch == nullptr || args.ll128SlotBytes % 128 != 0 || lines * sizeof(LL128Line) > args.ll128SlotBytes) return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(args.ll128Scratch) % 128 != 0) return cudaErrorInvalidValue;
  if (nBlocks < 1 || nThreads < 32 || nThreads > 512 || nThreads % 32 != 0) return cudaErrorInvalidValue;
  if (args.norm || args.nvls) return cudaErrorInvalidValue;
  MSCCLPP_DISPATCH_TYPE_OP(launchLL128Typed, dtype, op, args, nBlocks, nThreads, stream);
}

cudaError_t launchTwoShot(const CollArgs& argsIn, DataType dtype, ReduceOp op, int nBlocks, int nThreads,
                          cudaStream_t stream) {
  CollArgs args = argsIn;
  if (args.oneShot == 0) {
    // measured on two B200s: the one-shot form is slower than the two-shot form at every size from 1 MB to 128 MB (56 vs
    // 52 us at 16 MB with 128 blocks): loads over NVLink are the scarcer direction, and the two-shot form turns half of
    // them into stores. It stays available on request.
    args.oneShot = 2;
  }
  if (args.bytes % 16 != 0) return cudaErrorInvalidValue;
  if (nBlocks < 1 || nBlocks > kBarrierSlots || nThreads < 32 || nThreads > 512) return cudaErrorInvalidValue;
  if (nThreads < args.comm.world) return cudaErrorInvalidValue;
  if ((args.mode == kReduceScatter || args.mode == kAllGather || args.mode == kAllToAll) && (args.bytes / 16) % args.comm.world != 0) return cudaErrorInvalidValue;
  if (args.mode == kBroadcast && (args.root < 0 || args.root >= args.comm.world)) return cudaErrorInvalidValue;
  if (args.norm && ((static_cast<uint64_t>(args.hidden) * dataTypeSize(dtype)) % 16 != 0)) return cudaErrorInvalidValue;
  MSCCLPP_DISPATCH_TYPE_OP(launchTwoShotTyped, dtype, op, args, nBlocks, nThreads, stream);
}

}  // namespace mscclpp
