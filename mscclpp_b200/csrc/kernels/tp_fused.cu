// ONE kernel for the tensor-parallel row-parallel layer:
//
//     h   = sum over ranks ( X_r[M,K] * W_r[N,K]^T ) + residual          (bf16, fp32 accumulation)
//     out = h * rsqrt(mean(h^2) + eps) * gamma
//
// CTAs [0, numGemmCtas) run the tcgen05/TMEM GEMM (gemm_sm100.cuh) and store their bf16 partial tile
// into the rank's symmetric heap; when a tile is complete they stamp the launch epoch into a ready
// flag in the heap of every rank that owns rows of that tile (st.release.sys over NVLink).
// The remaining CTAs are reducers: a reducer waits until all ranks have finished every tile of a row
// block it owns rows in, then pulls those rows reduced over all ranks - one multimem.ld_reduce through
// the NVSwitch, or peer loads with an fp32 accumulator - adds the residual, takes the row norm and
// writes the new residual stream and the normalised output into every rank (multimem.st or peer
// stores). The transfer of row block i therefore overlaps the matmul of row blocks i+1.., tile by tile.
//
// Row ownership is cyclic in units of `rowsPerUnit` rows (unit u belongs to rank u % world), so every
// rank's reducers have work as soon as the first row blocks are done.
//
// mode 0: the owner writes `out` and `residualOut` to every rank.
// mode 1: the owner writes `residualOut` (= h) and one fp32 1/rms per row to every rank; `out` is then
//         produced by a cheap local pass (tpScaleRows), which halves the bytes that cross NVLink.
// mode 2: GEMM + reduce-scatter (sequence parallelism): rank r keeps the reduced rows [r*M/world, (r+1)*M/world)
//         in its local `out` [M/world, N]; no residual, no norm, nothing is broadcast.
//
// The reference library has no counterpart: it provides the allreduce only.
#include "tp_fused.cuh"

#include <cstdlib>

#include <mscclpp/gpu_data_types.hpp>

#include "gemm2_sm100.cuh"
#include "gemm_sm100.cuh"

namespace mscclpp {

namespace {

using bf16 = __nv_bfloat16;
constexpr int kMaxNBlk = 128;

// Packed bf16 arithmetic for the element-wise parts of the single-GPU layer. With a dozen warps per SM these loops are
// bound by instruction latency, not by memory: one HADD2 / HMUL2 / HFMA2 per two elements instead of a convert - operate -
// convert chain per element is what makes them fit in the shadow of the MMAs.
MSCCLPP_DEVICE_INLINE __nv_bfloat162 asBf162(uint32_t w) { return *reinterpret_cast<__nv_bfloat162*>(&w); }
MSCCLPP_DEVICE_INLINE uint32_t asWord(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
// a + b per element, each sum rounded once to bf16 (the adder works in fp32 internally: same result as an fp32 add + round)
MSCCLPP_DEVICE_INLINE uint4 addBf16x8(uint4 a, uint4 b) {
  return make_uint4(asWord(__hadd2(asBf162(a.x), asBf162(b.x))), asWord(__hadd2(asBf162(a.y), asBf162(b.y))),
                    asWord(__hadd2(asBf162(a.z), asBf162(b.z))), asWord(__hadd2(asBf162(a.w), asBf162(b.w))));
}
MSCCLPP_DEVICE_INLINE float sumSquaresBf16x8(uint4 v) {
  const float2 a = __bfloat1622float2(asBf162(v.x)), b = __bfloat1622float2(asBf162(v.y));
  const float2 c = __bfloat1622float2(asBf162(v.z)), d = __bfloat1622float2(asBf162(v.w));
  float s0 = a.x * a.x, s1 = b.x * b.x;
  s0 = fmaf(a.y, a.y, s0);
  s1 = fmaf(b.y, b.y, s1);
  s0 = fmaf(c.x, c.x, s0);
  s1 = fmaf(d.x, d.x, s1);
  s0 = fmaf(c.y, c.y, s0);
  s1 = fmaf(d.y, d.y, s1);
  return s0 + s1;
}
// v * g * s with the fp32 scale s split into a bf16 head and a bf16 tail (s = hi + lo up to 2^-17 relative), so that the
// result carries the two product roundings of bf16 arithmetic but not a third from rounding s itself.
MSCCLPP_DEVICE_INLINE uint32_t scaleBf16x2(uint32_t v, uint32_t g, __nv_bfloat162 hi, __nv_bfloat162 lo, bool hasGamma) {
  const __nv_bfloat162 p = hasGamma ? __hmul2(asBf162(v), asBf162(g)) : asBf162(v);
  return asWord(__hfma2(p, lo, __hmul2(p, hi)));
}

struct TmapSet {
  CUtensorMap a[8];
  CUtensorMap b[8];
};

constexpr int kMaxMBlk = kTpMaxMBlk;
// Aux flag region of every heap: [kMaxMBlk][kMaxRanks] epoch-stamped "row block of rank src is complete"
// flags written by the producers, followed by kMaxMBlk local tile counters.
MSCCLPP_DEVICE_INLINE uint32_t* readyFlag(const DeviceComm& c, int owner, int mBlk, int src) {
  return reinterpret_cast<uint32_t*>(c.peerBase[owner] + c.auxFlagsOff) + (static_cast<size_t>(mBlk) * kMaxRanks + src);
}
MSCCLPP_DEVICE_INLINE uint32_t* tileCounter(const DeviceComm& c, int rank, int mBlk) {
  return reinterpret_cast<uint32_t*>(c.peerBase[rank] + c.auxFlagsOff + kTpTileCounterOffset) + mBlk;
}

MSCCLPP_DEVICE_INLINE uint32_t* landedFlag(const DeviceComm& c, int onRank, int unit) {
  return reinterpret_cast<uint32_t*>(c.peerBase[onRank] + c.auxFlagsOff + kTpLandedOffset) + unit;
}
MSCCLPP_DEVICE_INLINE uint32_t* unitDoneCounter(const DeviceComm& c, int rank, int unit) {
  return reinterpret_cast<uint32_t*>(c.peerBase[rank] + c.auxFlagsOff + kTpUnitDoneOffset) + unit;
}

struct PartialStoreSignal {
  static constexpr bool kNeedsTileBarrier = true;
  const DeviceComm* comm;
  bf16* partial;  // this rank's partial product [M, N]
  int M, N;
  int rank;
  int rowsPerUnit;
  int numUnits;
  int numNBlk;
  uint32_t epoch;
  unsigned long long* tl;  // this CTA's time-line words or null
  int sysFence;            // publish with a system-scope fence and release stores

  static constexpr bool kBulkStore = false;
  MSCCLPP_DEVICE_INLINE static float convert(float x) { return x; }
  MSCCLPP_DEVICE_INLINE void tileBegin(int, int, int) const {}
  // Plain (generic-proxy) stores, four complete 128-byte lines per warp instruction: the flag that tileDone() publishes
  // afterwards orders them for the peers' reducers with ordinary fences.
  MSCCLPP_DEVICE_INLINE void block(const uint8_t* stage, int row0, int col0, int lane, int /*b*/) const {
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int row = row0 + gemm::stagedRow(i, lane);
      if (row < M) {
        *reinterpret_cast<uint4*>(partial + static_cast<size_t>(row) * N + col0 + gemm::stagedCol(lane)) = gemm::stagedRead(stage, i, lane);
      }
    }
    __syncwarp();  // the staging buffer may be overwritten from here on
  }

  // Called by one warp after every epilogue warp has stored its part. One thread counts the tile; the CTA that
  // completes the LAST tile of a row block publishes one flag per owner rank (the classic last-block
  // pattern: fence, count, fence), so a row block costs `world` small NVLink stores, not world x tiles.
  MSCCLPP_DEVICE_INLINE void tileDone(int mBlk, int /*nBlk*/, int tid) const {
    if (tid != 0) return;
    unsigned long long tIn = 0;
    if (tl) {
      tIn = ptx::globaltimer();
      if (tl[14] != 0 && tIn - tl[14] > tl[15]) {
        tl[15] = tIn - tl[14];  // longest time between two finished tiles of this CTA ...
        tl[7] = tIn;            // ... and when it ended
      }
      tl[14] = tIn;
    }
    __threadfence();
    uint32_t* counter = tileCounter(*comm, rank, mBlk);
    const uint32_t done = atomicAdd(counter, 1u) + 1u;
    if (tl) {
      const unsigned long long dt = ptx::globaltimer() - tIn;
      tl[11] += dt;
      if (dt > tl[12]) tl[12] = dt;
    }
    if (done != static_cast<uint32_t>(numNBlk)) return;
    *counter = 0;  // every tile of this row block has been counted: ready for the next launch
    if (sysFence) __threadfence_system(); else __threadfence();
    const int world = comm->world;
    const int u0 = (mBlk * gemm::kBlockM) / rowsPerUnit;
    int u1 = ((mBlk + 1) * gemm::kBlockM + rowsPerUnit - 1) / rowsPerUnit;
    if (u1 > numUnits) u1 = numUnits;
    // The fence above has GPU scope on purpose. The tiles live in THIS GPU's memory, whose L2 every peer's load (plain
    // or multimem) goes through, so "performed at this GPU's L2" is all a reader needs; the flag goes out after it.
    // A system-scope fence here also waits for this SM's share of the NVLink queues to drain: once the reducers
    // saturate the links that took tens of microseconds per row block and stalled the GEMM CTA that published it.
    // sysFence restores the conservative form (system-scope fence, release stores) for comparison and for fabrics
    // where a peer's load might not go through this GPU's L2.
    for (int o = 0; o < world; o++) {
      // does rank o own one of the units [u0, u1)?
      const int first = (o - (u0 % world) + world) % world;
      if (first < u1 - u0) {
        if (sysFence) ptx::st_release_sys(readyFlag(*comm, o, mBlk, rank), epoch);
        else ptx::st_relaxed_sys(readyFlag(*comm, o, mBlk, rank), epoch);
      }
    }
    if (tl) tl[13] += ptx::globaltimer() - tIn;
  }
  MSCCLPP_DEVICE_INLINE void warpTileDone(int, int) const {}
  MSCCLPP_DEVICE_INLINE void warpDrain(int) const {}
  MSCCLPP_DEVICE_INLINE void auxWarp(int, int) const {}
};

// Reducer CTAs are split into independent groups of kGroupThreads threads; a group owns one row at a
// time and keeps the whole row in registers (kWordsPerThread 16-byte words per thread), so that
//  * 5 groups x 16 KB of loads are in flight per CTA (NVLink needs ~2 MB in flight per GPU), and
//  * the code stays small: one copy of the row pipeline, loops unrolled over the words only.
constexpr int kGroupThreads = 64;
constexpr int kGroupsPerCta = gemm::kNumThreads / kGroupThreads;
constexpr int kWordsPerThread = 16;  // N <= kGroupThreads * kWordsPerThread * 8 = 8192 elements

MSCCLPP_DEVICE_INLINE void groupBarrier(int group) { ptx::named_barrier(2 + group, kGroupThreads); }

// Sum over the 64 threads of a group (two warps).
MSCCLPP_DEVICE_INLINE float groupSum(float v, float* smem2, int group) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warpInGroup = (threadIdx.x >> 5) & 1;
  groupBarrier(group);  // smem2 free again
  if ((threadIdx.x & 31) == 0) smem2[warpInGroup] = v;
  groupBarrier(group);
  return smem2[0] + smem2[1];
}

template <bool kNvls>
MSCCLPP_DEVICE_INLINE void scatterWord(const DeviceComm& c, int rank, uint64_t heapOff, uint4 v) {
  if constexpr (kNvls) {
    ptx::multimem_st_v4(reinterpret_cast<void*>(c.mcBase + heapOff), v);
  } else {
#pragma unroll 1
    for (int i = 0; i < c.world; i++) {
      const int p = (rank + i) % c.world;
      ptx::st_na_v4(reinterpret_cast<void*>(c.peerBase[p] + heapOff), v);
    }
  }
}

// ---- mode 3: the local scale pass inside the launch -------------------------------------------------------------
// One warp turns landed rows into out = h * rinv * gamma, local memory only. Rows are handed out in ascending order
// from a per-rank counter; a row's ownership unit must have been announced by its owner (landedFlag, written behind a
// system-scope fence that covers every store of the unit's rows - see publisherWarp). h and rinv were written by other
// GPUs: they are read through L2 (ld.global.cg), behind an acquire on the flag.
constexpr int kPubQueue = 64;  // finished rows a reducer group may have waiting for the publisher

MSCCLPP_DEVICE_INLINE bool scaleRowsWarp(const TpFusedArgs& a, int rank, uint32_t epoch, int lane) {
  const DeviceComm& c = a.comm;
  const int M = a.shape.M, N = a.shape.N, rpu = a.rowsPerUnit;
  const uint64_t local = c.peerBase[rank];
  const uint64_t base = c.peerBase[c.rank];
  const uint4* hBase = reinterpret_cast<const uint4*>(local + (reinterpret_cast<uint64_t>(a.residualOut) - base));
  uint4* outBase = reinterpret_cast<uint4*>(local + (reinterpret_cast<uint64_t>(a.out) - base));
  const float* rinv = reinterpret_cast<const float*>(local + (reinterpret_cast<uint64_t>(a.rinv) - base));
  const uint4* g4 = reinterpret_cast<const uint4*>(a.gamma);
  const bool hasGamma = a.gamma != nullptr;
  const int words = N / 8;
  uint32_t* scaleCounter = &control(c, rank)->gridSync[6];  // zero at launch start (finishLaunch re-arms it)
  int knownUnit = -1;
  for (;;) {
    int s = 0;
    if (lane == 0) s = static_cast<int>(atomicAdd(scaleCounter, 1u));
    s = __shfl_sync(0xffffffffu, s, 0);
    if (s >= M) return true;
    const int unit = s / rpu;
    if (unit != knownUnit) {
      int ok = 1;
      if (lane == 0) {
        ok = waitGreaterEqualBackoff(landedFlag(c, rank, unit), epoch, c.status, c.timeoutNs, kDevTimeoutFlag, rank, 7600 + (unit & 255),
                                     unit % c.world)
                 ? 1
                 : 0;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);  // (the shuffle also orders the other lanes' loads behind lane 0's acquire)
      if (!ok) return false;
      knownUnit = unit;
    }
    const float sc = __ldcg(rinv + s);
    const __nv_bfloat16 hi1 = __float2bfloat16_rn(sc);
    const __nv_bfloat162 hi = __bfloat162bfloat162(hi1);
    const __nv_bfloat162 lo = __float2bfloat162_rn(sc - __bfloat162float(hi1));
    const uint4* src = hBase + static_cast<size_t>(s) * words;
    uint4* dst = outBase + static_cast<size_t>(s) * words;
    constexpr int kDepth = 16;
    for (int w0 = lane; w0 < words; w0 += 32 * kDepth) {
      uint4 v[kDepth];
#pragma unroll
      for (int k = 0; k < kDepth; k++) {
        const int w = w0 + 32 * k;
        if (w < words) v[k] = ptx::ld_cg_v4(src + w);
      }
#pragma unroll
      for (int k = 0; k < kDepth; k++) {
        const int w = w0 + 32 * k;
        if (w < words) {
          const uint4 g = hasGamma ? __ldg(g4 + w) : make_uint4(0, 0, 0, 0);
          dst[w] = make_uint4(scaleBf16x2(v[k].x, g.x, hi, lo, hasGamma), scaleBf16x2(v[k].y, g.y, hi, lo, hasGamma),
                              scaleBf16x2(v[k].z, g.z, hi, lo, hasGamma), scaleBf16x2(v[k].w, g.w, hi, lo, hasGamma));
        }
      }
    }
  }
}

// The publisher warp of a CTA (mode 3). Reducer groups push the unit of every row they have finished into their ring;
// this warp, and only this warp, pays for making those rows' stores system-visible: it takes what has been pushed, issues
// ONE system-scope fence (cumulative: it covers the stores of the threads whose pushes it has observed), and then counts
// the rows on their unit's counter in this rank's memory. Whoever completes a unit resets the counter, fences again (the
// acquire side of the counter chain: the other CTAs' publishers fenced before they counted) and writes the launch epoch
// into the unit's "landed" word on every rank. The reducer groups never wait for a fence.
MSCCLPP_DEVICE_INLINE void publisherWarp(const TpFusedArgs& a, int rank, uint32_t epoch, int lane, int numProducers, const int (*queue)[kPubQueue],
                                         volatile int* tails, volatile int* heads, volatile int* producersLeft) {
  const DeviceComm& c = a.comm;
  const int M = a.shape.M, rpu = a.rowsPerUnit;
  int head = 0;
  SpinGuard guard(c.status, c.timeoutNs);
  for (;;) {
    const int left = *producersLeft;  // read BEFORE the tails: a group pushes its last row before it signs off
    __syncwarp();
    int tail = head;
    if (lane < numProducers) tail = tails[lane];
    if (!__any_sync(0xffffffffu, tail != head)) {
      if (left == 0) return;
      __nanosleep(200);
      if (!guard.keepSpinning()) {
        if (lane == 0) guard.report(kDevTimeoutFlag, rank, 7700, 0, left, 0);
        return;
      }
      continue;
    }
    __threadfence_system();
    if (lane < numProducers) {
      for (int i = head; i != tail; i++) {
        const int unit = queue[lane][i % kPubQueue];
        const uint32_t prev = atomicAdd(unitDoneCounter(c, rank, unit), 1u);
        const int rowsInUnit = M - unit * rpu < rpu ? M - unit * rpu : rpu;
        if (static_cast<int>(prev) + 1 == rowsInUnit) {
          *unitDoneCounter(c, rank, unit) = 0;  // nobody else counts on this unit in this launch: ready for the next one
          __threadfence_system();
          for (int p = 0; p < c.world; p++) ptx::st_relaxed_sys(landedFlag(c, (rank + p) % c.world, unit), epoch);
        }
      }
      head = tail;
      heads[lane] = head;
    }
  }
}

template <bool kNvls>
// `slot` names this CTA in the closing cross-rank barrier (the same grid runs on every rank). Rows are handed out
// dynamically, in ascending order, from a per-rank counter: CTAs that were GEMM CTAs join in when their tiles are done,
// so after the matmul the whole GPU works on the reduction.
MSCCLPP_DEVICE_INLINE void reducerCta(const TpFusedArgs& a, int rank, uint32_t epoch, int slot) {
  const DeviceComm& c = a.comm;
  const int world = c.world;
  const int M = a.shape.M, N = a.shape.N;
  const int rpu = a.rowsPerUnit;
  const int numUnits = (M + rpu - 1) / rpu;
  const int ownedUnits = numUnits > rank ? (numUnits - rank + world - 1) / world : 0;
  const int ownedRows = ownedUnits * rpu;  // some may fall beyond M in the last unit
  const int unitsPerRow = N * 2 / 16;
  const uint64_t local = c.peerBase[rank];
  const uint64_t partialOff = reinterpret_cast<uint64_t>(a.partial) - c.peerBase[c.rank];
  const uint64_t outOff = reinterpret_cast<uint64_t>(a.out) - c.peerBase[c.rank];
  const uint64_t resOutOff = reinterpret_cast<uint64_t>(a.residualOut) - c.peerBase[c.rank];
  const uint64_t resInOff = a.residualIn ? reinterpret_cast<uint64_t>(a.residualIn) - c.peerBase[c.rank] : 0;
  const uint64_t rinvOff = a.rinv ? reinterpret_cast<uint64_t>(a.rinv) - c.peerBase[c.rank] : 0;
  const char* gamma = reinterpret_cast<const char*>(a.gamma);

  __shared__ float sumSmem[kGroupsPerCta][2];
  __shared__ int okSmem[kGroupsPerCta];
  // readiness of row blocks is learned once per CTA: one group polls the (remote-written) flags, the
  // others watch a bitmap in shared memory. Few pollers per flag line keep its L2 slice responsive.
  __shared__ uint32_t readyBits[kMaxMBlk / 32];
  __shared__ int pollLock;
  __shared__ int groupState[kGroupsPerCta];
  for (int i = threadIdx.x; i < kMaxMBlk / 32; i += blockDim.x) readyBits[i] = 0;
  if (threadIdx.x == 0) pollLock = 0;
  __syncthreads();
  const int group = threadIdx.x / kGroupThreads;
  const int lane = threadIdx.x % kGroupThreads;
  if (lane == 0) okSmem[group] = 1;
  groupBarrier(group);

  // mode 3: the last group of the CTA does not reduce - its first warp publishes finished rows, its second warp scales
  // landed rows from the start; the other groups scale when they run out of rows to reduce
  const bool fold = a.mode == 3;
  constexpr int kProducers = kGroupsPerCta - 1;
  __shared__ int pubQueue[kProducers][kPubQueue];
  __shared__ volatile int pubTail[kProducers], pubHead[kProducers];
  __shared__ volatile int producersLeft;
  if (threadIdx.x < kProducers) pubTail[threadIdx.x] = pubHead[threadIdx.x] = 0;
  if (threadIdx.x == 0) producersLeft = fold ? kProducers : 0;
  __syncthreads();
  if (fold && group == kGroupsPerCta - 1) {
    const int lane32 = threadIdx.x & 31;
    if (((threadIdx.x >> 5) & 1) == 0) {
      publisherWarp(a, rank, epoch, lane32, kProducers, pubQueue, pubTail, pubHead, &producersLeft);
    }
    if (!scaleRowsWarp(a, rank, epoch, lane32) && lane32 == 0) okSmem[group] = 0;
    __syncthreads();
    bool everyOk = true;
    for (int g = 0; g < kGroupsPerCta; g++) everyOk = everyOk && okSmem[g] != 0;
    if (everyOk) rankBarrier(c, rank, 2, slot, epoch);
    return;
  }

  __shared__ int nextRow[kGroupsPerCta];
  uint32_t* rowCounter = &control(c, rank)->gridSync[7];  // zero at launch start (finishLaunch re-arms it)
  int readyMb = -1;
  bool healthy = true;
  // optional stamps (group 0, lane 0 of every CTA)
  unsigned long long* tl = (a.timeline != nullptr && blockIdx.y == 0 && threadIdx.x == 0) ? a.timeline + static_cast<size_t>(blockIdx.x) * kTimelineWords : nullptr;
  unsigned long long tlRows = 0, tlWait = 0, tlWork = 0, tlMark = 0, tlGather = 0, tlMath = 0, tlScatter = 0, tlPhase = 0;
  // owned row j -> global row: unit = rank + (j / rpu) * world, row = unit * rpu + j % rpu
#pragma unroll 1
  // Lane 0 draws the row after the current one while the current one is in flight, so the atomic's round trip to L2
  // is off the per-row critical path. (A drawn row is always processed or lies beyond the last one.)
  int drawn = 0;
  if (lane == 0) drawn = static_cast<int>(atomicAdd(rowCounter, 1u));
  for (;;) {
    if (lane == 0) {
      nextRow[group] = healthy ? drawn : ownedRows;
      if (healthy && drawn < ownedRows) drawn = static_cast<int>(atomicAdd(rowCounter, 1u));
    }
    groupBarrier(group);
    const int j = nextRow[group];
    groupBarrier(group);  // nextRow may be rewritten from here on
    if (j >= ownedRows) break;
    const int row = (rank + (j / rpu) * world) * rpu + (j % rpu);
    if (row >= M) continue;
    // The residual does not depend on anybody's GEMM: with the switch doing the reduction there are registers to
    // spare, so its loads are put in flight before the readiness wait and the gather.
    [[maybe_unused]] uint4 resEarly[kWordsPerThread];
    if constexpr (kNvls) {
      if (a.residualIn && a.mode != 2) {
        const uint64_t resRow = local + resInOff + static_cast<uint64_t>(row) * unitsPerRow * 16;
#pragma unroll
        for (int k = 0; k < kWordsPerThread; k++) {
          const int w = lane + k * kGroupThreads;
          resEarly[k] = make_uint4(0, 0, 0, 0);
          if (w < unitsPerRow) resEarly[k] = ptx::ld_nc_na_v4(reinterpret_cast<const void*>(resRow + w * 16));
        }
      }
    }
    // ---- wait until every rank has produced every tile of the row block this row lives in
    const int mb = row / gemm::kBlockM;
    if (tl) tlMark = ptx::globaltimer();
    if (mb != readyMb && !a.noFlags) {
      // Every decision below is taken by lane 0 and read by the group after a barrier, so all 64
      // threads always agree on which barriers they execute.
      for (;;) {
        if (lane == 0) {
          int st;
          if ((*reinterpret_cast<volatile uint32_t*>(&readyBits[mb >> 5]) >> (mb & 31)) & 1u) st = 2;       // known ready
          else if (c.status != nullptr && *reinterpret_cast<volatile uint32_t*>(&c.status->poisoned) != 0) st = 3;  // abort
          else st = (atomicCAS(&pollLock, 0, 1) == 0) ? 1 : 0;                                               // poll / watch
          groupState[group] = st;
        }
        groupBarrier(group);
        const int st = groupState[group];
        if (st == 1) {
          if (lane < world) {
            if (!waitGreaterEqualBackoff(readyFlag(c, rank, mb, lane), epoch, c.status, c.timeoutNs, kDevTimeoutFlag, rank,
                                         7000 + mb, lane)) {
              okSmem[group] = 0;
            }
          }
          groupBarrier(group);
          if (lane == 0) {
            if (okSmem[group]) atomicOr(&readyBits[mb >> 5], 1u << (mb & 31));
            __threadfence_block();
            atomicExch(&pollLock, 0);
          }
        } else if (st == 0) {
          __nanosleep(300);
        }
        groupBarrier(group);  // groupState may be rewritten from here on
        if (st == 2) break;
        if (st == 3 || okSmem[group] == 0) {
          healthy = false;
          break;
        }
      }
      if (!healthy) {
        if (lane == 0) okSmem[group] = 0;
        break;
      }
      // The poller took a system-scope acquire on the flags before it set the bit in shared memory; a CTA-scope
      // fence after reading the bit completes the chain for this thread. (A system-scope fence here would also wait
      // for this thread's outstanding peer stores of the previous row - microseconds per row.)
      __threadfence_block();
      readyMb = mb;
    }
    const uint64_t rowOff = static_cast<uint64_t>(row) * unitsPerRow * 16;
    if (tl) {
      const unsigned long long now = ptx::globaltimer();
      tlWait += now - tlMark;
      tlMark = now;
    }

    // ---- gather: the row summed over all ranks, packed bf16 in registers
    uint4 h[kWordsPerThread];
    if constexpr (kNvls) {
#pragma unroll
      for (int k = 0; k < kWordsPerThread; k++) {
        const int w = lane + k * kGroupThreads;
        h[k] = make_uint4(0, 0, 0, 0);
        if (w < unitsPerRow)
          h[k] = ptx::multimem_ld_reduce_add_bf16x2_acc32(reinterpret_cast<const void*>(c.mcBase + partialOff + rowOff + w * 16));
      }
    } else {
      // Two halves of 8 words, one fp32 accumulator set per half. The loads of the next peer (and, at the end of the
      // first half, of the second half's first peer) are put in flight before the current peer's words are added, so
      // a row costs about one NVLink round trip plus the issue time instead of 2 x world round trips in series.
      // Peers are visited starting with this rank (local memory answers first) - every rank a different order.
      const uint64_t rowBase = partialOff + rowOff;
      auto issue = [&](uint4 (&buf)[8], int half, int step) {
        const int p = (rank + step) % world;
        const uint64_t base = c.peerBase[p] + rowBase;
#pragma unroll
        for (int k = 0; k < 8; k++) {
          const int w = lane + (half * 8 + k) * kGroupThreads;
          buf[k] = make_uint4(0, 0, 0, 0);
          if (w < unitsPerRow) buf[k] = ptx::ld_nc_na_v4(reinterpret_cast<const void*>(base + w * 16));
        }
      };
      uint4 va[8], vb[8];
      issue(va, 0, 0);
#pragma unroll
      for (int half = 0; half < 2; half++) {
        float acc[8][8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
#pragma unroll
          for (int i = 0; i < 8; i++) acc[k][i] = 0.f;
        }
#pragma unroll 1
        for (int step = 0; step < world; step += 2) {
          if (step + 1 < world) issue(vb, half, step + 1);
#pragma unroll
          for (int k = 0; k < 8; k++) accumulate16<bf16, SUM>(acc[k], va[k]);
          if (step + 2 < world) {
            issue(va, half, step + 2);
          } else if (half == 0) {
            issue(va, 1, 0);
          }
          if (step + 1 < world) {
#pragma unroll
            for (int k = 0; k < 8; k++) accumulate16<bf16, SUM>(acc[k], vb[k]);
          }
        }
#pragma unroll
        for (int k = 0; k < 8; k++) h[half * 8 + k] = Vec16<bf16>::fromFloat(acc[k]);
      }
    }
    if (tl) {
      // (the first use of h below waits for the loads, so this stamp is taken after a dependent read)
      const unsigned long long now = ptx::globaltimer() + (h[0].x == 0x7fc07fc1u ? 1 : 0);
      tlGather += now - tlMark;
      tlPhase = now;
    }
    if (a.mode == 2) {
      // reduce-scatter: the reduced row stays here, in row j of this rank's [ownedRows, N] output
      const uint64_t dstOff = outOff + static_cast<uint64_t>(j) * unitsPerRow * 16;
#pragma unroll
      for (int k = 0; k < kWordsPerThread; k++) {
        const int w = lane + k * kGroupThreads;
        if (w < unitsPerRow) ptx::st_na_v4(reinterpret_cast<void*>(local + dstOff + w * 16), h[k]);
      }
      continue;
    }

    // ---- residual add (rounded to bf16 like the unfused composition), sum of squares
    float ss = 0.f;
#pragma unroll
    for (int half = 0; half < 2; half++) {
      uint4 res[8];
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int w = lane + (half * 8 + k) * kGroupThreads;
        if constexpr (kNvls) {
          res[k] = resEarly[half * 8 + k];
        } else {
          res[k] = make_uint4(0, 0, 0, 0);
          if (a.residualIn && w < unitsPerRow) res[k] = ptx::ld_nc_na_v4(reinterpret_cast<const void*>(local + resInOff + rowOff + w * 16));
        }
      }
#pragma unroll
      for (int k = 0; k < 8; k++) {
        float f[8], rf[8];
        Vec16<bf16>::toFloat(h[half * 8 + k], f);
        if (a.residualIn) {
          Vec16<bf16>::toFloat(res[k], rf);
#pragma unroll
          for (int i = 0; i < 8; i++) f[i] += rf[i];
          h[half * 8 + k] = Vec16<bf16>::fromFloat(f);
          Vec16<bf16>::toFloat(h[half * 8 + k], f);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) ss += f[i] * f[i];
      }
    }
    if (tl) {
      const unsigned long long now = ptx::globaltimer() + (ss == -1.f ? 1 : 0);
      tlMath += now - tlPhase;
      tlPhase = now;
    }
    if (a.residualOut) {
#pragma unroll
      for (int k = 0; k < kWordsPerThread; k++) {
        const int w = lane + k * kGroupThreads;
        if (w < unitsPerRow) scatterWord<kNvls>(c, rank, resOutOff + rowOff + w * 16, h[k]);
      }
    }
    if (tl) {
      const unsigned long long now = ptx::globaltimer();
      tlScatter += now - tlPhase;
    }
    const float total = groupSum(ss, sumSmem[group], group);
    const float rinv = rsqrtf(total / static_cast<float>(N) + a.eps);

    // ---- normalise and publish (mode 0), or publish 1/rms only (modes 1 and 3)
    if (a.mode == 1 || fold) {
      if (lane == 0) {
        const uint64_t off = rinvOff + static_cast<uint64_t>(row) * 4;
        if constexpr (kNvls) {
          ptx::multimem_st_u32(reinterpret_cast<void*>(c.mcBase + off), __float_as_uint(rinv));
        } else {
          for (int p = 0; p < world; p++) ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peerBase[p] + off), __float_as_uint(rinv));
        }
        if (fold) {
          // hand the row to the publisher (every thread of the group issued its stores before the barriers of groupSum)
          const int t = pubTail[group];
          SpinGuard g(c.status, c.timeoutNs);
          bool room = true;
          while (t - pubHead[group] >= kPubQueue) {
            __nanosleep(100);
            if (!g.keepSpinning()) {
              g.report(kDevTimeoutFlag, rank, 7800 + group, 0, t, pubHead[group]);
              room = false;
              break;
            }
          }
          if (room) {
            pubQueue[group][t % kPubQueue] = row / rpu;
            __threadfence_block();
            pubTail[group] = t + 1;
          } else {
            okSmem[group] = 0;
          }
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < kWordsPerThread; k++) {
        const int w = lane + k * kGroupThreads;
        if (w < unitsPerRow) {
          float f[8];
          Vec16<bf16>::toFloat(h[k], f);
          if (gamma) {
            float g[8];
            Vec16<bf16>::toFloat(*reinterpret_cast<const uint4*>(gamma + static_cast<size_t>(w) * 16), g);
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = f[i] * rinv * g[i];
          } else {
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = f[i] * rinv;
          }
          scatterWord<kNvls>(c, rank, outOff + rowOff + w * 16, Vec16<bf16>::fromFloat(f));
        }
      }
    }
    if (tl) {
      const unsigned long long now = ptx::globaltimer();
      tlWork += now - tlMark;
      if (tlRows == 0) tl[6] = now;
      tlRows++;
    }
  }
  if (tl) {
    tl[3] = tlRows;
    tl[4] = tlWait;
    tl[5] = tlWork;
    tl[8] = tlGather;
    tl[9] = tlMath;
    tl[10] = tlScatter;
  }
  if (fold) {
    // this group has pushed its last row: tell the publisher, then join the scale pass (every warp for itself)
    groupBarrier(group);
    if (lane == 0) {
      __threadfence_block();
      atomicSub(const_cast<int*>(&producersLeft), 1);
    }
    if (okSmem[group] != 0 && !scaleRowsWarp(a, rank, epoch, threadIdx.x & 31) && (threadIdx.x & 31) == 0) okSmem[group] = 0;
  }
  // every store of mine is issued: meet the peers' reducers with the same index. After it, everything
  // their reducers wrote into my buffers has landed.
  __syncthreads();
  bool allOk = true;
  for (int g = 0; g < kGroupsPerCta; g++) allOk = allOk && okSmem[g] != 0;
  if (allOk) rankBarrier(c, rank, 2, slot, epoch);
  if (tl) tl[2] = ptx::globaltimer();
}

// kBlockN == 0 selects the two-SM GEMM core (256 x 256 tiles on CTA pairs; the launch uses clusters of two).
template <int kBlockN, bool kNvls>
__global__ void __launch_bounds__(gemm::kNumThreads, 1)
    tpFusedKernel(const __grid_constant__ TmapSet maps, const __grid_constant__ TpFusedArgs a) {
  extern __shared__ uint8_t smemRaw[];
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const uint32_t epoch = launchEpoch(c, rank);
  const bool stamp = a.timeline != nullptr && blockIdx.y == 0 && threadIdx.x == 0;
  if (stamp) a.timeline[static_cast<size_t>(blockIdx.x) * kTimelineWords] = ptx::globaltimer();
  if (static_cast<int>(blockIdx.x) < a.numGemmCtas) {
    gemm::NoGate gate;
    const uint64_t partialOff = reinterpret_cast<uint64_t>(a.partial) - c.peerBase[c.rank];
    const int numUnits = (a.shape.M + a.rowsPerUnit - 1) / a.rowsPerUnit;
    constexpr int kTileN = kBlockN == 0 ? gemm::Config2::kBlockN : kBlockN;
    PartialStoreSignal epi{&c, reinterpret_cast<bf16*>(c.peerBase[rank] + partialOff), a.shape.M, a.shape.N, rank,
                           a.rowsPerUnit, numUnits, a.shape.N / kTileN, epoch,
                           (a.timeline != nullptr && blockIdx.y == 0) ? a.timeline + static_cast<size_t>(blockIdx.x) * kTimelineWords : nullptr,
                           a.sysFence};
    if constexpr (kBlockN == 0) {
      gemm::gemmCtaPair(&maps.a[blockIdx.y], &maps.b[blockIdx.y], a.shape, blockIdx.x / 2, a.numGemmCtas / 2, gate, epi, c.status,
                        c.timeoutNs, smemRaw);
    } else {
      gemm::gemmCta<kBlockN>(&maps.a[blockIdx.y], &maps.b[blockIdx.y], a.shape, blockIdx.x, a.numGemmCtas, gate, epi,
                             c.status, c.timeoutNs, smemRaw);
    }
  }
  if (stamp) a.timeline[static_cast<size_t>(blockIdx.x) * kTimelineWords + 1] = ptx::globaltimer();
  // dedicated reducer CTAs start here at once; GEMM CTAs arrive when their last tile is stored
  reducerCta<kNvls>(a, rank, epoch, blockIdx.x);
  finishLaunch(c, rank, epoch);
}

template <bool kNvls>
__global__ void __launch_bounds__(gemm::kNumThreads, 1) tpReduceNormKernel(const __grid_constant__ TpFusedArgs a) {
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const uint32_t epoch = launchEpoch(c, rank);
  // every rank's partial product is final once its kernel runs
  if (rankBarrier(c, rank, 0, blockIdx.x, epoch)) reducerCta<kNvls>(a, rank, epoch, blockIdx.x);
  finishLaunch(c, rank, epoch);
}

// Epilogue of the single-GPU layer: h = bf16(acc) + residual (rounded to bf16 like the unfused composition), stored;
// the sum of squares of the rounded values over the columns that ONE epilogue warp handles in a tile goes to
// sumsq[part][row] (part = those columns' index, N / (64 * blocksPerWarp) parts per row): every word of the table is
// written exactly once per launch, so nothing has to be cleared before it and no atomics are involved. Whoever needs a
// row's sum adds up its parts.
// The residual of a block is requested one block ahead (the first at tileBegin, before the accumulator is ready), with the
// row-contiguous lane mapping of the staging buffer: every load and store covers complete 128-byte lines.
struct ResidualSumsqStore {
  static constexpr bool kNeedsTileBarrier = false;
  static constexpr bool kBulkStore = false;
  const bf16* residual;  // [M, N] or null
  bf16* h;               // [M, N]
  float* sumsq;          // [N / (64 * blocksPerWarp)][M]
  int M, N;
  int blocksPerWarp;  // 64-column blocks per warp and tile
  int probe;          // diagnostics, 0 in production: bit 4 no residual loads, bit 5 no sum-of-squares stores, bit 6 no h
                      // stores, bit 7 no normalisation (results are then wrong; timing only)
  uint4 pre[8];       // residual words of the block that comes next
  float ssAcc[8];     // this lane's rows: sum of squares over the blocks of the current tile so far
  MSCCLPP_DEVICE_INLINE int numParts() const { return N / (64 * blocksPerWarp); }
  MSCCLPP_DEVICE_INLINE static float convert(float x) { return x; }
  MSCCLPP_DEVICE_INLINE void prefetch(int row0, int col0, int lane) {
    if (residual == nullptr || (probe & 16)) return;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int row = row0 + gemm::stagedRow(i, lane);
      pre[i] = make_uint4(0, 0, 0, 0);
      if (row < M) pre[i] = ptx::ld_input_v4(residual + static_cast<size_t>(row) * N + col0 + gemm::stagedCol(lane));
    }
  }
  MSCCLPP_DEVICE_INLINE void tileBegin(int row0, int col0, int lane) { prefetch(row0, col0, lane); }
  MSCCLPP_DEVICE_INLINE void block(const uint8_t* stage, int row0, int col0, int lane, int b) {
    uint4 res[8];
#pragma unroll
    for (int i = 0; i < 8; i++) res[i] = pre[i];
    if (b + 1 < blocksPerWarp) prefetch(row0, col0 + 64, lane);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int row = row0 + gemm::stagedRow(i, lane);
      uint4 packed = gemm::stagedRead(stage, i, lane);
      if (residual != nullptr) packed = addBf16x8(packed, res[i]);
      float ss = sumSquaresBf16x8(packed);
      // the eight lanes that share a row
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      ss += __shfl_xor_sync(0xffffffffu, ss, 4);
      ssAcc[i] = b == 0 ? ss : ssAcc[i] + ss;
      if (row < M) {
        if (!(probe & 64)) *reinterpret_cast<uint4*>(h + static_cast<size_t>(row) * N + col0 + gemm::stagedCol(lane)) = packed;
        if (b == blocksPerWarp - 1 && (lane & 7) == 0 && !(probe & 32)) {
          sumsq[static_cast<size_t>((col0 - b * 64) / (64 * blocksPerWarp)) * M + row] = ssAcc[i];
        }
      }
    }
    __syncwarp();
  }
  MSCCLPP_DEVICE_INLINE void tileDone(int, int, int) const {}
  MSCCLPP_DEVICE_INLINE void warpTileDone(int, int) const {}
  MSCCLPP_DEVICE_INLINE void warpDrain(int) const {}
  MSCCLPP_DEVICE_INLINE void auxWarp(int, int) const {}
};

// The whole single-GPU layer in ONE kernel: the epilogue of ResidualSumsqStore, plus the normalisation. Every epilogue
// warp counts its finished part of a tile on the tile's 128-row block; once a block has all its arrivals its rows are
// final (h stored, sums of squares added) and become units of follow-up work, two rows each, handed out in ascending
// order from one counter. A warp takes at most one unit after each tile part (without ever waiting: a unit is only
// taken when its block is already complete), so the normalisation of block i runs in the shadow of the MMAs of the
// blocks after it and h is re-read from L2. The units are taken by kAuxWarps extra warps per CTA that have no other job
// (an epilogue warp that stopped for a row would hold up the accumulator hand-over of its tile); the epilogue warps join
// them after their last tile. All waits are bounded.
struct ResidualNormStore {
  static constexpr bool kNeedsTileBarrier = false;
  static constexpr bool kBulkStore = false;
  static constexpr int kRowsPerUnit = 2;
  static constexpr int kAuxWarps = 4;
  ResidualSumsqStore base;
  bf16* out;            // [M, N]
  const bf16* gamma;    // [N] or null
  uint32_t* blockCount;  // [ceil(M / 128)] arrivals per row block, zero at launch
  uint32_t* nextUnit;    // zero at launch
  uint32_t fullCount;    // arrivals that complete a row block: N tiles x epilogue warps per tile
  float eps;
  DeviceStatus* status;
  uint64_t budgetNs;
  uint32_t pendingUnit;  // per thread (lane 0 of each epilogue warp): a claimed unit whose block was not complete yet
  int pendingArrive;     // per thread: row block whose arrival this warp still owes (-1 = none)
  unsigned long long* stamps;  // optional time line (gemm::Shape::stamps): words 9-12 of a CTA are its first extra warp's
                               // units done, ns waited for blocks, ns spent normalising, finish time
  MSCCLPP_DEVICE_INLINE static float convert(float x) { return x; }
  MSCCLPP_DEVICE_INLINE void tileBegin(int row0, int col0, int lane) { base.tileBegin(row0, col0, lane); }
  MSCCLPP_DEVICE_INLINE void block(const uint8_t* stage, int row0, int col0, int lane, int b) {
    if (b == 0) flushArrival(lane);  // the previous tile's arrival (see warpTileDone)
    base.block(stage, row0, col0, lane, b);
  }
  MSCCLPP_DEVICE_INLINE void tileDone(int, int, int) const {}

  MSCCLPP_DEVICE_INLINE void normaliseRow(int row, int lane) const {
    const int N = base.N;
    float total = 0.f;
    for (int p = lane; p < base.numParts(); p += 32) total += __ldcg(base.sumsq + static_cast<size_t>(p) * base.M + row);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    const float rinv = rsqrtf(total / static_cast<float>(N) + eps);
    const __nv_bfloat16 hi1 = __float2bfloat16_rn(rinv);
    const __nv_bfloat162 hi = __bfloat162bfloat162(hi1);
    const __nv_bfloat162 lo = __float2bfloat162_rn(rinv - __bfloat162float(hi1));
    const int words = N / 8;
    const uint4* src = reinterpret_cast<const uint4*>(base.h + static_cast<size_t>(row) * N);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * N);
    const uint4* g4 = reinterpret_cast<const uint4*>(gamma);
    const bool hasGamma = gamma != nullptr;
    constexpr int kDepth = 16;  // 16-byte loads in flight per lane
    for (int w0 = lane; w0 < words; w0 += 32 * kDepth) {
      uint4 v[kDepth];
#pragma unroll
      for (int k = 0; k < kDepth; k++) {
        const int w = w0 + 32 * k;
        if (w < words) v[k] = ptx::ld_cg_v4(src + w);  // written by other SMs during this launch: through L2, never L1
      }
#pragma unroll
      for (int k = 0; k < kDepth; k++) {
        const int w = w0 + 32 * k;
        if (w < words) {
          const uint4 g = hasGamma ? __ldg(g4 + w) : make_uint4(0, 0, 0, 0);
          dst[w] = make_uint4(scaleBf16x2(v[k].x, g.x, hi, lo, hasGamma), scaleBf16x2(v[k].y, g.y, hi, lo, hasGamma),
                              scaleBf16x2(v[k].z, g.z, hi, lo, hasGamma), scaleBf16x2(v[k].w, g.w, hi, lo, hasGamma));
        }
      }
    }
  }

  MSCCLPP_DEVICE_INLINE void normaliseUnit(uint32_t u, int lane) const {
    if (base.probe & 128) return;
    const int r0 = static_cast<int>(u) * kRowsPerUnit;
#pragma unroll 1
    for (int r = r0; r < r0 + kRowsPerUnit && r < base.M; r++) normaliseRow(r, lane);
  }
  MSCCLPP_DEVICE_INLINE bool blockComplete(uint32_t unit) const {
    return ptx::ld_acquire_gpu(blockCount + unit * kRowsPerUnit / gemm::kBlockM) >= fullCount;
  }

  // An epilogue warp only counts its finished part of a tile (normalising rows between tiles would sit on the critical
  // path of the accumulator hand-over: the MMA waits for the slowest of the eight warps). The count needs a fence after
  // the warp's h stores and sum-of-squares updates, and a fence right behind the stores waits out their whole latency;
  // so the arrival for a tile is only NOTED here and made one tile later (flushArrival, called when the next tile's
  // accumulator has been read), when those stores have long been performed and the fence returns at once.
  MSCCLPP_DEVICE_INLINE void warpTileDone(int mBlk, int /*lane*/) { pendingArrive = mBlk; }
  MSCCLPP_DEVICE_INLINE void flushArrival(int lane) {
    if (pendingArrive < 0) return;
    __syncwarp();
    if (lane == 0) {
      __threadfence();
      atomicAdd(blockCount + pendingArrive, 1u);
    }
    pendingArrive = -1;
  }
  // The extra warps of the launch do nothing but normalise: claim the next unit, wait (bounded) for its block, scale.
  MSCCLPP_DEVICE_INLINE void auxWarp(int idx, int lane) {
    drain(lane, (stamps != nullptr && idx == 0 && lane == 0) ? stamps + static_cast<size_t>(blockIdx.x) * gemm::kStampWords : nullptr);
  }

  // The warp has no tile left: finish the unit it holds, then claim and finish units until none is left. Waiting is
  // safe here (bounded all the same): what a block still lacks is produced by warps that do not depend on this one.
  MSCCLPP_DEVICE_INLINE void warpDrain(int lane) { drain(lane, nullptr); }
  MSCCLPP_DEVICE_INLINE void drain(int lane, unsigned long long* tl) {
    constexpr uint32_t kNone = 0xffffffffu;
    const uint32_t totalUnits = static_cast<uint32_t>((base.M + kRowsPerUnit - 1) / kRowsPerUnit);
    flushArrival(lane);  // the last tile's arrival
    for (;;) {
      uint32_t go = kNone;
      unsigned long long t0 = 0;
      if (tl != nullptr) t0 = ptx::globaltimer();
      if (lane == 0) {
        uint32_t mine = pendingUnit;
        pendingUnit = kNone;
        if (mine == kNone && ptx::ld_volatile(nextUnit) < totalUnits) {
          mine = atomicAdd(nextUnit, 1u);
          if (mine >= totalUnits) mine = kNone;
        }
        if (mine != kNone) {
          SpinGuard g(status, budgetNs);
          bool ready = true;
          while (!blockComplete(mine)) {
            __nanosleep(200);
            if (!g.keepSpinning()) {
              g.report(kDevTimeoutFlag, 0, 7500, 0, fullCount, mine);
              ready = false;
              break;
            }
          }
          if (ready) go = mine;
        }
      }
      go = __shfl_sync(0xffffffffu, go, 0);
      unsigned long long t1 = 0;
      if (tl != nullptr) {
        t1 = ptx::globaltimer();
        tl[10] += t1 - t0;
      }
      if (go == kNone) {
        if (tl != nullptr) tl[12] = t1;
        return;
      }
      normaliseUnit(go, lane);
      if (tl != nullptr) {
        tl[11] += ptx::globaltimer() - t1;
        tl[9] += 1;
      }
    }
  }
};

template <int kBlockN>
__global__ void __launch_bounds__(gemm::kNumThreads + 32 * ResidualNormStore::kAuxWarps, 1)
    tpLocalFusedKernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, gemm::Shape shape,
                       ResidualNormStore epi) {
  extern __shared__ uint8_t smemRaw[];
  gemm::NoGate gate;
  if constexpr (kBlockN == 0) {
    gemm::gemmCtaPair(&tmapA, &tmapB, shape, blockIdx.x / 2, gridDim.x / 2, gate, epi, epi.status, epi.budgetNs, smemRaw);
  } else {
    gemm::gemmCta<kBlockN>(&tmapA, &tmapB, shape, blockIdx.x, gridDim.x, gate, epi, epi.status, epi.budgetNs, smemRaw);
  }
}

template <int kBlockN>
__global__ void __launch_bounds__(gemm::kNumThreads, 1)
    gemmResidualSumsqKernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, gemm::Shape shape,
                            ResidualSumsqStore epi, DeviceStatus* status, uint64_t budgetNs) {
  extern __shared__ uint8_t smemRaw[];
  gemm::NoGate gate;
  if constexpr (kBlockN == 0) {
    gemm::gemmCtaPair(&tmapA, &tmapB, shape, blockIdx.x / 2, gridDim.x / 2, gate, epi, status, budgetNs, smemRaw);
  } else {
    gemm::gemmCta<kBlockN>(&tmapA, &tmapB, shape, blockIdx.x, gridDim.x, gate, epi, status, budgetNs, smemRaw);
  }
}

// out[row] = h[row] * rsqrt(sum of the row's parts / N + eps) * gamma. `tpr` threads (a multiple of 32) share a row; every
// warp adds up the parts for itself. Eight 16-byte loads are in flight per thread.
__global__ void __launch_bounds__(512) tpScaleRowsPartsKernel(const bf16* h, const float* parts, int numParts, const bf16* gamma, bf16* out,
                                                              int M, int N, float eps, int tpr) {
  const int lane = threadIdx.x & 31;
  const int groupsPerBlock = blockDim.x / tpr;
  const int inGroup = threadIdx.x % tpr;
  const int words = N / 8;
  const uint4* g4 = reinterpret_cast<const uint4*>(gamma);
  for (int row = blockIdx.x * groupsPerBlock + threadIdx.x / tpr; row < M; row += gridDim.x * groupsPerBlock) {
    float total = 0.f;
    for (int p = lane; p < numParts; p += 32) total += parts[static_cast<size_t>(p) * M + row];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    const float sc = rsqrtf(total / static_cast<float>(N) + eps);
    const uint4* src = reinterpret_cast<const uint4*>(h + static_cast<size_t>(row) * N);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * N);
    for (int w0 = inGroup; w0 < words; w0 += tpr * 8) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int w = w0 + k * tpr;
        if (w < words) v[k] = ptx::ld_input_v4(src + w);
      }
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int w = w0 + k * tpr;
        if (w < words) {
          float f[8];
          Vec16<bf16>::toFloat(v[k], f);
          if (gamma != nullptr) {
            float g[8];
            Vec16<bf16>::toFloat(__ldg(g4 + w), g);
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = f[i] * sc * g[i];
          } else {
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = f[i] * sc;
          }
          dst[w] = Vec16<bf16>::fromFloat(f);
        }
      }
    }
  }
}

// out[row] = h[row] * rinv[row] * gamma (local pass of mode 1)
__global__ void __launch_bounds__(512) tpScaleRowsKernel(const bf16* h, const float* rinv, const bf16* gamma, bf16* out,
                                                         int M, int N) {
  const int unitsPerRow = N / 8;
  const size_t total = static_cast<size_t>(M) * unitsPerRow;
  // The rows arrived in ascending order during the launch before this one, so the LAST rows are the ones still in L2:
  // the pass walks the rows from the end.
  for (size_t v = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < total;
       v += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t u = total - 1 - v;
    const int row = static_cast<int>(u / unitsPerRow), ru = static_cast<int>(u % unitsPerRow);
    float f[8];
    Vec16<bf16>::toFloat(*reinterpret_cast<const uint4*>(h + u * 8), f);
    const float s = rinv[row];
    if (gamma) {
      float g[8];
      Vec16<bf16>::toFloat(*reinterpret_cast<const uint4*>(gamma + static_cast<size_t>(ru) * 8), g);
#pragma unroll
      for (int i = 0; i < 8; i++) f[i] = f[i] * s * g[i];
    } else {
#pragma unroll
      for (int i = 0; i < 8; i++) f[i] = f[i] * s;
    }
    *reinterpret_cast<uint4*>(out + u * 8) = Vec16<bf16>::fromFloat(f);
  }
}

template <int kBlockN>
struct SmemOf {
  static constexpr int kSmemBytes = gemm::Config<kBlockN>::kSmemBytes;
};
template <>
struct SmemOf<0> {
  static constexpr int kSmemBytes = gemm::Config2::kSmemBytes;
};

template <int kBlockN>
cudaError_t launchTyped(const TmapSet& maps, const TpFusedArgs& args, int grid, cudaStream_t stream) {
  using Cfg = SmemOf<kBlockN>;
  auto kernelNvls = tpFusedKernel<kBlockN, true>;
  auto kernelP2p = tpFusedKernel<kBlockN, false>;
  cudaError_t e = gemm::ensureDynamicSmem(reinterpret_cast<const void*>(kernelNvls), Cfg::kSmemBytes);
  if (e == cudaSuccess) e = gemm::ensureDynamicSmem(reinterpret_cast<const void*>(kernelP2p), Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 g(grid, args.emuRanks > 1 ? args.emuRanks : 1, 1);
  dim3 b(gemm::kNumThreads, 1, 1);
  auto kernel = args.nvls ? kernelNvls : kernelP2p;
  if constexpr (kBlockN == 0) {
    TmapSet m = maps;
    TpFusedArgs a = args;
    void* params[] = {&m, &a};
    return gemm::launchClusterPair(reinterpret_cast<const void*>(kernel), g, b, Cfg::kSmemBytes, params, args.emuRanks > 1, stream);
  }
  if (args.emuRanks > 1) {
    TmapSet m = maps;
    TpFusedArgs a = args;
    void* params[] = {&m, &a};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), g, b, params, Cfg::kSmemBytes, stream);
  }
  kernel<<<g, b, Cfg::kSmemBytes, stream>>>(maps, args);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launchTpFused(const TpFusedArgs& argsIn, const void* const* A, const void* const* B, int numReducers,
                          cudaStream_t stream) {
  TpFusedArgs args = argsIn;
  const int M = args.shape.M, N = args.shape.N, K = args.shape.K;
  const int world = args.comm.world;
  const bool twoSm = args.blockN == 0;  // block_n 0 = 256 x 256 tiles on SM pairs
  const int tileN = twoSm ? gemm::Config2::kBlockN : args.blockN;
  if (M <= 0 || N % tileN != 0 || K % gemm::kBlockK != 0) return cudaErrorInvalidValue;
  if (twoSm && M < gemm::Config2::kPairM) return cudaErrorInvalidValue;
  if (N / tileN > kMaxNBlk || world > 8) return cudaErrorInvalidValue;
  if (N * 2 / 16 > kWordsPerThread * kGroupThreads) return cudaErrorInvalidValue;
  const int numMBlk = (M + gemm::kBlockM - 1) / gemm::kBlockM;
  if (numMBlk > kMaxMBlk) return cudaErrorInvalidValue;
  if ((args.mode == 1 || args.mode == 3) && args.rinv == nullptr) return cudaErrorInvalidValue;
  if (args.nvls && args.comm.mcBase == 0) return cudaErrorInvalidValue;
  const int emu = args.emuRanks > 1 ? args.emuRanks : 1;
  if (emu > 8) return cudaErrorInvalidValue;
  if (args.sysFence < 0) {
    const char* env = std::getenv("MSCCLPP_TP_SYS_FENCE");
    args.sysFence = (env != nullptr && env[0] != '\0' && env[0] != '0') ? 1 : 0;
  }
  args.shape.aBoxRows = M < gemm::kBlockM ? M : gemm::kBlockM;
  args.shape.rowMajorTiles = 1;
  if (args.mode == 2) {
    // reduce-scatter: rank r owns rows [r * M / world, (r + 1) * M / world); the GEMM visits the row blocks
    // interleaved over the owners so that every owner's reducers have a finished block per round
    if (M % (world * (twoSm ? gemm::Config2::kPairM : gemm::kBlockM)) != 0) return cudaErrorInvalidValue;
    args.rowsPerUnit = M / world;
    args.shape.mOrder = 1;
    args.shape.mOrderParam = world;
  }
  if (args.rowsPerUnit <= 0) {
    int rpu = gemm::kBlockM;
    while (rpu > 1 && M < rpu * world) rpu >>= 1;
    args.rowsPerUnit = rpu;
  }
  if (args.mode == 3 && (args.residualOut == nullptr || (M + args.rowsPerUnit - 1) / args.rowsPerUnit > kTpMaxUnits)) return cudaErrorInvalidValue;
  TmapSet maps;
  for (int e = 0; e < emu; e++) {
    cudaError_t err = gemm::makeTensorMapBf16(&maps.a[e], A[e], M, K, static_cast<uint64_t>(K) * 2, args.shape.aBoxRows);
    if (err != cudaSuccess) return err;
    err = gemm::makeTensorMapBf16(&maps.b[e], B[e], N, K, static_cast<uint64_t>(K) * 2, twoSm ? tileN / 2 : tileN);
    if (err != cudaSuccess) return err;
  }
  const int tiles = twoSm ? 2 * ((M + gemm::Config2::kPairM - 1) / gemm::Config2::kPairM) * (N / tileN) : numMBlk * (N / tileN);
  int sms = gemm::smCount() / emu;
  // Measured on 2 and 8 B200s with K = 1024 per rank: from about a thousand tokens on the reduction is the longer half and
  // wants ~48 CTAs from the first finished row block; below that the GEMM is short and few dedicated reducers keep more
  // SMs on it. With a long reduction dimension the matmul is the longer half again and gets the SMs back.
  if (numReducers <= 0) numReducers = sms >= 64 ? (M < 1024 ? 8 : (K <= 2048 ? 48 : 24)) : 2;
  if (numReducers > kBarrierSlots) numReducers = kBarrierSlots;
  int gemmCtas = args.numGemmCtas > 0 ? args.numGemmCtas : sms - numReducers;
  if (gemmCtas > tiles) gemmCtas = tiles;
  if (gemmCtas < 1) gemmCtas = 1;
  if (twoSm) {
    // CTA pairs: an even number of GEMM CTAs and of reducers, so that clusters never straddle the two roles
    gemmCtas &= ~1;
    if (gemmCtas < 2) gemmCtas = 2;
    numReducers = (numReducers + 1) & ~1;
  }
  args.numGemmCtas = gemmCtas;
  const int grid = gemmCtas + numReducers;
  switch (args.blockN) {
    case 0:
      return launchTyped<0>(maps, args, grid, stream);
    case 64:
      return launchTyped<64>(maps, args, grid, stream);
    case 128:
      return launchTyped<128>(maps, args, grid, stream);
    case 256:
      return launchTyped<256>(maps, args, grid, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

cudaError_t launchTpReduceNorm(const TpFusedArgs& argsIn, int numCtas, cudaStream_t stream) {
  TpFusedArgs args = argsIn;
  const int M = args.shape.M, N = args.shape.N;
  const int world = args.comm.world;
  if (M <= 0 || N % 8 != 0 || N * 2 / 16 > kWordsPerThread * kGroupThreads || world > 8) return cudaErrorInvalidValue;
  if (args.mode != 0 && args.mode != 1) return cudaErrorInvalidValue;
  if ((args.mode == 1 || args.mode == 3) && args.rinv == nullptr) return cudaErrorInvalidValue;
  if (args.nvls && args.comm.mcBase == 0) return cudaErrorInvalidValue;
  const int emu = args.emuRanks > 1 ? args.emuRanks : 1;
  if (emu > 8) return cudaErrorInvalidValue;
  if (args.rowsPerUnit <= 0) {
    int rpu = 64;  // smaller units than the fused kernel's: nothing ties ownership to GEMM row blocks here
    while (rpu > 1 && M < rpu * world) rpu >>= 1;
    args.rowsPerUnit = rpu;
  }
  args.noFlags = 1;
  args.numGemmCtas = 0;
  const int sms = gemm::smCount() / emu;
  if (numCtas <= 0) numCtas = sms < 128 ? sms : 128;
  if (numCtas > kBarrierSlots) numCtas = kBarrierSlots;
  dim3 g(numCtas, emu, 1), b(gemm::kNumThreads, 1, 1);
  auto kernel = args.nvls ? tpReduceNormKernel<true> : tpReduceNormKernel<false>;
  if (emu > 1) {
    void* params[] = {&args};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), g, b, params, 0, stream);
  }
  kernel<<<g, b, 0, stream>>>(args);
  return cudaGetLastError();
}

template <int kBlockN>
cudaError_t launchLocalTyped(const CUtensorMap& ta, const CUtensorMap& tb, gemm::Shape shape, ResidualSumsqStore epi, DeviceStatus* status,
                             cudaStream_t stream) {
  using Cfg = SmemOf<kBlockN>;
  auto kernel = gemmResidualSumsqKernel<kBlockN>;
  cudaError_t e = gemm::ensureDynamicSmem(reinterpret_cast<const void*>(kernel), Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  uint64_t budget = 2000000000ull;
  if constexpr (kBlockN == 0) {
    const int tiles = ((shape.M + gemm::Config2::kPairM - 1) / gemm::Config2::kPairM) * (shape.N / gemm::Config2::kBlockN);
    int grid = gemm::smCount() & ~1;
    if (grid > 2 * tiles) grid = 2 * tiles;
    void* params[] = {const_cast<CUtensorMap*>(&ta), const_cast<CUtensorMap*>(&tb), &shape, &epi, &status, &budget};
    return gemm::launchClusterPair(reinterpret_cast<const void*>(kernel), dim3(grid), dim3(gemm::kNumThreads), Cfg::kSmemBytes, params, false,
                                   stream);
  } else {
    const int tiles = ((shape.M + gemm::kBlockM - 1) / gemm::kBlockM) * (shape.N / kBlockN);
    int grid = gemm::smCount();
    if (grid > tiles) grid = tiles;
    kernel<<<grid, gemm::kNumThreads, Cfg::kSmemBytes, stream>>>(ta, tb, shape, epi, status, budget);
    return cudaGetLastError();
  }
}

int tpSumsqParts(int N, int blockN, bool twoSm) {
  const int blocksPerWarp = twoSm ? gemm::Config2::kColsPerWarp / 64 : (blockN >= 128 ? blockN / 128 : 1);
  return N / (64 * blocksPerWarp);
}

cudaError_t launchGemmResidualSumsq(const void* A, const void* B, const void* residual, void* h, float* sumsq, int M, int N, int K,
                                    int blockN, bool twoSm, DeviceStatus* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % gemm::kBlockK != 0 || N % 8 != 0) return cudaErrorInvalidValue;
  if (twoSm && (M < gemm::Config2::kPairM || N % gemm::Config2::kBlockN != 0)) return cudaErrorInvalidValue;
  if (!twoSm && (blockN != 64 && blockN != 128 && blockN != 256)) return cudaErrorInvalidValue;
  if (!twoSm && N % blockN != 0) return cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
  gemm::Shape shape{M, N, K, M < gemm::kBlockM ? M : gemm::kBlockM, 0, 0, 0};
  if (twoSm) shape.aBoxRows = gemm::kBlockM;
  CUtensorMap ta, tb;
  e = gemm::makeTensorMapBf16(&ta, A, M, K, static_cast<uint64_t>(K) * 2, shape.aBoxRows);
  if (e != cudaSuccess) return e;
  e = gemm::makeTensorMapBf16(&tb, B, N, K, static_cast<uint64_t>(K) * 2, twoSm ? gemm::Config2::kBlockN / 2 : blockN);
  if (e != cudaSuccess) return e;
  ResidualSumsqStore epi{};
  epi.residual = static_cast<const bf16*>(residual);
  epi.h = static_cast<bf16*>(h);
  epi.sumsq = sumsq;
  epi.M = M;
  epi.N = N;
  epi.blocksPerWarp = twoSm ? gemm::Config2::kColsPerWarp / 64 : (blockN >= 128 ? blockN / 128 : 1);
  if (twoSm) return launchLocalTyped<0>(ta, tb, shape, epi, status, stream);
  switch (blockN) {
    case 64:
      return launchLocalTyped<64>(ta, tb, shape, epi, status, stream);
    case 128:
      return launchLocalTyped<128>(ta, tb, shape, epi, status, stream);
    default:
      return launchLocalTyped<256>(ta, tb, shape, epi, status, stream);
  }
}

constexpr int kLocalFusedThreads = gemm::kNumThreads + 32 * ResidualNormStore::kAuxWarps;

template <int kBlockN>
cudaError_t launchLocalFusedTyped(const CUtensorMap& ta, const CUtensorMap& tb, gemm::Shape shape, ResidualNormStore epi, cudaStream_t stream) {
  using Cfg = SmemOf<kBlockN>;
  auto kernel = tpLocalFusedKernel<kBlockN>;
  cudaError_t e = gemm::ensureDynamicSmem(reinterpret_cast<const void*>(kernel), Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  if constexpr (kBlockN == 0) {
    const int tiles = ((shape.M + gemm::Config2::kPairM - 1) / gemm::Config2::kPairM) * (shape.N / gemm::Config2::kBlockN);
    int grid = gemm::smCount() & ~1;
    if (grid > 2 * tiles) grid = 2 * tiles;
    void* params[] = {const_cast<CUtensorMap*>(&ta), const_cast<CUtensorMap*>(&tb), &shape, &epi};
    return gemm::launchClusterPair(reinterpret_cast<const void*>(kernel), dim3(grid), dim3(kLocalFusedThreads), Cfg::kSmemBytes, params,
                                   false, stream);
  } else {
    const int tiles = ((shape.M + gemm::kBlockM - 1) / gemm::kBlockM) * (shape.N / kBlockN);
    int grid = gemm::smCount();
    if (grid > tiles) grid = tiles;
    kernel<<<grid, kLocalFusedThreads, Cfg::kSmemBytes, stream>>>(ta, tb, shape, epi);
    return cudaGetLastError();
  }
}

namespace {
// words of counters at the start of the one-kernel path's workspace: [row blocks, rounded up to the pair core's 256-row
// tiles] arrival counters and one unit counter, rounded up to a multiple of four words
size_t localFusedCounterWords(int M) {
  const size_t blocks = 2 * static_cast<size_t>((M + gemm::Config2::kPairM - 1) / gemm::Config2::kPairM);
  return (blocks + 1 + 3) / 4 * 4;
}
}  // namespace

size_t tpLocalFusedWorkspaceBytes(int M, int N) {
  // the counters (cleared before every launch), then the [N / 64][M] parts of the rows' sums of squares (never cleared)
  return (localFusedCounterWords(M) + static_cast<size_t>(M) * (N / 64)) * 4;
}

cudaError_t launchTpLocalFused(const void* A, const void* B, const void* residual, void* h, void* out, const void* gamma, void* workspace,
                               int M, int N, int K, float eps, int blockN, bool twoSm, DeviceStatus* status, cudaStream_t stream, int probe,
                               unsigned long long* stamps) {
  if (M <= 0 || N <= 0 || K <= 0 || K % gemm::kBlockK != 0 || N % 8 != 0) return cudaErrorInvalidValue;
  if (twoSm && (M < gemm::Config2::kPairM || N % gemm::Config2::kBlockN != 0)) return cudaErrorInvalidValue;
  if (!twoSm && (blockN != 64 && blockN != 128 && blockN != 256)) return cudaErrorInvalidValue;
  if (!twoSm && N % blockN != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(residual) |
       reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(workspace)) & 15)
    return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(workspace, 0, localFusedCounterWords(M) * 4, stream);
  if (e != cudaSuccess) return e;
  // row blocks are walked one after the other (all their N tiles first), so that they complete in order and early
  gemm::Shape shape{M, N, K, M < gemm::kBlockM ? M : gemm::kBlockM, 1, 0, 0, probe & 15, stamps};
  if (twoSm) shape.aBoxRows = gemm::kBlockM;
  CUtensorMap ta, tb;
  e = gemm::makeTensorMapBf16(&ta, A, M, K, static_cast<uint64_t>(K) * 2, shape.aBoxRows);
  if (e != cudaSuccess) return e;
  const int tileN = twoSm ? gemm::Config2::kBlockN : blockN;
  e = gemm::makeTensorMapBf16(&tb, B, N, K, static_cast<uint64_t>(K) * 2, twoSm ? tileN / 2 : tileN);
  if (e != cudaSuccess) return e;
  const int epiWarps = tileN >= 128 ? gemm::kNumEpilogueWarps : 4;
  ResidualNormStore epi{};
  epi.base.residual = static_cast<const bf16*>(residual);
  epi.base.h = static_cast<bf16*>(h);
  epi.base.sumsq = static_cast<float*>(workspace) + localFusedCounterWords(M);
  epi.base.M = M;
  epi.base.N = N;
  epi.base.blocksPerWarp = tileN / (epiWarps / 4) / 64;
  epi.base.probe = probe;
  epi.out = static_cast<bf16*>(out);
  epi.gamma = static_cast<const bf16*>(gamma);
  epi.blockCount = static_cast<uint32_t*>(workspace);
  epi.nextUnit = epi.blockCount + 2 * ((M + gemm::Config2::kPairM - 1) / gemm::Config2::kPairM);
  epi.fullCount = static_cast<uint32_t>((N / tileN) * epiWarps);
  epi.eps = eps;
  epi.status = status;
  epi.budgetNs = 2000000000ull;
  epi.pendingUnit = 0xffffffffu;
  epi.pendingArrive = -1;
  epi.stamps = stamps;
  if (twoSm) return launchLocalFusedTyped<0>(ta, tb, shape, epi, stream);
  switch (blockN) {
    case 64:
      return launchLocalFusedTyped<64>(ta, tb, shape, epi, stream);
    case 128:
      return launchLocalFusedTyped<128>(ta, tb, shape, epi, stream);
    default:
      return launchLocalFusedTyped<256>(ta, tb, shape, epi, stream);
  }
}

cudaError_t launchTpScaleRowsFromSumsq(const void* h, const float* sumsqParts, int numParts, const void* gamma, void* out, int M, int N,
                                       float eps, cudaStream_t stream) {
  if (N % 8 != 0 || numParts < 1 || M < 1) return cudaErrorInvalidValue;
  // few rows: a whole thread block per row (one batch of loads); many rows: a warp per row
  const int sms = gemm::smCount();
  const int tpr = M <= 2 * sms ? 512 : (M <= 16 * sms ? 128 : 32);
  const int groupsPerBlock = 512 / tpr;
  int blocks = (M + groupsPerBlock - 1) / groupsPerBlock;
  if (blocks > sms * 4) blocks = sms * 4;
  tpScaleRowsPartsKernel<<<blocks, 512, 0, stream>>>(static_cast<const bf16*>(h), sumsqParts, numParts, static_cast<const bf16*>(gamma),
                                                      static_cast<bf16*>(out), M, N, eps, tpr);
  return cudaGetLastError();
}

cudaError_t launchTpScaleRows(const void* h, const float* rinv, const void* gamma, void* out, int M, int N,
                              cudaStream_t stream) {
  if (N % 8 != 0) return cudaErrorInvalidValue;
  const size_t total = static_cast<size_t>(M) * (N / 8);
  int blocks = static_cast<int>((total + 511) / 512);
  const int cap = gemm::smCount() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  tpScaleRowsKernel<<<blocks, 512, 0, stream>>>(static_cast<const bf16*>(h), rinv, static_cast<const bf16*>(gamma),
                                                static_cast<bf16*>(out), M, N);
  return cudaGetLastError();
}

}  // namespace mscclpp
