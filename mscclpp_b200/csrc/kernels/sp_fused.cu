// All-gather -> GEMM in ONE kernel (sequence parallelism, the column-parallel half of an MLP):
//
//     D[M, N] = act( concat_r(A_r)[M, K] * W[N, K]^T )        A_r = rank r's [M / world, K] rows
//
// CTAs [0, numGemmCtas) run the tcgen05/TMEM GEMM. They visit the row blocks of this rank first (operands come
// straight from aLocal) and then the peers' in the order rank+1, rank+2, ... The remaining CTAs are copiers: one
// thread each drives a ring of TMA bulk copies (peer memory -> shared memory -> aFull) and, per 128-row block,
// publishes an epoch-stamped flag; the GEMM's TMA producer waits for that flag before it loads the block's
// tiles. Every A row therefore crosses NVLink exactly once (a GEMM that read its tiles from peer memory would
// fetch them N / blockN times) and the gather of block i+1 overlaps the MMAs of block i.
//
// No load here uses cluster multicast; peers' memory is only ever the source of plain bulk copies.
// The reference library has no counterpart (it offers the all-gather alone).
#include "sp_fused.cuh"

#include <mscclpp/gpu_data_types.hpp>

#include "gemm2_sm100.cuh"
#include "gemm_sm100.cuh"

namespace mscclpp {

namespace {

using bf16 = __nv_bfloat16;

constexpr int kAgMaxMBlk = 4096;
// The first 4096 * 17 words of the aux flag region belong to the fused tensor-parallel kernel; the
// all-gather's row-block flags follow.
constexpr uint64_t kAgFlagWordOffset = 4096ull * (kMaxRanks + 1);
static_assert((kAgFlagWordOffset + kAgMaxMBlk) * 4 <= kAuxFlagBytes, "aux flag region too small");

MSCCLPP_DEVICE_INLINE uint32_t* blockFlag(const DeviceComm& c, int rank, int mBlk) {
  return reinterpret_cast<uint32_t*>(c.peerBase[rank] + c.auxFlagsOff) + kAgFlagWordOffset + mBlk;
}

struct AgTmaps {
  CUtensorMap aLocal[8];
  CUtensorMap aFull[8];
  CUtensorMap b[8];
  CUtensorMap d[8];  // output, 64-column x 32-row boxes (epilogue bulk stores)
};

// Gate of the GEMM's TMA producer: own row blocks come from aLocal at once, the others from aFull when landed.
struct GatherGate {
  const DeviceComm* comm;
  const CUtensorMap* tmapLocal;
  int rank;
  int ownFirst, ownCount;  // this rank's row blocks
  uint32_t epoch;

  MSCCLPP_DEVICE_INLINE bool waitRowBlock(int mBlk) const {
    if (mBlk >= ownFirst && mBlk < ownFirst + ownCount) return true;
    const bool ok = waitGreaterEqualBackoff(blockFlag(*comm, rank, mBlk), epoch, comm->status, comm->timeoutNs, kDevTimeoutFlag, rank,
                                            8000 + mBlk, 0);
    // the rows were written through the async proxy by a copier and are read through it by the loads that follow
    ptx::fence_proxy_async();
    return ok;
  }
  MSCCLPP_DEVICE_INLINE const CUtensorMap* tmapA(int mBlk, const CUtensorMap* full, int& row) const {
    if (mBlk >= ownFirst && mBlk < ownFirst + ownCount) {
      row = (mBlk - ownFirst) * gemm::kBlockM;
      return tmapLocal;
    }
    row = mBlk * gemm::kBlockM;
    return full;
  }
};

// Activation in fp32 on the accumulator, then one tiled bulk store per staged 32 x 64 block.
template <int kAct>
struct StoreAct {
  static constexpr bool kNeedsTileBarrier = false;
  static constexpr bool kBulkStore = true;
  const CUtensorMap* tmapD;
  int M;
  MSCCLPP_DEVICE_INLINE static float convert(float x) {
    if constexpr (kAct == 1) {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    } else if constexpr (kAct == 2) {
      return x / (1.f + __expf(-x));
    } else {
      return x;
    }
  }
  MSCCLPP_DEVICE_INLINE void tileBegin(int, int, int) const {}
  MSCCLPP_DEVICE_INLINE void block(const uint8_t* stage, int row0, int col0, int lane, int /*b*/) const {
    if (lane == 0 && row0 < M) {
      ptx::tma_store_2d(tmapD, stage, col0, row0);
      ptx::bulk_commit();
    }
  }
  MSCCLPP_DEVICE_INLINE void tileDone(int, int, int) const {}
  MSCCLPP_DEVICE_INLINE void warpTileDone(int, int) const {}
  MSCCLPP_DEVICE_INLINE void warpDrain(int) const {}
  MSCCLPP_DEVICE_INLINE void auxWarp(int, int) const {}
};

// Gated activation (SwiGLU): the GEMM's N columns are gate/up features interleaved in groups of 32 (columns [64 b, 64 b +
// 32) gate features 32 b .., columns [64 b + 32, 64 b + 64) the matching up features); the output has N / 2 columns,
// out[:, 32 b + j] = silu(gate) * up, taken in fp32 on the accumulators. Rows leave with plain 64-byte-contiguous stores.
struct StoreGated {
  static constexpr bool kNeedsTileBarrier = false;
  static constexpr bool kBulkStore = false;
  static constexpr bool kGatedPairs = true;
  __nv_bfloat16* out;  // [M, N / 2]
  int M, halfN;
  MSCCLPP_DEVICE_INLINE static float convert(float x) { return x; }
  MSCCLPP_DEVICE_INLINE static float gatePair(float g, float u) { return g / (1.f + __expf(-g)) * u; }
  MSCCLPP_DEVICE_INLINE void tileBegin(int, int, int) const {}
  MSCCLPP_DEVICE_INLINE void block(const uint8_t* stage, int row0, int col0, int lane, int /*b*/) const {
    // four lanes per row (chunks 0-3), eight rows per step
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int r = 8 * i + (lane >> 2), ch = lane & 3;
      const int row = row0 + r;
      if (row < M) {
        *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * halfN + col0 / 2 + ch * 8) =
            *reinterpret_cast<const uint4*>(stage + gemm::stagedOffset(r, ch));
      }
    }
    __syncwarp();  // the staging buffer may be overwritten from here on
  }
  MSCCLPP_DEVICE_INLINE void tileDone(int, int, int) const {}
  MSCCLPP_DEVICE_INLINE void warpTileDone(int, int) const {}
  MSCCLPP_DEVICE_INLINE void warpDrain(int) const {}
  MSCCLPP_DEVICE_INLINE void auxWarp(int, int) const {}
};

constexpr uint32_t kPieceBytes = 32768;
constexpr int kRingStages = 6;  // 192 KiB of the CTA's dynamic shared memory

// One copier CTA. Thread 0 runs the copy pipeline; the block as a whole takes part in the two rank barriers.
MSCCLPP_DEVICE_INLINE void copierCta(const AgGemmArgs& a, int rank, uint32_t epoch, int copierIdx, int numCopiers, uint8_t* smemRaw) {
  const DeviceComm& c = a.comm;
  const int world = c.world;
  const int per = a.shape.M / gemm::kBlockM / world;  // row blocks per rank
  const uint64_t blockBytes = static_cast<uint64_t>(gemm::kBlockM) * a.shape.K * 2;
  const int piecesPerBlock = static_cast<int>(blockBytes / kPieceBytes);
  const uint64_t aLocalOff = reinterpret_cast<uint64_t>(a.aLocal) - c.peerBase[c.rank];
  const uint64_t aFullOff = reinterpret_cast<uint64_t>(a.aFull) - c.peerBase[c.rank];
  __shared__ __align__(8) uint64_t full[kRingStages];
  __shared__ int healthyS;
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 127) & ~uintptr_t(127));

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRingStages; s++) ptx::mbar_init(&full[s], 1);
    ptx::fence_mbar_init();
    healthyS = 1;
  }
  // every rank's aLocal is final once its kernel runs: meet the peers' copiers with my index
  const bool peersHere = rankBarrier(c, rank, 0, copierIdx, epoch);

  if (threadIdx.x == 0 && peersHere) {
    const int totalChunks = (world - 1) * per;
    int myChunks = 0;
    for (int idx = copierIdx; idx < totalChunks; idx += numCopiers) myChunks++;
    const int P = myChunks * piecesPerBlock;
    // piece p of mine -> source / destination address and the row block it belongs to
    auto locate = [&](int p, uint64_t& src, uint64_t& dst, int& mBlk) {
      const int chunk = copierIdx + (p / piecesPerBlock) * numCopiers;
      const int peer = (rank + 1 + chunk / per) % world;
      const int b = chunk % per;
      const uint64_t within = static_cast<uint64_t>(p % piecesPerBlock) * kPieceBytes;
      src = c.peerBase[peer] + aLocalOff + b * blockBytes + within;
      mBlk = peer * per + b;
      dst = c.peerBase[rank] + aFullOff + static_cast<uint64_t>(mBlk) * blockBytes + within;
    };
    auto issueLoad = [&](int p) {
      uint64_t src, dst;
      int mBlk;
      locate(p, src, dst, mBlk);
      const int stage = p % kRingStages;
      ptx::mbar_expect_tx(&full[stage], kPieceBytes);
      ptx::bulk_g2s(ring + static_cast<size_t>(stage) * kPieceBytes, reinterpret_cast<const void*>(src), kPieceBytes, &full[stage]);
    };
    auto publish = [&](int p) {  // piece p (the last of its row block) has been written
      uint64_t src, dst;
      int mBlk;
      locate(p, src, dst, mBlk);
      ptx::fence_proxy_async();
      __threadfence();  // GPU scope is enough: the flag and the rows are in this GPU's memory and read by its own GEMM CTAs
      ptx::st_relaxed_sys(blockFlag(c, rank, mBlk), epoch);
    };
    int issued = 0;
    for (; issued < kRingStages - 1 && issued < P; issued++) issueLoad(issued);
    bool ok = true;
    int i = 0;
    for (; i < P; i++) {
      const int stage = i % kRingStages;
      ok = mbarWait(&full[stage], (i / kRingStages) & 1u, c.status, c.timeoutNs, 500 + stage);
      if (!ok) break;
      uint64_t src, dst;
      int mBlk;
      locate(i, src, dst, mBlk);
      ptx::bulk_s2g(reinterpret_cast<void*>(dst), ring + static_cast<size_t>(stage) * kPieceBytes, kPieceBytes);
      ptx::bulk_commit();
      ptx::bulk_wait<1>();  // every store but the newest is complete: piece i-1 is in aFull
      if (i >= 1 && (i - 1) % piecesPerBlock == piecesPerBlock - 1) publish(i - 1);
      // the stage of piece i-1 (never used yet when i == 0) is free again
      if (issued < P) issueLoad(issued++);
    }
    ptx::bulk_wait<0>();
    if (ok && P > 0) publish(P - 1);
    if (!ok) {
      // drain the loads still in flight (bounded), so that nothing lands in shared memory after the CTA is gone
      for (int p = i; p < issued; p++) mbarWait(&full[p % kRingStages], (p / kRingStages) & 1u, nullptr, 2000000ull, 0);
      healthyS = 0;
    }
  }
  __syncthreads();
  // my pulls are done: peers may overwrite their aLocal after this
  if (peersHere && healthyS) rankBarrier(c, rank, 1, copierIdx, epoch);
}

template <int kBlockN, int kAct>
__global__ void __launch_bounds__(gemm::kNumThreads, 1)
    agGemmKernel(const __grid_constant__ AgTmaps maps, const __grid_constant__ AgGemmArgs a) {
  extern __shared__ uint8_t smemRaw[];
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const uint32_t epoch = launchEpoch(c, rank);
  if (static_cast<int>(blockIdx.x) < a.numGemmCtas) {
    const int per = a.shape.M / gemm::kBlockM / c.world;
    GatherGate gate{&c, &maps.aLocal[blockIdx.y], rank, rank * per, per, epoch};
    auto makeEpilogue = [&] {
      if constexpr (kAct == 3) {
        // D of (emulated) rank blockIdx.y: same heap offset as a.D
        const uint64_t dOff = reinterpret_cast<uint64_t>(a.D) - c.peerBase[c.rank];
        return StoreGated{reinterpret_cast<__nv_bfloat16*>(c.peerBase[rank] + dOff), a.shape.M, a.shape.N / 2};
      } else {
        return StoreAct<kAct>{&maps.d[blockIdx.y], a.shape.M};
      }
    };
    auto epi = makeEpilogue();
    gemm::Shape shape = a.shape;
    shape.mOrder = 2;
    if constexpr (kBlockN == 0) {
      shape.mOrderParam = rank * per / 2;  // the pair core orders 256-row blocks
      gemm::gemmCtaPair(&maps.aFull[blockIdx.y], &maps.b[blockIdx.y], shape, blockIdx.x / 2, a.numGemmCtas / 2, gate, epi, c.status,
                        c.timeoutNs, smemRaw);
    } else {
      shape.mOrderParam = rank * per;
      gemm::gemmCta<kBlockN>(&maps.aFull[blockIdx.y], &maps.b[blockIdx.y], shape, blockIdx.x, a.numGemmCtas, gate, epi, c.status,
                             c.timeoutNs, smemRaw);
    }
  } else {
    copierCta(a, rank, epoch, blockIdx.x - a.numGemmCtas, gridDim.x - a.numGemmCtas, smemRaw);
  }
  finishLaunch(c, rank, epoch);
}

template <int kBlockN>
struct SmemOf {
  static constexpr int kSmemBytes = gemm::Config<kBlockN>::kSmemBytes;
};
template <>
struct SmemOf<0> {
  static constexpr int kSmemBytes = gemm::Config2::kSmemBytes;
};

// kBlockN == 0 selects the two-SM GEMM core (256 x 256 tiles on CTA pairs, clusters of two CTAs).
template <int kBlockN, int kAct>
cudaError_t launchTyped(const AgTmaps& maps, const AgGemmArgs& args, int grid, cudaStream_t stream) {
  using Cfg = SmemOf<kBlockN>;
  static_assert(Cfg::kSmemBytes >= kRingStages * static_cast<int>(kPieceBytes) + 128, "ring must fit");
  auto kernel = agGemmKernel<kBlockN, kAct>;
  cudaError_t e = gemm::ensureDynamicSmem(reinterpret_cast<const void*>(kernel), Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 g(grid, args.emuRanks > 1 ? args.emuRanks : 1, 1);
  dim3 b(gemm::kNumThreads, 1, 1);
  // GEMM CTAs wait for copier CTAs of the same launch: co-residency is required, so the launch is cooperative
  AgTmaps m = maps;
  AgGemmArgs a = args;
  void* params[] = {&m, &a};
  if constexpr (kBlockN == 0) {
    return gemm::launchClusterPair(reinterpret_cast<const void*>(kernel), g, b, Cfg::kSmemBytes, params, true, stream);
  }
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), g, b, params, Cfg::kSmemBytes, stream);
}

template <int kBlockN>
cudaError_t launchAct(const AgTmaps& maps, const AgGemmArgs& args, int grid, cudaStream_t stream) {
  switch (args.activation) {
    case 0:
      return launchTyped<kBlockN, 0>(maps, args, grid, stream);
    case 1:
      return launchTyped<kBlockN, 1>(maps, args, grid, stream);
    case 2:
      return launchTyped<kBlockN, 2>(maps, args, grid, stream);
    case 3:
      return launchTyped<kBlockN, 3>(maps, args, grid, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launchAllGatherGemm(const AgGemmArgs& argsIn, const void* const* B, int numCopiers, cudaStream_t stream) {
  AgGemmArgs args = argsIn;
  const int M = args.shape.M, N = args.shape.N, K = args.shape.K;
  const int world = args.comm.world;
  if (M <= 0 || world < 1 || world > 8 || M % (world * gemm::kBlockM) != 0) return cudaErrorInvalidValue;
  const bool twoSm = args.blockN == 0;  // block_n 0 = 256 x 256 tiles on SM pairs
  const int tileN = twoSm ? gemm::Config2::kBlockN : args.blockN;
  if (N % tileN != 0 || K % 128 != 0) return cudaErrorInvalidValue;
  if (twoSm && M % (world * gemm::Config2::kPairM) != 0) return cudaErrorInvalidValue;
  if ((static_cast<uint64_t>(gemm::kBlockM) * K * 2) % kPieceBytes != 0) return cudaErrorInvalidValue;
  const int numMBlk = M / gemm::kBlockM;
  if (numMBlk > kAgMaxMBlk) return cudaErrorInvalidValue;
  // the copy ring lives in the GEMM's dynamic shared memory: only the two larger tile configurations have room
  if (args.blockN != 256 && args.blockN != 128 && !twoSm) return cudaErrorInvalidValue;
  const int emu = args.emuRanks > 1 ? args.emuRanks : 1;
  if (emu > 8 || (emu > 1 && emu != world)) return cudaErrorInvalidValue;
  args.shape.aBoxRows = gemm::kBlockM;
  args.shape.rowMajorTiles = 1;
  const uint64_t base = args.comm.peerBase[args.comm.rank];
  const uint64_t aLocalOff = reinterpret_cast<uint64_t>(args.aLocal) - base;
  const uint64_t aFullOff = reinterpret_cast<uint64_t>(args.aFull) - base;
  const uint64_t dOff = reinterpret_cast<uint64_t>(args.D) - base;
  AgTmaps maps;
  for (int e = 0; e < emu; e++) {
    const uint64_t heap = emu > 1 ? args.comm.peerBase[e] : base;
    cudaError_t err = gemm::makeTensorMapBf16(&maps.aLocal[e], reinterpret_cast<const void*>(heap + aLocalOff), M / world, K,
                                              static_cast<uint64_t>(K) * 2, gemm::kBlockM);
    if (err != cudaSuccess) return err;
    err = gemm::makeTensorMapBf16(&maps.aFull[e], reinterpret_cast<const void*>(heap + aFullOff), M, K, static_cast<uint64_t>(K) * 2,
                                  gemm::kBlockM);
    if (err != cudaSuccess) return err;
    err = gemm::makeTensorMapBf16(&maps.b[e], B[e], N, K, static_cast<uint64_t>(K) * 2, twoSm ? tileN / 2 : tileN);
    if (err != cudaSuccess) return err;
    const int dCols = args.activation == 3 ? N / 2 : N;  // (the gated epilogue stores without this map)
    err = gemm::makeTensorMapBf16(&maps.d[e], reinterpret_cast<const void*>(heap + dOff), M, dCols, static_cast<uint64_t>(dCols) * 2, 32);
    if (err != cudaSuccess) return err;
  }
  const int tiles = numMBlk * (N / tileN);
  const int sms = gemm::smCount() / emu;
  if (numCopiers <= 0) numCopiers = world == 1 ? 1 : (sms >= 64 ? 12 : 2);
  if (numCopiers > kBarrierSlots) numCopiers = kBarrierSlots;
  int gemmCtas = args.numGemmCtas > 0 ? args.numGemmCtas : sms - numCopiers;
  if (gemmCtas > tiles) gemmCtas = tiles;
  if (gemmCtas < 1) gemmCtas = 1;
  if (twoSm) {
    gemmCtas &= ~1;
    if (gemmCtas < 2) gemmCtas = 2;
    numCopiers = (numCopiers + 1) & ~1;
  }
  args.numGemmCtas = gemmCtas;
  const int grid = gemmCtas + numCopiers;
  if (twoSm) return launchAct<0>(maps, args, grid, stream);
  if (args.blockN == 256) return launchAct<256>(maps, args, grid, stream);
  return launchAct<128>(maps, args, grid, stream);
}

}  // namespace mscclpp
