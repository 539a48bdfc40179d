// Warp-specialised persistent bf16 GEMM core for sm_100a: TMA (cp.async.bulk.tensor, no cluster
// multicast) stages 128B-swizzled A/B tiles in shared memory, ONE thread issues tcgen05.mma with
// the fp32 accumulator in tensor memory (TMEM), and four epilogue warps read the accumulator back
// with tcgen05.ld while the next tile's MMAs already run on the second TMEM buffer.
//
//   D[M,N] = A[M,K] * B[N,K]^T        A, B bf16 K-major (row-major [rows, K]); fp32 accumulate
//
// The reference library has no GEMM (it is a pure communication library); this core exists so that
// the tensor-parallel collectives can be fused with the matmul that produces or consumes them.
// Hooks for that fusion:
//   * AGate     - called by the TMA producer before it loads the A tiles of a row block, so an
//                 all-gather that is still in flight can be waited for block by block;
//   * Epilogue  - receives each 32-column slice of the accumulator (one row per thread) and a
//                 tileDone() call after all 128 epilogue threads have stored their part, where a
//                 fused kernel signals consumers (reduce-scatter / allreduce owners);
//   * aux CTAs  - blocks with blockIdx.x >= number of GEMM CTAs run a caller-supplied role
//                 (reducer, copier) inside the same launch.
// Every wait is bounded; on expiry the kernel records a DeviceStatus, drains its own TMA copies,
// frees its TMEM and returns.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mscclpp/device/ptx.cuh>
#include <mscclpp/poll_device.hpp>

#include "gemm.cuh"

namespace mscclpp {
namespace gemm {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;           // K of one tcgen05.mma for 16-bit inputs
constexpr int kNumEpilogueWarps = 8;  // two warps per TMEM lane quarter, each takes half of the tile's columns
constexpr int kNumEpilogueThreads = kNumEpilogueWarps * 32;
constexpr int kNumThreads = 64 + kNumEpilogueThreads;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-9: epilogue

template <int kBlockN>
struct Config {
  static_assert(kBlockN == 64 || kBlockN == 128 || kBlockN == 256, "unsupported N tile");
  static constexpr int kStageABytes = kBlockM * kBlockK * 2;
  static constexpr int kStageBBytes = kBlockN * kBlockK * 2;
  static constexpr int kStageBytes = kStageABytes + kStageBBytes;
  static constexpr int kStages = kBlockN == 256 ? 4 : (kBlockN == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * kBlockN;  // two accumulator buffers (power of two >= 32)
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;  // +1024: manual alignment
};

MSCCLPP_DEVICE_INLINE void tileCoord(const Shape& s, int tile, int numMBlk, int numNBlk, int& mBlk, int& nBlk) {
  if (s.rowMajorTiles) {
    mBlk = tile / numNBlk;
    nBlk = tile % numNBlk;
  } else {
    mBlk = tile % numMBlk;
    nBlk = tile / numMBlk;
  }
  if (s.mOrder == 1) {
    const int per = numMBlk / s.mOrderParam;
    mBlk = (mBlk % s.mOrderParam) * per + mBlk / s.mOrderParam;
  } else if (s.mOrder == 2) {
    mBlk += s.mOrderParam;
    if (mBlk >= numMBlk) mBlk -= numMBlk;
  }
}

// 64-bit shared-memory matrix descriptor: K-major operand, 128-byte swizzle, tile base 1024B-aligned.
// bits [0,14) start address >> 4; [16,30) leading byte offset >> 4 (unused for swizzled K-major, 1);
// [32,46) stride byte offset >> 4 (8 rows x 128 B = 1024 B between 8-row groups); [46,48) version = 1
// on sm_100; [61,64) layout = 2 (SWIZZLE_128B).
MSCCLPP_DEVICE_INLINE uint64_t makeSmemDesc(uint32_t smemAddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smemAddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// 32-bit instruction descriptor for kind::f16: bf16 x bf16 -> fp32, both operands K-major.
// [4,6) D format (1 = f32); [7,10) A format (1 = bf16); [10,13) B format (1 = bf16);
// bit 15 / 16 A / B major (0 = K); [17,23) N >> 3; [24,29) M >> 4.
template <int kBlockN>
MSCCLPP_HOST_DEVICE_INLINE constexpr uint32_t makeInstrDesc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kBlockN >> 3) << 17) |
         (static_cast<uint32_t>(kBlockM >> 4) << 24);
}

struct NoGate {
  MSCCLPP_DEVICE_INLINE bool waitRowBlock(int /*mBlk*/) const { return true; }
  // Tensor map and first row (in that map) of row block mBlk's A tiles.
  MSCCLPP_DEVICE_INLINE const CUtensorMap* tmapA(int mBlk, const CUtensorMap* dflt, int& row) const {
    row = mBlk * kBlockM;
    return dflt;
  }
};

struct SharedState {
  uint64_t* full;       // [stages] TMA -> MMA
  uint64_t* empty;      // [stages] MMA -> TMA
  uint64_t* tmemFull;   // [2] MMA -> epilogue
  uint64_t* tmemEmpty;  // [2] epilogue -> MMA
  uint32_t* tmemBase;
  volatile uint32_t* abortFlag;
  volatile uint32_t* epiArrivals;  // epilogue warps that finished storing, summed over the tiles so far
};

// Body of a GEMM CTA. All 192 threads call it. `ctaIdx`/`numCtas` index the persistent tile loop.
template <int kBlockN, typename AGate, typename Epilogue>
MSCCLPP_DEVICE_INLINE void gemmCta(const CUtensorMap* tmapA, const CUtensorMap* tmapB, Shape shape, int ctaIdx,
                                   int numCtas, AGate& gate, Epilogue& epi, DeviceStatus* status, uint64_t budgetNs,
                                   uint8_t* smemRaw) {
  using Cfg = Config<kBlockN>;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- carve shared memory (tiles need 1024-byte alignment for the 128B swizzle)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  SharedState st;
  st.full = bars;
  st.empty = bars + Cfg::kStages;
  st.tmemFull = bars + 2 * Cfg::kStages;
  st.tmemEmpty = bars + 2 * Cfg::kStages + 2;
  st.tmemBase = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::kStages + 4);
  st.abortFlag = reinterpret_cast<volatile uint32_t*>(st.tmemBase + 1);
  st.epiArrivals = reinterpret_cast<volatile uint32_t*>(st.tmemBase + 2);

  const int numMBlk = (shape.M + kBlockM - 1) / kBlockM;
  const int numNBlk = shape.N / kBlockN;
  const int numTiles = numMBlk * numNBlk;
  const int numKBlk = shape.K / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; s++) {
      ptx::mbar_init(&st.full[s], 1);
      ptx::mbar_init(&st.empty[s], 1);
    }
    for (int s = 0; s < 2; s++) {
      ptx::mbar_init(&st.tmemFull[s], 1);
      ptx::mbar_init(&st.tmemEmpty[s], kNumEpilogueWarps);  // one arrival per epilogue warp
    }
    *st.abortFlag = 0;
    *st.epiArrivals = 0;
    ptx::fence_mbar_init();
    ptx::tma_prefetch_desc(tmapA);
    ptx::tma_prefetch_desc(tmapB);
  }
  if (warp == 1) {
    ptx::tmem_alloc(st.tmemBase, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_sync();
  const uint32_t tmemBase = *st.tmemBase;

  if (warp == 0) {
    // ===================================================== TMA producer (one thread)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0;        // bit s: stage s has a load in flight that nobody has waited for yet
      uint32_t armedParity = 0;  // parity those loads complete
      bool ok = true;
      for (int tile = ctaIdx; tile < numTiles && ok; tile += numCtas) {
        int mBlk, nBlk;
        tileCoord(shape, tile, numMBlk, numNBlk, mBlk, nBlk);
        ok = gate.waitRowBlock(mBlk);
        int aRow;
        const CUtensorMap* tmapARows = gate.tmapA(mBlk, tmapA, aRow);
        for (int kb = 0; kb < numKBlk && ok; kb++) {
          ok = mbarWait(&st.empty[stage], phase ^ 1u, status, budgetNs, 100 + stage);
          if (!ok || *st.abortFlag) {
            ok = false;
            break;
          }
          uint8_t* sa = tiles + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kStageABytes;
          ptx::mbar_expect_tx(&st.full[stage], shape.aBoxRows * kBlockK * 2 + Cfg::kStageBBytes);
          ptx::tma_load_2d(sa, tmapARows, kb * kBlockK, aRow, &st.full[stage]);
          ptx::tma_load_2d(sb, tmapB, kb * kBlockK, nBlk * kBlockN, &st.full[stage]);
          armed |= 1u << stage;
          armedParity = (armedParity & ~(1u << stage)) | (phase << stage);
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        *st.abortFlag = 1;
        // drain: wait (bounded) until every load this thread issued has landed
        for (int s = 0; s < Cfg::kStages; s++) {
          if (armed & (1u << s)) mbarWait(&st.full[s], (armedParity >> s) & 1u, nullptr, 2000000ull, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ===================================================== MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc = makeInstrDesc<kBlockN>();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = ctaIdx; tile < numTiles && ok; tile += numCtas, it++) {
        const int acc = it & 1;
        const uint32_t accPhase = (it >> 1) & 1;
        ok = mbarWait(&st.tmemEmpty[acc], accPhase ^ 1u, status, budgetNs, 200 + acc);
        if (!ok || *st.abortFlag) {
          ok = false;
          break;
        }
        ptx::tcgen05_fence_after_sync();
        const uint32_t tmemD = tmemBase + acc * kBlockN;
        for (int kb = 0; kb < numKBlk; kb++) {
          ok = mbarWait(&st.full[stage], phase, status, budgetNs, 300 + stage);
          if (!ok || *st.abortFlag) {
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after_sync();
          const uint32_t sa = ptx::smem_u32(tiles + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kStageABytes;
          const uint64_t descA = makeSmemDesc(sa);
          const uint64_t descB = makeSmemDesc(sb);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; k++) {
            // advancing K by 16 elements = 32 bytes inside the 128-byte swizzle row: +2 in the (>>4) address field
            ptx::tcgen05_mma_f16(tmemD, descA + 2 * k, descB + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ptx::tcgen05_commit(&st.empty[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) ptx::tcgen05_commit(&st.tmemFull[acc]);
      }
      if (!ok) *st.abortFlag = 1;
    }
  } else if (warp < 2 + kNumEpilogueWarps) {
    // ===================================================== epilogue (8 warps: lane quarter x column half)
    const int quarter = warp & 3;  // a warp may only touch TMEM lanes [32*(warpid%4), +32)
    const int half = (warp - 2) >> 2;
    constexpr int kChunksPerWarp = kBlockN / 32 / (kNumEpilogueWarps / 4);
    bool ok = true;
    int it = 0;
    for (int tile = ctaIdx; tile < numTiles && ok; tile += numCtas, it++) {
      int mBlk, nBlk;
      tileCoord(shape, tile, numMBlk, numNBlk, mBlk, nBlk);
      const int acc = it & 1;
      const uint32_t accPhase = (it >> 1) & 1;
      const int row = mBlk * kBlockM + quarter * 32 + lane;
      // lets the epilogue put loads it will need (a residual, a bias) in flight while the MMAs of this tile still run
      epi.tileBegin(row, nBlk * kBlockN + half * kChunksPerWarp * 32);
      ok = mbarWait(&st.tmemFull[acc], accPhase, status, budgetNs, 400 + acc);
      ok = __all_sync(0xffffffffu, ok) && (*st.abortFlag == 0);
      if (!ok) break;
      ptx::tcgen05_fence_after_sync();
      const uint32_t taddr = tmemBase + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kBlockN;
#pragma unroll
      for (int i = 0; i < kChunksPerWarp; i++) {
        const int c = half * kChunksPerWarp + i;
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(taddr + c * 32, v);
        ptx::tmem_ld_wait();
        epi.store(row, nBlk * kBlockN + c * 32, v, i);  // i: index of the slice within this warp's part of the tile
      }
      // accumulator buffer can be overwritten by the MMA warp from here on
      ptx::tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&st.tmemEmpty[acc]);
      if constexpr (Epilogue::kNeedsTileBarrier) {
        // All epilogue warps have issued their stores -> let the fused kernel publish the tile. The
        // meeting point is a counter with a bounded wait (not bar.sync): if one warp gave up on the
        // accumulator barrier above, the others must not wait for it forever.
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          atomicAdd(const_cast<uint32_t*>(st.epiArrivals), 1u);
          const uint32_t target = static_cast<uint32_t>(it + 1) * kNumEpilogueWarps;
          SpinGuard g(status, budgetNs);
          while (static_cast<int32_t>(*st.epiArrivals - target) < 0) {
            if (*st.abortFlag || !g.keepSpinning()) {
              *st.abortFlag = 1;
              break;
            }
          }
          __threadfence_block();
        }
        __syncwarp();
        if (*st.abortFlag) {
          ok = false;
          break;
        }
        if (warp == 2) epi.tileDone(mBlk, nBlk, lane);
      }
    }
    if (!ok && lane == 0) *st.abortFlag = 1;
  }

  // ---- teardown: everybody meets, then the allocating warp frees TMEM
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_sync();
  if (warp == 1) ptx::tmem_dealloc(tmemBase, Cfg::kTmemCols);
}

// Plain epilogue: convert to bf16 and store row-major D[M, ldd].
struct StoreBf16 {
  static constexpr bool kNeedsTileBarrier = false;
  __nv_bfloat16* D;
  int ldd;
  int M;
  MSCCLPP_DEVICE_INLINE void tileBegin(int, int) const {}
  MSCCLPP_DEVICE_INLINE void store(int row, int col, const uint32_t (&v)[32], int /*slice*/ = 0) const {
    if (row >= M) return;
    uint4* dst = reinterpret_cast<uint4*>(D + static_cast<size_t>(row) * ldd + col);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  MSCCLPP_DEVICE_INLINE void tileDone(int, int, int) const {}
};

}  // namespace gemm
}  // namespace mscclpp
