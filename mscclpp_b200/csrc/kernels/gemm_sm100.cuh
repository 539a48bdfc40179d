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
//   * Epilogue  - each epilogue warp converts a 32-row x 64-column block of the accumulator to bf16 and
//                 writes it into its own 4 KB of shared memory in the 128-byte-swizzled layout of a TMA
//                 box; Epilogue::block() then moves it out with ONE cp.async.bulk.tensor store, or re-reads
//                 it with a row-contiguous lane mapping (stagedRead) so that every global load and store
//                 of a fused epilogue (residual add, partial products for a collective) covers whole
//                 128-byte lines. tileDone() follows once all epilogue warps have stored their part; there
//                 a fused kernel signals consumers (reduce-scatter / allreduce owners);
//   * aux CTAs  - blocks with blockIdx.x >= number of GEMM CTAs run a caller-supplied role
//                 (reducer, copier) inside the same launch.
// Every wait is bounded; on expiry the kernel records a DeviceStatus, drains its own TMA copies,
// frees its TMEM and returns.
#pragma once

#include <type_traits>
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
constexpr int kStagingBytesPerWarp = 32 * 128;  // 32 rows x 64 bf16 columns
constexpr int kEpilogueStagingBytes = kNumEpilogueWarps * kStagingBytesPerWarp;

template <int kBlockN>
struct Config {
  static_assert(kBlockN == 64 || kBlockN == 128 || kBlockN == 256, "unsupported N tile");
  static constexpr int kStageABytes = kBlockM * kBlockK * 2;
  static constexpr int kStageBBytes = kBlockN * kBlockK * 2;
  static constexpr int kStageBytes = kStageABytes + kStageBBytes;
  static constexpr int kStages = kBlockN == 256 ? 4 : (kBlockN == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * kBlockN;  // two accumulator buffers (power of two >= 32)
  static constexpr int kBarrierBytes = 256;
  // epilogue warps that take part: every warp owns 32 rows (its TMEM lane quarter) x a multiple of 64 columns
  static constexpr int kEpiWarps = kBlockN >= 128 ? kNumEpilogueWarps : 4;
  static constexpr int kColsPerWarp = kBlockN / (kEpiWarps / 4);
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpilogueStagingBytes + kBarrierBytes + 1024;  // +1024: manual alignment
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
  } else if (s.mOrder == 3) {
    // bands of mOrderParam row blocks, walked row-block-first inside a band: the tiles that run at the same time cover
    // a near-square region, so each wave re-reads a band of A and a few column panels of B from L2 instead of all of A
    const int g = s.mOrderParam;
    const int perBand = g * numNBlk;
    const int band = tile / perBand;
    const int first = band * g;
    const int rows = numMBlk - first < g ? numMBlk - first : g;  // the last band may be shorter
    const int t = tile - band * perBand;
    mBlk = first + t % rows;
    nBlk = t / rows;
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

// ---- epilogue staging: a warp's 32 x 64 bf16 block in shared memory, laid out like a SWIZZLE_128B TMA box
// (row r at byte r * 128, its 16-byte chunk c at position c ^ (r & 7)); the buffer is 1024-byte aligned.
MSCCLPP_DEVICE_INLINE uint32_t stagedOffset(int r, int c) { return static_cast<uint32_t>(r * 128 + ((c ^ (r & 7)) << 4)); }
// Row-contiguous view for fused epilogues: in step i (0..7) lane l holds chunk (l & 7) of row 4 * i + (l >> 3), so a
// warp-wide global access built on it touches four complete 128-byte lines.
MSCCLPP_DEVICE_INLINE int stagedRow(int i, int lane) { return 4 * i + (lane >> 3); }
MSCCLPP_DEVICE_INLINE int stagedCol(int lane) { return (lane & 7) * 8; }
MSCCLPP_DEVICE_INLINE uint4 stagedRead(const uint8_t* stage, int i, int lane) {
  return *reinterpret_cast<const uint4*>(stage + stagedOffset(stagedRow(i, lane), lane & 7));
}

struct SharedState {
  uint64_t* full;       // [stages] TMA -> MMA
  uint64_t* empty;      // [stages] MMA -> TMA
  uint64_t* tmemFull;   // [2] MMA -> epilogue
  uint64_t* tmemEmpty;  // [2] epilogue -> MMA
  uint32_t* tmemBase;
  volatile uint32_t* abortFlag;
  volatile uint32_t* epiArrivals;  // epilogue warps that finished storing, summed over the tiles so far
};

// Columns [8k, 8k+8) of a thread's 32 accumulator values as packed bf16.
template <typename Epilogue>
MSCCLPP_DEVICE_INLINE uint4 packChunk(const uint32_t (&v)[32], int k) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    __nv_bfloat162 h = __floats2bfloat162_rn(Epilogue::convert(__uint_as_float(v[8 * k + 2 * j])),
                                             Epilogue::convert(__uint_as_float(v[8 * k + 2 * j + 1])));
    w[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Epilogues that combine the two 32-column halves of every 64-column block into 32 output columns (gated activations: the
// weight rows are interleaved so that columns [0, 32) of a block are "gate" features and [32, 64) the matching "up"
// features) say so with `static constexpr bool kGatedPairs = true` and a `static float gatePair(float gate, float up)`.
// Only chunks 0-3 of a staged row then carry data.
template <typename E, typename = void>
struct IsGatedEpilogue : std::false_type {};
template <typename E>
struct IsGatedEpilogue<E, std::void_t<decltype(E::kGatedPairs)>> : std::bool_constant<E::kGatedPairs> {};

// One epilogue warp, one tile: `taddr` is the TMEM address of the warp's lane quarter at its first column,
// (row0, col0) the global coordinates of that corner. Calls arriveEmpty() as soon as the warp's last accumulator
// read has completed, i.e. before the last block is written out.
template <int kColsPerWarp, typename Epilogue, typename ArriveEmpty>
MSCCLPP_DEVICE_INLINE void stagedEpilogueTile(Epilogue& epi, uint32_t taddr, uint8_t* stage, int row0, int col0, int lane,
                                              ArriveEmpty&& arriveEmpty, int probe = 0) {
  static_assert(kColsPerWarp % 64 == 0, "an epilogue warp works in blocks of 64 columns");
  constexpr int kBlocks = kColsPerWarp / 64;
  const bool drop = (probe & 4) != 0;
  if (probe & 8) {  // diagnostics: hand the accumulator back unread
    ptx::tcgen05_fence_before_sync();
    __syncwarp();
    if (lane == 0) arriveEmpty();
    return;
  }
#pragma unroll
  for (int b = 0; b < kBlocks; b++) {
    uint32_t v0[32], v1[32];
    ptx::tmem_ld_32x32b_x32(taddr + b * 64, v0);
    ptx::tmem_ld_32x32b_x32(taddr + b * 64 + 32, v1);
    ptx::tmem_ld_wait();
    if (b == kBlocks - 1) {
      ptx::tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) arriveEmpty();
    }
    // the buffer is free once the bulk store of the previous block has read it (or block() has ended)
    if constexpr (Epilogue::kBulkStore) {
      if (lane == 0) ptx::bulk_wait_read<0>();
    }
    __syncwarp();
    if constexpr (IsGatedEpilogue<Epilogue>::value) {
#pragma unroll
      for (int i = 0; i < 32; i++) v0[i] = __float_as_uint(Epilogue::gatePair(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
#pragma unroll
      for (int c = 0; c < 4; c++) *reinterpret_cast<uint4*>(stage + stagedOffset(lane, c)) = packChunk<Epilogue>(v0, c);
    } else {
#pragma unroll
      for (int c = 0; c < 4; c++) {
        *reinterpret_cast<uint4*>(stage + stagedOffset(lane, c)) = packChunk<Epilogue>(v0, c);
        *reinterpret_cast<uint4*>(stage + stagedOffset(lane, c + 4)) = packChunk<Epilogue>(v1, c);
      }
    }
    if constexpr (Epilogue::kBulkStore) ptx::fence_proxy_async_smem();
    __syncwarp();
    if (!drop) epi.block(stage, row0, col0 + b * 64, lane, b);
  }
}

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
  uint8_t* staging = smem + Cfg::kStages * Cfg::kStageBytes;  // 1024-byte aligned: every stage is a multiple of 1024 bytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kEpilogueStagingBytes);
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
  unsigned long long* tl = shape.stamps != nullptr ? shape.stamps + static_cast<size_t>(blockIdx.x) * kStampWords : nullptr;
  if (tl != nullptr && threadIdx.x == 0) tl[0] = ptx::globaltimer();

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; s++) {
      ptx::mbar_init(&st.full[s], 1);
      ptx::mbar_init(&st.empty[s], 1);
    }
    for (int s = 0; s < 2; s++) {
      ptx::mbar_init(&st.tmemFull[s], 1);
      ptx::mbar_init(&st.tmemEmpty[s], Cfg::kEpiWarps);  // one arrival per epilogue warp that takes part
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
          if (tl != nullptr) {
            const unsigned long long t0 = ptx::globaltimer();
            ok = mbarWaitFast(&st.empty[stage], phase ^ 1u, status, budgetNs, 100 + stage, st.abortFlag);
            tl[8] += ptx::globaltimer() - t0;
          } else {
            ok = mbarWaitFast(&st.empty[stage], phase ^ 1u, status, budgetNs, 100 + stage, st.abortFlag);
          }
          if (!ok) break;
          uint8_t* sa = tiles + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kStageABytes;
          if (shape.probe & 1) {
            ptx::mbar_arrive(&st.full[stage]);
          } else {
            ptx::mbar_expect_tx(&st.full[stage], shape.aBoxRows * kBlockK * 2 + Cfg::kStageBBytes);
            ptx::tma_load_2d(sa, tmapARows, kb * kBlockK, aRow, &st.full[stage]);
            ptx::tma_load_2d(sb, tmapB, kb * kBlockK, nBlk * kBlockN, &st.full[stage]);
          }
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
      // The issue loop is ONE thread feeding the tensor core: every instruction in it is on the critical path of the
      // whole SM. Descriptors are formed once and stepped by adds; the common case of each wait is one instruction.
      const uint64_t descA0 = makeSmemDesc(ptx::smem_u32(tiles));
      const uint64_t descB0 = makeSmemDesc(ptx::smem_u32(tiles) + Cfg::kStageABytes);
      constexpr uint64_t kStageStep = Cfg::kStageBytes >> 4;  // a stage, in the descriptor's 16-byte address units
      const bool issue = (shape.probe & 2) == 0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = ctaIdx; tile < numTiles && ok; tile += numCtas, it++) {
        const int acc = it & 1;
        const uint32_t accPhase = (it >> 1) & 1;
        if (tl != nullptr) {
          const unsigned long long t0 = ptx::globaltimer();
          ok = mbarWaitFast(&st.tmemEmpty[acc], accPhase ^ 1u, status, budgetNs, 200 + acc, st.abortFlag);
          tl[2] += ptx::globaltimer() - t0;
        } else {
          ok = mbarWaitFast(&st.tmemEmpty[acc], accPhase ^ 1u, status, budgetNs, 200 + acc, st.abortFlag);
        }
        if (!ok) break;
        ptx::tcgen05_fence_after_sync();
        const uint32_t tmemD = tmemBase + acc * kBlockN;
        for (int kb = 0; kb < numKBlk; kb++) {
          if (tl != nullptr) {
            const unsigned long long t0 = ptx::globaltimer();
            ok = mbarWaitFast(&st.full[stage], phase, status, budgetNs, 300 + stage, st.abortFlag);
            tl[3] += ptx::globaltimer() - t0;
          } else {
            ok = mbarWaitFast(&st.full[stage], phase, status, budgetNs, 300 + stage, st.abortFlag);
          }
          if (!ok) break;
          ptx::tcgen05_fence_after_sync();
          const uint64_t descA = descA0 + stage * kStageStep;
          const uint64_t descB = descB0 + stage * kStageStep;
          if (issue) {
            // advancing K by 16 elements = 32 bytes inside the 128-byte swizzle row: +2 in the (>>4) address field
            ptx::tcgen05_mma_f16(tmemD, descA, descB, idesc, kb != 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < kBlockK / kUmmaK; k++) ptx::tcgen05_mma_f16_acc(tmemD, descA + 2 * k, descB + 2 * k, idesc);
          }
          ptx::tcgen05_commit(&st.empty[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) ptx::tcgen05_commit(&st.tmemFull[acc]);
      }
      if (tl != nullptr) tl[1] = ptx::globaltimer();
      if (!ok) *st.abortFlag = 1;
    }
  } else if (warp < 2 + Cfg::kEpiWarps) {
    // ===================================================== epilogue (lane quarter x column part per warp)
    const int quarter = warp & 3;  // a warp may only touch TMEM lanes [32*(warpid%4), +32)
    const int part = (warp - 2) >> 2;
    uint8_t* stage = staging + (warp - 2) * kStagingBytesPerWarp;
    bool ok = true;
    int it = 0;
    for (int tile = ctaIdx; tile < numTiles && ok; tile += numCtas, it++) {
      int mBlk, nBlk;
      tileCoord(shape, tile, numMBlk, numNBlk, mBlk, nBlk);
      const int acc = it & 1;
      const uint32_t accPhase = (it >> 1) & 1;
      const int row0 = mBlk * kBlockM + quarter * 32;
      const int col0 = nBlk * kBlockN + part * Cfg::kColsPerWarp;
      // lets the epilogue put loads it will need (a residual, a bias) in flight while the MMAs of this tile still run
      epi.tileBegin(row0, col0, lane);
      const bool stampIt = tl != nullptr && warp == 2 && lane == 0;
      unsigned long long tw0 = 0;
      if (stampIt) tw0 = ptx::globaltimer();
      ok = mbarWait(&st.tmemFull[acc], accPhase, status, budgetNs, 400 + acc);
      ok = __all_sync(0xffffffffu, ok) && (*st.abortFlag == 0);
      if (!ok) break;
      if (stampIt) {
        const unsigned long long now = ptx::globaltimer();
        tl[5] += now - tw0;
        tw0 = now;
      }
      ptx::tcgen05_fence_after_sync();
      const uint32_t taddr = tmemBase + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kBlockN + part * Cfg::kColsPerWarp;
      // the accumulator buffer can be overwritten by the MMA warp as soon as every warp has read its part
      stagedEpilogueTile<Cfg::kColsPerWarp>(epi, taddr, stage, row0, col0, lane, [&] { ptx::mbar_arrive(&st.tmemEmpty[acc]); }, shape.probe);
      if (stampIt) {
        const unsigned long long now = ptx::globaltimer();
        tl[6] += now - tw0;
        tl[4] = now;
      }
      if constexpr (Epilogue::kNeedsTileBarrier) {
        // All epilogue warps have issued their stores -> let the fused kernel publish the tile. The
        // meeting point is a counter with a bounded wait (not bar.sync): if one warp gave up on the
        // accumulator barrier above, the others must not wait for it forever.
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          atomicAdd(const_cast<uint32_t*>(st.epiArrivals), 1u);
          const uint32_t target = static_cast<uint32_t>(it + 1) * Cfg::kEpiWarps;
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
      // per-warp hook: this warp's part of the tile is stored (fused epilogues count it and may take on follow-up work)
      epi.warpTileDone(mBlk, lane);
    }
    if (ok) epi.warpDrain(lane);  // follow-up work that is left once the warp has no tile of its own any more
    if (tl != nullptr && warp == 2 && lane == 0) tl[7] = ptx::globaltimer();
    if (!ok && lane == 0) *st.abortFlag = 1;
    // bulk stores of this warp still read its staging buffer: the CTA must not end before they have
    if constexpr (Epilogue::kBulkStore) {
      if (lane == 0) ptx::bulk_wait<0>();
    }
  } else if (warp >= 2 + kNumEpilogueWarps) {
    // warps beyond the ten of the GEMM roles (a kernel may launch more threads): follow-up work of a fused epilogue that
    // must stay off the epilogue warps' critical path
    epi.auxWarp(warp - (2 + kNumEpilogueWarps), lane);
  }

  // ---- teardown: everybody meets, then the allocating warp frees TMEM
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_sync();
  if (warp == 1) ptx::tmem_dealloc(tmemBase, Cfg::kTmemCols);
}

// Plain epilogue: every staged 32 x 64 block leaves with one tiled bulk store (rows beyond M are clipped by the
// tensor map, whose box is 64 columns x 32 rows with the 128-byte swizzle of the staging layout).
struct StoreBf16 {
  static constexpr bool kNeedsTileBarrier = false;
  static constexpr bool kBulkStore = true;
  const CUtensorMap* tmapD;
  int M;
  MSCCLPP_DEVICE_INLINE static float convert(float x) { return x; }
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

}  // namespace gemm
}  // namespace mscclpp
