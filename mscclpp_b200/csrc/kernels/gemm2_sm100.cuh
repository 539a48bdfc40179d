// Two-SM variant of the persistent bf16 GEMM core: a cluster of two CTAs works on one 256 x 256 tile with
// tcgen05.mma.cta_group::2. Each CTA stages its own 128 rows of A and 128 of the tile's 256 B rows (so a k-block
// costs 32 KB of shared-memory fill per SM instead of 48 KB, and each MMA reads half of B from the peer SM), holds
// the accumulator rows of its A half in its own TMEM and runs its own epilogue. The leader CTA (cluster rank 0)
// issues every MMA; completion is signalled to both CTAs with tcgen05.commit ... multicast::cluster.
//
//   D[M,N] = A[M,K] * B[N,K]^T        A, B bf16 K-major; fp32 accumulate; N % 256 == 0; K % 64 == 0
//
// Loads never use cluster multicast: both CTAs fetch their halves with plain tiled TMA loads whose byte counts
// land on the leader's mbarrier. Same hooks as the one-SM core (AGate, Epilogue); row blocks handed to them are
// 128-row blocks (block = 2 * pairRowBlock + cluster rank). Every wait is bounded.
#pragma once

#include "gemm_sm100.cuh"

namespace mscclpp {
namespace gemm {

struct Config2 {
  static constexpr int kBlockN = 256;
  static constexpr int kPairM = 2 * kBlockM;                       // 256 rows per tile
  static constexpr int kStageABytes = kBlockM * kBlockK * 2;       // this CTA's A half: 16 KB
  static constexpr int kStageBBytes = (kBlockN / 2) * kBlockK * 2;  // this CTA's B half: 16 KB
  static constexpr int kStageBytes = kStageABytes + kStageBBytes;
  static constexpr int kStages = 6;
  static constexpr int kTmemCols = 2 * kBlockN;  // two accumulator buffers of 256 columns
  static constexpr int kBarrierBytes = 256;
  static constexpr int kEpiWarps = kNumEpilogueWarps;
  static constexpr int kColsPerWarp = kBlockN / 2;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpilogueStagingBytes + kBarrierBytes + 1024;
};

MSCCLPP_HOST_DEVICE_INLINE constexpr uint32_t makeInstrDescPair() {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(Config2::kBlockN >> 3) << 17) |
         (static_cast<uint32_t>(Config2::kPairM >> 4) << 24);
}

// Body of one CTA of a pair. All threads call it; `pairIdx` / `numPairs` index the persistent tile loop.
// shape.mOrder / mOrderParam apply to 256-row blocks here.
template <typename AGate, typename Epilogue>
MSCCLPP_DEVICE_INLINE void gemmCtaPair(const CUtensorMap* tmapA, const CUtensorMap* tmapB, Shape shape, int pairIdx, int numPairs,
                                       AGate& gate, Epilogue& epi, DeviceStatus* status, uint64_t budgetNs, uint8_t* smemRaw) {
  using Cfg = Config2;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t ctaRank = ptx::cluster_ctarank();
  const bool leader = ctaRank == 0;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* staging = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kEpilogueStagingBytes);
  SharedState st;
  st.full = bars;
  st.empty = bars + Cfg::kStages;
  st.tmemFull = bars + 2 * Cfg::kStages;
  st.tmemEmpty = bars + 2 * Cfg::kStages + 2;
  st.tmemBase = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::kStages + 4);
  st.abortFlag = reinterpret_cast<volatile uint32_t*>(st.tmemBase + 1);
  st.epiArrivals = reinterpret_cast<volatile uint32_t*>(st.tmemBase + 2);

  const int numMBlk2 = (shape.M + Cfg::kPairM - 1) / Cfg::kPairM;
  const int numNBlk = shape.N / Cfg::kBlockN;
  const int numTiles = numMBlk2 * numNBlk;
  const int numKBlk = shape.K / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; s++) {
      ptx::mbar_init(&st.full[s], 1);   // the leader's producer arrives once and announces both CTAs' bytes
      ptx::mbar_init(&st.empty[s], 1);  // one multicast commit per use
    }
    for (int s = 0; s < 2; s++) {
      ptx::mbar_init(&st.tmemFull[s], 1);
      ptx::mbar_init(&st.tmemEmpty[s], 2 * kNumEpilogueWarps);  // the epilogue warps of both CTAs arrive at the leader's
    }
    *st.abortFlag = 0;
    *st.epiArrivals = 0;
    ptx::fence_mbar_init();
    ptx::tma_prefetch_desc(tmapA);
    ptx::tma_prefetch_desc(tmapB);
  }
  __syncthreads();
  // the peer's barriers must exist before anything of mine can signal them
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tmem_alloc_pair(st.tmemBase, Cfg::kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_sync();
  const uint32_t tmemBase = *st.tmemBase;

  if (warp == 0) {
    // ===================================================== TMA producer (one thread per CTA)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issuedUses = 0;
      for (int tile = pairIdx; tile < numTiles && ok; tile += numPairs) {
        int mBlk2, nBlk;
        tileCoord(shape, tile, numMBlk2, numNBlk, mBlk2, nBlk);
        const int mBlk = 2 * mBlk2 + static_cast<int>(ctaRank);
        ok = gate.waitRowBlock(mBlk);
        int aRow;
        const CUtensorMap* tmapARows = gate.tmapA(mBlk, tmapA, aRow);
        for (int kb = 0; kb < numKBlk && ok; kb++) {
          ok = mbarWaitFast(&st.empty[stage], phase ^ 1u, status, budgetNs, 100 + stage, st.abortFlag);
          if (!ok) break;
          uint8_t* sa = tiles + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kStageABytes;
          const uint32_t leaderFull = ptx::mapa_shared(ptx::smem_u32(&st.full[stage]), 0);
          if (shape.probe & 1) {
            if (leader) ptx::mbar_arrive(&st.full[stage]);
          } else {
            if (leader) ptx::mbar_expect_tx(&st.full[stage], 2 * Cfg::kStageBytes);
            ptx::tma_load_2d_pair(sa, tmapARows, kb * kBlockK, aRow, leaderFull);
            ptx::tma_load_2d_pair(sb, tmapB, kb * kBlockK, nBlk * Cfg::kBlockN + static_cast<int>(ctaRank) * (Cfg::kBlockN / 2), leaderFull);
          }
          issuedUses++;
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) *st.abortFlag = 1;
      // Loads in flight land in this CTA's shared memory: the CTA stays resident until the cluster barrier at the
      // end, which every thread of both CTAs reaches, and the leader's consumer either uses them or has given up.
      (void)issuedUses;
    }
  } else if (warp == 1) {
    // ===================================================== MMA issuer (one thread of the leader CTA)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = makeInstrDescPair();
      // one thread feeds the tensor cores of both SMs: descriptors are stepped by adds, waits cost one instruction when
      // the data is already there
      const uint64_t descA0 = makeSmemDesc(ptx::smem_u32(tiles));
      const uint64_t descB0 = makeSmemDesc(ptx::smem_u32(tiles) + Cfg::kStageABytes);
      constexpr uint64_t kStageStep = Cfg::kStageBytes >> 4;
      const bool issue = (shape.probe & 2) == 0;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = pairIdx; tile < numTiles && ok; tile += numPairs, it++) {
        const int acc = it & 1;
        const uint32_t accPhase = (it >> 1) & 1;
        ok = mbarWaitFast(&st.tmemEmpty[acc], accPhase ^ 1u, status, budgetNs, 200 + acc, st.abortFlag);
        if (!ok) break;
        ptx::tcgen05_fence_after_sync();
        const uint32_t tmemD = tmemBase + acc * Cfg::kBlockN;
        for (int kb = 0; kb < numKBlk; kb++) {
          ok = mbarWaitFast(&st.full[stage], phase, status, budgetNs, 300 + stage, st.abortFlag);
          if (!ok) break;
          ptx::tcgen05_fence_after_sync();
          const uint64_t descA = descA0 + stage * kStageStep;
          const uint64_t descB = descB0 + stage * kStageStep;
          if (issue) {
            ptx::tcgen05_mma_f16_pair(tmemD, descA, descB, idesc, kb != 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < kBlockK / kUmmaK; k++) ptx::tcgen05_mma_f16_pair_acc(tmemD, descA + 2 * k, descB + 2 * k, idesc);
          }
          ptx::tcgen05_commit_pair(&st.empty[stage], 3);  // both CTAs may refill this stage once the MMAs retire
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) ptx::tcgen05_commit_pair(&st.tmemFull[acc], 3);
      }
      if (!ok) *st.abortFlag = 1;
    }
  } else if (warp < 2 + kNumEpilogueWarps) {
    // ===================================================== epilogue (8 warps per CTA, on this CTA's accumulator rows)
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    uint8_t* stage = staging + (warp - 2) * kStagingBytesPerWarp;
    bool ok = true;
    int it = 0;
    for (int tile = pairIdx; tile < numTiles && ok; tile += numPairs, it++) {
      int mBlk2, nBlk;
      tileCoord(shape, tile, numMBlk2, numNBlk, mBlk2, nBlk);
      const int mBlk = 2 * mBlk2 + static_cast<int>(ctaRank);
      const int acc = it & 1;
      const uint32_t accPhase = (it >> 1) & 1;
      const int row0 = mBlk * kBlockM + quarter * 32;
      const int col0 = nBlk * Cfg::kBlockN + part * Cfg::kColsPerWarp;
      // lets the epilogue put loads it will need (a residual, a bias) in flight while the MMAs of this tile still run
      epi.tileBegin(row0, col0, lane);
      ok = mbarWait(&st.tmemFull[acc], accPhase, status, budgetNs, 400 + acc);
      ok = __all_sync(0xffffffffu, ok) && (*st.abortFlag == 0);
      if (!ok) break;
      ptx::tcgen05_fence_after_sync();
      const uint32_t taddr = tmemBase + (static_cast<uint32_t>(quarter * 32) << 16) + acc * Cfg::kBlockN + part * Cfg::kColsPerWarp;
      const uint32_t leaderEmpty = ptx::mapa_shared(ptx::smem_u32(&st.tmemEmpty[acc]), 0);
      stagedEpilogueTile<Cfg::kColsPerWarp>(epi, taddr, stage, row0, col0, lane, [&] { ptx::mbar_arrive_cluster(leaderEmpty); }, shape.probe);
      if constexpr (Epilogue::kNeedsTileBarrier) {
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
      // per-warp hook: this warp's part of the tile is stored (fused epilogues count it and may take on follow-up work)
      epi.warpTileDone(mBlk, lane);
    }
    if (ok) epi.warpDrain(lane);  // follow-up work that is left once the warp has no tile of its own any more
    if (!ok && lane == 0) *st.abortFlag = 1;
    if constexpr (Epilogue::kBulkStore) {
      if (lane == 0) ptx::bulk_wait<0>();
    }
  } else if (warp >= 2 + kNumEpilogueWarps) {
    // warps beyond the ten of the GEMM roles (a kernel may launch more threads): follow-up work of a fused epilogue that
    // must stay off the epilogue warps' critical path
    epi.auxWarp(warp - (2 + kNumEpilogueWarps), lane);
  }

  // ---- teardown: both CTAs meet (the peer may still read my shared memory or signal my barriers until then)
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();
  ptx::tcgen05_fence_after_sync();
  if (warp == 1) ptx::tmem_dealloc_pair(tmemBase, Cfg::kTmemCols);
}

}  // namespace gemm
}  // namespace mscclpp
