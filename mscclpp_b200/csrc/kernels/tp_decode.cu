// The tensor-parallel layer for a handful of tokens (decode), ONE launch:
//
//     h   = sum over ranks ( X_r[T,K] * W_r[N,K]^T ) + residual            T <= kTpDecodeMaxTokens
//     out = h * rsqrt(mean(h^2) + eps) * gamma
//
// With so few rows the layer is a stream over the weight shard (16 MB at the headline shape), not a matrix product of
// 128-row tiles: those would be empty, and their set-up (tensor memory, barriers, tensor maps) costs more than the work.
// What the launch costs is its chain of dependent memory round trips, so the kernel is built to have few:
//   * every SM takes a slab of up to 64 output columns and fetches the weight rows of the slab with bulk copies
//     (cp.async.bulk global -> shared, one per row and 512-element chunk of the reduction dimension, no multicast) into
//     two shared-memory buffers. The copies of the first two chunks are issued before anything else happens, so at the
//     headline shape the whole shard is in flight while the activations are still being staged;
//   * the products are taken by warp-level tensor-core instructions with the WEIGHTS as the 16-row operand and the (up
//     to eight) tokens as the 8-column operand (m16n8k16, fp32 accumulation): one instruction covers 16 output columns
//     x 8 tokens x 16 reduction elements, so eight tokens cost what one costs. (tcgen05 tiles start at 64 rows and want
//     tensor memory and descriptors set up first; for 16 MFLOP that set-up is the longer part.) Sixteen warps split the
//     slab four ways by columns and four ways along the reduction dimension;
//   * the slab's [T, columns] results meet the other ranks in a one-shot packet allreduce done by the SAME thread
//     blocks: each rank stores its slab as LL16 {data, flag} packets into every peer's scratch (plain peer stores, or
//     one multimem.st that the NVSwitch replicates) and sums what arrives - no barrier between the ranks at all;
//   * the residual and gamma words a thread will need are requested at kernel start;
//   * the rows' sums of squares cross the thread blocks the same way as the packets cross the ranks: every block
//     writes {its share, launch epoch} as one 8-byte word per row, and every block reads all shares (all loads in flight
//     at once) until their stamps match - one round trip instead of a grid barrier followed by the reads;
//   * a block counts itself out of the launch (the counter that moves the launch epoch on) at its start, where the
//     round trip of that atomic is hidden, not at its end.
// Every rank ends up with the whole result.
//
// The reference library has no counterpart (it offers the allreduce alone, allreduce_packet.cu).
#include "tp_fused.cuh"

#include <mscclpp/gpu_data_types.hpp>
#include <mscclpp/packet_device.hpp>

#include "gemm.cuh"

namespace mscclpp {

namespace {

using bf16 = __nv_bfloat16;
constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxCols = 64;            // output columns per thread block: four groups of 16
constexpr int kChunkK = 512;            // reduction elements per chunk
constexpr int kRowBytes = kChunkK * 2 + 16;  // a weight row of a chunk in shared memory; the 16 bytes of padding spread the
                                             // rows of an 8 x 8 matrix load over all banks
constexpr int kChunkBytes = kMaxCols * kRowBytes;
constexpr int kSlices = 4;              // warps that share a column group, each with kChunkK / kSlices of a chunk

// {share of the row's sum of squares, epoch} words of the thread blocks: [gridDim.x][kTpDecodeMaxTokens]
MSCCLPP_DEVICE_INLINE uint2* shareTable(const DeviceComm& c, int rank) {
  return reinterpret_cast<uint2*>(c.peerBase[rank] + c.auxFlagsOff + kTpDecodeAuxOffset);
}

MSCCLPP_DEVICE_INLINE void ldmatrix_x4(uint32_t (&r)[4], const void* smemRow) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(ptx::smem_u32(smemRow)));
}
// D[16 x 8] += A[16 x 16] (row-major) * B[16 x 8] (column-major), bf16 operands, fp32 accumulation
MSCCLPP_DEVICE_INLINE void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool kNvls>
__global__ void __launch_bounds__(kThreads, 1) tpDecodeKernel(TpDecodeArgs a) {
  static_assert(kWarps == 4 * kSlices, "sixteen warps: four column groups x four slices");
  extern __shared__ __align__(128) uint8_t smemRaw[];
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const int world = c.world;
  const int T = a.T, N = a.N, K = a.K;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* x = a.x[blockIdx.y];
  const bf16* w = a.w[blockIdx.y];
  const uint64_t local = c.peerBase[rank];
  const uint64_t heap0 = c.peerBase[c.rank];
  unsigned long long* tl = (a.stamps != nullptr && threadIdx.x == 0 && blockIdx.y == 0) ? a.stamps + static_cast<size_t>(blockIdx.x) * 8 : nullptr;
  if (tl) tl[0] = ptx::globaltimer();

  // columns of this block: a.colsPerCta (a multiple of 8) from col0 on, worked off in passes of up to kMaxCols columns
  // (one pass at the shapes this kernel is meant for: N / #SMs <= 64)
  const int col0 = blockIdx.x * a.colsPerCta;
  const int cols = col0 < N ? (N - col0 < a.colsPerCta ? N - col0 : a.colsPerCta) : 0;
  const int passes = (cols + kMaxCols - 1) / kMaxCols;
  auto passCols = [&](int ps) { return cols - ps * kMaxCols < kMaxCols ? cols - ps * kMaxCols : kMaxCols; };

  const int xStride = K + 8;                                                // bf16 elements; the padding spreads the tokens over the banks
  uint8_t* wch = smemRaw;                                                   // [2][kMaxCols][kRowBytes]
  bf16* xs = reinterpret_cast<bf16*>(smemRaw + 2 * kChunkBytes);            // [kTpDecodeMaxTokens][xStride], rows >= T zero
  float* part = reinterpret_cast<float*>(xs + kTpDecodeMaxTokens * xStride);  // [kSlices][kTpDecodeMaxTokens][kMaxCols] fp32
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ float rinvSmem[kTpDecodeMaxTokens];
  __shared__ float rowSum[kTpDecodeMaxTokens];
  __shared__ int shareOk;

  // ---- the weight stream starts first. Its items are (pass, chunk of the reduction dimension) in order; item q goes to
  // buffer q % 2 with one bulk copy per weight row, and is requested as soon as item q - 2 has been consumed.
  const int chunks = (K + kChunkK - 1) / kChunkK;  // the last chunk may be 256 elements short
  const int items = passes * chunks;
  auto chunkLen = [&](int ch) { return K - ch * kChunkK < kChunkK ? K - ch * kChunkK : kChunkK; };
  auto arm = [&](int q) {  // thread 0
    ptx::mbar_expect_tx(&bars[q & 1], static_cast<uint32_t>(passCols(q / chunks)) * chunkLen(q % chunks) * 2);
  };
  auto requestRow = [&](int q) {  // every thread, after the item's barrier has been armed
    const int ps = q / chunks, ch = q % chunks;
    if (static_cast<int>(threadIdx.x) < passCols(ps)) {
      ptx::bulk_g2s(wch + (q & 1) * kChunkBytes + threadIdx.x * kRowBytes,
                    w + static_cast<size_t>(col0 + ps * kMaxCols + threadIdx.x) * K + static_cast<size_t>(ch) * kChunkK,
                    static_cast<uint32_t>(chunkLen(ch)) * 2, &bars[q & 1]);
    }
  };
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars[0], 1);
    ptx::mbar_init(&bars[1], 1);
    ptx::fence_mbar_init();
    for (int q = 0; q < 2 && q < items; q++) arm(q);
    shareOk = 1;
  }
  if (threadIdx.x < kTpDecodeMaxTokens) rowSum[threadIdx.x] = 0.f;
  __syncthreads();
  for (int q = 0; q < 2 && q < items; q++) requestRow(q);
  int requested = items < 2 ? items : 2;  // items requested so far (the same in every thread)
  int waited = 0;                         // items this warp has seen land

  const uint32_t epoch = launchEpoch(c, rank);
  // ---- the tail works with one thread per 16-byte word of a pass's [T, <= 64] results; what the first pass will need is
  // requested now
  const int t = threadIdx.x / (kMaxCols / 8), ju = threadIdx.x % (kMaxCols / 8);
  const uint64_t outOff = reinterpret_cast<uint64_t>(a.out) - heap0;
  const uint64_t resOutOff = a.residualOut ? reinterpret_cast<uint64_t>(a.residualOut) - heap0 : 0;
  const uint64_t resInOff = a.residualIn ? reinterpret_cast<uint64_t>(a.residualIn) - heap0 : 0;
  uint4 resWord = make_uint4(0, 0, 0, 0), gammaWord = make_uint4(0, 0, 0, 0);
  if (t < T && ju * 8 < passCols(0)) {
    const int col = col0 + ju * 8;
    if (a.residualIn != nullptr) resWord = ptx::ld_input_v4(reinterpret_cast<const void*>(local + resInOff + (static_cast<uint64_t>(t) * N + col) * 2));
    if (a.gamma != nullptr) gammaWord = __ldg(reinterpret_cast<const uint4*>(a.gamma + col));
  }

  // ---- activations to shared memory (bf16, the rows of absent tokens zero)
  const int wordsPerRow = K / 8;
  for (int i = threadIdx.x; i < kTpDecodeMaxTokens * wordsPerRow; i += kThreads) {
    const int tt = i / wordsPerRow, kw = i % wordsPerRow;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tt < T) v = ptx::ld_input_v4(x + static_cast<size_t>(tt) * K + kw * 8);
    *reinterpret_cast<uint4*>(xs + tt * xStride + kw * 8) = v;
  }
  // (the barrier in it also publishes the staged activations)
  retireLaunchEarly(c, rank, epoch);
  if (tl) tl[1] = ptx::globaltimer();

  // warp (g, sl) multiplies columns [16 g, 16 g + 16) of a pass by slice sl of every chunk. This lane's row of the four
  // 8 x 8 matrices of an A fragment, and its word of the B fragment:
  const int g = warp / kSlices, sl = warp % kSlices;
  const int aRow = g * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
  const int aKoff = ((lane >> 4) & 1) * 8;
  const bf16* xLane = xs + (lane >> 2) * xStride + (lane & 3) * 2;
  bool healthy = true;
  uint4 hWord = make_uint4(0, 0, 0, 0);

  for (int ps = 0; ps < passes; ps++) {
    const int pcols = passCols(ps);
    const int pcol0 = col0 + ps * kMaxCols;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int ch = 0; ch < chunks; ch++) {
      const int q = ps * chunks + ch;
      bool ok = healthy && mbarWait(&bars[q & 1], (q >> 1) & 1, c.status, c.timeoutNs, 600 + ch);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) waited = q + 1;
      if (ok && g * 16 < pcols) {
        const int len = chunkLen(ch);
        const int k0 = sl * (kChunkK / kSlices);
        const uint8_t* rowBase = wch + (q & 1) * kChunkBytes + aRow * kRowBytes;
#pragma unroll
        for (int kk = 0; kk < kChunkK / kSlices; kk += 16) {
          if (k0 + kk < len) {
            uint32_t af[4];
            ldmatrix_x4(af, rowBase + (k0 + kk + aKoff) * 2);
            const bf16* xb = xLane + ch * kChunkK + k0 + kk;
            mma_m16n8k16(acc, af, *reinterpret_cast<const uint32_t*>(xb), *reinterpret_cast<const uint32_t*>(xb + 8));
          }
        }
      }
      healthy = healthy && ok;
      if (q + 2 < items) {
        // refill the buffer once every warp has read item q out of it (the decision to go on is taken by the whole block)
        if (!__syncthreads_and(healthy ? 1 : 0)) healthy = false;
        if (healthy) {
          if (threadIdx.x == 0) arm(q + 2);
          __syncthreads();
          requestRow(q + 2);
          requested = q + 3;
        }
      }
    }
    if (healthy && g * 16 < pcols) {
      // accumulator layout: rows lane / 4 and lane / 4 + 8 (output columns), columns 2 (lane % 4) and + 1 (tokens)
      float* dst = part + sl * (kTpDecodeMaxTokens * kMaxCols) + g * 16 + (lane >> 2);
      const int tok = (lane & 3) * 2;
      dst[tok * kMaxCols] = acc[0];
      dst[(tok + 1) * kMaxCols] = acc[1];
      dst[tok * kMaxCols + 8] = acc[2];
      dst[(tok + 1) * kMaxCols + 8] = acc[3];
    }
    if (tl && ps == 0) tl[2] = ptx::globaltimer();
    if (!__syncthreads_and(healthy ? 1 : 0)) healthy = false;
    if (tl && ps == 0) tl[3] = ptx::globaltimer();

    // ---- one thread per 16-byte word of the pass: allreduce, residual, sum of squares
    const bool active = t < T && ju * 8 < pcols;
    float ss = 0.f;
    if (active && healthy) {
      const int col = pcol0 + ju * 8;
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; j++) {
        f[j] = 0.f;
#pragma unroll
        for (int q = 0; q < kSlices; q++) f[j] += part[q * (kTpDecodeMaxTokens * kMaxCols) + t * kMaxCols + ju * 8 + j];
      }
      uint4 mine = Vec16<bf16>::fromFloat(f);  // the partial product leaves the rank rounded to bf16, like a GEMM output would
      if (world > 1) {
        const uint64_t bufOff = c.llScratchOff + static_cast<uint64_t>(epoch & 1u) * (static_cast<uint64_t>(world) * c.llSlotBytes);
        const uint64_t u = static_cast<uint64_t>(t) * (N / 8) + col / 8;  // word index inside the [T, N] activation
        if constexpr (kNvls) {
          char* mc = reinterpret_cast<char*>(c.mcBase + bufOff + static_cast<uint64_t>(rank) * c.llSlotBytes + u * 32);
          ptx::multimem_st_v4(mc, make_uint4(mine.x, epoch, mine.y, epoch));
          ptx::multimem_st_v4(mc + 16, make_uint4(mine.z, epoch, mine.w, epoch));
        } else {
          for (int k = 1; k < world; k++) {
            const int p = (rank + k) % world;
            LL16Packet* pk = reinterpret_cast<LL16Packet*>(c.peerBase[p] + bufOff + static_cast<uint64_t>(rank) * c.llSlotBytes + u * 32);
            pk[0].write(mine.x, mine.y, epoch);
            pk[1].write(mine.z, mine.w, epoch);
          }
        }
        // contributions are added in rank order, so that every rank computes bit-identical sums. All peers' packets are
        // requested before any flag is looked at, and polled together until all carry this launch's flag (the wait for the
        // slowest peer is paid once, one round trip after it everything is in registers).
        float sum[8];
        const uint64_t slotBase = local + bufOff + u * 32;
        uint4 word[8];
        SpinGuard guard(c.status, c.timeoutNs);
        for (;;) {
          bool allHere = true;
#pragma unroll
          for (int p = 0; p < 8; p++) {
            if (p < world && p != rank) {
              const char* pk = reinterpret_cast<const char*>(slotBase + static_cast<uint64_t>(p) * c.llSlotBytes);
              const uint4 a0 = ptx::ld_volatile_v4(pk), a1 = ptx::ld_volatile_v4(pk + 16);
              word[p] = make_uint4(a0.x, a0.z, a1.x, a1.z);
              allHere = allHere && a0.y == epoch && a0.w == epoch && a1.y == epoch && a1.w == epoch;
            }
          }
          if (allHere) break;
          if (!guard.keepSpinning()) {
            guard.report(kDevTimeoutPacket, rank, 16, 0, epoch, 0);
            healthy = false;
            break;
          }
        }
        if (healthy) {
#pragma unroll
          for (int p = 0; p < 8; p++) {
            if (p < world) {
              const uint4 v = p == rank ? mine : word[p];
              if (p == 0) Vec16<bf16>::toFloat(v, sum);
              else accumulate16<bf16, SUM>(sum, v);
            }
          }
        }
        mine = Vec16<bf16>::fromFloat(sum);
      }
      if (healthy) {
        Vec16<bf16>::toFloat(mine, f);
        if (a.residualIn != nullptr) {
          if (ps > 0) resWord = ptx::ld_input_v4(reinterpret_cast<const void*>(local + resInOff + (static_cast<uint64_t>(t) * N + col) * 2));
          float r[8];
          Vec16<bf16>::toFloat(resWord, r);
#pragma unroll
          for (int j = 0; j < 8; j++) f[j] += r[j];
          mine = Vec16<bf16>::fromFloat(f);
          Vec16<bf16>::toFloat(mine, f);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) ss += f[j] * f[j];
        hWord = mine;
        if (a.residualOut != nullptr) *reinterpret_cast<uint4*>(local + resOutOff + (static_cast<uint64_t>(t) * N + col) * 2) = mine;
        // with several passes h waits in `out` for the row's 1/rms (same thread writes and re-reads it)
        if (passes > 1) *reinterpret_cast<uint4*>(local + outOff + (static_cast<uint64_t>(t) * N + col) * 2) = mine;
      }
    }
    if (active && healthy) atomicAdd(&rowSum[t], ss);  // shared-memory atomic: a few contributions per row
    if (passes > 1) __syncthreads();                    // `part` is rewritten by the next pass
  }
  if (tl) tl[4] = ptx::globaltimer();
  if (!healthy) {
    // give the copies still in flight a (bounded) chance to land before the block may exit
    for (int q = waited; q < requested; q++) (void)mbarWait(&bars[q & 1], (q >> 1) & 1, nullptr, 2000000ull, 0);
  }

  // ---- sums of squares: this block's share of every row goes to the rank's table stamped with the launch epoch; every
  // block then reads all shares, waiting (bounded) for stamps of this launch. Nothing in the table needs clearing.
  if (!__syncthreads_and(healthy ? 1 : 0)) healthy = false;
  uint2* table = shareTable(c, rank);  // [gridDim.x][kTpDecodeMaxTokens]
  if (healthy && static_cast<int>(threadIdx.x) < T) {
    ptx::st_volatile_v2(&table[blockIdx.x * kTpDecodeMaxTokens + threadIdx.x], make_uint2(__float_as_uint(rowSum[threadIdx.x]), epoch));
  }
  if (healthy && warp < T) {  // one warp per row: gridDim.x shares, all requested before the first is looked at
    constexpr int kPerLane = (kBarrierSlots + 31) / 32;
    uint2 v[kPerLane];
#pragma unroll
    for (int q = 0; q < kPerLane; q++) {
      const int b = lane + q * 32;
      v[q] = make_uint2(0, epoch);
      if (b < static_cast<int>(gridDim.x)) v[q] = ptx::ld_volatile_v2(&table[b * kTpDecodeMaxTokens + warp]);
    }
    float sAll = 0.f;
    bool ok = true;
#pragma unroll
    for (int q = 0; q < kPerLane; q++) {
      const int b = lane + q * 32;
      if (v[q].y != epoch && ok) {
        const uint2* src = &table[b * kTpDecodeMaxTokens + warp];
        SpinGuard sg(c.status, c.timeoutNs);
        while ((v[q] = ptx::ld_volatile_v2(src)).y != epoch) {
          if (!sg.keepSpinning()) {
            sg.report(kDevTimeoutFlag, rank, 9100, b, epoch, v[q].y);
            ok = false;
            break;
          }
        }
      }
      sAll += __uint_as_float(v[q].x);
    }
    ok = __all_sync(0xffffffffu, ok);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sAll += __shfl_xor_sync(0xffffffffu, sAll, o);
    if (lane == 0) {
      rinvSmem[warp] = rsqrtf(sAll / static_cast<float>(N) + a.eps);
      if (!ok) shareOk = 0;
    }
  }
  __syncthreads();
  if (tl) tl[5] = ptx::globaltimer();
  if (healthy && shareOk && t < T) {
    const float rinv = rinvSmem[t];
    for (int ps = 0; ps < passes; ps++) {
      if (ju * 8 >= passCols(ps)) continue;
      const int col = col0 + ps * kMaxCols + ju * 8;
      uint4* dst = reinterpret_cast<uint4*>(local + outOff + (static_cast<uint64_t>(t) * N + col) * 2);
      if (passes > 1) {
        hWord = *dst;
        if (a.gamma != nullptr) gammaWord = __ldg(reinterpret_cast<const uint4*>(a.gamma + col));
      }
      float f[8];
      Vec16<bf16>::toFloat(hWord, f);
      if (a.gamma != nullptr) {
        float gm[8];
        Vec16<bf16>::toFloat(gammaWord, gm);
#pragma unroll
        for (int j = 0; j < 8; j++) f[j] = f[j] * rinv * gm[j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; j++) f[j] = f[j] * rinv;
      }
      *dst = Vec16<bf16>::fromFloat(f);
    }
  }
  if (tl) tl[6] = ptx::globaltimer();
}

}  // namespace

cudaError_t launchTpDecode(const TpDecodeArgs& argsIn, cudaStream_t stream) {
  TpDecodeArgs args = argsIn;
  const int T = args.T, N = args.N, K = args.K;
  const int world = args.comm.world;
  if (T < 1 || T > kTpDecodeMaxTokens || N % 8 != 0 || K % 256 != 0 || world < 1 || world > 8) return cudaErrorInvalidValue;
  // bulk copies want 16-byte aligned sources: weight rows start on multiples of K * 2 bytes, segments on multiples of 1 KB
  if (reinterpret_cast<uintptr_t>(args.w[0]) % 16 != 0) return cudaErrorInvalidValue;
  if (args.nvls && args.comm.mcBase == 0) return cudaErrorInvalidValue;
  const int emu = args.emuRanks > 1 ? args.emuRanks : 1;
  if (emu > 8) return cudaErrorInvalidValue;
  // the packets of one rank must fit its slot of the LL scratch (two bytes of scratch per byte of payload)
  if (static_cast<uint64_t>(T) * N * 2 * 2 > args.comm.llSlotBytes) return cudaErrorInvalidValue;
  int ctas = args.numCtas > 0 ? args.numCtas : gemm::smCount() / emu;
  if (ctas > kBarrierSlots) ctas = kBarrierSlots;
  int colsPerCta = ((N + ctas - 1) / ctas + 7) / 8 * 8;
  ctas = (N + colsPerCta - 1) / colsPerCta;
  args.colsPerCta = colsPerCta;
  constexpr size_t kMaxSmem = 200u * 1024;
  const size_t smem = 2 * static_cast<size_t>(kChunkBytes) + static_cast<size_t>(kTpDecodeMaxTokens) * (K + 8) * 2 +
                      static_cast<size_t>(kSlices) * kTpDecodeMaxTokens * kMaxCols * sizeof(float);
  if (smem > kMaxSmem) return cudaErrorInvalidValue;
  auto kernel = args.nvls ? tpDecodeKernel<true> : tpDecodeKernel<false>;
  cudaError_t e = gemm::ensureDynamicSmem(reinterpret_cast<const void*>(kernel), static_cast<int>(kMaxSmem));
  if (e != cudaSuccess) return e;
  dim3 grid(ctas, emu, 1), block(kThreads, 1, 1);
  void* params[] = {&args};
  // the blocks of a rank wait for one another's shares of the row sums: the launch has to be co-resident
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, params, smem, stream);
}

}  // namespace mscclpp
