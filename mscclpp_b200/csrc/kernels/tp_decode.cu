// The tensor-parallel layer for a handful of tokens (decode), ONE launch:
//
//     h   = sum over ranks ( X_r[T,K] * W_r[N,K]^T ) + residual            T <= kTpDecodeMaxTokens
//     out = h * rsqrt(mean(h^2) + eps) * gamma
//
// With so few rows the layer is a stream over the weight shard (16 MB at the headline shape), not a matrix product:
// tensor-core tiles of 128 rows would be empty and their set-up (tensor memory, barriers, tensor maps) costs more than
// the work. What the launch costs is its chain of dependent memory round trips, so the kernel is built to have few:
//   * every SM takes a slab of output columns; each warp owns groups of four columns and fetches their weight rows with
//     bulk copies (cp.async.bulk global -> shared, no multicast) into its own two shared-memory buffers. The copies of a
//     warp's first two pieces are issued before anything else happens, so at the headline shape the whole shard is in
//     flight while the activations are still being staged (as fp32, in shared memory);
//   * the slab's [T, columns] results meet the other ranks in a one-shot packet allreduce done by the SAME thread
//     blocks: each rank stores its slab as LL16 {data, flag} packets into every peer's scratch (plain peer stores, or
//     one multimem.st that the NVSwitch replicates) and sums what arrives - no barrier between the ranks at all;
//   * the residual and gamma words a thread will need are requested at kernel start;
//   * the rows' sums of squares cross the thread blocks the same way as the packets cross the ranks: every block
//     writes {its share, launch epoch} as one 8-byte word per row, and every block reads all shares until their stamps
//     match - one round trip instead of a grid barrier (arrive, spin) followed by the reads;
//   * a block counts itself out of the launch as soon as it has read the shares, before its final stores.
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
constexpr int kColsPerIter = 4;   // columns a warp works on at a time
constexpr int kSegK = 512;        // reduction elements per piece: a piece is [kColsPerIter][kSegK] bf16 = 4 KB
constexpr int kPieceBytes = kColsPerIter * kSegK * 2;
constexpr int kPiecesPerWarp = 2; // buffers per warp

// {share of the row's sum of squares, epoch} words of the thread blocks: [gridDim.x][kTpDecodeMaxTokens]
MSCCLPP_DEVICE_INLINE uint2* shareTable(const DeviceComm& c, int rank) {
  return reinterpret_cast<uint2*>(c.peerBase[rank] + c.auxFlagsOff + kTpDecodeAuxOffset);
}

MSCCLPP_DEVICE_INLINE void unpack8(uint4 v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <bool kNvls>
__global__ void __launch_bounds__(kThreads, 1) tpDecodeKernel(TpDecodeArgs a) {
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

  // columns of this block: slabs of a.colsPerCta (a multiple of 8)
  const int col0 = blockIdx.x * a.colsPerCta;
  const int cols = col0 < N ? (N - col0 < a.colsPerCta ? N - col0 : a.colsPerCta) : 0;

  uint8_t* wbuf = smemRaw + static_cast<size_t>(warp) * kPiecesPerWarp * kPieceBytes;   // this warp's pieces
  float* xs = reinterpret_cast<float*>(smemRaw + static_cast<size_t>(kWarps) * kPiecesPerWarp * kPieceBytes);  // [T][K] fp32
  float* part = xs + static_cast<size_t>(T) * K;                                        // [T][colsPerCta] fp32
  __shared__ __align__(8) uint64_t bars[kWarps][kPiecesPerWarp];
  __shared__ float rinvSmem[kTpDecodeMaxTokens];
  __shared__ float rowSum[kTpDecodeMaxTokens];
  __shared__ int shareOk;

  // ---- the weight stream starts first. A warp's work is a list of pieces: (column group g, segment s of the reduction
  // dimension), g = warp, warp + kWarps, ...; piece i uses buffer i % 2 and is requested two pieces ahead.
  const int segs = (K + kSegK - 1) / kSegK;  // the last segment may be 256 elements short
  const int groups = (cols + kColsPerIter - 1) / kColsPerIter;
  const int myGroups = groups > warp ? (groups - warp + kWarps - 1) / kWarps : 0;
  const int myPieces = myGroups * segs;
  if (lane == 0) {
    for (int b = 0; b < kPiecesPerWarp; b++) ptx::mbar_init(&bars[warp][b], 1);
    ptx::fence_mbar_init();
  }
  __syncwarp();
  auto request = [&](int piece) {
    // lanes 0..3 fetch one column's segment each (1 KB, contiguous in the weight row); lane 0 arms the barrier first
    const int g = warp + (piece / segs) * kWarps, sg = piece % segs;
    const int cc = g * kColsPerIter;
    const int valid = cols - cc < kColsPerIter ? cols - cc : kColsPerIter;
    const int segLen = K - sg * kSegK < kSegK ? K - sg * kSegK : kSegK;
    uint64_t* bar = &bars[warp][piece % kPiecesPerWarp];
    if (lane == 0) ptx::mbar_expect_tx(bar, static_cast<uint32_t>(valid) * segLen * 2);
    __syncwarp();
    if (lane < valid) {
      ptx::bulk_g2s(wbuf + (piece % kPiecesPerWarp) * kPieceBytes + lane * kSegK * 2,
                    w + static_cast<size_t>(col0 + cc + lane) * K + static_cast<size_t>(sg) * kSegK, static_cast<uint32_t>(segLen) * 2, bar);
    }
  };
  for (int i = 0; i < kPiecesPerWarp && i < myPieces; i++) request(i);

  const uint32_t epoch = launchEpoch(c, rank);
  if (threadIdx.x < kTpDecodeMaxTokens) rowSum[threadIdx.x] = 0.f;
  if (threadIdx.x == 0) shareOk = 1;

  // ---- what the tail will need, requested now: one thread per 16-byte word of the slab
  const int unitsPerRow = a.colsPerCta / 8;
  const int myUnits = T * unitsPerRow;
  const int t = threadIdx.x / unitsPerRow, ju = threadIdx.x % unitsPerRow;
  const bool active = static_cast<int>(threadIdx.x) < myUnits && ju * 8 < cols;
  const int col = col0 + ju * 8;
  const uint64_t outOff = reinterpret_cast<uint64_t>(a.out) - heap0;
  const uint64_t resOutOff = reinterpret_cast<uint64_t>(a.residualOut) - heap0;
  const uint64_t resInOff = a.residualIn ? reinterpret_cast<uint64_t>(a.residualIn) - heap0 : 0;
  uint4 resWord = make_uint4(0, 0, 0, 0), gammaWord = make_uint4(0, 0, 0, 0);
  if (active) {
    if (a.residualIn != nullptr) resWord = ptx::ld_input_v4(reinterpret_cast<const void*>(local + resInOff + (static_cast<uint64_t>(t) * N + col) * 2));
    if (a.gamma != nullptr) gammaWord = __ldg(reinterpret_cast<const uint4*>(a.gamma + col));
  }

  // ---- activations to shared memory, as fp32
  for (int i = threadIdx.x; i < T * K / 8; i += kThreads) {
    float f[8];
    unpack8(ptx::ld_input_v4(x + static_cast<size_t>(i) * 8), f);
    *reinterpret_cast<float4*>(xs + static_cast<size_t>(i) * 8) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(xs + static_cast<size_t>(i) * 8 + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
  __syncthreads();

  // ---- the slab. Every activation word read from shared memory serves four weight rows (with fewer, eight tokens are
  // bound by shared-memory bandwidth, not by the weight stream); lane l covers k = 256 j + 8 l .. + 8 of a segment.
  bool healthy = true;
  float acc[kColsPerIter][kTpDecodeMaxTokens];
  for (int piece = 0; piece < myPieces && healthy; piece++) {
    const int sg = piece % segs;
    const int cc = (warp + (piece / segs) * kWarps) * kColsPerIter;
    if (sg == 0) {
#pragma unroll
      for (int q = 0; q < kColsPerIter; q++) {
#pragma unroll
        for (int tt = 0; tt < kTpDecodeMaxTokens; tt++) acc[q][tt] = 0.f;
      }
    }
    healthy = mbarWait(&bars[warp][piece % kPiecesPerWarp], (piece / kPiecesPerWarp) & 1, c.status, c.timeoutNs, 600 + warp);
    healthy = __all_sync(0xffffffffu, healthy);
    if (!healthy) break;
    const uint8_t* wp = wbuf + (piece % kPiecesPerWarp) * kPieceBytes + lane * 16;
    const int segLen = K - sg * kSegK < kSegK ? K - sg * kSegK : kSegK;
#pragma unroll
    for (int j = 0; j < kSegK / 256; j++) {
      if (j * 256 >= segLen) break;
      float fw[kColsPerIter][8];
#pragma unroll
      for (int q = 0; q < kColsPerIter; q++) unpack8(*reinterpret_cast<const uint4*>(wp + q * kSegK * 2 + j * 512), fw[q]);
      const float* xk = xs + static_cast<size_t>(sg) * kSegK + j * 256 + lane * 8;
#pragma unroll
      for (int tt = 0; tt < kTpDecodeMaxTokens; tt++) {
        if (tt < T) {
          const float4 xlo = *reinterpret_cast<const float4*>(xk + static_cast<size_t>(tt) * K);
          const float4 xhi = *reinterpret_cast<const float4*>(xk + static_cast<size_t>(tt) * K + 4);
#pragma unroll
          for (int q = 0; q < kColsPerIter; q++) {
            acc[q][tt] += fw[q][0] * xlo.x + fw[q][1] * xlo.y + fw[q][2] * xlo.z + fw[q][3] * xlo.w + fw[q][4] * xhi.x + fw[q][5] * xhi.y +
                          fw[q][6] * xhi.z + fw[q][7] * xhi.w;
          }
        }
      }
    }
    __syncwarp();  // every lane has read the buffer: it may be refilled
    if (piece + kPiecesPerWarp < myPieces) request(piece + kPiecesPerWarp);
    if (sg == segs - 1) {
#pragma unroll
      for (int tt = 0; tt < kTpDecodeMaxTokens; tt++) {
        if (tt < T) {
#pragma unroll
          for (int q = 0; q < kColsPerIter; q++) {
            float v = acc[q][tt];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && cc + q < cols) part[tt * a.colsPerCta + cc + q] = v;
          }
        }
      }
    }
  }
  if (!healthy) {
    // give the copies this warp still has in flight a (bounded) chance to land before the block may exit
    for (int b = 0; b < kPiecesPerWarp; b++) (void)mbarWait(&bars[warp][b], 0, nullptr, 2000000ull, 0);
  }
  if (!__syncthreads_and(healthy ? 1 : 0)) healthy = false;

  // ---- one thread per 16-byte word of the slab: allreduce, residual, sum of squares
  uint4 hWord = make_uint4(0, 0, 0, 0);
  float ss = 0.f;
  if (active && healthy) {
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; j++) f[j] = part[t * a.colsPerCta + ju * 8 + j];
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
      // contributions are added in rank order, so that every rank computes bit-identical sums
      float sum[8];
      for (int p = 0; p < world && healthy; p++) {
        uint4 v = mine;
        if (p != rank) {
          const LL16Packet* pk = reinterpret_cast<const LL16Packet*>(local + bufOff + static_cast<uint64_t>(p) * c.llSlotBytes + u * 32);
          uint2 lo, hi;
          healthy = pk[0].read(epoch, lo, c.status, c.timeoutNs, rank, p) && pk[1].read(epoch, hi, c.status, c.timeoutNs, rank, p);
          v = make_uint4(lo.x, lo.y, hi.x, hi.y);
        }
        if (p == 0) Vec16<bf16>::toFloat(v, sum);
        else accumulate16<bf16, SUM>(sum, v);
      }
      mine = Vec16<bf16>::fromFloat(sum);
    }
    if (healthy) {
      Vec16<bf16>::toFloat(mine, f);
      if (a.residualIn != nullptr) {
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
    }
  }
  // ---- sums of squares: this block's share of every row goes to the rank's table stamped with the launch epoch; every
  // block then reads all shares, waiting (bounded) for stamps of this launch. Nothing in the table needs clearing.
  if (active && healthy) atomicAdd(&rowSum[t], ss);  // shared-memory atomic: at most unitsPerRow contributions per row
  if (!__syncthreads_and(healthy ? 1 : 0)) healthy = false;
  uint2* table = shareTable(c, rank);  // [gridDim.x][kTpDecodeMaxTokens]
  if (healthy && static_cast<int>(threadIdx.x) < T) {
    ptx::st_volatile_v2(&table[blockIdx.x * kTpDecodeMaxTokens + threadIdx.x], make_uint2(__float_as_uint(rowSum[threadIdx.x]), epoch));
  }
  if (healthy && warp < T) {  // one warp per row: gridDim.x shares
    float sAll = 0.f;
    bool ok = true;
    for (int b = lane; b < static_cast<int>(gridDim.x) && ok; b += 32) {
      const uint2* src = &table[b * kTpDecodeMaxTokens + warp];
      uint2 v = ptx::ld_volatile_v2(src);
      if (v.y != epoch) {
        SpinGuard g(c.status, c.timeoutNs);
        while ((v = ptx::ld_volatile_v2(src)).y != epoch) {
          if (!g.keepSpinning()) {
            g.report(kDevTimeoutFlag, rank, 9100, b, epoch, v.y);
            ok = false;
            break;
          }
        }
      }
      sAll += __uint_as_float(v.x);
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
  // this block has taken everything it needs from the launch's shared state: count it out now, so that the round trip of
  // that atomic overlaps the final stores
  if (threadIdx.x == 0) {
    SymmControl* ctl = control(c, rank);
    __threadfence();
    const uint32_t prev = atomicAdd(&ctl->done, 1u);
    if (prev == gridDim.x - 1) {
      ctl->done = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&ctl->epoch) = epoch;
    }
  }
  if (active && healthy && shareOk) {
    const float rinv = rinvSmem[t];
    float f[8];
    Vec16<bf16>::toFloat(hWord, f);
    if (a.gamma != nullptr) {
      float g[8];
      Vec16<bf16>::toFloat(gammaWord, g);
#pragma unroll
      for (int j = 0; j < 8; j++) f[j] = f[j] * rinv * g[j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) f[j] = f[j] * rinv;
    }
    *reinterpret_cast<uint4*>(local + outOff + (static_cast<uint64_t>(t) * N + col) * 2) = Vec16<bf16>::fromFloat(f);
  }
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
  // one thread per 16-byte word of the slab
  if (T * (colsPerCta / 8) > kThreads) return cudaErrorInvalidValue;
  ctas = (N + colsPerCta - 1) / colsPerCta;
  args.colsPerCta = colsPerCta;
  constexpr size_t kMaxSmem = 200u * 1024;
  const size_t smem = static_cast<size_t>(kWarps) * kPiecesPerWarp * kPieceBytes + (static_cast<size_t>(T) * K + static_cast<size_t>(T) * colsPerCta) * sizeof(float);
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
