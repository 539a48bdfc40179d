// The tensor-parallel layer for a handful of tokens (decode), ONE launch:
//
//     h   = sum over ranks ( X_r[T,K] * W_r[N,K]^T ) + residual            T <= kTpDecodeMaxTokens
//     out = h * rsqrt(mean(h^2) + eps) * gamma
//
// With so few rows the layer is a stream over the weight shard (16 MB at the headline shape), not a matrix product:
// tensor-core tiles of 128 rows would be empty and their set-up (tensor memory, barriers, tensor maps) costs more than
// the work. So every SM takes a slab of output columns; its warps stream the weight rows of their columns with 16-byte
// loads (four columns per warp in flight), multiply them with the activations kept as fp32 in shared memory, and the
// slab's [T, columns] results meet the other ranks in a one-shot packet allreduce done by the SAME thread blocks:
// each rank stores its slab as LL16 {data, flag} packets into every peer's scratch (plain peer stores, or one
// multimem.st that the NVSwitch replicates) and sums what arrives - no barrier between the ranks at all. The residual
// add follows in registers; the rows' sums of squares cross the thread blocks through one grid barrier, after which the
// same threads scale and store their words. Every rank ends up with the whole result.
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

MSCCLPP_DEVICE_INLINE float* partialSums(const DeviceComm& c, int rank) {
  return reinterpret_cast<float*>(c.peerBase[rank] + c.auxFlagsOff + kTpDecodeAuxOffset);
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
  extern __shared__ __align__(16) uint8_t smemRaw[];
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const int world = c.world;
  const uint32_t epoch = launchEpoch(c, rank);
  const int T = a.T, N = a.N, K = a.K;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* x = a.x[blockIdx.y];
  const bf16* w = a.w[blockIdx.y];
  const uint64_t local = c.peerBase[rank];
  const uint64_t heap0 = c.peerBase[c.rank];

  // columns of this block: slabs of a.colsPerCta (a multiple of 8)
  const int col0 = blockIdx.x * a.colsPerCta;
  const int cols = col0 < N ? (N - col0 < a.colsPerCta ? N - col0 : a.colsPerCta) : 0;

  float* xs = reinterpret_cast<float*>(smemRaw);                          // [T][K] fp32
  float* part = xs + static_cast<size_t>(T) * K;                          // [T][colsPerCta] fp32
  __shared__ float rinvSmem[kTpDecodeMaxTokens];
  __shared__ float rowSum[kTpDecodeMaxTokens];
  if (threadIdx.x < kTpDecodeMaxTokens) rowSum[threadIdx.x] = 0.f;

  // ---- activations to shared memory, as fp32
  for (int i = threadIdx.x; i < T * K / 8; i += kThreads) {
    float f[8];
    unpack8(ptx::ld_input_v4(x + static_cast<size_t>(i) * 8), f);
#pragma unroll
    for (int j = 0; j < 8; j++) xs[static_cast<size_t>(i) * 8 + j] = f[j];
  }
  __syncthreads();

  // ---- the slab: a warp takes four columns at a time (every activation word read from shared memory then serves four
  // weight rows: with fewer, eight tokens are bound by shared-memory bandwidth, not by the weight stream); lane l covers
  // k = 256 j + 8 l .. + 8. Eight 16-byte weight loads are in flight per lane.
  constexpr int kColsPerIter = 4;
  const int kSteps = K / 256;
  for (int cc = warp * kColsPerIter; cc < cols; cc += kWarps * kColsPerIter) {
    const bf16* wr[kColsPerIter];
#pragma unroll
    for (int q = 0; q < kColsPerIter; q++) wr[q] = w + static_cast<size_t>(col0 + (cc + q < cols ? cc + q : cc)) * K + lane * 8;
    float acc[kColsPerIter][kTpDecodeMaxTokens];
#pragma unroll
    for (int q = 0; q < kColsPerIter; q++) {
#pragma unroll
      for (int tt = 0; tt < kTpDecodeMaxTokens; tt++) acc[q][tt] = 0.f;
    }
    for (int j0 = 0; j0 < kSteps; j0 += 2) {
      uint4 wv[2][kColsPerIter];
#pragma unroll
      for (int jj = 0; jj < 2; jj++) {
        if (j0 + jj < kSteps) {
#pragma unroll
          for (int q = 0; q < kColsPerIter; q++) wv[jj][q] = ptx::ld_input_v4(wr[q] + (j0 + jj) * 256);
        }
      }
#pragma unroll
      for (int jj = 0; jj < 2; jj++) {
        if (j0 + jj < kSteps) {
          float fw[kColsPerIter][8];
#pragma unroll
          for (int q = 0; q < kColsPerIter; q++) unpack8(wv[jj][q], fw[q]);
          const float* xk = xs + (j0 + jj) * 256 + lane * 8;
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
      }
    }
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
  __syncthreads();

  // ---- one thread per 16-byte word of the slab: allreduce, residual, sum of squares
  const int unitsPerRow = a.colsPerCta / 8;
  const int myUnits = T * unitsPerRow;
  const int i = threadIdx.x;
  const int t = i / unitsPerRow, ju = i % unitsPerRow;
  const bool active = i < myUnits && ju * 8 < cols;
  const uint64_t outOff = reinterpret_cast<uint64_t>(a.out) - heap0;
  const uint64_t resOutOff = reinterpret_cast<uint64_t>(a.residualOut) - heap0;
  const uint64_t resInOff = a.residualIn ? reinterpret_cast<uint64_t>(a.residualIn) - heap0 : 0;
  uint4 hWord = make_uint4(0, 0, 0, 0);
  float ss = 0.f;
  bool healthy = true;
  if (active) {
    const int col = col0 + ju * 8;
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
      float acc[8];
      for (int p = 0; p < world && healthy; p++) {
        uint4 v = mine;
        if (p != rank) {
          const LL16Packet* pk = reinterpret_cast<const LL16Packet*>(local + bufOff + static_cast<uint64_t>(p) * c.llSlotBytes + u * 32);
          uint2 lo, hi;
          healthy = pk[0].read(epoch, lo, c.status, c.timeoutNs, rank, p) && pk[1].read(epoch, hi, c.status, c.timeoutNs, rank, p);
          v = make_uint4(lo.x, lo.y, hi.x, hi.y);
        }
        if (p == 0) Vec16<bf16>::toFloat(v, acc);
        else accumulate16<bf16, SUM>(acc, v);
      }
      mine = Vec16<bf16>::fromFloat(acc);
    }
    if (healthy) {
      Vec16<bf16>::toFloat(mine, f);
      if (a.residualIn != nullptr) {
        float r[8];
        Vec16<bf16>::toFloat(ptx::ld_input_v4(reinterpret_cast<const void*>(local + resInOff + (static_cast<uint64_t>(t) * N + col) * 2)), r);
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
  // ---- sums of squares: this block's share of every row to the rank's table, then a grid barrier, then every block adds
  // up the table for itself (no word of the table is ever shared between launches: nothing to clear)
  if (active) atomicAdd(&rowSum[t], ss);  // shared-memory atomic: at most unitsPerRow contributions per row
  __syncthreads();
  float* table = partialSums(c, rank);  // [gridDim.x][kTpDecodeMaxTokens]
  if (threadIdx.x < T) table[blockIdx.x * kTpDecodeMaxTokens + threadIdx.x] = rowSum[threadIdx.x];
  if (!__syncthreads_and(healthy ? 1 : 0)) healthy = false;
  const bool gridOk = gridBarrier(c, rank, &control(c, rank)->gridSync[5], gridDim.x);
  if (gridOk) {
    if (warp < T) {  // one warp per row: gridDim.x partial sums
      float s = 0.f;
      for (int b = lane; b < static_cast<int>(gridDim.x); b += 32) s += __ldcg(&table[b * kTpDecodeMaxTokens + warp]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) rinvSmem[warp] = rsqrtf(s / static_cast<float>(N) + a.eps);
    }
    __syncthreads();
    if (active && healthy) {
      const int col = col0 + ju * 8;
      const float rinv = rinvSmem[t];
      float f[8];
      Vec16<bf16>::toFloat(hWord, f);
      if (a.gamma != nullptr) {
        float g[8];
        Vec16<bf16>::toFloat(__ldg(reinterpret_cast<const uint4*>(a.gamma + col)), g);
#pragma unroll
        for (int j = 0; j < 8; j++) f[j] = f[j] * rinv * g[j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; j++) f[j] = f[j] * rinv;
      }
      *reinterpret_cast<uint4*>(local + outOff + (static_cast<uint64_t>(t) * N + col) * 2) = Vec16<bf16>::fromFloat(f);
    }
  }
  finishLaunch(c, rank, epoch);
}

}  // namespace

cudaError_t launchTpDecode(const TpDecodeArgs& argsIn, cudaStream_t stream) {
  TpDecodeArgs args = argsIn;
  const int T = args.T, N = args.N, K = args.K;
  const int world = args.comm.world;
  if (T < 1 || T > kTpDecodeMaxTokens || N % 8 != 0 || K % 256 != 0 || world < 1 || world > 8) return cudaErrorInvalidValue;
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
  const size_t smem = (static_cast<size_t>(T) * K + static_cast<size_t>(T) * colsPerCta) * sizeof(float);
  if (smem > kMaxSmem) return cudaErrorInvalidValue;
  auto kernel = args.nvls ? tpDecodeKernel<true> : tpDecodeKernel<false>;
  cudaError_t e = gemm::ensureDynamicSmem(reinterpret_cast<const void*>(kernel), static_cast<int>(kMaxSmem));
  if (e != cudaSuccess) return e;
  dim3 grid(ctas, emu, 1), block(kThreads, 1, 1);
  void* params[] = {&args};
  // the blocks of a rank meet in a grid barrier: the launch has to be co-resident
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, params, smem, stream);
}

}  // namespace mscclpp
