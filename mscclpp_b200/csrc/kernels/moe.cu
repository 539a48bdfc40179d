// MoE expert-parallel dispatch and combine, one kernel each, over peer memory.
//
// dispatch: every (token, expert) pair of this rank is PUSHED into the hosting rank's receive buffer, directly
//   into its place in an expert-grouped layout (rows of local expert 0 from source ranks 0..n-1, then expert 1,
//   ...), so the grouped expert GEMM can run on the buffer as it is. The sizes are data dependent:
//     A. one pass over topkIdx assigns each pair its position inside its (source rank, expert) group and counts
//        the groups (atomics on 64..256 counters);
//     B. the counts travel to every rank as (value, epoch) pairs - 8-byte stores, no separate flag;
//     C. every block reads the full [rank][expert] count matrix and derives the first row of each of its groups
//        at the destination;
//     D. one warp per token loads the row once and stores it to its top-k destinations (16-byte peer stores);
//        with fp8 = 1 the row is quantised in registers to e4m3 with one scale per 128 elements, which halves the
//        bytes on NVLink.
// combine: the reverse direction is a PULL - the source rank reads the expert outputs of its tokens out of the
//   hosting ranks' buffers (16-byte peer loads), applies the routing weights in fp32 and writes the bf16 result.
//   No staging buffer and no second pass. With fp8 = 1 the expert outputs are e4m3 with 1 x 128 scales (quantised by
//   the expert GEMM's epilogue or by launchMoeQuantizeRows), half the bytes over NVLink.
// Both end with a cross-rank barrier: after dispatch returns every row sent to this rank has landed; after combine
// returns the peers are done reading this rank's expert outputs.
//
// The reference library has no MoE kernels of its own; its bulk-copy device primitives
// (include/mscclpp/bulk_device.hpp) exist to let users write them.
#include "moe.cuh"

#include <mscclpp/gpu_data_types.hpp>
#include <mscclpp/poll_device.hpp>

namespace mscclpp {

namespace {

using bf16 = __nv_bfloat16;
constexpr int kThreads = 512;
constexpr int kMaxWordsPerLane = 32;  // hidden <= 32 lanes * 32 words * 8 elements = 8192

struct Workspace {
  uint32_t* cnt;      // [kMoeMaxExperts] pairs of this rank per expert (zero between launches)
  uint2* matrix;      // [kMaxRanks][kMoeMaxExperts] (count, epoch) written by the source ranks
};

MSCCLPP_DEVICE_INLINE Workspace workspaceOf(const DeviceComm& c, int rank, uint64_t wsOff) {
  Workspace w;
  w.cnt = reinterpret_cast<uint32_t*>(c.peerBase[rank] + wsOff);
  w.matrix = reinterpret_cast<uint2*>(c.peerBase[rank] + wsOff + kMoeMaxExperts * sizeof(uint32_t));
  return w;
}


// Quantises the 8 values of one lane to e4m3 with the scale of its 128-element group (the 16 consecutive lanes that
// hold the group): returns the packed bytes, sets `scale` (the same on all 16 lanes).
MSCCLPP_DEVICE_INLINE uint2 quantizeWordE4m3(const float (&f)[8], float& scale) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  scale = amax > 0.f ? amax * (1.f / 448.f) : 1.f;
  const float inv = 1.f / scale;
  uint32_t q2[2];
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i] * inv, f[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i + 2] * inv, f[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    q2[i] = lo | (hi << 16);
  }
  return make_uint2(q2[0], q2[1]);
}

// 16 e4m3 bytes -> 16 floats (not yet scaled).
MSCCLPP_DEVICE_INLINE void e4m3x16ToFloat(const uint4& v, float (&f)[16]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffffu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    f[4 * i] = a.x;
    f[4 * i + 1] = a.y;
    f[4 * i + 2] = b.x;
    f[4 * i + 3] = b.y;
  }
}

__global__ void __launch_bounds__(kThreads, 1) moeDispatchKernel(MoeDispatchArgs a) {
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const int world = c.world;
  const uint32_t epoch = launchEpoch(c, rank);
  const uint64_t base = c.peerBase[c.rank];
  const uint64_t local = c.peerBase[rank];
  const uint64_t wsOff = reinterpret_cast<uint64_t>(a.workspace) - base;
  const Workspace ws = workspaceOf(c, rank, wsOff);
  // local operands: addressed through the (emulated) rank's heap base
  const bf16* x = reinterpret_cast<const bf16*>(local + (reinterpret_cast<uint64_t>(a.x) - base));
  const int32_t* topkIdx = reinterpret_cast<const int32_t*>(local + (reinterpret_cast<uint64_t>(a.topkIdx) - base));
  int32_t* slotMap = reinterpret_cast<int32_t*>(local + (reinterpret_cast<uint64_t>(a.slotMap) - base));
  int32_t* recvCounts = reinterpret_cast<int32_t*>(local + (reinterpret_cast<uint64_t>(a.recvCounts) - base));
  const uint64_t recvXOff = reinterpret_cast<uint64_t>(a.recvX) - base;
  const uint64_t recvScalesOff = a.recvScales ? reinterpret_cast<uint64_t>(a.recvScales) - base : 0;
  const uint64_t recvSrcOff = reinterpret_cast<uint64_t>(a.recvSrc) - base;
  const int E = a.numExperts, El = E / world;
  const int pairs = a.tokens * a.topk;
  SymmControl* ctl = control(c, rank);

  __shared__ uint32_t counts[kMaxRanks][kMoeMaxExperts];  // [source rank][expert]
  __shared__ uint32_t firstRow[kMoeMaxExperts];           // first destination row of my group of expert e
  __shared__ int overflow;

  // ---- A. position of every pair inside its (me, expert) group
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += gridDim.x * blockDim.x) {
    const int e = topkIdx[i];
    slotMap[i] = (e >= 0 && e < E) ? static_cast<int32_t>(atomicAdd(&ws.cnt[e], 1u)) : -1;
  }
  bool healthy = gridBarrier(c, rank, &ctl->gridSync[0], gridDim.x);

  // ---- B. block 0 sends my counts to everybody (its own matrix row included), then re-arms the counters
  if (blockIdx.x == 0 && healthy) {
    for (int i = threadIdx.x; i < world * E; i += blockDim.x) {
      const int p = i / E, e = i % E;
      uint2* dst = workspaceOf(c, p, wsOff).matrix + rank * kMoeMaxExperts + e;
      ptx::st_volatile_v2(dst, make_uint2(ws.cnt[e], epoch));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) ws.cnt[e] = 0;
  }

  // ---- C. every block collects the whole matrix and derives the first row of each of its groups
  if (threadIdx.x == 0) overflow = 0;
  __syncthreads();
  if (healthy) {
    for (int i = threadIdx.x; i < world * E; i += blockDim.x) {
      const int s = i / E, e = i % E;
      const uint2* src = ws.matrix + s * kMoeMaxExperts + e;
      SpinGuard g(c.status, c.timeoutNs);
      uint2 v = ptx::ld_volatile_v2(src);
      while (v.y != epoch) {
        if (!g.keepSpinning()) {
          g.report(kDevTimeoutFlag, rank, 6000 + s, e, epoch, v.y);
          overflow = 2;
          break;
        }
        v = ptx::ld_volatile_v2(src);
      }
      counts[s][e] = v.x;
    }
  }
  __syncthreads();
  if (healthy && overflow == 0) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const int d = e / El;
      uint32_t row = 0, rankTotal = 0;
      for (int e2 = d * El; e2 < (d + 1) * El; e2++) {
        uint32_t tot = 0;
        for (int s = 0; s < world; s++) tot += counts[s][e2];
        if (e2 < e) row += tot;
        rankTotal += tot;
      }
      for (int s = 0; s < rank; s++) row += counts[s][e];
      firstRow[e] = row;
      if (rankTotal > static_cast<uint32_t>(a.capacity)) atomicExch(&overflow, 1);
      if (blockIdx.x == 0 && d == rank) {
        uint32_t tot = 0;
        for (int s = 0; s < world; s++) tot += counts[s][e];
        recvCounts[e - d * El] = static_cast<int32_t>(tot);
        if (e == d * El) recvCounts[El] = static_cast<int32_t>(rankTotal);
      }
    }
  }
  __syncthreads();
  if (overflow == 1 && blockIdx.x == 0 && threadIdx.x == 0 && c.status != nullptr) {
    // a destination would receive more rows than its buffer holds: nothing is sent, the host sees the error
    SpinGuard g(c.status, c.timeoutNs);
    g.report(kDevErrorCapacity, rank, 6100, 0, static_cast<uint64_t>(a.capacity), 0);
  }
  const bool send = healthy && overflow == 0;

  // ---- D. one warp per token: load the row once, store it to each destination
  const int lane = threadIdx.x & 31;
  const int warpsPerBlock = blockDim.x >> 5;
  const int warp = blockIdx.x * warpsPerBlock + (threadIdx.x >> 5);
  const int numWarps = gridDim.x * warpsPerBlock;
  const int words = a.hidden / 8;  // 16-byte words per bf16 row
  const int scalesPerRow = a.hidden / kMoeScaleGroup;
  if (send) {
    for (int t = warp; t < a.tokens; t += numWarps) {
      int dstRank[kMoeMaxTopk], dstRow[kMoeMaxTopk], dstK[kMoeMaxTopk];
      int nd = 0;
      for (int k = 0; k < a.topk; k++) {
        const int e = topkIdx[t * a.topk + k];
        if (e < 0 || e >= E) continue;
        dstRank[nd] = e / El;
        dstRow[nd] = static_cast<int>(firstRow[e]) + slotMap[t * a.topk + k];  // slotMap holds the position in the group
        dstK[nd] = k;
        nd++;
      }
      __syncwarp();  // every lane has read the positions before lane 0 replaces them by the final rows
      if (lane == 0) {
        for (int q = 0; q < nd; q++) slotMap[t * a.topk + dstK[q]] = dstRow[q];
      }
      if (nd == 0) continue;
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * a.hidden);
      if (!a.fp8) {
#pragma unroll 1
        for (int w0 = 0; w0 < words; w0 += 32 * 8) {
          uint4 v[8];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int w = w0 + j * 32 + lane;
            v[j] = w < words ? ptx::ld_nc_na_v4(src + w) : make_uint4(0, 0, 0, 0);
          }
          for (int q = 0; q < nd; q++) {
            const uint64_t rowBase = c.peerBase[dstRank[q]] + recvXOff + static_cast<uint64_t>(dstRow[q]) * a.hidden * 2;
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const int w = w0 + j * 32 + lane;
              if (w < words) ptx::st_na_v4(reinterpret_cast<void*>(rowBase + static_cast<uint64_t>(w) * 16), v[j]);
            }
          }
        }
      } else {
        // 32 lanes x 8 elements = 256 elements per step = two scale groups (lanes 0-15, 16-31). Eight steps are loaded
        // before the first is quantised, so a lane keeps 128 bytes of the row in flight instead of 16.
#pragma unroll 1
        for (int w0 = 0; w0 < words; w0 += 32 * 8) {
          uint4 v[8];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int w = w0 + j * 32 + lane;
            v[j] = w < words ? ptx::ld_nc_na_v4(src + w) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int w = w0 + j * 32 + lane;
            float f[8];
            Vec16<bf16>::toFloat(v[j], f);
            float scale;
            const uint2 packed = quantizeWordE4m3(f, scale);
            if (w < words) {
              for (int q = 0; q < nd; q++) {
                const uint64_t peer = c.peerBase[dstRank[q]];
                ptx::st_volatile_v2(reinterpret_cast<void*>(peer + recvXOff + static_cast<uint64_t>(dstRow[q]) * a.hidden + static_cast<uint64_t>(w) * 8), packed);
                if ((lane & 15) == 0) {
                  float* sc = reinterpret_cast<float*>(peer + recvScalesOff) + static_cast<uint64_t>(dstRow[q]) * scalesPerRow + w / 16;
                  ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(sc), __float_as_uint(scale));
                }
              }
            }
          }
        }
      }
      if (lane == 0) {
        for (int q = 0; q < nd; q++) {
          int32_t* dst = reinterpret_cast<int32_t*>(c.peerBase[dstRank[q]] + recvSrcOff) + dstRow[q];
          ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(dst), (static_cast<uint32_t>(rank) << 24) | static_cast<uint32_t>(t));
        }
      }
    }
  } else {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += gridDim.x * blockDim.x) slotMap[i] = -1;
  }
  // every row of mine is on its way: after this barrier the rows sent TO me have landed
  if (healthy) rankBarrier(c, rank, 0, blockIdx.x, epoch);
  finishLaunch(c, rank, epoch);
}

__global__ void __launch_bounds__(kThreads, 1) moeCombineKernel(MoeCombineArgs a) {
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const int world = c.world;
  const uint32_t epoch = launchEpoch(c, rank);
  const uint64_t base = c.peerBase[c.rank];
  const uint64_t local = c.peerBase[rank];
  const int32_t* topkIdx = reinterpret_cast<const int32_t*>(local + (reinterpret_cast<uint64_t>(a.topkIdx) - base));
  const float* weights = reinterpret_cast<const float*>(local + (reinterpret_cast<uint64_t>(a.topkWeights) - base));
  const int32_t* slotMap = reinterpret_cast<const int32_t*>(local + (reinterpret_cast<uint64_t>(a.slotMap) - base));
  bf16* y = reinterpret_cast<bf16*>(local + (reinterpret_cast<uint64_t>(a.y) - base));
  const uint64_t outOff = reinterpret_cast<uint64_t>(a.expertOut) - base;
  const uint64_t scalesOff = a.fp8 ? reinterpret_cast<uint64_t>(a.outScales) - base : 0;
  const int scalesPerRow = a.hidden / kMoeScaleGroup;
  const int El = a.numExperts / world;
  const int words = a.hidden / 8;

  // the peers' expert outputs are final once their kernels run
  const bool healthy = rankBarrier(c, rank, 0, blockIdx.x, epoch);
  const int lane = threadIdx.x & 31;
  const int warpsPerBlock = blockDim.x >> 5;
  const int numWarps = gridDim.x * warpsPerBlock;
  if (healthy) {
    for (int t = blockIdx.x * warpsPerBlock + (threadIdx.x >> 5); t < a.tokens; t += numWarps) {
      uint64_t rowBase[kMoeMaxTopk];
      uint64_t scaleBase[kMoeMaxTopk];
      float wgt[kMoeMaxTopk];
      int nd = 0;
      for (int k = 0; k < a.topk; k++) {
        const int e = topkIdx[t * a.topk + k];
        const int row = slotMap[t * a.topk + k];
        if (e < 0 || e >= a.numExperts || row < 0) continue;
        rowBase[nd] = c.peerBase[e / El] + outOff + static_cast<uint64_t>(row) * a.hidden * (a.fp8 ? 1 : 2);
        scaleBase[nd] = c.peerBase[e / El] + scalesOff + static_cast<uint64_t>(row) * scalesPerRow * 4;
        wgt[nd] = weights[t * a.topk + k];
        nd++;
      }
      uint4* dst = reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * a.hidden);
      if (a.fp8) {
        // a lane's 16-byte word holds 16 values; the 8 lanes of a 128-element group share one scale
        const int words16 = a.hidden / 16;
#pragma unroll 1
        for (int w0 = 0; w0 < words16; w0 += 32 * 4) {
          float acc[4][16];
#pragma unroll
          for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int i = 0; i < 16; i++) acc[j][i] = 0.f;
          }
          for (int q = 0; q < nd; q++) {
            uint4 v[4];
            float sc[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const int w = w0 + j * 32 + lane;
              v[j] = make_uint4(0, 0, 0, 0);
              sc[j] = 0.f;
              if (w < words16) {
                v[j] = ptx::ld_nc_na_v4(reinterpret_cast<const void*>(rowBase[q] + static_cast<uint64_t>(w) * 16));
                sc[j] = __uint_as_float(ptx::ld_relaxed_sys(reinterpret_cast<const uint32_t*>(scaleBase[q]) + w / 8));
              }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
              float f[16];
              e4m3x16ToFloat(v[j], f);
              const float m = wgt[q] * sc[j];
#pragma unroll
              for (int i = 0; i < 16; i++) acc[j][i] += m * f[i];
            }
          }
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int w = w0 + j * 32 + lane;
            if (w < words16) {
              float lo[8], hi[8];
#pragma unroll
              for (int i = 0; i < 8; i++) {
                lo[i] = acc[j][i];
                hi[i] = acc[j][8 + i];
              }
              dst[2 * w] = Vec16<bf16>::fromFloat(lo);
              dst[2 * w + 1] = Vec16<bf16>::fromFloat(hi);
            }
          }
        }
        continue;
      }
#pragma unroll 1
      for (int w0 = 0; w0 < words; w0 += 32 * 4) {
        float acc[4][8];
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
          for (int i = 0; i < 8; i++) acc[j][i] = 0.f;
        }
        for (int q = 0; q < nd; q++) {
          uint4 v[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int w = w0 + j * 32 + lane;
            v[j] = w < words ? ptx::ld_nc_na_v4(reinterpret_cast<const void*>(rowBase[q] + static_cast<uint64_t>(w) * 16)) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int j = 0; j < 4; j++) {
            float f[8];
            Vec16<bf16>::toFloat(v[j], f);
#pragma unroll
            for (int i = 0; i < 8; i++) acc[j][i] += wgt[q] * f[i];
          }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int w = w0 + j * 32 + lane;
          if (w < words) dst[w] = Vec16<bf16>::fromFloat(acc[j]);
        }
      }
    }
  }
  // my reads are done: the peers may overwrite their expert outputs after this
  if (healthy) rankBarrier(c, rank, 1, blockIdx.x, epoch);
  finishLaunch(c, rank, epoch);
}

// One warp per row: the dispatch's quantiser as a stand-alone pass (for expert outputs that are to be combined as fp8).
__global__ void __launch_bounds__(kThreads) moeQuantizeRowsKernel(const bf16* x, uint8_t* q, float* scales, int rows, int hidden) {
  const int lane = threadIdx.x & 31;
  const int warpsPerBlock = blockDim.x >> 5;
  const int words = hidden / 8;
  const int scalesPerRow = hidden / kMoeScaleGroup;
  for (int r = blockIdx.x * warpsPerBlock + (threadIdx.x >> 5); r < rows; r += gridDim.x * warpsPerBlock) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * hidden);
#pragma unroll 1
    for (int w0 = 0; w0 < words; w0 += 32 * 8) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int w = w0 + j * 32 + lane;
        v[j] = w < words ? src[w] : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int w = w0 + j * 32 + lane;
        float f[8];
        Vec16<bf16>::toFloat(v[j], f);
        float scale;
        const uint2 packed = quantizeWordE4m3(f, scale);
        if (w < words) {
          *reinterpret_cast<uint2*>(q + static_cast<size_t>(r) * hidden + static_cast<size_t>(w) * 8) = packed;
          if ((lane & 15) == 0) scales[static_cast<size_t>(r) * scalesPerRow + w / 16] = scale;
        }
      }
    }
  }
}

template <typename Kernel, typename Args>
cudaError_t launchCoop(Kernel kernel, const Args& args, int nBlocks, int emu, cudaStream_t stream) {
  dim3 grid(nBlocks, emu > 1 ? emu : 1, 1);
  dim3 block(kThreads, 1, 1);
  Args copy = args;
  void* params[] = {&copy};
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, params, 0, stream);
}

int defaultBlocks(int emu) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int n = sms / (emu > 1 ? emu : 1);
  if (n > 64) n = 64;  // NVLink-bound: 64 blocks x 16 warps x 8 KB rows keep several MB in flight
  return n < 1 ? 1 : n;
}

bool validCommon(const DeviceComm& c, int tokens, int hidden, int topk, int numExperts, int emu) {
  if (tokens < 0 || tokens >= (1 << 24) || hidden <= 0 || hidden % 256 != 0 || hidden > 32 * kMaxWordsPerLane * 8) return false;
  if (topk < 1 || topk > kMoeMaxTopk || numExperts < c.world || numExperts > kMoeMaxExperts || numExperts % c.world != 0) return false;
  if (emu > 1 && emu != c.world) return false;
  return true;
}

}  // namespace

cudaError_t launchMoeDispatch(const MoeDispatchArgs& args, int nBlocks, cudaStream_t stream) {
  const int emu = args.emuRanks > 1 ? args.emuRanks : 1;
  if (!validCommon(args.comm, args.tokens, args.hidden, args.topk, args.numExperts, emu)) return cudaErrorInvalidValue;
  if (args.capacity <= 0 || (args.fp8 && args.recvScales == nullptr)) return cudaErrorInvalidValue;
  if (nBlocks <= 0) nBlocks = defaultBlocks(emu);
  if (nBlocks > kBarrierSlots) return cudaErrorInvalidValue;
  return launchCoop(moeDispatchKernel, args, nBlocks, emu, stream);
}

cudaError_t launchMoeQuantizeRows(const __nv_bfloat16* x, void* q, float* scales, int rows, int hidden, cudaStream_t stream) {
  if (rows < 0 || hidden <= 0 || hidden % 256 != 0) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  const int warpsPerBlock = kThreads / 32;
  int blocks = (rows + warpsPerBlock - 1) / warpsPerBlock;
  if (blocks > 148 * 4) blocks = 148 * 4;
  moeQuantizeRowsKernel<<<blocks, kThreads, 0, stream>>>(x, static_cast<uint8_t*>(q), scales, rows, hidden);
  return cudaGetLastError();
}

cudaError_t launchMoeCombine(const MoeCombineArgs& args, int nBlocks, cudaStream_t stream) {
  const int emu = args.emuRanks > 1 ? args.emuRanks : 1;
  if (!validCommon(args.comm, args.tokens, args.hidden, args.topk, args.numExperts, emu)) return cudaErrorInvalidValue;
  if (args.fp8 && args.outScales == nullptr) return cudaErrorInvalidValue;
  if (nBlocks <= 0) nBlocks = defaultBlocks(emu);
  if (nBlocks > kBarrierSlots) return cudaErrorInvalidValue;
  return launchCoop(moeCombineKernel, args, nBlocks, emu, stream);
}

}  // namespace mscclpp
