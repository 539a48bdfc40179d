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
//   No staging buffer and no second pass.
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
        // 32 lanes x 8 elements = 256 elements per step = two scale groups (lanes 0-15, 16-31)
#pragma unroll 1
        for (int w0 = 0; w0 < words; w0 += 32) {
          const int w = w0 + lane;
          float f[8];
          Vec16<bf16>::toFloat(w < words ? ptx::ld_nc_na_v4(src + w) : make_uint4(0, 0, 0, 0), f);
          float amax = 0.f;
#pragma unroll
          for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          const float scale = amax > 0.f ? amax * (1.f / 448.f) : 1.f;
          const float inv = 1.f / scale;
          uint32_t q2[2];
#pragma unroll
          for (int i = 0; i < 2; i++) {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i] * inv, f[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i + 2] * inv, f[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
            q2[i] = lo | (hi << 16);
          }
          if (w < words) {
            for (int q = 0; q < nd; q++) {
              const uint64_t peer = c.peerBase[dstRank[q]];
              ptx::st_volatile_v2(reinterpret_cast<void*>(peer + recvXOff + static_cast<uint64_t>(dstRow[q]) * a.hidden + static_cast<uint64_t>(w) * 8),
                                  make_uint2(q2[0], q2[1]));
              if ((lane & 15) == 0) {
                float* sc = reinterpret_cast<float*>(peer + recvScalesOff) + static_cast<uint64_t>(dstRow[q]) * scalesPerRow + w / 16;
                ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(sc), __float_as_uint(scale));
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
      float wgt[kMoeMaxTopk];
      int nd = 0;
      for (int k = 0; k < a.topk; k++) {
        const int e = topkIdx[t * a.topk + k];
        const int row = slotMap[t * a.topk + k];
        if (e < 0 || e >= a.numExperts || row < 0) continue;
        rowBase[nd] = c.peerBase[e / El] + outOff + static_cast<uint64_t>(row) * a.hidden * 2;
        wgt[nd] = weights[t * a.topk + k];
        nd++;
      }
      uint4* dst = reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * a.hidden);
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

cudaError_t launchMoeCombine(const MoeCombineArgs& args, int nBlocks, cudaStream_t stream) {
  const int emu = args.emuRanks > 1 ? args.emuRanks : 1;
  if (!validCommon(args.comm, args.tokens, args.hidden, args.topk, args.numExperts, emu)) return cudaErrorInvalidValue;
  if (nBlocks <= 0) nBlocks = defaultBlocks(emu);
  if (nBlocks > kBarrierSlots) return cudaErrorInvalidValue;
  return launchCoop(moeCombineKernel, args, nBlocks, emu, stream);
}

}  // namespace mscclpp
