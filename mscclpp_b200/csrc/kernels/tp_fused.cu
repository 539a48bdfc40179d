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
//
// The reference library has no counterpart: it provides the allreduce only.
#include "tp_fused.cuh"

#include <mscclpp/gpu_data_types.hpp>

#include "gemm_sm100.cuh"

namespace mscclpp {

namespace {

using bf16 = __nv_bfloat16;
constexpr int kMaxNBlk = 128;
constexpr int kRowsPerPass = 2;
constexpr int kUnitsPerThread = 4;  // 16-byte words of one row held by one thread (N <= 4 * 8 * blockDim)

struct TmapSet {
  CUtensorMap a[8];
  CUtensorMap b[8];
};

MSCCLPP_DEVICE_INLINE uint32_t* readyFlag(const DeviceComm& c, int owner, int mBlk, int src, int nBlk) {
  return reinterpret_cast<uint32_t*>(c.peerBase[owner] + c.auxFlagsOff) +
         ((static_cast<size_t>(mBlk) * kMaxRanks + src) * kMaxNBlk + nBlk);
}

struct PartialStoreSignal {
  const DeviceComm* comm;
  bf16* partial;  // this rank's partial product [M, N]
  int M, N;
  int rank;
  int rowsPerUnit;
  int numUnits;
  uint32_t epoch;

  MSCCLPP_DEVICE_INLINE void store(int row, int col, const uint32_t (&v)[32]) const {
    if (row >= M) return;
    uint4* dst = reinterpret_cast<uint4*>(partial + static_cast<size_t>(row) * N + col);
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

  // Called by all epilogue threads after a CTA-wide (epilogue) barrier: thread o tells rank o.
  MSCCLPP_DEVICE_INLINE void tileDone(int mBlk, int nBlk, int tid) const {
    const int world = comm->world;
    if (tid >= world) return;
    const int u0 = (mBlk * gemm::kBlockM) / rowsPerUnit;
    int u1 = ((mBlk + 1) * gemm::kBlockM + rowsPerUnit - 1) / rowsPerUnit;
    if (u1 > numUnits) u1 = numUnits;
    // does rank `tid` own one of the units [u0, u1)?
    const int first = (tid - (u0 % world) + world) % world;
    if (first >= u1 - u0) return;
    ptx::fence_acq_rel_sys();
    ptx::st_release_sys(readyFlag(*comm, tid, mBlk, rank, nBlk), epoch);
  }
};

// Sum of kRowsPerPass floats per thread over the CTA.
template <int R>
MSCCLPP_DEVICE_INLINE void blockSumMulti(float (&v)[R], float (&total)[R], float* smem /* [32 * R + R] */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int r = 0; r < R; r++) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[r] += __shfl_xor_sync(0xffffffffu, v[r], o);
  }
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < R; r++) smem[warp * R + r] = v[r];
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int r = 0; r < R; r++) {
      float s = lane < nwarps ? smem[lane * R + r] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) smem[32 * R + r] = s;
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; r++) total[r] = smem[32 * R + r];
}

template <bool kNvls>
MSCCLPP_DEVICE_INLINE uint4 gatherRowWord(const DeviceComm& c, uint64_t heapOff) {
  if constexpr (kNvls) {
    return ptx::multimem_ld_reduce_add_bf16x2_acc32(reinterpret_cast<const void*>(c.mcBase + heapOff));
  } else {
    uint4 v[8];
    float acc[8];
#pragma unroll
    for (int p = 0; p < 8; p++)
      if (p < c.world) v[p] = ptx::ld_nc_na_v4(reinterpret_cast<const void*>(c.peerBase[p] + heapOff));
    Vec16<bf16>::toFloat(v[0], acc);
#pragma unroll
    for (int p = 1; p < 8; p++)
      if (p < c.world) accumulate16<bf16, SUM>(acc, v[p]);
    for (int p = 8; p < c.world; p++)
      accumulate16<bf16, SUM>(acc, ptx::ld_nc_na_v4(reinterpret_cast<const void*>(c.peerBase[p] + heapOff)));
    return Vec16<bf16>::fromFloat(acc);
  }
}

template <bool kNvls>
MSCCLPP_DEVICE_INLINE void scatterWord(const DeviceComm& c, int rank, uint64_t heapOff, uint4 v) {
  if constexpr (kNvls) {
    ptx::multimem_st_v4(reinterpret_cast<void*>(c.mcBase + heapOff), v);
  } else {
    for (int i = 0; i < c.world; i++) {
      const int p = (rank + i) % c.world;
      ptx::st_na_v4(reinterpret_cast<void*>(c.peerBase[p] + heapOff), v);
    }
  }
}

template <bool kNvls>
MSCCLPP_DEVICE_INLINE void reducerCta(const TpFusedArgs& a, int rank, uint32_t epoch, int reducerIdx, int numReducers) {
  const DeviceComm& c = a.comm;
  const int world = c.world;
  const int M = a.shape.M, N = a.shape.N;
  const int numNBlk = N / a.blockN;
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

  __shared__ float redSmem[32 * kRowsPerPass + kRowsPerPass];
  __shared__ int okSmem;
  if (threadIdx.x == 0) okSmem = 1;
  __syncthreads();

  int readyMb = -1;
  bool healthy = true;
  // owned row j -> global row: unit = rank + (j / rpu) * world, row = unit * rpu + j % rpu
  for (int j0 = reducerIdx * kRowsPerPass; j0 < ownedRows && healthy; j0 += numReducers * kRowsPerPass) {
    int rows[kRowsPerPass];
#pragma unroll
    for (int r = 0; r < kRowsPerPass; r++) {
      const int j = j0 + r;
      const int row = (rank + (j / rpu) * world) * rpu + (j % rpu);
      rows[r] = (j < ownedRows && row < M) ? row : -1;
    }
    // ---- wait until every rank has produced every tile of the row blocks these rows live in
#pragma unroll
    for (int r = 0; r < kRowsPerPass; r++) {
      if (rows[r] < 0) continue;
      const int mb = rows[r] / gemm::kBlockM;
      if (mb == readyMb) continue;
      for (int i = threadIdx.x; i < world * numNBlk; i += blockDim.x) {
        const int src = i / numNBlk, nb = i % numNBlk;
        if (!waitGreaterEqual(readyFlag(c, rank, mb, src, nb), epoch, c.status, c.timeoutNs, kDevTimeoutFlag, rank,
                              7000 + mb, src)) {
          okSmem = 0;
        }
      }
      __syncthreads();
      readyMb = mb;
      if (okSmem == 0) healthy = false;
    }
    if (!healthy) break;

    // ---- pass 1: reduced partial + residual, kept in registers; row sum of squares.
    // All loads of the pass are issued before the first use, so one CTA keeps
    // 2 x kRowsPerPass x kUnitsPerThread x 16 B per thread in flight.
    uint4 h[kRowsPerPass][kUnitsPerThread];
    uint4 res[kRowsPerPass][kUnitsPerThread];
    float ss[kRowsPerPass];
#pragma unroll
    for (int r = 0; r < kRowsPerPass; r++) {
#pragma unroll
      for (int k = 0; k < kUnitsPerThread; k++) {
        const int ru = threadIdx.x + k * blockDim.x;
        h[r][k] = make_uint4(0, 0, 0, 0);
        res[r][k] = make_uint4(0, 0, 0, 0);
        if (rows[r] >= 0 && ru < unitsPerRow) {
          const uint64_t off = (static_cast<uint64_t>(rows[r]) * unitsPerRow + ru) * 16;
          h[r][k] = gatherRowWord<kNvls>(c, partialOff + off);
          if (a.residualIn) res[r][k] = ptx::ld_nc_na_v4(reinterpret_cast<const void*>(local + resInOff + off));
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerPass; r++) {
      ss[r] = 0.f;
#pragma unroll
      for (int k = 0; k < kUnitsPerThread; k++) {
        const int ru = threadIdx.x + k * blockDim.x;
        if (rows[r] >= 0 && ru < unitsPerRow) {
          float f[8];
          Vec16<bf16>::toFloat(h[r][k], f);
          if (a.residualIn) {
            float rf[8];
            Vec16<bf16>::toFloat(res[r][k], rf);
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] += rf[i];
            h[r][k] = Vec16<bf16>::fromFloat(f);
            Vec16<bf16>::toFloat(h[r][k], f);
          }
#pragma unroll
          for (int i = 0; i < 8; i++) ss[r] += f[i] * f[i];
        }
      }
    }
    if (a.residualOut) {
#pragma unroll
      for (int r = 0; r < kRowsPerPass; r++) {
#pragma unroll
        for (int k = 0; k < kUnitsPerThread; k++) {
          const int ru = threadIdx.x + k * blockDim.x;
          if (rows[r] >= 0 && ru < unitsPerRow) {
            const uint64_t off = (static_cast<uint64_t>(rows[r]) * unitsPerRow + ru) * 16;
            scatterWord<kNvls>(c, rank, resOutOff + off, h[r][k]);
          }
        }
      }
    }
    float total[kRowsPerPass];
    blockSumMulti<kRowsPerPass>(ss, total, redSmem);

    // ---- pass 2: normalise (mode 0) or publish 1/rms (mode 1)
    uint4 gam[kUnitsPerThread];
    if (a.mode != 1 && gamma) {
#pragma unroll
      for (int k = 0; k < kUnitsPerThread; k++) {
        const int ru = threadIdx.x + k * blockDim.x;
        gam[k] = ru < unitsPerRow ? *reinterpret_cast<const uint4*>(gamma + static_cast<size_t>(ru) * 16) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerPass; r++) {
      if (rows[r] < 0) continue;
      const float rinv = rsqrtf(total[r] / static_cast<float>(N) + a.eps);
      if (a.mode == 1) {
        if (threadIdx.x == 0) {
          const uint64_t off = rinvOff + static_cast<uint64_t>(rows[r]) * 4;
          if constexpr (kNvls) {
            ptx::multimem_st_u32(reinterpret_cast<void*>(c.mcBase + off), __float_as_uint(rinv));
          } else {
            for (int p = 0; p < world; p++) ptx::st_relaxed_sys(reinterpret_cast<uint32_t*>(c.peerBase[p] + off), __float_as_uint(rinv));
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < kUnitsPerThread; k++) {
          const int ru = threadIdx.x + k * blockDim.x;
          if (ru < unitsPerRow) {
            const uint64_t off = (static_cast<uint64_t>(rows[r]) * unitsPerRow + ru) * 16;
            float f[8];
            Vec16<bf16>::toFloat(h[r][k], f);
            if (gamma) {
              float g[8];
              Vec16<bf16>::toFloat(gam[k], g);
#pragma unroll
              for (int i = 0; i < 8; i++) f[i] = f[i] * rinv * g[i];
            } else {
#pragma unroll
              for (int i = 0; i < 8; i++) f[i] = f[i] * rinv;
            }
            scatterWord<kNvls>(c, rank, outOff + off, Vec16<bf16>::fromFloat(f));
          }
        }
      }
    }
  }
  // every store of mine is issued: meet the peers' reducers with the same index. After it, everything
  // their reducers wrote into my buffers has landed.
  if (healthy) rankBarrier(c, rank, 2, reducerIdx, epoch);
}

template <int kBlockN, bool kNvls>
__global__ void __launch_bounds__(gemm::kNumThreads, 1)
    tpFusedKernel(const __grid_constant__ TmapSet maps, const __grid_constant__ TpFusedArgs a) {
  extern __shared__ uint8_t smemRaw[];
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const uint32_t epoch = launchEpoch(c, rank);
  if (static_cast<int>(blockIdx.x) < a.numGemmCtas) {
    gemm::NoGate gate;
    const uint64_t partialOff = reinterpret_cast<uint64_t>(a.partial) - c.peerBase[c.rank];
    const int numUnits = (a.shape.M + a.rowsPerUnit - 1) / a.rowsPerUnit;
    PartialStoreSignal epi{&c, reinterpret_cast<bf16*>(c.peerBase[rank] + partialOff), a.shape.M, a.shape.N, rank,
                           a.rowsPerUnit, numUnits, epoch};
    gemm::gemmCta<kBlockN>(&maps.a[blockIdx.y], &maps.b[blockIdx.y], a.shape, blockIdx.x, a.numGemmCtas, gate, epi,
                           c.status, c.timeoutNs, smemRaw);
  } else {
    reducerCta<kNvls>(a, rank, epoch, blockIdx.x - a.numGemmCtas, gridDim.x - a.numGemmCtas);
  }
  finishLaunch(c, rank, epoch);
}

// out[row] = h[row] * rinv[row] * gamma (local pass of mode 1)
__global__ void __launch_bounds__(512) tpScaleRowsKernel(const bf16* h, const float* rinv, const bf16* gamma, bf16* out,
                                                         int M, int N) {
  const int unitsPerRow = N / 8;
  const size_t total = static_cast<size_t>(M) * unitsPerRow;
  for (size_t u = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < total;
       u += static_cast<size_t>(gridDim.x) * blockDim.x) {
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
cudaError_t launchTyped(const TmapSet& maps, const TpFusedArgs& args, int grid, cudaStream_t stream) {
  using Cfg = gemm::Config<kBlockN>;
  auto kernelNvls = tpFusedKernel<kBlockN, true>;
  auto kernelP2p = tpFusedKernel<kBlockN, false>;
  static bool attrSet = false;
  if (!attrSet) {
    cudaError_t e = cudaFuncSetAttribute(kernelNvls, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kernelP2p, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attrSet = true;
  }
  dim3 g(grid, args.emuRanks > 1 ? args.emuRanks : 1, 1);
  dim3 b(gemm::kNumThreads, 1, 1);
  auto kernel = args.nvls ? kernelNvls : kernelP2p;
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
  if (M <= 0 || N % args.blockN != 0 || K % gemm::kBlockK != 0) return cudaErrorInvalidValue;
  if (N / args.blockN > kMaxNBlk || world > 8) return cudaErrorInvalidValue;
  if (N * 2 / 16 > kUnitsPerThread * gemm::kNumThreads) return cudaErrorInvalidValue;
  const int numMBlk = (M + gemm::kBlockM - 1) / gemm::kBlockM;
  if (static_cast<uint64_t>(numMBlk) * kMaxRanks * kMaxNBlk * 4 > kAuxFlagBytes) return cudaErrorInvalidValue;
  if (args.mode == 1 && args.rinv == nullptr) return cudaErrorInvalidValue;
  if (args.nvls && args.comm.mcBase == 0) return cudaErrorInvalidValue;
  const int emu = args.emuRanks > 1 ? args.emuRanks : 1;
  if (emu > 8) return cudaErrorInvalidValue;
  args.shape.aBoxRows = M < gemm::kBlockM ? M : gemm::kBlockM;
  args.shape.rowMajorTiles = 1;
  if (args.rowsPerUnit <= 0) {
    int rpu = gemm::kBlockM;
    while (rpu > 1 && M < rpu * world) rpu >>= 1;
    args.rowsPerUnit = rpu;
  }
  TmapSet maps;
  for (int e = 0; e < emu; e++) {
    cudaError_t err = gemm::makeTensorMapBf16(&maps.a[e], A[e], M, K, static_cast<uint64_t>(K) * 2, args.shape.aBoxRows);
    if (err != cudaSuccess) return err;
    err = gemm::makeTensorMapBf16(&maps.b[e], B[e], N, K, static_cast<uint64_t>(K) * 2, args.blockN);
    if (err != cudaSuccess) return err;
  }
  const int tiles = numMBlk * (N / args.blockN);
  int sms = gemm::smCount() / emu;
  if (numReducers <= 0) numReducers = sms >= 64 ? 24 : 2;
  if (numReducers > kBarrierSlots) numReducers = kBarrierSlots;
  int gemmCtas = args.numGemmCtas > 0 ? args.numGemmCtas : sms - numReducers;
  if (gemmCtas > tiles) gemmCtas = tiles;
  if (gemmCtas < 1) gemmCtas = 1;
  args.numGemmCtas = gemmCtas;
  const int grid = gemmCtas + numReducers;
  switch (args.blockN) {
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
