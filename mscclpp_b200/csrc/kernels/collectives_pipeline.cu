// Allreduce for buffers that are NOT in the symmetric heap (ordinary cudaMalloc / framework tensors), in ONE kernel.
//
// Peers cannot address such buffers, so the data takes a detour through heap scratch; what matters is that the three
// legs overlap instead of running as copy-in -> collective -> copy-out launches. Every thread block owns one slice
// (sliceBytes) of each "round" of the message and runs, per round,
//
//   1. copy-in     user input  -> its slice of the local scratch-in            (local stores)
//   2. barrier A   with the blocks of the same index on every rank            (all slices of this index are staged)
//   3. reduce      this rank's 1/world of the slice: multimem.ld_reduce through the NVSwitch (or peer loads with an fp32
//                  accumulator), result to EVERY rank's scratch-out            (multimem.st or peer stores)
//   4. barrier B   (every rank's part of my scratch-out slice has landed)
//   5. copy-out    scratch-out -> user output                                  (local loads, L1 bypassed)
//
// Blocks never wait for other blocks of their own rank, so while one block sits in a barrier the others copy and
// reduce: with a few blocks per SM the NVLink transfers, the local copies and the barrier latencies overlap. Scratch is
// double buffered per block (round parity), which is what makes two barriers per round enough.
// One round that covers the whole message is the un-pipelined "reduce-scatter + all-gather through scratch" form.
//
// Role of the reference's allreduce_nvls_block_pipeline.cu:16-147 / allreduce_nvls_warp_pipeline.cu:14-112 (NVLS) and
// allreduce_rsag_pipeline.cu:85-221 / allreduce_rsag.cu:33-128 (peer loads). Those specialise warps or blocks per leg
// and chain them with device semaphores; here every block runs all legs on its own slice and the overlap comes from
// the blocks being out of step with one another.
#include "collectives.cuh"

namespace mscclpp {

namespace {

// Barrier words of this kernel live in the aux flag region behind those of the fused tensor-parallel kernels:
// u64 flags[2 phases][kBarrierSlots][kMaxRanks], value = (launch epoch << 32) | round + 1.
constexpr uint64_t kPipeFlagByteOffset = (4096ull * (kMaxRanks + 1) + 4096ull) * 4ull;
static_assert(kPipeFlagByteOffset % 8 == 0, "u64 flags");
static_assert(kPipeFlagByteOffset + 2ull * kBarrierSlots * kMaxRanks * 8ull <= kAuxFlagBytes, "aux flag region too small");

MSCCLPP_DEVICE_INLINE uint64_t* pipeFlag(const DeviceComm& c, int owner, int phase, int slot, int src) {
  return reinterpret_cast<uint64_t*>(c.peerBase[owner] + c.auxFlagsOff + kPipeFlagByteOffset) +
         ((static_cast<uint64_t>(phase) * kBarrierSlots + slot) * kMaxRanks + src);
}

// All threads of the block call it. Stores made by the block before the call are visible to the peers' blocks of the same
// slot after their call returns.
MSCCLPP_DEVICE_INLINE bool pipeBarrier(const DeviceComm& c, int rank, int phase, int slot, uint64_t token, int* okSmem) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < c.world && t != rank) {
    ptx::fence_acq_rel_sys();
    ptx::st_release_sys(pipeFlag(c, t, phase, slot, rank), token);
    if (!waitGreaterEqual(pipeFlag(c, rank, phase, slot, t), token, c.status, c.timeoutNs, kDevTimeoutBarrier, rank,
                          20000 + phase * 1000 + slot, t)) {
      *okSmem = 0;
    }
  }
  __syncthreads();
  return *okSmem != 0;
}

MSCCLPP_DEVICE_INLINE uint4 loadUnitTail(const char* base, uint64_t u, uint64_t bytes) {
  const uint64_t off = u * 16;
  if (off + 16 <= bytes) return *reinterpret_cast<const uint4*>(base + off);
  uint32_t w[4] = {0, 0, 0, 0};
  for (uint64_t i = off; i < bytes; i++) w[(i - off) >> 2] |= static_cast<uint32_t>(static_cast<uint8_t>(base[i])) << (8 * ((i - off) & 3));
  return make_uint4(w[0], w[1], w[2], w[3]);
}
MSCCLPP_DEVICE_INLINE void storeUnitTail(char* base, uint64_t u, uint64_t bytes, uint4 v) {
  const uint64_t off = u * 16;
  if (off + 16 <= bytes) {
    *reinterpret_cast<uint4*>(base + off) = v;
    return;
  }
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  for (uint64_t i = off; i < bytes; i++) base[i] = static_cast<char>(w[(i - off) >> 2] >> (8 * ((i - off) & 3)));
}

template <typename T, ReduceOp Op>
MSCCLPP_DEVICE_INLINE uint4 switchReduce(const void* mc) {
  if constexpr (__is_same(T, __half)) {
    if constexpr (Op == SUM) return ptx::multimem_ld_reduce_add_f16x2_acc32(mc);
    else return ptx::multimem_ld_reduce_min_f16x2(mc);
  } else if constexpr (__is_same(T, __nv_bfloat16)) {
    if constexpr (Op == SUM) return ptx::multimem_ld_reduce_add_bf16x2_acc32(mc);
    else return ptx::multimem_ld_reduce_min_bf16x2(mc);
  } else if constexpr (__is_same(T, f8e4m3)) {
    return ptx::multimem_ld_reduce_add_e4m3x4(mc);
  } else if constexpr (__is_same(T, f8e5m2)) {
    return ptx::multimem_ld_reduce_add_e5m2x4(mc);
  } else {
    return ptx::multimem_ld_reduce_add_f32(mc);
  }
}

template <typename T, ReduceOp Op>
constexpr bool switchReducible() {
  if (__is_same(T, __half) || __is_same(T, __nv_bfloat16)) return true;
  if (Op != SUM) return false;
  return __is_same(T, float) || __is_same(T, f8e4m3) || __is_same(T, f8e5m2);
}

template <typename T, ReduceOp Op, bool kFloat = IsFloatLike<T>::value>
struct PipeAccum;
template <typename T, ReduceOp Op>
struct PipeAccum<T, Op, true> {
  float acc[Vec16<T>::kElems];
  MSCCLPP_DEVICE_INLINE void init(uint4 v) { Vec16<T>::toFloat(v, acc); }
  MSCCLPP_DEVICE_INLINE void add(uint4 v) { accumulate16<T, Op>(acc, v); }
  MSCCLPP_DEVICE_INLINE uint4 result() const { return Vec16<T>::fromFloat(acc); }
};
template <typename T, ReduceOp Op>
struct PipeAccum<T, Op, false> {
  uint4 acc;
  MSCCLPP_DEVICE_INLINE void init(uint4 v) { acc = v; }
  MSCCLPP_DEVICE_INLINE void add(uint4 v) { acc = reduce16<T, Op>(acc, v); }
  MSCCLPP_DEVICE_INLINE uint4 result() const { return acc; }
};

template <typename T, ReduceOp Op, bool kNvls>
__global__ void __launch_bounds__(512, 2) pipelineAllreduceKernel(PipeArgs a) {
  const DeviceComm& c = a.comm;
  const int rank = deviceRank(c);
  const int world = c.world;
  const uint32_t epoch = launchEpoch(c, rank);
  const int slot = blockIdx.x;
  const uint64_t emu = static_cast<uint64_t>(blockIdx.y) * a.emuStride;
  const char* in = reinterpret_cast<const char*>(a.in) + emu;
  char* out = reinterpret_cast<char*>(a.out) + emu;
  const uint64_t bytes = a.bytes;
  const uint64_t nunits = (bytes + 15) / 16;
  const uint64_t sliceUnits = a.sliceBytes / 16;  // a multiple of `world`
  const uint64_t subUnits = sliceUnits / world;
  const uint64_t roundUnits = sliceUnits * gridDim.x;
  const uint64_t rounds = (nunits + roundUnits - 1) / roundUnits;
  // scratch (heap offset, equal on every rank): [parity][in | out][slot][sliceBytes]
  const uint64_t scratchOff = reinterpret_cast<uint64_t>(a.scratch) - c.peerBase[c.rank];
  const uint64_t local = c.peerBase[rank];
  __shared__ int okSmem;
  if (threadIdx.x == 0) okSmem = 1;
  __syncthreads();

  bool healthy = true;
  for (uint64_t r = 0; r < rounds && healthy; r++) {
    const uint64_t first = r * roundUnits + static_cast<uint64_t>(slot) * sliceUnits;  // first global unit of my slice
    const uint64_t parityOff = scratchOff + (r & 1) * (2ull * gridDim.x * a.sliceBytes);
    const uint64_t inSlice = parityOff + static_cast<uint64_t>(slot) * a.sliceBytes;
    const uint64_t outSlice = parityOff + (static_cast<uint64_t>(gridDim.x) + slot) * a.sliceBytes;
    const uint64_t token = (static_cast<uint64_t>(epoch) << 32) | (r + 1);
    const uint64_t have = first < nunits ? (nunits - first < sliceUnits ? nunits - first : sliceUnits) : 0;  // units of this slice that exist

    // 1. copy-in (nothing to do for a slice beyond the end of the message, but the barriers still run: peers may not know)
    for (uint64_t u = threadIdx.x; u < have; u += blockDim.x) {
      *reinterpret_cast<uint4*>(local + inSlice + u * 16) = loadUnitTail(in, first + u, bytes);
    }
    // 2. every rank has staged its slice of this index
    healthy = pipeBarrier(c, rank, 0, slot, token, &okSmem);
    if (!healthy) break;
    // 3. reduce my part of the slice, result to everybody's scratch-out
    {
      const uint64_t begin = static_cast<uint64_t>(rank) * subUnits;
      const uint64_t end = begin + subUnits < have ? begin + subUnits : have;
      constexpr int kUnroll = kNvls ? 4 : 2;  // peer loads hold `world` words per unit in registers
      for (uint64_t u0 = begin + threadIdx.x; u0 < end; u0 += static_cast<uint64_t>(blockDim.x) * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int k = 0; k < kUnroll; k++) {
          const uint64_t u = u0 + static_cast<uint64_t>(k) * blockDim.x;
          if (u >= end) continue;
          if constexpr (kNvls) {
            v[k] = switchReduce<T, Op>(reinterpret_cast<const void*>(c.mcBase + inSlice + u * 16));
          } else {
            PipeAccum<T, Op> acc;
            uint4 w[8];
#pragma unroll
            for (int p = 0; p < 8; p++)
              if (p < world) w[p] = ptx::ld_nc_na_v4(reinterpret_cast<const void*>(c.peerBase[p] + inSlice + u * 16));
            acc.init(w[0]);
#pragma unroll
            for (int p = 1; p < 8; p++)
              if (p < world) acc.add(w[p]);
            v[k] = acc.result();
          }
        }
#pragma unroll
        for (int k = 0; k < kUnroll; k++) {
          const uint64_t u = u0 + static_cast<uint64_t>(k) * blockDim.x;
          if (u >= end) continue;
          if constexpr (kNvls) {
            ptx::multimem_st_v4(reinterpret_cast<void*>(c.mcBase + outSlice + u * 16), v[k]);
          } else {
            for (int i = 0; i < world; i++) {
              const int p = (rank + i) % world;
              ptx::st_na_v4(reinterpret_cast<void*>(c.peerBase[p] + outSlice + u * 16), v[k]);
            }
          }
        }
      }
    }
    // 4. every rank's part of my scratch-out slice has landed
    healthy = pipeBarrier(c, rank, 1, slot, token, &okSmem);
    if (!healthy) break;
    // 5. copy-out
    for (uint64_t u = threadIdx.x; u < have; u += blockDim.x) {
      storeUnitTail(out, first + u, bytes, ptx::ld_nc_na_v4(reinterpret_cast<const void*>(local + outSlice + u * 16)));
    }
  }
  finishLaunch(c, rank, epoch);
}

template <typename T, ReduceOp Op>
cudaError_t launchPipeTyped(const PipeArgs& a, int nBlocks, int nThreads, cudaStream_t stream) {
  dim3 grid(nBlocks, a.emuRanks > 1 ? a.emuRanks : 1, 1);
  dim3 block(nThreads, 1, 1);
  const void* kernel;
  if (a.nvls) {
    if constexpr (switchReducible<T, Op>()) {
      kernel = reinterpret_cast<const void*>(pipelineAllreduceKernel<T, Op, true>);
    } else {
      kernel = reinterpret_cast<const void*>(pipelineAllreduceKernel<T, Op, false>);  // the switch cannot reduce this type: peer loads
    }
  } else {
    kernel = reinterpret_cast<const void*>(pipelineAllreduceKernel<T, Op, false>);
  }
  PipeArgs copy = a;
  void* params[] = {&copy};
  if (a.emuRanks > 1) return cudaLaunchCooperativeKernel(kernel, grid, block, params, 0, stream);
  return cudaLaunchKernel(kernel, grid, block, params, 0, stream);
}

}  // namespace

size_t pipelineScratchBytes(int nBlocks, uint64_t sliceBytes) { return 4ull * static_cast<size_t>(nBlocks) * sliceBytes; }

cudaError_t launchPipelineAllreduce(const PipeArgs& args, DataType dtype, ReduceOp op, int nBlocks, int nThreads, cudaStream_t stream) {
  const int world = args.comm.world;
  if (args.bytes == 0 || world < 1 || world > 8) return cudaErrorInvalidValue;
  if (nBlocks < 1 || nBlocks > kBarrierSlots || nThreads < 32 || nThreads > 512 || nThreads < world) return cudaErrorInvalidValue;
  if (args.sliceBytes == 0 || args.sliceBytes % (16ull * world) != 0) return cudaErrorInvalidValue;
  if (args.scratch == nullptr || (reinterpret_cast<uintptr_t>(args.scratch) & 15) != 0) return cudaErrorInvalidValue;
  if (args.nvls && args.comm.mcBase == 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(args.in) & 15) != 0 || (reinterpret_cast<uintptr_t>(args.out) & 15) != 0) return cudaErrorInvalidValue;
  const bool isMin = op == MIN;
  switch (dtype) {
    case DataType::FLOAT16:
      return isMin ? launchPipeTyped<__half, MIN>(args, nBlocks, nThreads, stream) : launchPipeTyped<__half, SUM>(args, nBlocks, nThreads, stream);
    case DataType::BFLOAT16:
      return isMin ? launchPipeTyped<__nv_bfloat16, MIN>(args, nBlocks, nThreads, stream)
                   : launchPipeTyped<__nv_bfloat16, SUM>(args, nBlocks, nThreads, stream);
    case DataType::FLOAT32:
      return isMin ? launchPipeTyped<float, MIN>(args, nBlocks, nThreads, stream) : launchPipeTyped<float, SUM>(args, nBlocks, nThreads, stream);
    case DataType::INT32:
      return isMin ? launchPipeTyped<int32_t, MIN>(args, nBlocks, nThreads, stream) : launchPipeTyped<int32_t, SUM>(args, nBlocks, nThreads, stream);
    case DataType::UINT32:
      return isMin ? launchPipeTyped<uint32_t, MIN>(args, nBlocks, nThreads, stream) : launchPipeTyped<uint32_t, SUM>(args, nBlocks, nThreads, stream);
    case DataType::UINT8:
      return isMin ? launchPipeTyped<uint8_t, MIN>(args, nBlocks, nThreads, stream) : launchPipeTyped<uint8_t, SUM>(args, nBlocks, nThreads, stream);
    case DataType::FLOAT8_E4M3:
      return isMin ? launchPipeTyped<f8e4m3, MIN>(args, nBlocks, nThreads, stream) : launchPipeTyped<f8e4m3, SUM>(args, nBlocks, nThreads, stream);
    case DataType::FLOAT8_E5M2:
      return isMin ? launchPipeTyped<f8e5m2, MIN>(args, nBlocks, nThreads, stream) : launchPipeTyped<f8e5m2, SUM>(args, nBlocks, nThreads, stream);
    case DataType::FLOAT8_E4M3B15:
      return isMin ? launchPipeTyped<f8e4m3b15, MIN>(args, nBlocks, nThreads, stream)
                   : launchPipeTyped<f8e4m3b15, SUM>(args, nBlocks, nThreads, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace mscclpp
