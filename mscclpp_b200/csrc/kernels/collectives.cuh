// Argument block and launch entry points of the native collective kernels (allreduce, allgather,
// reduce-scatter, with an optional fused residual-add + RMSNorm epilogue).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include <mscclpp/device/symm.cuh>
#include <mscclpp/gpu_data_types.hpp>

namespace mscclpp {

enum CollMode : int { kAllReduce = 0, kReduceScatter = 1, kAllGather = 2, kBroadcast = 3, kAllToAll = 4 };

struct CollArgs {
  DeviceComm comm;
  const void* in;      // local buffer of rank comm.rank; emulated rank e uses in + e * emuStride
  void* out;
  uint64_t bytes;      // allreduce / broadcast / all-to-all: buffer bytes; reduce-scatter: input bytes; allgather: output bytes
  uint64_t emuStride;  // 0 unless several ranks are emulated in one launch on one GPU
  int emuRanks;        // gridDim.y (1 = real multi-GPU mode)
  int mode;            // CollMode
  int nvls;            // use multimem through comm.mcBase
  // fused epilogue: out = rmsnorm(allreduce(in) + residualIn) * gamma, residualOut = allreduce(in) + residualIn
  int norm;
  int rows;
  int hidden;          // elements per row
  float eps;
  const void* residualIn;   // [rows, hidden] local, replicated on every rank (may be null)
  void* residualOut;        // [rows, hidden] local (may be null)
  const void* gamma;        // [hidden] (may be null = all ones)
  int broadcastResidual;    // two-shot only: write residualOut on every rank, not just the owner's rows
  int root;                 // kBroadcast: the rank whose `in` is copied into everybody's `out`
  int ll8;                  // one-shot allreduce only: 8-byte {data, flag} packets instead of 16-byte ones (peer stores, no norm)
  void* ll128Scratch;       // launchAllreduceLL128: symmetric-heap scratch of ll128ScratchBytes(world, slot) bytes at the same offset
  uint64_t ll128SlotBytes;  // on every rank, zeroed once before its first use; a slot takes ceil(bytes / 120) lines of 128 bytes
  unsigned long long* stamps;  // launchTwoShot, optional: five globaltimer reads of block 0 (entry, after the opening barrier,
                               // after its share of the work, after the closing barrier, at the end); null = none
  int oneShot;              // launchTwoShot, allreduce over peer loads: every rank reduces the whole buffer for itself (no stores
                            // to peers). 0 = the launcher decides (currently: never), 1 = always, 2 = never.
};

// One-shot LL16 allreduce (every rank sends its whole buffer to every peer as packets).
// Buffers may live anywhere in local memory. bytes <= comm.llSlotBytes / 2.
cudaError_t launchAllreduceLL(const CollArgs& args, DataType dtype, ReduceOp op, int nBlocks, int nThreads,
                              cudaStream_t stream);

// One-shot LL128 allreduce: as launchAllreduceLL with 128-byte lines (120 bytes of payload + flag) instead of 16-byte packets,
// for messages too long for 50 % scratch efficiency and too short for the two-shot algorithms. Any size and alignment (8-byte
// aligned buffers take the fast path); ceil(bytes / 120) * 128 <= args.ll128SlotBytes; peer stores only (no multimem form, no
// fused norm).
constexpr size_t ll128ScratchBytes(int world, size_t slotBytes) { return 2 * static_cast<size_t>(world) * slotBytes; }
cudaError_t launchAllreduceLL128(const CollArgs& args, DataType dtype, ReduceOp op, int nBlocks, int nThreads, cudaStream_t stream);

// Two-shot zero-copy allreduce / reduce-scatter / allgather over peer pointers or NVLS multimem.
// `in` and `out` must be symmetric-heap buffers at the same offset on every rank; bytes % 16 == 0.
cudaError_t launchTwoShot(const CollArgs& args, DataType dtype, ReduceOp op, int nBlocks, int nThreads,
                          cudaStream_t stream);

// Allreduce of buffers outside the symmetric heap through heap scratch, pipelined inside one kernel (see
// collectives_pipeline.cu). `scratch`: pipelineScratchBytes(nBlocks, sliceBytes) bytes of symmetric-heap memory at the
// same offset on every rank. sliceBytes: a multiple of 16 * world; one round moves nBlocks * sliceBytes of the message.
struct PipeArgs {
  DeviceComm comm;
  const void* in;      // local buffer, anywhere in device memory, 16-byte aligned; emulated rank e uses in + e * emuStride
  void* out;
  uint64_t bytes;      // any size (a tail shorter than 16 bytes is zero-padded inside the scratch)
  void* scratch;
  uint64_t sliceBytes;
  uint64_t emuStride;
  int emuRanks;
  int nvls;
};
size_t pipelineScratchBytes(int nBlocks, uint64_t sliceBytes);
cudaError_t launchPipelineAllreduce(const PipeArgs& args, DataType dtype, ReduceOp op, int nBlocks, int nThreads, cudaStream_t stream);

}  // namespace mscclpp
