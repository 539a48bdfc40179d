// Expert-parallel MoE dispatch / combine over NVLink peer memory (all-to-all with data-dependent sizes).
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mscclpp/device/symm.cuh>

namespace mscclpp {

constexpr int kMoeMaxExperts = 256;
constexpr int kMoeMaxTopk = 8;
constexpr int kMoeScaleGroup = 128;  // elements per fp8 scale (1 x 128 blocks along the hidden dimension)

// Bytes of symmetric workspace the dispatch kernel needs (counters + count matrix).
constexpr size_t moeWorkspaceBytes() { return (kMoeMaxExperts + 2ull * kMaxRanks * kMoeMaxExperts) * sizeof(uint32_t) + 256; }

struct MoeDispatchArgs {
  DeviceComm comm;
  int tokens, hidden, topk, numExperts;  // numExperts over all ranks; rank r hosts experts [r * E/world, (r+1) * E/world)
  int capacity;                 // rows of recvX on every rank
  int fp8;                      // 0: rows travel as bf16; 1: as e4m3 with one fp32 scale per 128 elements
  const __nv_bfloat16* x;       // [tokens, hidden] (symmetric-heap memory when ranks are emulated)
  const int32_t* topkIdx;       // [tokens, topk] expert ids, -1 = unused slot
  int32_t* slotMap;             // [tokens, topk] out: row of the destination rank's recvX that holds this copy (-1 = none)
  void* recvX;                  // symmetric [capacity, hidden] bf16 (or uint8 e4m3): rows grouped by local expert
  float* recvScales;            // symmetric [capacity, hidden / 128] (fp8 only)
  int32_t* recvSrc;             // symmetric [capacity]: (source rank << 24) | source token
  int32_t* recvCounts;          // [E/world + 1] out: rows per local expert, then their total
  uint32_t* workspace;          // symmetric, moeWorkspaceBytes(), zero-initialised once
  int emuRanks;
};

struct MoeCombineArgs {
  DeviceComm comm;
  int tokens, hidden, topk, numExperts;
  const int32_t* topkIdx;       // [tokens, topk]
  const float* topkWeights;     // [tokens, topk]
  const int32_t* slotMap;       // [tokens, topk] from dispatch
  const void* expertOut;        // symmetric [capacity, hidden]: expert outputs in the rows dispatch assigned (bf16, or
                                // e4m3 bytes when fp8 is set)
  __nv_bfloat16* y;             // [tokens, hidden] out: sum_k w[t,k] * expertOut_{rank(e_k)}[slot(t,k)]
  int emuRanks;
  int fp8;                      // 1: expertOut holds e4m3 with one fp32 scale per 128 elements in outScales (half the
                                // bytes pulled over NVLink); the weighted sum is still taken in fp32
  const float* outScales;       // symmetric [capacity, hidden / 128] (fp8 only)
};

// Quantiser for the fp8 form of the combine (and for tests): q[r] = e4m3(x[r] / scale), scale = amax of each 128-element
// group / 448. x [rows, hidden] bf16, q [rows, hidden] bytes, scales [rows, hidden / 128]; hidden % 256 == 0.
cudaError_t launchMoeQuantizeRows(const __nv_bfloat16* x, void* q, float* scales, int rows, int hidden, cudaStream_t stream);

// nBlocks <= 0 picks a default. Both launches are cooperative (grid barriers, and emulated ranks wait on each other).
cudaError_t launchMoeDispatch(const MoeDispatchArgs& args, int nBlocks, cudaStream_t stream);
cudaError_t launchMoeCombine(const MoeCombineArgs& args, int nBlocks, cudaStream_t stream);

}  // namespace mscclpp
