// Sequence-parallel fused kernels: all-gather -> GEMM and GEMM -> reduce-scatter, each ONE launch.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mscclpp/device/symm.cuh>

#include "gemm.cuh"

namespace mscclpp {

struct AgGemmArgs {
  DeviceComm comm;
  gemm::Shape shape;          // M = rows after the gather (all ranks), N = this rank's output columns, K
  const __nv_bfloat16* aLocal;  // symmetric [M / world, K]: this rank's rows (global rows rank * M / world ...)
  __nv_bfloat16* aFull;       // symmetric [M, K] workspace; peers' rows land here (own rows are read from aLocal)
  __nv_bfloat16* D;           // symmetric [M, N] output ([M, N / 2] with the gated activation)
  int blockN;                 // 128 or 256; 0 = 256 x 256 tiles on pairs of SMs (M % (world * 256) == 0)
  int numGemmCtas;            // 0 = all SMs but the copiers
  int activation;             // 0 none, 1 GELU (tanh form), 2 SiLU - applied to the fp32 accumulator; 3 SwiGLU: B's rows are
                              // gate / up features interleaved in groups of 32, D[:, 32 b + j] = silu(gate) * up, N / 2 columns
  int emuRanks;               // > 1: emulated ranks in one cooperative launch (tests)
};

// B[e]: [N, K] bf16 row-major weights of (emulated) rank e. numCopiers <= 0 picks a default.
// Requires M % (world * 128) == 0 and K % 128 == 0.
cudaError_t launchAllGatherGemm(const AgGemmArgs& args, const void* const* B, int numCopiers, cudaStream_t stream);

}  // namespace mscclpp
