// Host entry points of the tcgen05 bf16 GEMM and helpers shared by the fused GEMM+collective kernels.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include <mscclpp/poll_device.hpp>

namespace mscclpp {
namespace gemm {

struct Shape {
  int M, N, K;
  int aBoxRows;  // rows of the A tensor-map box: min(kBlockM, M); rows beyond it are never stored
  int rowMajorTiles;  // 0: consecutive tiles walk M (share a B tile); 1: walk N inside one row block, so
                      // that row blocks complete in order (what a fused consumer of whole rows wants)
  int mOrder;       // order in which row blocks are visited: 0 natural; 1 interleaved over mOrderParam equal groups
                    // (0, per, 2*per, ..., 1, per+1, ...: every group completes a block per round - reduce-scatter
                    // owners all have work at once); 2 rotated by mOrderParam blocks (all-gather: own rows first);
                    // 3 bands of mOrderParam row blocks walked row-block-first (L2-friendly order of a plain GEMM)
  int mOrderParam;
  int probe;  // diagnostics, 0 in production: bit 0 = the producer issues no loads (stages are handed over empty), bit 1 = no
              // MMAs are issued (barriers only), bit 2 = the epilogue drops its blocks instead of storing them, bit 3 = it does not even read the accumulator. Timing the
              // kernel with each bit shows which of the three pipelines bounds a shape; results are then meaningless.
  unsigned long long* stamps;  // optional time line, kStampWords words per CTA (null = off), all in globaltimer ns:
                               // [0] CTA start, [1] last MMA issued, [2] ns the MMA thread waited for a free accumulator,
                               // [3] ns it waited for operands, [4] epilogue warp 2: last tile part stored, [5] ns it
                               // waited for a full accumulator, [6] ns it spent in Epilogue::block, [7] its drain done,
                               // [8] ns the producer waited for a free stage; [9..15] belong to the epilogue
};
constexpr int kStampWords = 16;


// Encodes a 2-D bf16 tensor map (row-major [rows, cols], 128-byte swizzle, box = [boxRows, 64]).
// Returns cudaErrorNotSupported when the driver entry point is unavailable.
cudaError_t makeTensorMapBf16(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t rowStrideBytes,
                              uint32_t boxRows);

// D[M, ldd] (bf16) = A[M, K] * B[N, K]^T, fp32 accumulation on the 5th-generation tensor cores.
// blockN in {64, 128, 256}; N % blockN == 0; K % 64 == 0; numCtas <= 0 picks one CTA per SM.
// band: row blocks per band of the tile order (0 = default, < 0 = none); probe: see Shape::probe.
cudaError_t gemmBf16(const void* A, const void* B, void* D, int M, int N, int K, int ldd, int blockN, int numCtas,
                     DeviceStatus* status, cudaStream_t stream, int probe = 0, int band = 0);

// Same product on 256 x 256 tiles shared by pairs of SMs (tcgen05 cta_group::2, clusters of two CTAs).
// N % 256 == 0; K % 64 == 0; numCtas <= 0 picks one CTA per SM (rounded down to an even number).
cudaError_t gemmBf16TwoSm(const void* A, const void* B, void* D, int M, int N, int K, int ldd, int numCtas, DeviceStatus* status,
                          cudaStream_t stream, int probe = 0, int band = 0);

// Raises the kernel's dynamic shared-memory limit once per (kernel, device); call before every launch that needs > 48 KB.
cudaError_t ensureDynamicSmem(const void* kernel, int bytes);

// Launch helper for kernels built on the two-SM core: clusters of two CTAs along x, optionally cooperative.
cudaError_t launchClusterPair(const void* kernel, dim3 grid, dim3 block, size_t smemBytes, void** params, bool cooperative,
                              cudaStream_t stream);

int smCount();

}  // namespace gemm
}  // namespace mscclpp
