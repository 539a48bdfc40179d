// Fused tensor-parallel layer: GEMM (tcgen05) + allreduce + residual add + RMSNorm in one launch.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mscclpp/device/symm.cuh>

#include "gemm.cuh"

namespace mscclpp {

struct TpFusedArgs {
  DeviceComm comm;
  gemm::Shape shape;            // M tokens, N = hidden, K = this rank's shard of the reduction dimension
  __nv_bfloat16* partial;       // symmetric [M, N]: this rank's partial product (written by the GEMM CTAs)
  const __nv_bfloat16* residualIn;   // symmetric-heap [M, N], replicated content (may be null)
  __nv_bfloat16* residualOut;   // symmetric [M, N]: receives h on every rank (may be null in mode 0)
  __nv_bfloat16* out;           // symmetric [M, N]: normalised output (mode 0: written by the owners everywhere)
  const __nv_bfloat16* gamma;   // [N] local (may be null)
  float* rinv;                  // symmetric [M] fp32, mode 1 only
  float eps;
  int blockN;                   // GEMM N tile: 64, 128 or 256; 0 = 256 x 256 tiles on pairs of SMs (M >= 256, N % 256 == 0)
  int numGemmCtas;              // 0 = all SMs but the reducers
  int rowsPerUnit;              // ownership granule, power of two <= 128; 0 = pick from M and world
  int mode;                     // 0: owners broadcast out + residualOut; 1: owners broadcast residualOut + rinv;
                                // 2: reduce-scatter, out is this rank's [M / world, N] block (M % (world * 128) == 0);
                                // 3: as 1, and `out` is produced inside the same launch: owners announce every ownership
                                // unit whose rows have landed everywhere, and warps that have no row to reduce turn
                                // landed rows into out = h * rinv * gamma locally (no second launch)
  int nvls;                     // multimem through comm.mcBase instead of peer loads/stores
  int emuRanks;                 // > 1: that many emulated ranks in one cooperative launch (tests)
  int noFlags;                  // set by launchTpReduceNorm: rows are complete at kernel start, no per-block flags
  int sysFence;                 // 1: row-block flags go out as fence.acq_rel.sys + st.release.sys (the conservative form);
                                // 0 (default): GPU-scope fence + relaxed system-scope store. -1 on entry = read the
                                // environment variable MSCCLPP_TP_SYS_FENCE (unset = 0).
  unsigned long long* timeline; // optional device buffer, kTimelineWords words per CTA (of emulated rank 0's grid layout):
                                // [0] CTA start, [1] GEMM part done, [2] reducer part done (all globaltimer ns),
                                // [3] rows reduced by group 0, [4] ns group 0 waited for readiness, [5] ns it spent on rows,
                                // [6] time group 0 finished its first row, [8] ns of [5] in the gather (loads of all ranks'
                                // partial rows), [9] ns in residual add + sum of squares, [10] ns issuing the broadcast
                                // stores of h; GEMM CTAs: [11] ns spent counting finished tiles (fence + atomic), [12] the
                                // longest such call, [13] ns spent in calls that published row-block flags, [14] time of
                                // the last finished tile, [15] longest time between two finished tiles, [7] when that ended.
                                // The caller zeroes the buffer. Null = no stamps.
};

constexpr int kTimelineWords = 16;

// Layout of the fused kernel's part of a heap's aux flag region (DeviceComm::auxFlagsOff), shared with every host file
// that has to clear or place it: [kTpMaxMBlk][kMaxRanks] epoch-stamped "row block of rank src is complete" words, then
// kTpMaxMBlk tile counters (zero between launches).
constexpr int kTpMaxMBlk = 4096;
constexpr size_t kTpReadyFlagBytes = static_cast<size_t>(kTpMaxMBlk) * kMaxRanks * 4;
constexpr size_t kTpTileCounterOffset = kTpReadyFlagBytes;  // bytes from the start of the aux region
constexpr size_t kTpTileCounterBytes = static_cast<size_t>(kTpMaxMBlk) * 4;
static_assert(kTpTileCounterOffset + kTpTileCounterBytes <= kAuxFlagBytes, "aux flag region too small");
// mode 3: [kTpMaxUnits] "unit has landed on this rank" words written by the unit's owner (epoch-stamped), then [kTpMaxUnits]
// counters of finished rows per unit in the owner's own memory (zero between launches)
constexpr int kTpMaxUnits = 4096;
constexpr size_t kTpLandedOffset = 512u << 10;
constexpr size_t kTpUnitDoneOffset = kTpLandedOffset + static_cast<size_t>(kTpMaxUnits) * 4;
static_assert(kTpLandedOffset >= kTpTileCounterOffset + kTpTileCounterBytes && kTpUnitDoneOffset + static_cast<size_t>(kTpMaxUnits) * 4 <= kAuxFlagBytes,
              "aux flag region too small");

// A[e], B[e]: operands of (emulated) rank e; real multi-GPU use passes one entry each.
// A: [M, K] bf16 row-major activations, B: [N, K] bf16 row-major weights (nn.Linear layout).
cudaError_t launchTpFused(const TpFusedArgs& args, const void* const* A, const void* const* B, int numReducers,
                          cudaStream_t stream);

// The reducer half alone: allreduce + residual + RMSNorm of an existing [M, N] bf16 `partial` (modes 0 and 1 as above).
// Starts with a cross-rank barrier (every rank's partial is final), then every CTA is a reducer.
cudaError_t launchTpReduceNorm(const TpFusedArgs& args, int numCtas, cudaStream_t stream);

// One GPU, no collective: h = bf16(A * B^T) + residual written by the GEMM epilogue, which also writes every row's
// sum of squares in parts: sumsq[part][row], tpSumsqParts(N, blockN, twoSm) parts of M floats each, every word written
// exactly once (no clearing, no atomics); launchTpScaleRowsFromSumsq adds the parts up and produces the RMSNorm.
// twoSm selects the 256 x 256 pair tiles (M >= 256, N % 256 == 0), else one-SM tiles of blockN columns.
int tpSumsqParts(int N, int blockN, bool twoSm);
cudaError_t launchGemmResidualSumsq(const void* A, const void* B, const void* residual, void* h, float* sumsq, int M, int N, int K,
                                    int blockN, bool twoSm, DeviceStatus* status, cudaStream_t stream);
// out = h * rsqrt(sum_p sumsqParts[p][row] / N + eps) * gamma
cudaError_t launchTpScaleRowsFromSumsq(const void* h, const float* sumsqParts, int numParts, const void* gamma, void* out, int M, int N,
                                       float eps, cudaStream_t stream);

// The same single-GPU layer in ONE launch: h = bf16(A * B^T) + residual and out = h * rsqrt(mean(h^2) + eps) * gamma.
// Rows are normalised by the epilogue warps as soon as their 128-row block is complete, while the MMAs of later blocks
// run. `stamps`: optional zeroed device buffer of gemm::kStampWords words per CTA that receives a time line (one-SM tiles).
// `workspace`: tpLocalFusedWorkspaceBytes(M, N) bytes of device memory, 16-byte aligned (its counters are cleared here on `stream`).
size_t tpLocalFusedWorkspaceBytes(int M, int N);
cudaError_t launchTpLocalFused(const void* A, const void* B, const void* residual, void* h, void* out, const void* gamma, void* workspace,
                               int M, int N, int K, float eps, int blockN, bool twoSm, DeviceStatus* status, cudaStream_t stream,
                               int probe = 0, unsigned long long* stamps = nullptr);

// The layer for a handful of tokens (decode): one launch, no tensor-core tiles - every SM streams the weight rows of its
// slab of output columns, the slabs meet the other ranks in a one-shot LL packet allreduce done by the same thread
// blocks, residual add and RMSNorm follow in registers (see tp_decode.cu). Every rank ends up with the whole result.
constexpr int kTpDecodeMaxTokens = 8;
// this kernel's words in a heap's aux flag region: [kBarrierSlots][kTpDecodeMaxTokens] {fp32 row sum, epoch} pairs, behind the flags of
// the fused layer, of the all-gather GEMM and of the pipelined allreduce
constexpr uint64_t kTpDecodeAuxOffset = (4096ull * (kMaxRanks + 1) + 4096ull) * 4ull + 2ull * kBarrierSlots * kMaxRanks * 8ull;
static_assert(kTpDecodeAuxOffset % 8 == 0 && kTpDecodeAuxOffset + static_cast<uint64_t>(kBarrierSlots) * kTpDecodeMaxTokens * 8 <= kAuxFlagBytes, "aux flag region too small");
struct TpDecodeArgs {
  DeviceComm comm;
  const __nv_bfloat16* x[8];      // [T, K] activations of (emulated) rank e; real multi-GPU use fills entry 0
  const __nv_bfloat16* w[8];      // [N, K] weight shard of (emulated) rank e
  const __nv_bfloat16* residualIn;  // symmetric-heap [T, N], replicated content (may be null)
  __nv_bfloat16* residualOut;     // symmetric-heap [T, N] (may be null)
  __nv_bfloat16* out;             // symmetric-heap [T, N]
  const __nv_bfloat16* gamma;     // [N] local (may be null)
  int T, N, K;                    // T <= kTpDecodeMaxTokens, N % 8 == 0, K % 256 == 0, 128 KB + T * K * 4 bytes of shared memory
  float eps;
  int nvls;                       // packets leave through one multimem.st instead of world - 1 peer stores
  int emuRanks;
  int numCtas;                    // 0 = one thread block per SM
  int colsPerCta;                 // set by the launcher
  unsigned long long* stamps;     // optional time line: 8 words per thread block (globaltimer ns, thread 0): [0] entry,
                                  // [1] activations staged, [2] its warp's weight pieces consumed, [3] all warps done,
                                  // [4] allreduce + residual done, [5] row-sum shares of all blocks read, [6] last store
};
cudaError_t launchTpDecode(const TpDecodeArgs& args, cudaStream_t stream);

// Local pass of mode 1: out = h * rinv[row] * gamma.
cudaError_t launchTpScaleRows(const void* h, const float* rinv, const void* gamma, void* out, int M, int N,
                              cudaStream_t stream);

}  // namespace mscclpp
