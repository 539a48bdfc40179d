// Plain bf16 GEMM on tcgen05/TMEM (see gemm_sm100.cuh for the kernel body) and tensor-map helpers.
#include "gemm.cuh"

#include <mutex>
#include <set>
#include <utility>

#include "gemm2_sm100.cuh"
#include "gemm_sm100.cuh"

namespace mscclpp {
namespace gemm {

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encodeFn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(p);
    }
  });
  return fn;
}

template <int kBlockN>
__global__ void __launch_bounds__(kNumThreads, 1)
    gemmBf16Kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                   const __grid_constant__ CUtensorMap tmapD, Shape shape, DeviceStatus* status, uint64_t budgetNs) {
  extern __shared__ uint8_t smemRaw[];
  NoGate gate;
  StoreBf16 epi{&tmapD, shape.M};
  if (threadIdx.x == 0) ptx::tma_prefetch_desc(&tmapD);
  gemmCta<kBlockN>(&tmapA, &tmapB, shape, blockIdx.x, gridDim.x, gate, epi, status, budgetNs, smemRaw);
}

template <int kBlockN>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, Shape shape, int numCtas,
                   DeviceStatus* status, cudaStream_t stream) {
  using Cfg = Config<kBlockN>;
  cudaError_t e = ensureDynamicSmem(reinterpret_cast<const void*>(gemmBf16Kernel<kBlockN>), Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int tiles = ((shape.M + kBlockM - 1) / kBlockM) * (shape.N / kBlockN);
  int grid = numCtas > 0 ? numCtas : smCount();
  if (grid > tiles) grid = tiles;
  gemmBf16Kernel<kBlockN><<<grid, kNumThreads, Cfg::kSmemBytes, stream>>>(ta, tb, td, shape, status, 2000000000ull);
  return cudaGetLastError();
}

__global__ void __launch_bounds__(kNumThreads, 1)
    gemmBf16PairKernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                       const __grid_constant__ CUtensorMap tmapD, Shape shape, DeviceStatus* status, uint64_t budgetNs) {
  extern __shared__ uint8_t smemRaw[];
  NoGate gate;
  StoreBf16 epi{&tmapD, shape.M};
  if (threadIdx.x == 0) ptx::tma_prefetch_desc(&tmapD);
  gemmCtaPair(&tmapA, &tmapB, shape, blockIdx.x / 2, gridDim.x / 2, gate, epi, status, budgetNs, smemRaw);
}

// Tile order of a plain GEMM: bands of `band` row blocks (0 = the default for the tile shape, < 0 = plain column-major walk).
void setBandOrder(Shape& shape, int numMBlk, int band, int dflt) {
  if (band == 0) band = dflt;
  if (band > 0 && numMBlk > band) {
    shape.mOrder = 3;
    shape.mOrderParam = band;
  }
}

}  // namespace

cudaError_t ensureDynamicSmem(const void* kernel, int bytes) {
  // the attribute belongs to the (kernel, device) pair: a process that drives several GPUs sets it on each of them
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({kernel, dev})) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done.insert({kernel, dev});
  return e;
}

cudaError_t launchClusterPair(const void* kernel, dim3 grid, dim3 block, size_t smemBytes, void** params, bool cooperative,
                              cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 2;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeCooperative;
  attrs[1].val.cooperative = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = cooperative ? 2 : 1;
  return cudaLaunchKernelExC(&cfg, kernel, params);
}

cudaError_t gemmBf16TwoSm(const void* A, const void* B, void* D, int M, int N, int K, int ldd, int numCtas, DeviceStatus* status,
                          cudaStream_t stream, int probe, int band) {
  if (M <= 0 || N <= 0 || K <= 0 || K % kBlockK != 0 || N % Config2::kBlockN != 0 || ldd % 8 != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(D) & 15) != 0) return cudaErrorInvalidValue;
  Shape shape{M, N, K, kBlockM, 0, 0, 0, probe};
  setBandOrder(shape, (M + Config2::kPairM - 1) / Config2::kPairM, band, 8);
  CUtensorMap ta, tb, td;
  cudaError_t e = makeTensorMapBf16(&ta, A, M, K, static_cast<uint64_t>(K) * 2, kBlockM);
  if (e != cudaSuccess) return e;
  e = makeTensorMapBf16(&tb, B, N, K, static_cast<uint64_t>(K) * 2, Config2::kBlockN / 2);
  if (e != cudaSuccess) return e;
  e = makeTensorMapBf16(&td, D, M, N, static_cast<uint64_t>(ldd) * 2, 32);
  if (e != cudaSuccess) return e;
  e = ensureDynamicSmem(reinterpret_cast<const void*>(gemmBf16PairKernel), Config2::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int tiles = ((M + Config2::kPairM - 1) / Config2::kPairM) * (N / Config2::kBlockN);
  int grid = numCtas > 0 ? numCtas : smCount();
  grid &= ~1;
  if (grid > 2 * tiles) grid = 2 * tiles;
  if (grid < 2) grid = 2;
  uint64_t budget = 2000000000ull;
  void* params[] = {&ta, &tb, &td, &shape, &status, &budget};
  return launchClusterPair(reinterpret_cast<const void*>(gemmBf16PairKernel), dim3(grid), dim3(kNumThreads), Config2::kSmemBytes, params,
                           false, stream);
}

int smCount() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

cudaError_t makeTensorMapBf16(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t rowStrideBytes,
                              uint32_t boxRows) {
  EncodeFn fn = encodeFn();
  if (fn == nullptr) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (rowStrideBytes & 15) != 0) return cudaErrorInvalidValue;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {rowStrideBytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockK), boxRows};
  cuuint32_t elemStrides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elemStrides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t gemmBf16(const void* A, const void* B, void* D, int M, int N, int K, int ldd, int blockN, int numCtas,
                     DeviceStatus* status, cudaStream_t stream, int probe, int band) {
  if (M <= 0 || N <= 0 || K <= 0 || K % kBlockK != 0 || N % blockN != 0 || ldd % 8 != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(D) & 15) != 0) return cudaErrorInvalidValue;
  Shape shape{M, N, K, M < kBlockM ? M : kBlockM, 0, 0, 0, probe};
  setBandOrder(shape, (M + kBlockM - 1) / kBlockM, band, 16);
  CUtensorMap ta, tb, td;
  cudaError_t e = makeTensorMapBf16(&ta, A, M, K, static_cast<uint64_t>(K) * 2, shape.aBoxRows);
  if (e != cudaSuccess) return e;
  e = makeTensorMapBf16(&tb, B, N, K, static_cast<uint64_t>(K) * 2, blockN);
  if (e != cudaSuccess) return e;
  e = makeTensorMapBf16(&td, D, M, N, static_cast<uint64_t>(ldd) * 2, 32);  // 64-column x 32-row boxes of the output
  if (e != cudaSuccess) return e;
  switch (blockN) {
    case 64:
      return launch<64>(ta, tb, td, shape, numCtas, status, stream);
    case 128:
      return launch<128>(ta, tb, td, shape, numCtas, status, stream);
    case 256:
      return launch<256>(ta, tb, td, shape, numCtas, status, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace gemm
}  // namespace mscclpp
