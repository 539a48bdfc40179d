// Allocation-free variant of the fused tensor-parallel layer kernel for one GPU: the kernel is the
// one in tp_fused.cu, its intermediates live in a file-scope device array instead of the symmetric
// heap. See include/mscclpp/ext/tp_layer_noalloc.h for the contract. No counterpart in the reference.
#include <mscclpp/ext/tp_layer_noalloc.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "tp_fused.cuh"

namespace {

using namespace mscclpp;

constexpr size_t kControlBytes = (sizeof(SymmControl) + 4095) / 4096 * 4096;
constexpr size_t kStatusOff = kControlBytes;
constexpr size_t kAuxOff = kStatusOff + 4096;
constexpr size_t kPartialOff = kAuxOff + kAuxFlagBytes;
constexpr size_t kPartialBytes = static_cast<size_t>(MSCCLPP_B200_NOALLOC_MAX_ELEMS) * 2;
constexpr size_t kScratchBytes = kPartialOff + kPartialBytes;
// tile counters inside the aux region: the layout constants are the fused kernel's own (tp_fused.cuh)
constexpr size_t kTileCounterOff = kAuxOff + kTpTileCounterOffset;
constexpr size_t kTileCounterBytes = kTpTileCounterBytes;

// The scratch. In host code this name is only a handle for cudaGetSymbolAddress, never an address a
// kernel could use.
static __device__ __align__(256) unsigned char g_noallocScratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned char* g_scratchPtr[kMaxDevices] = {nullptr};

int fail(cudaError_t code, char* err, size_t errLen, const char* what) {
  if (err != nullptr && errLen > 0) {
    std::snprintf(err, errLen, "mscclpp_b200_tp_layer_noalloc: %s (%s)", what, cudaGetErrorString(code));
  }
  return static_cast<int>(code);
}

}  // namespace

extern "C" int mscclpp_b200_tp_layer_noalloc(const void* x, const void* w, const void* residual, const void* gamma,
                                             void* out, void* residual_out, int m, int n, int k, float eps,
                                             void* cuda_stream, char* err, size_t err_len) {
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (x == nullptr || w == nullptr || out == nullptr || residual_out == nullptr) {
    return fail(cudaErrorInvalidValue, err, err_len, "x, w, out and residual_out must not be NULL");
  }
  if (m <= 0 || n <= 0 || k <= 0 || n % 64 != 0 || k % 64 != 0 || n > 8192) {
    return fail(cudaErrorInvalidValue, err, err_len, "need m > 0, n a multiple of 64 and <= 8192, k a multiple of 64");
  }
  if (static_cast<size_t>(m) * static_cast<size_t>(n) > MSCCLPP_B200_NOALLOC_MAX_ELEMS) {
    return fail(cudaErrorInvalidValue, err, err_len,
                "m * n exceeds MSCCLPP_B200_NOALLOC_MAX_ELEMS (4 Mi elements): the built-in scratch is too small");
  }
  const void* ptrs[] = {x, w, residual, gamma, out, residual_out};
  for (const void* p : ptrs) {
    if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) return fail(cudaErrorInvalidValue, err, err_len, "pointers must be 16-byte aligned");
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(e, err, err_len, "cudaGetDevice failed");
  if (dev < 0 || dev >= kMaxDevices) return fail(cudaErrorInvalidDevice, err, err_len, "device index out of range");

  // ---- once per device, with that device current: device address of the scratch
  unsigned char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratchPtr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noallocScratch);
      if (e != cudaSuccess || p == nullptr) return fail(e != cudaSuccess ? e : cudaErrorUnknown, err, err_len, "cudaGetSymbolAddress failed");
      g_scratchPtr[dev] = static_cast<unsigned char*>(p);
    }
    scratch = g_scratchPtr[dev];
  }

  // ---- what must start from zero: tile counters, block counters of the launch bookkeeping, error block
  e = cudaMemsetAsync(scratch + kTileCounterOff, 0, kTileCounterBytes, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(scratch + offsetof(SymmControl, done), 0, sizeof(uint32_t), stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(scratch + offsetof(SymmControl, gridSync), 0, sizeof(uint32_t) * 64, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(scratch + kStatusOff, 0, sizeof(DeviceStatus), stream);
  if (e != cudaSuccess) return fail(e, err, err_len, "clearing the scratch failed");

  TpFusedArgs args{};
  std::memset(&args.comm, 0, sizeof(args.comm));
  args.comm.peerBase[0] = reinterpret_cast<uint64_t>(scratch);  // "heap" of the only rank = the scratch
  args.comm.mcBase = 0;
  args.comm.heapBytes = kScratchBytes;
  args.comm.auxFlagsOff = kAuxOff;
  args.comm.status = reinterpret_cast<DeviceStatus*>(scratch + kStatusOff);
  args.comm.timeoutNs = 2000000000ull;
  args.comm.rank = 0;
  args.comm.world = 1;
  args.shape.M = m;
  args.shape.N = n;
  args.shape.K = k;
  args.partial = reinterpret_cast<__nv_bfloat16*>(scratch + kPartialOff);
  // The kernel was written for buffers inside a heap and turns every pointer into "heap base + offset". The caller's
  // buffers are outside the scratch, so their "offsets" (pointer minus scratch base, in unsigned 64-bit arithmetic) wrap
  // around; adding the base again gives back the original pointer exactly. Only this rank's base is ever used (world 1).
  args.residualIn = static_cast<const __nv_bfloat16*>(residual);
  args.residualOut = static_cast<__nv_bfloat16*>(residual_out);
  args.out = static_cast<__nv_bfloat16*>(out);
  args.gamma = static_cast<const __nv_bfloat16*>(gamma);
  args.rinv = nullptr;
  args.eps = eps;
  const int tilesM = (m + 127) / 128;
  args.blockN = 64;
  for (int bn : {256, 128}) {
    if (n % bn == 0 && tilesM * (n / bn) >= 60) {
      args.blockN = bn;
      break;
    }
  }
  args.numGemmCtas = 0;
  args.rowsPerUnit = 0;
  args.mode = 0;
  args.nvls = 0;
  args.emuRanks = 1;
  const void* A[1] = {x};
  const void* B[1] = {w};
  e = launchTpFused(args, A, B, /*numReducers=*/64, stream);
  if (e != cudaSuccess) return fail(e, err, err_len, "kernel launch failed");
  return 0;
}

extern "C" int mscclpp_b200_tp_layer_noalloc_status(void* cuda_stream, unsigned int* status_words, char* err, size_t err_len) {
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (status_words == nullptr) return fail(cudaErrorInvalidValue, err, err_len, "status_words must not be NULL");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(e, err, err_len, "cudaGetDevice failed");
  if (dev < 0 || dev >= kMaxDevices) return fail(cudaErrorInvalidDevice, err, err_len, "device index out of range");
  unsigned char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    scratch = g_scratchPtr[dev];
  }
  static_assert(sizeof(DeviceStatus) == 64, "the status block is 16 words");
  if (scratch == nullptr) {  // the entry point never ran on this device: nothing can have gone wrong yet
    std::memset(status_words, 0, sizeof(DeviceStatus));
    return 0;
  }
  e = cudaMemcpyAsync(status_words, scratch + kStatusOff, sizeof(DeviceStatus), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(e, err, err_len, "reading the status block failed");
  return 0;
}
