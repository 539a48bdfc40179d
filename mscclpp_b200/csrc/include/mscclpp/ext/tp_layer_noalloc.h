/* Allocation-free entry point of the fused projection + residual + RMSNorm layer (single GPU).
 *
 * This entry point has no counterpart in the reference library.
 *
 * Who needs it: code that runs where device memory must not be allocated or freed - for example a
 * plugin called from inside another framework's memory-planned region, a real-time serving loop whose
 * memory budget is fixed at start-up, or a host that forbids cudaMalloc after initialisation because
 * an allocation may synchronise the device or fragment a pre-sized pool. The regular entry points of
 * this library take their intermediate buffers from the symmetric heap, which is created with CUDA
 * allocation calls; this one keeps the same intermediates (the bf16 partial product of the GEMM, the
 * tile-completion counters and flags, the launch bookkeeping and the error block) in one fixed array
 * that is part of the library image.
 *
 *   out          = RMSNorm(x * w^T + residual) * gamma        [m, n] bf16
 *   residual_out = x * w^T + residual                          [m, n] bf16
 *
 * x [m, k] and w [n, k] are bf16, row-major (w in nn.Linear layout); residual and gamma may be NULL.
 * All pointers are device pointers of the CURRENT device, 16-byte aligned. Inputs and outputs are the
 * caller's; the function calls no cudaMalloc / cudaFree nor any other allocating routine.
 *
 * Limits (fixed when the library is built): m * n <= MSCCLPP_B200_NOALLOC_MAX_ELEMS (4 Mi elements, an
 * 8 MiB intermediate), n a multiple of 64 and <= 8192, k a multiple of 64. Larger sizes are rejected
 * with cudaErrorInvalidValue and a message; the whole array is about 10.3 MiB and every GPU on which the
 * library is used holds it until the process exits.
 *
 * The array is shared by all calls and keeps what the last call left in it. The function clears the
 * parts that must start from zero (tile counters, block counters, error block) on `stream` before it
 * launches; the launch counter deliberately carries over, because the completion flags are stamped
 * with it and therefore never need clearing. Two calls that overlap on the GPU (different streams, or
 * different host threads) use the same intermediates and race: serialise them.
 *
 * The first call on each device looks up the device address of the array (cudaGetSymbolAddress) and
 * raises the kernel's shared-memory limit on that device (both are remembered per device, so a process
 * that drives several GPUs pays this once on each). Make that first call outside of any stream capture.
 *
 * A device-side wait that runs out of time (every wait in the kernel is bounded) leaves out /
 * residual_out partly unwritten although the launch itself succeeded. The kernel records that in an
 * error block inside the array; mscclpp_b200_tp_layer_noalloc_status() copies the block out. The next
 * call of the entry point clears it, so ask before calling again when a result looks wrong.
 *
 * Returns 0 on success, otherwise a cudaError_t value; when `err` is not NULL a description of the
 * failure is written there (at most err_len bytes, always terminated).
 */
#ifndef MSCCLPP_B200_TP_LAYER_NOALLOC_H_
#define MSCCLPP_B200_TP_LAYER_NOALLOC_H_

#include <stddef.h>

#define MSCCLPP_B200_NOALLOC_MAX_ELEMS (4u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int mscclpp_b200_tp_layer_noalloc(const void* x, const void* w, const void* residual, const void* gamma, void* out,
                                  void* residual_out, int m, int n, int k, float eps, void* cuda_stream, char* err,
                                  size_t err_len);

/* Copies the 64-byte error block of the current device's array into status_words[16] (waits for `cuda_stream`, i.e. for
 * the calls queued on it so far). status_words[0] is 0 when no wait gave up; otherwise it is the kind of wait, words 2-5
 * say where (rank, thread block, site, peer). Allocates nothing. Returns 0 when the block could be read. No counterpart
 * in the reference. */
int mscclpp_b200_tp_layer_noalloc_status(void* cuda_stream, unsigned int* status_words, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif

#endif /* MSCCLPP_B200_TP_LAYER_NOALLOC_H_ */
