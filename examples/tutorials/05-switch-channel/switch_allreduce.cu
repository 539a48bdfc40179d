// Tutorial 05 - SwitchChannel: an allreduce in which the NVSwitch does the arithmetic. Every GPU binds its buffer into
// one multicast object; a kernel then reads "the sum over all GPUs" with one multimem.ld_reduce per 16 bytes and
// writes the result to every GPU with one multimem.st. One process per GPU (2 to 8), forked by the parent.
//
// (Same exercise as the reference's examples/tutorials/05-switch-channel/.)
#include <cstdio>
#include <cstdlib>
#include <sys/wait.h>
#include <unistd.h>
#include <vector>

#include <cuda_fp16.h>

#include <mscclpp/core.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/switch_channel.hpp>

using namespace mscclpp;

// Rank r reduces and broadcasts the r-th slice of the buffer; barriers in front (inputs written) and behind
// (results landed) run over the switch as well.
__global__ void switchAllReduce(SwitchChannelDeviceHandle ch, int rank, int nRanks, uint64_t units16, int* failed) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ch.barrier.signal();
    ok = ch.barrier.wait(5000000000ull) ? 1 : 0;
  }
  __syncthreads();
  if (ok) {
    const uint64_t per = units16 / nRanks, begin = rank * per;
    for (uint64_t i = begin + threadIdx.x; i < begin + per; i += blockDim.x) ch.broadcast(i, ch.reduce<__half>(i));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (ok) {
      ch.barrier.signal();
      ok = ch.barrier.wait(5000000000ull) ? 1 : 0;
    }
    if (!ok) *failed = 1;
  }
}

static int worker(int rank, int nRanks, const char* ipPort) {
  MSCCLPP_CUDATHROW(cudaSetDevice(rank));
  if (!isNvlsSupported()) {
    if (rank == 0) std::printf("NVLink multicast is not available on this machine\n");
    return 0;
  }
  auto bootstrap = std::make_shared<TcpBootstrap>(rank, nRanks);
  bootstrap->initialize(ipPort);
  auto comm = std::make_shared<Communicator>(bootstrap);
  std::vector<int> all(nRanks);
  for (int i = 0; i < nRanks; i++) all[i] = i;
  const size_t bytes = 64 << 20;
  GpuBuffer<__half> buf(bytes / sizeof(__half));  // VMM allocation with the multicast granularity
  auto nvls = connectNvlsCollective(comm, all, bytes);
  SwitchChannel channel = nvls->bindAllocatedMemory(buf.data(), buf.bytes());
  std::vector<__half> host(bytes / sizeof(__half), __float2half(static_cast<float>(rank + 1)));
  gpuMemcpy(buf.data(), host.data(), bytes, cudaMemcpyHostToDevice);
  int* failed = static_cast<int*>(detail::gpuCalloc(sizeof(int)));
  bootstrap->barrier();
  cudaEvent_t start, stop;
  MSCCLPP_CUDATHROW(cudaEventCreate(&start));
  MSCCLPP_CUDATHROW(cudaEventCreate(&stop));
  MSCCLPP_CUDATHROW(cudaEventRecord(start));
  switchAllReduce<<<1, 1024>>>(channel.deviceHandle(), rank, nRanks, bytes / 16, failed);
  MSCCLPP_CUDATHROW(cudaEventRecord(stop));
  MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
  float ms = 0;
  MSCCLPP_CUDATHROW(cudaEventElapsedTime(&ms, start, stop));
  gpuMemcpy(host.data(), buf.data(), bytes, cudaMemcpyDeviceToHost);
  int f = 0;
  gpuMemcpy(&f, failed, sizeof(int), cudaMemcpyDeviceToHost);
  const float expect = nRanks * (nRanks + 1) / 2.0f;
  const bool good = !f && __half2float(host[0]) == expect && __half2float(host.back()) == expect;
  if (rank == 0) std::printf("allreduce of %zu MB over %d GPUs through the switch: %.1f us, result %s\n", bytes >> 20, nRanks, ms * 1e3f, good ? "correct" : "WRONG");
  bootstrap->barrier();
  return good ? 0 : 1;
}

int main(int argc, char** argv) {
  const int nRanks = argc > 1 ? std::atoi(argv[1]) : 2;
  const char* ipPort = argc > 2 ? argv[2] : "127.0.0.1:50544";
  std::vector<pid_t> pids(nRanks);
  for (int r = 0; r < nRanks; r++) {
    pids[r] = fork();
    if (pids[r] == 0) std::exit(worker(r, nRanks, ipPort));
  }
  int bad = 0;
  for (int r = 0; r < nRanks; r++) {
    int status = 0;
    waitpid(pids[r], &status, 0);
    bad |= !WIFEXITED(status) || WEXITSTATUS(status) != 0;
  }
  return bad;
}
