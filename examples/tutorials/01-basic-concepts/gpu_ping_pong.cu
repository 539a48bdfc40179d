// Tutorial 01 - basic concepts: Context, Endpoint, Connection, Semaphore.
// One process, two GPUs. Each GPU runs a kernel; the kernels take turns signalling each other through
// MemoryDevice2DeviceSemaphore (a counter in the peer's memory written over NVLink). Needs two GPUs with peer access.
//
// (Same exercise as the reference's examples/tutorials/01-basic-concepts/gpu_ping_pong.cu.)
#include <cstdio>
#include <mscclpp/core.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/semaphore.hpp>

using namespace mscclpp;

// Every wait is bounded: a kernel that gives up reports it through `failed` instead of hanging the GPU.
__global__ void pingPong(MemoryDevice2DeviceSemaphoreDeviceHandle sem, int myTurnFirst, int iters, int* failed) {
  if (threadIdx.x != 0) return;
  for (int i = 0; i < iters; i++) {
    if (myTurnFirst) {
      sem.signal();
      if (!sem.wait(2000000000ull)) { *failed = 1; return; }
    } else {
      if (!sem.wait(2000000000ull)) { *failed = 1; return; }
      sem.signal();
    }
  }
}

int main() {
  int n = 0;
  MSCCLPP_CUDATHROW(cudaGetDeviceCount(&n));
  if (n < 2) {
    std::printf("this tutorial needs two GPUs (found %d)\n", n);
    return 0;
  }
  const int iters = 1000;
  auto ctx = Context::create();
  // one endpoint per GPU, both in this process
  MSCCLPP_CUDATHROW(cudaSetDevice(0));
  Endpoint ep0 = ctx->createEndpoint(EndpointConfig(Transport::CudaIpc, Device(DeviceType::GPU, 0)));
  MSCCLPP_CUDATHROW(cudaSetDevice(1));
  Endpoint ep1 = ctx->createEndpoint(EndpointConfig(Transport::CudaIpc, Device(DeviceType::GPU, 1)));
  Connection c01 = ctx->connect(ep0, ep1);  // GPU 0's side
  Connection c10 = ctx->connect(ep1, ep0);  // GPU 1's side
  // a semaphore is a pair of stubs (one counter each); each side combines its own with the peer's
  MSCCLPP_CUDATHROW(cudaSetDevice(0));
  SemaphoreStub stub0(c01);
  MSCCLPP_CUDATHROW(cudaSetDevice(1));
  SemaphoreStub stub1(c10);
  MSCCLPP_CUDATHROW(cudaSetDevice(0));
  MemoryDevice2DeviceSemaphore sem0(Semaphore(stub0, stub1));
  int* failed0 = static_cast<int*>(detail::gpuCalloc(sizeof(int)));
  MSCCLPP_CUDATHROW(cudaSetDevice(1));
  MemoryDevice2DeviceSemaphore sem1(Semaphore(stub1, stub0));
  int* failed1 = static_cast<int*>(detail::gpuCalloc(sizeof(int)));

  cudaEvent_t start, stop;
  MSCCLPP_CUDATHROW(cudaSetDevice(0));
  MSCCLPP_CUDATHROW(cudaEventCreate(&start));
  MSCCLPP_CUDATHROW(cudaEventCreate(&stop));
  MSCCLPP_CUDATHROW(cudaEventRecord(start));
  pingPong<<<1, 32>>>(sem0.deviceHandle(), 1, iters, failed0);
  MSCCLPP_CUDATHROW(cudaEventRecord(stop));
  MSCCLPP_CUDATHROW(cudaSetDevice(1));
  pingPong<<<1, 32>>>(sem1.deviceHandle(), 0, iters, failed1);
  MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
  MSCCLPP_CUDATHROW(cudaSetDevice(0));
  MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
  float ms = 0;
  MSCCLPP_CUDATHROW(cudaEventElapsedTime(&ms, start, stop));
  int f0 = 0, f1 = 0;
  gpuMemcpy(&f0, failed0, sizeof(int), cudaMemcpyDeviceToHost);
  gpuMemcpy(&f1, failed1, sizeof(int), cudaMemcpyDeviceToHost);
  if (f0 || f1) {
    std::printf("a wait ran out of time (gpu0 %d, gpu1 %d)\n", f0, f1);
    return 1;
  }
  std::printf("%d round trips, %.2f us each\n", iters, ms * 1e3f / iters);
  return 0;
}
