// Tutorial 04 - PortChannel: the GPU does not move the bytes itself; it pushes a request into a FIFO and a host proxy
// thread (ProxyService) performs the copy through the connection (here CUDA IPC on one node; the same code drives the
// Ethernet transport between nodes), then signals the peer. Two processes, put-with-signal in both directions.
//
// (Same exercise as the reference's examples/tutorials/04-port-channel/bidir_port_channel.cu.)
#include <cstdio>
#include <cstdlib>
#include <sys/wait.h>
#include <unistd.h>

#include <mscclpp/core.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/port_channel.hpp>

using namespace mscclpp;

__global__ void exchange(PortChannelDeviceHandle ch, uint64_t recvOffset, uint64_t bytes, int* failed) {
  if (threadIdx.x != 0) return;
  ch.putWithSignal(recvOffset, 0, bytes);     // request: copy my first half into the peer's second half, then raise its semaphore
  if (!ch.wait(5000000000ull)) *failed = 1;   // the peer's data has arrived in my buffer
  if (!ch.flush()) *failed = 1;               // my request has been carried out (the source may be reused)
}

static int worker(int rank, const char* ipPort) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n < 2) return 0;
  MSCCLPP_CUDATHROW(cudaSetDevice(rank));
  auto bootstrap = std::make_shared<TcpBootstrap>(rank, 2);
  bootstrap->initialize(ipPort);
  Communicator comm(bootstrap);
  const int peer = 1 - rank;
  const size_t maxBytes = 16 << 20;
  // one buffer, two halves: [0, maxBytes) is what I send, the peer writes its data into my second half
  GpuBuffer<char> buf(2 * maxBytes);
  Connection conn = comm.connect(EndpointConfig(Transport::CudaIpc), peer).get();
  RegisteredMemory local = comm.registerMemory(buf.data(), buf.bytes(), Transport::CudaIpc);
  comm.sendMemory(local, peer);
  RegisteredMemory remote = comm.recvMemory(peer).get();
  ProxyService proxy;
  const SemaphoreId sid = proxy.buildAndAddSemaphore(comm, conn);
  const MemoryId dst = proxy.addMemory(remote), src = proxy.addMemory(local);
  PortChannel channel = proxy.portChannel(sid, dst, src);
  proxy.startProxy();
  int* failed = static_cast<int*>(detail::gpuCalloc(sizeof(int)));
  cudaEvent_t start, stop;
  MSCCLPP_CUDATHROW(cudaEventCreate(&start));
  MSCCLPP_CUDATHROW(cudaEventCreate(&stop));
  for (size_t bytes : {size_t(1) << 10, size_t(1) << 20, maxBytes}) {
    const int iters = 20;
    bootstrap->barrier();
    MSCCLPP_CUDATHROW(cudaEventRecord(start));
    for (int i = 0; i < iters; i++) exchange<<<1, 32>>>(channel.deviceHandle(), maxBytes, bytes, failed);
    MSCCLPP_CUDATHROW(cudaEventRecord(stop));
    MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
    float ms = 0;
    MSCCLPP_CUDATHROW(cudaEventElapsedTime(&ms, start, stop));
    if (rank == 0) std::printf("putWithSignal %10zu bytes  %8.2f us  %7.1f GB/s\n", bytes, ms * 1e3f / iters, bytes / (ms * 1e-3 / iters) / 1e9);
  }
  int f = 0;
  gpuMemcpy(&f, failed, sizeof(int), cudaMemcpyDeviceToHost);
  bootstrap->barrier();
  proxy.stopProxy();
  return f;
}

int main(int argc, char** argv) {
  const char* ipPort = argc > 1 ? argv[1] : "127.0.0.1:50543";
  pid_t pids[2];
  for (int r = 0; r < 2; r++) {
    pids[r] = fork();
    if (pids[r] == 0) std::exit(worker(r, ipPort));
  }
  int bad = 0;
  for (int r = 0; r < 2; r++) {
    int status = 0;
    waitpid(pids[r], &status, 0);
    bad |= !WIFEXITED(status) || WEXITSTATUS(status) != 0;
  }
  return bad;
}
