// Tutorial 03 - MemoryChannel: two processes, each GPU writes into the other's buffer with put(), reads it with get()
// and sends LL packets with putPackets(); prints the bandwidth of each for a few sizes.
//
// (Same exercise as the reference's examples/tutorials/03-memory-channel/bidir_memory_channel.cu.)
#include <cstdio>
#include <cstdlib>
#include <sys/wait.h>
#include <unistd.h>

#include <mscclpp/core.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/memory_channel.hpp>

using namespace mscclpp;

constexpr uint64_t kWait = 5000000000ull;

__global__ void putKernel(MemoryChannelDeviceHandle ch, uint64_t bytes, int* failed) {
  const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
  ch.put(0, bytes, tid, nthreads);  // my buffer -> the peer's buffer, same offset
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    ch.signal();                    // "my data is in your buffer"
    if (!ch.wait(kWait)) *failed = 1;
  }
}

__global__ void getKernel(MemoryChannelDeviceHandle ch, uint64_t bytes, int* failed) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    ch.relaxedSignal();             // "you may read my buffer"
    if (!ch.relaxedWait(kWait)) *failed = 1;
  }
  __syncthreads();
  ch.get(0, bytes, threadIdx.x, blockDim.x);  // the peer's buffer -> mine (launched with one block)
}

__global__ void packetKernel(MemoryChannelDeviceHandle ch, uint64_t bytes, uint32_t flag, int* failed) {
  const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
  ch.putPackets<LL16Packet>(0, 0, bytes, tid, nthreads, flag);            // data + flag in one 16-byte store
  if (!ch.unpackPackets<LL16Packet>(0, 0, bytes, tid, nthreads, flag, nullptr, kWait)) *failed = 1;  // wait for the peer's packets
}

static int worker(int rank, const char* ipPort) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n < 2) return 0;
  MSCCLPP_CUDATHROW(cudaSetDevice(rank));
  auto bootstrap = std::make_shared<TcpBootstrap>(rank, 2);
  bootstrap->initialize(ipPort);
  Communicator comm(bootstrap);
  const int peer = 1 - rank;
  const size_t maxBytes = 64 << 20;
  GpuBuffer<char> data(maxBytes), packets(2 * maxBytes);
  Connection conn = comm.connect(EndpointConfig(Transport::CudaIpc), peer).get();
  Semaphore sem = comm.buildSemaphore(conn, peer).get();
  RegisteredMemory localData = comm.registerMemory(data.data(), data.bytes(), Transport::CudaIpc);
  RegisteredMemory localPkt = comm.registerMemory(packets.data(), packets.bytes(), Transport::CudaIpc);
  comm.sendMemory(localData, peer, 0);
  comm.sendMemory(localPkt, peer, 1);
  RegisteredMemory remoteData = comm.recvMemory(peer, 0).get();
  RegisteredMemory remotePkt = comm.recvMemory(peer, 1).get();
  MemoryChannel dataChannel(sem, remoteData, localData);
  // packets travel from my data buffer into the peer's packet buffer; mine receives the peer's
  MemoryChannel packetChannel(sem, remotePkt, localData, packets.data());
  int* failed = static_cast<int*>(detail::gpuCalloc(sizeof(int)));
  cudaEvent_t start, stop;
  MSCCLPP_CUDATHROW(cudaEventCreate(&start));
  MSCCLPP_CUDATHROW(cudaEventCreate(&stop));
  uint32_t flag = 1;
  for (size_t bytes : {size_t(1) << 10, size_t(1) << 20, size_t(64) << 20}) {
    for (int mode = 0; mode < 3; mode++) {
      if (mode == 2 && bytes > (4 << 20)) continue;  // packets are the small-message protocol
      const int iters = 20, blocks = bytes >= (1 << 20) ? 64 : 1;
      bootstrap->barrier();
      MSCCLPP_CUDATHROW(cudaEventRecord(start));
      for (int i = 0; i < iters; i++) {
        if (mode == 0) putKernel<<<blocks, 512>>>(dataChannel.deviceHandle(), bytes, failed);
        if (mode == 1) getKernel<<<1, 512>>>(dataChannel.deviceHandle(), bytes, failed);
        if (mode == 2) packetKernel<<<blocks, 512>>>(packetChannel.deviceHandle(), bytes, flag++, failed);
      }
      MSCCLPP_CUDATHROW(cudaEventRecord(stop));
      MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
      float ms = 0;
      MSCCLPP_CUDATHROW(cudaEventElapsedTime(&ms, start, stop));
      if (rank == 0)
        std::printf("%-10s %10zu bytes  %8.2f us  %7.1f GB/s\n", mode == 0 ? "put" : (mode == 1 ? "get" : "putPackets"), bytes,
                    ms * 1e3f / iters, bytes / (ms * 1e-3 / iters) / 1e9);
    }
  }
  int f = 0;
  gpuMemcpy(&f, failed, sizeof(int), cudaMemcpyDeviceToHost);
  bootstrap->barrier();
  return f;
}

int main(int argc, char** argv) {
  const char* ipPort = argc > 1 ? argv[1] : "127.0.0.1:50542";
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
