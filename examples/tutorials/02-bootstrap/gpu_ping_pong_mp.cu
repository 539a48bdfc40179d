// Tutorial 02 - bootstrap: the ping-pong of tutorial 01 with one PROCESS per GPU. The processes find each other
// through TcpBootstrap (rank 0 listens on 127.0.0.1:<port>), a Communicator exchanges endpoints and builds the
// semaphore. The parent forks the two ranks, so no MPI is needed.
//
// (Same exercise as the reference's examples/tutorials/02-bootstrap/gpu_ping_pong_mp.cu.)
#include <cstdio>
#include <cstdlib>
#include <sys/wait.h>
#include <unistd.h>

#include <mscclpp/core.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/semaphore.hpp>

using namespace mscclpp;

__global__ void pingPong(MemoryDevice2DeviceSemaphoreDeviceHandle sem, int rank, int iters, int* failed) {
  if (threadIdx.x != 0) return;
  for (int i = 0; i < iters; i++) {
    if (rank == 0) {
      sem.signal();
      if (!sem.wait(2000000000ull)) { *failed = 1; return; }
    } else {
      if (!sem.wait(2000000000ull)) { *failed = 1; return; }
      sem.signal();
    }
  }
}

static int worker(int rank, const char* ipPort) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n < 2) {
    if (rank == 0) std::printf("this tutorial needs two GPUs\n");
    return 0;
  }
  MSCCLPP_CUDATHROW(cudaSetDevice(rank));
  auto bootstrap = std::make_shared<TcpBootstrap>(rank, 2);
  bootstrap->initialize(ipPort);
  Communicator comm(bootstrap);
  const int peer = 1 - rank;
  Connection conn = comm.connect(EndpointConfig(Transport::CudaIpc), peer).get();
  Semaphore sem = comm.buildSemaphore(conn, peer).get();
  MemoryDevice2DeviceSemaphore devSem(sem);
  int* failed = static_cast<int*>(detail::gpuCalloc(sizeof(int)));
  bootstrap->barrier();
  const int iters = 1000;
  cudaEvent_t start, stop;
  MSCCLPP_CUDATHROW(cudaEventCreate(&start));
  MSCCLPP_CUDATHROW(cudaEventCreate(&stop));
  MSCCLPP_CUDATHROW(cudaEventRecord(start));
  pingPong<<<1, 32>>>(devSem.deviceHandle(), rank, iters, failed);
  MSCCLPP_CUDATHROW(cudaEventRecord(stop));
  MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
  int f = 0;
  gpuMemcpy(&f, failed, sizeof(int), cudaMemcpyDeviceToHost);
  float ms = 0;
  MSCCLPP_CUDATHROW(cudaEventElapsedTime(&ms, start, stop));
  if (rank == 0 && !f) std::printf("%d round trips between two processes, %.2f us each\n", iters, ms * 1e3f / iters);
  bootstrap->barrier();
  return f;
}

int main(int argc, char** argv) {
  const char* ipPort = argc > 1 ? argv[1] : "127.0.0.1:50541";
  pid_t pids[2];  // the parent never touches CUDA: a process must not fork after initialising it
  for (int r = 0; r < 2; r++) {
    pids[r] = fork();  // fork before any CUDA context exists in the parent
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
