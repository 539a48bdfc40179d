// Prints, for every pair of GPUs, whether peer access is possible and whether NVLink multicast is available: the two
// properties the symmetric heap needs. (The reference ships a similar checker, tools/peer-access-test/peer_access_test.cu.)
//   nvcc -o peer_access_test peer_access_test.cu -lcuda && ./peer_access_test
#include <cstdio>
#include <cuda.h>
#include <cuda_runtime.h>

int main() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    std::printf("no CUDA device\n");
    return 1;
  }
  int bad = 0;
  for (int i = 0; i < n; i++) {
    int mc = 0;
    cudaDeviceGetAttribute(&mc, static_cast<cudaDeviceAttr>(132) /* multicast supported */, i);
    std::printf("GPU %d: multicast %s; peers:", i, mc ? "yes" : "no");
    for (int j = 0; j < n; j++) {
      if (i == j) continue;
      int can = 0;
      cudaDeviceCanAccessPeer(&can, i, j);
      std::printf(" %d:%s", j, can ? "ok" : "NO");
      bad += !can;
    }
    std::printf("\n");
  }
  return bad ? 2 : 0;
}
