// Exit code 0 and one line on stdout when a device of compute capability 10.x is visible, 1 otherwise.
#include <cuda_runtime.h>

#include <cstdio>

int main() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 1;
  for (int d = 0; d < n; d++) {
    int major = 0, minor = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) != cudaSuccess) continue;
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, d);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d);
    if (major == 10) {
      std::printf("device %d: sm_%d%d, %d SMs", d, major, minor, sms);
      return 0;
    }
  }
  return 1;
}
