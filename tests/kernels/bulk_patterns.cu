// MoE-shaped patterns on the pointer-based bulk-copy (TMA) primitives: tokens are staged through shared memory and
// pushed to their destination row (dispatch), pulled back (combine) or added into the destination (combine-reduce).
// One block per token, one thread issues the copies. Every wait is bounded; a give-up sets *failed.
#include <mscclpp/bulk_device.hpp>

using namespace mscclpp;

// mode 0: dst[map[t]] = src[t]; mode 1: dst[t] = src[map[t]]; mode 2: dst[map[t]] += src[t] (fp32 adds in memory)
extern "C" __global__ void bulkPattern(const float* src, float* dst, const int* map, int rowFloats, int mode, int* failed) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ BulkBarrier bar;
  const int t = blockIdx.x;
  const unsigned bytes = rowFloats * 4;
  if (threadIdx.x == 0) {
    bar.init(1);
    const float* from = mode == 1 ? src + static_cast<size_t>(map[t]) * rowFloats : src + static_cast<size_t>(t) * rowFloats;
    float* to = mode == 1 ? dst + static_cast<size_t>(t) * rowFloats : dst + static_cast<size_t>(map[t]) * rowFloats;
    bar.arriveExpectTx(bytes);
    bulkLoad(smem, from, bytes, bar);
    if (!bar.wait(0, nullptr, 2000000000ull)) {
      *failed = 1;
    } else {
      if (mode == 2) bulkReduceStore<float>(to, smem, bytes);
      else bulkStore(to, smem, bytes);
      bulkCommit();
      bulkWait<0>();
    }
  }
}
