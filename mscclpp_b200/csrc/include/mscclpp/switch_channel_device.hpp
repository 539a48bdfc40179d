// Device handle of SwitchChannel: NVSwitch multimem operations on a buffer that every member of a
// group has bound to one multicast object (reference: include/mscclpp/switch_channel_device.hpp:27-278).
//   reduce<T>(i)        element-wise reduction over all members of the i-th 16-byte word -> registers
//   broadcast(i, v)     store v into the i-th 16-byte word of every member
//   storeReduce<T>(i,v) add v into the i-th word of every member (multimem.red)
// fp8 reductions (e4m3 / e5m2, accumulated in f16 inside the switch) exist on sm_100a only, which is
// the only target of this library.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device/ptx.cuh"
#include "gpu_data_types.hpp"
#include "semaphore_device.hpp"

namespace mscclpp {

struct SwitchChannelDeviceHandle {
  void* devicePtr;    // this rank's buffer (ordinary address)
  void* mcPtr;        // multicast alias of the same range
  uint64_t bufferSize;
  SwitchDevice2DeviceSemaphoreDeviceHandle barrier;  // group barrier on a word owned by the connection

#if defined(__CUDACC__)
  template <typename T, ReduceOp Op = SUM>
  MSCCLPP_DEVICE_INLINE uint4 reduce(uint64_t index16) const {
    const void* p = static_cast<const char*>(mcPtr) + index16 * 16;
    if constexpr (__is_same(T, __half)) {
      if constexpr (Op == SUM) return ptx::multimem_ld_reduce_add_f16x2(p);
      else return ptx::multimem_ld_reduce_min_f16x2(p);
    } else if constexpr (__is_same(T, __nv_bfloat16)) {
      if constexpr (Op == SUM) return ptx::multimem_ld_reduce_add_bf16x2(p);
      else return ptx::multimem_ld_reduce_min_bf16x2(p);
    } else if constexpr (__is_same(T, float)) {
      return ptx::multimem_ld_reduce_add_f32(p);
    } else if constexpr (__is_same(T, f8e4m3)) {
      return ptx::multimem_ld_reduce_add_e4m3x4(p);
    } else if constexpr (__is_same(T, f8e5m2)) {
      return ptx::multimem_ld_reduce_add_e5m2x4(p);
    } else if constexpr (__is_same(T, int32_t)) {
      const char* c = static_cast<const char*>(p);
      return make_uint4(ptx::multimem_ld_reduce_add_s32(c), ptx::multimem_ld_reduce_add_s32(c + 4),
                        ptx::multimem_ld_reduce_add_s32(c + 8), ptx::multimem_ld_reduce_add_s32(c + 12));
    } else {
      const char* c = static_cast<const char*>(p);
      return make_uint4(ptx::multimem_ld_reduce_add_u32(c), ptx::multimem_ld_reduce_add_u32(c + 4),
                        ptx::multimem_ld_reduce_add_u32(c + 8), ptx::multimem_ld_reduce_add_u32(c + 12));
    }
  }
  // 16-bit float sum with an fp32 accumulator inside the switch (more accurate, same bandwidth).
  template <typename T>
  MSCCLPP_DEVICE_INLINE uint4 reduceAcc32(uint64_t index16) const {
    const void* p = static_cast<const char*>(mcPtr) + index16 * 16;
    if constexpr (__is_same(T, __half)) return ptx::multimem_ld_reduce_add_f16x2_acc32(p);
    else return ptx::multimem_ld_reduce_add_bf16x2_acc32(p);
  }
  MSCCLPP_DEVICE_INLINE void broadcast(uint64_t index16, uint4 v) const {
    ptx::multimem_st_v4(static_cast<char*>(mcPtr) + index16 * 16, v);
  }
  MSCCLPP_DEVICE_INLINE void broadcast8(uint64_t index8, uint2 v) const {
    ptx::multimem_st_v2(static_cast<char*>(mcPtr) + index8 * 8, v);
  }
  MSCCLPP_DEVICE_INLINE void broadcast4(uint64_t index4, uint32_t v) const {
    ptx::multimem_st_u32(static_cast<char*>(mcPtr) + index4 * 4, v);
  }
  template <typename T>
  MSCCLPP_DEVICE_INLINE void storeReduce(uint64_t index16, uint4 v) const {
    void* p = static_cast<char*>(mcPtr) + index16 * 16;
    if constexpr (__is_same(T, __half)) ptx::multimem_red_add_f16x2x4(p, v);
    else if constexpr (__is_same(T, __nv_bfloat16)) ptx::multimem_red_add_bf16x2x4(p, v);
    else ptx::multimem_red_add_f32x4(p, v);
  }
#endif
};

}  // namespace mscclpp
