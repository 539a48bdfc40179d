// Device-side assertion that REPORTS and never traps (role of the reference's include/mscclpp/assert_device.hpp:17-41,
// whose debug build calls __assert_fail). A trap loses the CUDA context and, on a multi-GPU job, leaves every peer
// spinning on flags that will never come; the kernels of this library report protocol problems through their bounded
// waits and status block instead. So: nothing in release builds, one printf per failing thread in debug builds.
#pragma once

#include "device.hpp"

#if defined(MSCCLPP_DEVICE_COMPILE) && defined(DEBUG_BUILD)
#include <cstdio>
#define MSCCLPP_ASSERT_DEVICE(__cond, __msg)                                                                           \
  do {                                                                                                                 \
    if (!(__cond))                                                                                                     \
      printf("mscclpp device assertion failed: %s (%s) at %s:%d, block %d thread %d\n", #__cond, __msg, __FILE__,     \
             __LINE__, static_cast<int>(blockIdx.x), static_cast<int>(threadIdx.x));                                   \
  } while (0)
#else
#define MSCCLPP_ASSERT_DEVICE(__cond, __msg) \
  do {                                       \
  } while (0)
#endif
