// Compilation-mode macros shared by host and device headers (reference: include/mscclpp/device.hpp:8-29).
//   MSCCLPP_DEVICE_COMPILE / MSCCLPP_HOST_COMPILE   which pass is running
//   MSCCLPP_DEVICE_CUDA                             device code is CUDA (always, here: sm_100a)
//   MSCCLPP_INLINE, MSCCLPP_DEVICE_INLINE, MSCCLPP_HOST_DEVICE_INLINE
#pragma once

#if defined(__CUDACC__)
#include <cuda_runtime.h>
#define MSCCLPP_DEVICE_CUDA
#if defined(__CUDA_ARCH__)
#define MSCCLPP_DEVICE_COMPILE
#else
#define MSCCLPP_HOST_COMPILE
#endif
#ifndef MSCCLPP_INLINE
#define MSCCLPP_INLINE __forceinline__
#endif
#ifndef MSCCLPP_DEVICE_INLINE
#define MSCCLPP_DEVICE_INLINE __forceinline__ __device__
#endif
#ifndef MSCCLPP_HOST_DEVICE_INLINE
#define MSCCLPP_HOST_DEVICE_INLINE __forceinline__ __host__ __device__
#endif
#else  // plain host compiler
#define MSCCLPP_HOST_COMPILE
#ifndef MSCCLPP_INLINE
#define MSCCLPP_INLINE inline
#endif
#ifndef MSCCLPP_HOST_DEVICE_INLINE
#define MSCCLPP_HOST_DEVICE_INLINE inline
#endif
#endif
