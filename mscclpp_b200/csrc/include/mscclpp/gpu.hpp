// The GPU programming interface this library is written against: CUDA 12.x for Blackwell (sm_100a). The reference's
// header of the same name (include/mscclpp/gpu.hpp) maps CUDA names to HIP for AMD builds; there is one target here,
// so this header only gathers the CUDA includes and states the capabilities the rest of the code may assume.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#define MSCCLPP_B200 1
// cuMulticast* (NVLS) and the VMM allocation API are part of every toolkit this library builds with
#define CUDA_NVLS_API_AVAILABLE 1
#define MSCCLPP_WARP_SIZE 32
