#pragma once

#include <cuda_runtime.h>

#include <mscclpp/gpu_data_types.hpp>

#include "execution_common.hpp"

namespace mscclpp {

// Launches the plan interpreter: nBlocks = largest thread-block count over the (emulated) ranks.
cudaError_t launchExecutionKernel(const ExecArgs& args, DataType dtype, int nBlocks, int nThreads, cudaStream_t stream);

}  // namespace mscclpp
