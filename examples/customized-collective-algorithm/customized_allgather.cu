// A user-written allgather registered as a native algorithm: the kernel lives in this file, the glue makes it an
// `Algorithm` that an `AlgorithmCollection` (and through it the NCCL-API shim) can select. Build it at run time with
//
//     module = mscclpp_b200.compile_native("customized_allgather", "customized_allgather.cu")
//     algo   = mscclpp_b200.Algorithm.create_from_native_capsule(module.create_allgather(symm.heap))
//
// (see examples/torch-integration/customized_allgather.py). The reference ships the same kind of example
// (examples/customized-collective-algorithm/customized_allgather.cu) built on port channels; this one uses the
// symmetric heap: every rank stores its slice straight into every peer's output buffer.
#include <pybind11/pybind11.h>

#include <mscclpp/algorithm.hpp>
#include <mscclpp/device/symm.cuh>
#include <mscclpp/symmetric_heap.hpp>

namespace py = pybind11;
using namespace mscclpp;

// out (symmetric, same offset on every rank) [world * bytes]; in: my slice [bytes] (any device memory of mine).
__global__ void __launch_bounds__(512) customAllGather(DeviceComm c, const uint4* in, uint64_t outOff, uint64_t units16) {
  const int rank = c.rank;
  const uint32_t epoch = launchEpoch(c, rank);
  // peers must have entered the collective before their output buffers are written
  bool ok = rankBarrier(c, rank, 0, blockIdx.x, epoch);
  if (ok) {
    for (uint64_t u = blockIdx.x * blockDim.x + threadIdx.x; u < units16; u += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
      const uint4 v = in[u];
      for (int p = 0; p < c.world; p++) {
        uint4* dst = reinterpret_cast<uint4*>(c.peerBase[(rank + p) % c.world] + outOff) + static_cast<uint64_t>(rank) * units16 + u;
        ptx::st_na_v4(dst, v);
      }
    }
    rankBarrier(c, rank, 1, blockIdx.x, epoch);  // every slice has landed everywhere
  }
  finishLaunch(c, rank, epoch);
}

static py::capsule createAllgather(std::shared_ptr<SymmetricHeap> heap) {
  auto kernel = [heap](const void* in, void* out, size_t inBytes, size_t outBytes, DataType, ReduceOp, cudaStream_t stream, int nBlocks,
                       int nThreads, bool, const std::unordered_map<std::string, uintptr_t>&) {
    if (inBytes % 16 != 0 || outBytes != inBytes * heap->world() || !heap->contains(out, outBytes)) return CommResult::InvalidUsage;
    if (nBlocks <= 0) nBlocks = 32;
    if (nThreads <= 0) nThreads = 512;
    const DeviceComm comm = heap->deviceComm();
    const uint64_t outOff = reinterpret_cast<uint64_t>(out) - comm.peerBase[comm.rank];
    customAllGather<<<nBlocks, nThreads, 0, stream>>>(comm, static_cast<const uint4*>(in), outOff, inBytes / 16);
    return cudaGetLastError() == cudaSuccess ? CommResult::Success : CommResult::UnhandledCudaError;
  };
  std::shared_ptr<Algorithm> algo = std::make_shared<NativeAlgorithm>("customized_allgather", "allgather", nullptr, kernel);
  // the capsule format understood by mscclpp_b200.Algorithm.create_from_native_capsule
  auto* holder = new std::shared_ptr<Algorithm>(std::move(algo));
  return py::capsule(holder, "mscclpp::AlgorithmPtr",
                     [](PyObject* cap) { delete static_cast<std::shared_ptr<Algorithm>*>(PyCapsule_GetPointer(cap, "mscclpp::AlgorithmPtr")); });
}

PYBIND11_MODULE(customized_allgather, m) {
  py::module_::import("mscclpp_b200").attr("native")();  // registers SymmetricHeap and friends with pybind11
  m.def("create_allgather", &createAllgather, py::arg("heap"));
}
