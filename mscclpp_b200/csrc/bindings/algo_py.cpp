// Python bindings of the algorithm framework (reference: python/csrc/algorithm.cpp and
// python/csrc/ext/algorithm_collection_builder_py.cpp cover the same surface with nanobind).
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <mscclpp/algorithm.hpp>
#include <mscclpp/ext/collectives/algorithm_collection_builder.hpp>

#include <mscclpp/errors.hpp>
#include <mscclpp/npkit/npkit.hpp>

#include "../core/cuda_driver.hpp"
#include "bindings.hpp"

namespace py = pybind11;
using namespace mscclpp;

namespace {

constexpr const char* kCapsuleName = "mscclpp::AlgorithmPtr";

class PyAlgorithmBuilder : public AlgorithmBuilder {
 public:
  using AlgorithmBuilder::AlgorithmBuilder;
  std::shared_ptr<Algorithm> build() override { PYBIND11_OVERRIDE_PURE(std::shared_ptr<Algorithm>, AlgorithmBuilder, build); }
};

// Builder that hands back an algorithm that already exists (DSL algorithms compiled in Python).
class FixedAlgorithmBuilder : public AlgorithmBuilder {
 public:
  explicit FixedAlgorithmBuilder(std::shared_ptr<Algorithm> algo) : algo_(std::move(algo)) {}
  std::shared_ptr<Algorithm> build() override { return algo_; }

 private:
  std::shared_ptr<Algorithm> algo_;
};

// A cubin loaded into the current context, for kernels compiled at run time from user sources.
class CudaModule {
 public:
  explicit CudaModule(const std::string& image) {
    MSCCLPP_CUDATHROW(cudaFree(nullptr));  // make sure the primary context exists and is current
    MSCCLPP_CUTHROW(CudaDriver::get().cuModuleLoadData(&module_, image.data()));
  }
  ~CudaModule() {
    if (module_) (void)CudaDriver::get().cuModuleUnload(module_);
  }
  CudaModule(const CudaModule&) = delete;
  CudaModule& operator=(const CudaModule&) = delete;
  uintptr_t function(const std::string& name) {
    CUfunction f;
    MSCCLPP_CUTHROW(CudaDriver::get().cuModuleGetFunction(&f, module_, name.c_str()));
    return reinterpret_cast<uintptr_t>(f);
  }

 private:
  CUmodule module_ = nullptr;
};

// Launch with the whole parameter block given as packed bytes (the layout the compiler gives the kernel's
// parameter list: each parameter at its natural alignment).
void launchPacked(uintptr_t function, const std::string& params, unsigned gridX, unsigned gridY, unsigned blockX, unsigned shared,
                  uintptr_t stream, bool cooperative, const std::vector<size_t>& offsets) {
  const CudaDriver& drv = CudaDriver::get();
  CUfunction f = reinterpret_cast<CUfunction>(function);
  if (shared > 48 * 1024) MSCCLPP_CUTHROW(drv.cuFuncSetAttribute(f, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, static_cast<int>(shared)));
  if (cooperative) {
    // cooperative launches take one pointer per parameter: `offsets` says where each one starts in `params`
    std::vector<void*> ptrs;
    for (size_t off : offsets) ptrs.push_back(const_cast<char*>(params.data()) + off);
    MSCCLPP_CUTHROW(drv.cuLaunchCooperativeKernel(f, gridX, gridY, 1, blockX, 1, 1, shared, reinterpret_cast<CUstream>(stream), ptrs.data()));
    return;
  }
  size_t size = params.size();
  void* extra[] = {CU_LAUNCH_PARAM_BUFFER_POINTER, const_cast<char*>(params.data()), CU_LAUNCH_PARAM_BUFFER_SIZE, &size, CU_LAUNCH_PARAM_END};
  MSCCLPP_CUTHROW(drv.cuLaunchKernel(f, gridX, gridY, 1, blockX, 1, 1, shared, reinterpret_cast<CUstream>(stream), nullptr, extra));
}

}  // namespace

void registerAlgorithmBindings(py::module_& m) {
  py::enum_<CollectiveBufferMode>(m, "CollectiveBufferMode")
      .value("ANY", CollectiveBufferMode::Any)
      .value("IN_PLACE", CollectiveBufferMode::InPlace)
      .value("OUT_OF_PLACE", CollectiveBufferMode::OutOfPlace);
  py::enum_<AlgorithmType>(m, "AlgorithmType").value("NATIVE", AlgorithmType::Native).value("DSL", AlgorithmType::DSL);
  py::enum_<CommResult>(m, "CommResult")
      .value("Success", CommResult::Success)
      .value("UnhandledCudaError", CommResult::UnhandledCudaError)
      .value("SystemError", CommResult::SystemError)
      .value("InternalError", CommResult::InternalError)
      .value("InvalidArgument", CommResult::InvalidArgument)
      .value("InvalidUsage", CommResult::InvalidUsage)
      .value("RemoteError", CommResult::RemoteError)
      .value("InProgress", CommResult::InProgress)
      .value("Timeout", CommResult::Timeout);

  py::class_<CollectiveRequest>(m, "CollectiveRequest")
      .def(py::init<>())
      .def_readwrite("world_size", &CollectiveRequest::worldSize)
      .def_readwrite("n_ranks_per_node", &CollectiveRequest::nRanksPerNode)
      .def_readwrite("rank", &CollectiveRequest::rank)
      .def_property(
          "input_buffer", [](const CollectiveRequest& r) { return reinterpret_cast<uintptr_t>(r.inputBuffer); },
          [](CollectiveRequest& r, uintptr_t p) { r.inputBuffer = reinterpret_cast<const void*>(p); })
      .def_property(
          "output_buffer", [](const CollectiveRequest& r) { return reinterpret_cast<uintptr_t>(r.outputBuffer); },
          [](CollectiveRequest& r, uintptr_t p) { r.outputBuffer = reinterpret_cast<void*>(p); })
      .def_readwrite("message_size", &CollectiveRequest::messageSize)
      .def_property(
          "stream", [](const CollectiveRequest& r) { return reinterpret_cast<uintptr_t>(r.stream); },
          [](CollectiveRequest& r, uintptr_t p) { r.stream = reinterpret_cast<cudaStream_t>(p); })
      .def_readwrite("collective", &CollectiveRequest::collective)
      .def_readwrite("dtype", &CollectiveRequest::dtype)
      .def_readwrite("op", &CollectiveRequest::op)
      .def_readwrite("symmetric_memory", &CollectiveRequest::symmetricMemory)
      .def_readwrite("in_capture", &CollectiveRequest::inCapture)
      .def_readwrite("hints", &CollectiveRequest::hints)
      .def_property_readonly("buffer_mode", &CollectiveRequest::bufferMode);

  py::class_<Algorithm, std::shared_ptr<Algorithm>> algorithm(m, "Algorithm");
  py::class_<Algorithm::Constraint>(algorithm, "Constraint")
      .def(py::init<>())
      .def(py::init([](int worldSize, int nRanksPerNode) { return Algorithm::Constraint{worldSize, nRanksPerNode}; }),
           py::arg("world_size"), py::arg("n_ranks_per_node"))
      .def_readwrite("world_size", &Algorithm::Constraint::worldSize)
      .def_readwrite("n_ranks_per_node", &Algorithm::Constraint::nRanksPerNode);
  algorithm.def_property_readonly("name", &Algorithm::name)
      .def_property_readonly("collective", &Algorithm::collective)
      .def_property_readonly("message_range", &Algorithm::messageRange)
      .def("set_message_size_range", &Algorithm::setMessageSizeRange, py::arg("min_message_size"), py::arg("max_message_size"))
      .def_property_readonly("tags", &Algorithm::tags)
      .def_property_readonly("buffer_mode", &Algorithm::bufferMode)
      .def_property_readonly("constraint", &Algorithm::constraint)
      .def_property_readonly("type", &Algorithm::type)
      .def(
          "execute",
          [](Algorithm& self, std::shared_ptr<Communicator> comm, uintptr_t input, uintptr_t output, size_t inputSize, size_t outputSize,
             DataType dtype, ReduceOp op, uintptr_t stream, std::shared_ptr<Executor> executor, int nBlocks, int nThreadsPerBlock,
             bool symmetricMemory, std::unordered_map<std::string, uintptr_t> extras, DataType accumDtype) {
            return static_cast<int>(self.execute(comm, reinterpret_cast<const void*>(input), reinterpret_cast<void*>(output), inputSize,
                                                 outputSize, dtype, op, reinterpret_cast<cudaStream_t>(stream), executor, nBlocks,
                                                 nThreadsPerBlock, symmetricMemory, extras, accumDtype));
          },
          py::arg("comm"), py::arg("input"), py::arg("output"), py::arg("input_size"), py::arg("output_size"), py::arg("dtype"),
          py::arg("op") = NOP, py::arg("stream") = 0, py::arg("executor") = nullptr, py::arg("n_blocks") = 0,
          py::arg("n_threads_per_block") = 0, py::arg("symmetric_memory") = false,
          py::arg("extras") = std::unordered_map<std::string, uintptr_t>(), py::arg("accum_dtype") = DataType::AUTO)
      .def("reset", &Algorithm::reset)
      // A capsule holds a heap-allocated shared_ptr<Algorithm>: the exchange format between extension modules
      // that were compiled separately (for example by the native-code compiler) and this module.
      .def("to_native_capsule",
           [](std::shared_ptr<Algorithm> self) {
             auto* holder = new std::shared_ptr<Algorithm>(std::move(self));
             return py::capsule(holder, kCapsuleName, [](PyObject* cap) {
               delete static_cast<std::shared_ptr<Algorithm>*>(PyCapsule_GetPointer(cap, kCapsuleName));
             });
           })
      .def_static("from_native_capsule", [](py::capsule cap) {
        if (cap.name() == nullptr || std::string(cap.name()) != kCapsuleName) throw py::type_error("capsule does not hold an algorithm");
        return *static_cast<std::shared_ptr<Algorithm>*>(cap.get_pointer());
      });

  py::class_<NativeAlgorithm, Algorithm, std::shared_ptr<NativeAlgorithm>>(m, "NativeAlgorithm")
      .def(py::init([](std::string name, std::string collective, py::object init, py::function kernel, size_t minSize, size_t maxSize,
                       CollectiveBufferMode mode, std::unordered_map<std::string, uint64_t> tags, Algorithm::Constraint constraint) {
             NativeAlgorithm::InitFunc initFn;
             if (!init.is_none()) {
               py::function f = init.cast<py::function>();
               initFn = [f](std::shared_ptr<Communicator> comm) {
                 py::gil_scoped_acquire gil;
                 f(comm);
               };
             }
             // the Python callable gets integers for pointers and returns a CommResult or an int (0 = success)
             NativeAlgorithm::KernelFunc kernelFn = [kernel](const void* in, void* out, size_t inBytes, size_t outBytes, DataType dtype,
                                                             ReduceOp op, cudaStream_t stream, int nBlocks, int nThreads, bool symmetric,
                                                             const std::unordered_map<std::string, uintptr_t>& extras) {
               py::gil_scoped_acquire gil;
               py::object r = kernel(reinterpret_cast<uintptr_t>(in), reinterpret_cast<uintptr_t>(out), inBytes, outBytes, dtype, op,
                                     reinterpret_cast<uintptr_t>(stream), nBlocks, nThreads, symmetric, extras);
               if (r.is_none()) return CommResult::Success;
               if (py::isinstance<CommResult>(r)) return r.cast<CommResult>();
               return static_cast<CommResult>(r.cast<int>());
             };
             return std::make_shared<NativeAlgorithm>(std::move(name), std::move(collective), std::move(initFn), std::move(kernelFn),
                                                      minSize, maxSize, mode, std::move(tags), constraint);
           }),
           py::arg("name"), py::arg("collective"), py::arg("init") = py::none(), py::arg("kernel"), py::arg("min_message_size") = 0,
           py::arg("max_message_size") = UINT64_MAX, py::arg("buffer_mode") = CollectiveBufferMode::Any,
           py::arg("tags") = std::unordered_map<std::string, uint64_t>(), py::arg("constraint") = Algorithm::Constraint());

  py::class_<DslAlgorithm, Algorithm, std::shared_ptr<DslAlgorithm>>(m, "DslAlgorithm")
      .def(py::init<std::string, ExecutionPlan, std::unordered_map<std::string, uint64_t>, Algorithm::Constraint>(), py::arg("id"),
           py::arg("plan"), py::arg("tags") = std::unordered_map<std::string, uint64_t>(), py::arg("constraint") = Algorithm::Constraint())
      .def_property_readonly("id", &DslAlgorithm::id);

  py::class_<AlgorithmBuilder, PyAlgorithmBuilder, std::shared_ptr<AlgorithmBuilder>>(m, "AlgorithmBuilder")
      .def(py::init<>())
      .def("build", &AlgorithmBuilder::build);

  py::class_<AlgorithmCollection>(m, "AlgorithmCollection")
      .def(py::init<>())
      .def("select_algorithm", &AlgorithmCollection::selectAlgorithm, py::arg("request"))
      .def("register_algorithm", &AlgorithmCollection::registerAlgorithm, py::arg("collective"), py::arg("algo_name"), py::arg("algorithm"))
      .def("get_algorithms_by_collective", &AlgorithmCollection::getAlgorithmsByCollective, py::arg("collective"))
      .def("get_all_algorithms", &AlgorithmCollection::getAllAlgorithms)
      .def("set_selectors", &AlgorithmCollection::setSelectors, py::arg("selector"), py::arg("fallback_selector"))
      .def("extend", &AlgorithmCollection::extend, py::arg("other"));

  using Builder = collective::AlgorithmCollectionBuilder;
  py::class_<Builder, std::shared_ptr<Builder>>(m, "AlgorithmCollectionBuilder")
      .def_static("get_instance", &Builder::getInstance)
      .def_static("reset", &Builder::reset)
      .def("add_algorithm_builder", &Builder::addAlgorithmBuilder, py::arg("builder"))
      .def("add_dsl_algorithm_builder",
           [](Builder& self, std::shared_ptr<Algorithm> algo) { self.addAlgorithmBuilder(std::make_shared<FixedAlgorithmBuilder>(std::move(algo))); },
           py::arg("algorithm"))
      .def("set_algorithm_selector", &Builder::setAlgorithmSelector, py::arg("selector"))
      .def("set_fallback_algorithm_selector", &Builder::setFallbackAlgorithmSelector, py::arg("selector"))
      .def("build", &Builder::build)
      .def("build_default_algorithms", &Builder::buildDefaultAlgorithms, py::arg("heap"));
  m.def("select_default_algorithm", &collective::selectDefaultAlgorithm, py::arg("algo_map_by_collective"), py::arg("request"));

  py::class_<CudaModule, std::shared_ptr<CudaModule>>(m, "CudaModule")
      .def(py::init([](py::bytes image) { return std::make_shared<CudaModule>(std::string(image)); }), py::arg("image"))
      .def("function", &CudaModule::function, py::arg("name"));
  m.def(
      "launch_packed",
      [](uintptr_t function, py::bytes params, unsigned gridX, unsigned gridY, unsigned blockX, unsigned shared, uintptr_t stream,
         bool cooperative, std::vector<size_t> offsets) {
        launchPacked(function, std::string(params), gridX, gridY, blockX, shared, stream, cooperative, offsets);
      },
      py::arg("function"), py::arg("params"), py::arg("grid_x"), py::arg("grid_y") = 1, py::arg("block_x") = 1, py::arg("shared") = 0,
      py::arg("stream") = 0, py::arg("cooperative") = false, py::arg("offsets") = std::vector<size_t>());

  py::module_ npkit = m.def_submodule("npkit", "event tracer");
  npkit.def("init", &NpKit::Init, py::arg("rank"));
  npkit.def("dump", &NpKit::Dump, py::arg("dump_dir"));
  npkit.def("shutdown", &NpKit::Shutdown);
  npkit.def("enabled", &NpKit::Enabled);
  npkit.def("collect_cpu_event", &NpKit::CollectCpuEvent, py::arg("type"), py::arg("size"), py::arg("rsvd"), py::arg("timestamp"),
            py::arg("channel_id"));
  npkit.def("cpu_timestamp", &NpKit::GetCpuTimestamp);

  m.def("get_flag_buffer", [] {
    auto buf = getFlagBuffer();
    return py::make_tuple(reinterpret_cast<uintptr_t>(buf.first.get()), buf.second);
  });
}
