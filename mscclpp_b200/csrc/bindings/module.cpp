// pybind11 bindings of the native runtime (module mscclpp_b200.lib._native).
// Pointers and CUDA streams cross the boundary as integers, so the module needs no torch headers and
// works with any framework that can expose a device pointer (the reference's nanobind module does
// the same with raw handles: python/csrc/core_py.cpp:39-334).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include <mscclpp/core.hpp>
#include <mscclpp/env.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/symmetric_heap.hpp>

#include "../kernels/collectives.cuh"
#include "../kernels/gemm.cuh"
#include "bindings.hpp"

namespace py = pybind11;
using namespace mscclpp;

namespace {

void checkCuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw CudaError(std::string(what) + " failed", static_cast<int>(e));
}

CollArgs makeCollArgs(SymmetricHeap& heap, uintptr_t in, uintptr_t out, uint64_t bytes, int mode, bool nvls) {
  CollArgs a{};
  a.comm = heap.deviceComm();
  a.in = reinterpret_cast<const void*>(in);
  a.out = reinterpret_cast<void*>(out);
  a.bytes = bytes;
  a.emuRanks = heap.emulated() ? heap.world() : 1;
  a.emuStride = heap.emulated() ? heap.bytes() : 0;
  a.mode = mode;
  a.nvls = nvls ? 1 : 0;
  if (nvls && !heap.nvls()) throw Error("NVLS requested but the heap has no multicast mapping", ErrorCode::InvalidUsage);
  return a;
}

void setNorm(CollArgs& a, int rows, int hidden, float eps, uintptr_t residualIn, uintptr_t residualOut, uintptr_t gamma,
             bool broadcastResidual) {
  a.norm = 1;
  a.rows = rows;
  a.hidden = hidden;
  a.eps = eps;
  a.residualIn = reinterpret_cast<const void*>(residualIn);
  a.residualOut = reinterpret_cast<void*>(residualOut);
  a.gamma = reinterpret_cast<const void*>(gamma);
  a.broadcastResidual = broadcastResidual ? 1 : 0;
}

}  // namespace

PYBIND11_MODULE(_native, m) {
  m.doc() = "native runtime of mscclpp_b200 (sm_100a)";

  // ------------------------------------------------------------------ errors
  py::enum_<ErrorCode>(m, "ErrorCode")
      .value("SystemError", ErrorCode::SystemError)
      .value("InternalError", ErrorCode::InternalError)
      .value("RemoteError", ErrorCode::RemoteError)
      .value("InvalidUsage", ErrorCode::InvalidUsage)
      .value("Timeout", ErrorCode::Timeout)
      .value("Aborted", ErrorCode::Aborted)
      .value("ExecutorError", ErrorCode::ExecutorError);
  static py::exception<BaseError> baseError(m, "BaseError");
  static py::exception<Error> error(m, "Error", baseError.ptr());
  static py::exception<SysError> sysError(m, "SysError", baseError.ptr());
  static py::exception<CudaError> cudaError(m, "CudaError", baseError.ptr());
  static py::exception<CuError> cuError(m, "CuError", baseError.ptr());
  static py::exception<IbError> ibError(m, "IbError", baseError.ptr());
  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const Error& e) {
      // instantiate the Python exception so that it can carry the ErrorCode as an attribute
      py::object exc = error.attr("__call__")(e.what());
      exc.attr("error_code") = py::cast(e.getErrorCode());
      PyErr_SetObject(error.ptr(), exc.ptr());
    } catch (const SysError& e) {
      PyErr_SetString(sysError.ptr(), e.what());
    } catch (const CudaError& e) {
      PyErr_SetString(cudaError.ptr(), e.what());
    } catch (const CuError& e) {
      PyErr_SetString(cuError.ptr(), e.what());
    } catch (const IbError& e) {
      PyErr_SetString(ibError.ptr(), e.what());
    } catch (const BaseError& e) {
      PyErr_SetString(baseError.ptr(), e.what());
    }
  });

  m.def("version", &version);

  // ------------------------------------------------------------------ env
  py::class_<Env, std::shared_ptr<Env>>(m, "Env")
      .def_readonly("debug", &Env::debug)
      .def_readonly("debug_subsys", &Env::debugSubsys)
      .def_readonly("debug_file", &Env::debugFile)
      .def_readonly("log_level", &Env::logLevel)
      .def_readonly("log_subsys", &Env::logSubsys)
      .def_readonly("log_file", &Env::logFile)
      .def_readonly("hca_devices", &Env::hcaDevices)
      .def_readonly("ibv_so", &Env::ibvSo)
      .def_readonly("ibv_mode", &Env::ibvMode)
      .def_readonly("hostid", &Env::hostid)
      .def_readonly("socket_family", &Env::socketFamily)
      .def_readonly("socket_ifname", &Env::socketIfname)
      .def_readonly("comm_id", &Env::commId)
      .def_readonly("cache_dir", &Env::cacheDir)
      .def_readonly("npkit_dump_dir", &Env::npkitDumpDir)
      .def_readonly("cuda_ipc_use_default_stream", &Env::cudaIpcUseDefaultStream)
      .def_readonly("nccl_lib_path", &Env::ncclLibPath)
      .def_readonly("force_nccl_fallback_operation", &Env::forceNcclFallbackOperation)
      .def_readonly("nccl_symmetric_memory", &Env::ncclSymmetricMemory)
      .def_readonly("force_disable_nvls", &Env::forceDisableNvls)
      .def_readonly("force_disable_gdr", &Env::forceDisableGdr)
      .def_readonly("ib_gid_index", &Env::ibGidIndex)
      .def_readonly("device_timeout_ms", &Env::deviceTimeoutMs)
      .def_readonly("heap_bytes", &Env::heapBytes);
  m.def("env", &env);

  // ------------------------------------------------------------------ bootstrap
  py::class_<Bootstrap, std::shared_ptr<Bootstrap>>(m, "Bootstrap")
      .def("get_rank", &Bootstrap::getRank)
      .def("get_n_ranks", &Bootstrap::getNranks)
      .def("get_n_ranks_per_node", &Bootstrap::getNranksPerNode)
      // collective on first use (the ranks exchange their domains): other Python threads must be able to run
      .def("get_n_ranks_per_ipc_domain", &Bootstrap::getNranksPerIpcDomain, py::call_guard<py::gil_scoped_release>())
      .def(
          "send",
          [](Bootstrap& b, py::bytes data, int peer, int tag) {
            std::string s = data;
            py::gil_scoped_release rel;
            std::vector<char> v(s.begin(), s.end());
            b.send(v, peer, tag);
          },
          py::arg("data"), py::arg("peer"), py::arg("tag") = 0)
      .def(
          "recv",
          [](Bootstrap& b, int peer, int tag) {
            std::vector<char> v;
            {
              py::gil_scoped_release rel;
              b.recv(v, peer, tag);
            }
            return py::bytes(v.data(), v.size());
          },
          py::arg("peer"), py::arg("tag") = 0)
      .def("all_gather",
           [](Bootstrap& b, py::bytes mine) {
             std::string s = mine;
             const int n = b.getNranks();
             std::vector<char> all(s.size() * n);
             std::memcpy(all.data() + s.size() * b.getRank(), s.data(), s.size());
             {
               py::gil_scoped_release rel;
               b.allGather(all.data(), static_cast<int>(s.size()));
             }
             py::list out;
             for (int r = 0; r < n; r++) out.append(py::bytes(all.data() + s.size() * r, s.size()));
             return out;
           })
      .def("barrier", [](Bootstrap& b) {
        py::gil_scoped_release rel;
        b.barrier();
      })
      .def("group_barrier", [](Bootstrap& b, std::vector<int> ranks) {
        py::gil_scoped_release rel;
        b.groupBarrier(ranks);
      });

  py::class_<TcpBootstrap, Bootstrap, std::shared_ptr<TcpBootstrap>>(m, "TcpBootstrap")
      .def(py::init<int, int>(), py::arg("rank"), py::arg("n_ranks"))
      .def_static("create", [](int rank, int nRanks) { return std::make_shared<TcpBootstrap>(rank, nRanks); })
      .def_static("create_unique_id",
                  []() {
                    UniqueId id = TcpBootstrap::createUniqueId();
                    return py::bytes(reinterpret_cast<const char*>(id.data()), id.size());
                  })
      .def("get_unique_id",
           [](TcpBootstrap& b) {
             UniqueId id = b.getUniqueId();
             return py::bytes(reinterpret_cast<const char*>(id.data()), id.size());
           })
      .def(
          "initialize",
          [](TcpBootstrap& b, py::object idOrSpec, int64_t timeoutSec) {
            if (py::isinstance<py::bytes>(idOrSpec)) {
              std::string s = idOrSpec.cast<py::bytes>();
              if (s.size() != UniqueIdBytes) throw Error("UniqueId must be 128 bytes", ErrorCode::InvalidUsage);
              UniqueId id;
              std::memcpy(id.data(), s.data(), UniqueIdBytes);
              py::gil_scoped_release rel;
              b.initialize(id, timeoutSec);
            } else {
              std::string spec = idOrSpec.cast<std::string>();
              py::gil_scoped_release rel;
              b.initialize(spec, timeoutSec);
            }
          },
          py::arg("id_or_if_ip_port"), py::arg("timeout_sec") = 30)
      .def("abort", &TcpBootstrap::abort)
      .def("broadcast", [](TcpBootstrap& b, py::bytes data, int root) {
        std::string s = data;
        {
          py::gil_scoped_release rel;
          b.broadcast(s.data(), static_cast<int>(s.size()), root);
        }
        return py::bytes(s);
      });

  // ------------------------------------------------------------------ capability probes
  m.def("is_nvls_supported", &isNvlsSupported);
  m.def("is_bulk_supported", &isBulkSupported);
  m.def("is_fp8_multimem_supported", &isFp8MultimemSupported);
  m.def("is_cumem_map_allocated", [](uintptr_t p) { return isCuMemMapAllocated(reinterpret_cast<void*>(p)); });

  py::enum_<DataType>(m, "DataType")
      .value("int32", DataType::INT32)
      .value("uint32", DataType::UINT32)
      .value("float16", DataType::FLOAT16)
      .value("float32", DataType::FLOAT32)
      .value("bfloat16", DataType::BFLOAT16)
      .value("float8_e4m3", DataType::FLOAT8_E4M3)
      .value("float8_e4m3fn", DataType::FLOAT8_E4M3)  // the name torch and the reference use for the same format
      .value("float8_e5m2", DataType::FLOAT8_E5M2)
      .value("uint8", DataType::UINT8)
      .value("float8_e4m3b15", DataType::FLOAT8_E4M3B15)
      .value("auto", DataType::AUTO);
  py::enum_<ReduceOp>(m, "ReduceOp").value("SUM", SUM).value("MIN", MIN).value("NOP", NOP);

  // ------------------------------------------------------------------ symmetric heap
  py::class_<DeviceStatus>(m, "DeviceStatus")
      .def_readonly("code", &DeviceStatus::code)
      .def_readonly("poisoned", &DeviceStatus::poisoned)
      .def_readonly("rank", &DeviceStatus::rank)
      .def_readonly("block", &DeviceStatus::block)
      .def_readonly("where", &DeviceStatus::where)
      .def_readonly("peer", &DeviceStatus::peer)
      .def_readonly("expected", &DeviceStatus::expected)
      .def_readonly("observed", &DeviceStatus::observed)
      .def_readonly("count", &DeviceStatus::count);

  py::class_<SymmetricHeap, std::shared_ptr<SymmetricHeap>>(m, "SymmetricHeap")
      .def_static(
          "create",
          [](std::shared_ptr<Bootstrap> b, size_t bytes, size_t llSlotBytes, bool enableNvls, int64_t timeoutMs) {
            SymmetricHeap::Options o;
            o.bytes = bytes;
            if (llSlotBytes) o.llSlotBytes = llSlotBytes;
            o.enableNvls = enableNvls;
            o.timeoutMs = timeoutMs;
            py::gil_scoped_release rel;
            return SymmetricHeap::create(b, o);
          },
          py::arg("bootstrap"), py::arg("bytes") = 0, py::arg("ll_slot_bytes") = 0, py::arg("enable_nvls") = true,
          py::arg("timeout_ms") = -1)
      .def_static(
          "create_emulated",
          [](int world, size_t bytes, size_t llSlotBytes, int64_t timeoutMs) {
            SymmetricHeap::Options o;
            o.bytes = bytes;
            if (llSlotBytes) o.llSlotBytes = llSlotBytes;
            o.timeoutMs = timeoutMs;
            return SymmetricHeap::createEmulated(world, o);
          },
          py::arg("world"), py::arg("bytes") = 0, py::arg("ll_slot_bytes") = 0, py::arg("timeout_ms") = -1)
      .def("destroy", [](SymmetricHeap& h) {
        py::gil_scoped_release rel;
        h.destroy();
      })
      .def_property_readonly("rank", &SymmetricHeap::rank)
      .def_property_readonly("world", &SymmetricHeap::world)
      .def_property_readonly("emulated", &SymmetricHeap::emulated)
      .def_property_readonly("nvls", &SymmetricHeap::nvls)
      .def_property_readonly("bytes", &SymmetricHeap::bytes)
      .def_property_readonly("local_base", [](SymmetricHeap& h) { return reinterpret_cast<uintptr_t>(h.localBase()); })
      .def_property_readonly("mc_base", [](SymmetricHeap& h) { return reinterpret_cast<uintptr_t>(h.mcBase()); })
      .def("peer_base", [](SymmetricHeap& h, int r) { return reinterpret_cast<uintptr_t>(h.peerBase(r)); })
      .def("alloc", [](SymmetricHeap& h, size_t bytes, size_t align) { return reinterpret_cast<uintptr_t>(h.alloc(bytes, align)); },
           py::arg("bytes"), py::arg("alignment") = 256)
      .def("free", [](SymmetricHeap& h, uintptr_t p) { h.free(reinterpret_cast<void*>(p)); })
      .def("bytes_free", &SymmetricHeap::bytesFree)
      .def("symmetric_on_all_ranks",
           [](SymmetricHeap& h, uintptr_t p, size_t bytes) {
             py::gil_scoped_release release;  // may exchange offsets over the bootstrap
             return h.symmetricOnAllRanks(reinterpret_cast<void*>(p), bytes);
           },
           py::arg("ptr"), py::arg("bytes"))
      .def("contains", [](SymmetricHeap& h, uintptr_t p, size_t bytes) { return h.contains(reinterpret_cast<void*>(p), bytes); },
           py::arg("ptr"), py::arg("bytes") = 1)
      .def("emulated_ptr", [](SymmetricHeap& h, uintptr_t p, int r) {
        return reinterpret_cast<uintptr_t>(h.emulatedPtr(reinterpret_cast<void*>(p), r));
      })
      .def("status", [](SymmetricHeap& h) {
        h.refreshStatus();
        return h.status();
      })
      .def("check_status", &SymmetricHeap::checkStatus)
      .def("reset_status", &SymmetricHeap::resetStatus)
      .def("set_timeout_ms", &SymmetricHeap::setTimeoutMs)
      .def("device_comm_bytes", [](SymmetricHeap& h) {
        DeviceComm c = h.deviceComm();
        return py::bytes(reinterpret_cast<const char*>(&c), sizeof(c));
      });

  // ------------------------------------------------------------------ collectives
  m.def(
      "allreduce_ll",
      [](SymmetricHeap& heap, uintptr_t in, uintptr_t out, uint64_t bytes, DataType dtype, ReduceOp op, int nBlocks,
         int nThreads, uintptr_t stream, bool nvls, bool ll8) {
        CollArgs a = makeCollArgs(heap, in, out, bytes, kAllReduce, nvls);
        a.ll8 = ll8 ? 1 : 0;
        checkCuda(launchAllreduceLL(a, dtype, op, nBlocks, nThreads, reinterpret_cast<cudaStream_t>(stream)), "allreduce_ll");
      },
      py::arg("heap"), py::arg("input"), py::arg("output"), py::arg("bytes"), py::arg("dtype"), py::arg("op") = SUM,
      py::arg("n_blocks") = 8, py::arg("n_threads") = 512, py::arg("stream") = 0, py::arg("nvls") = false, py::arg("ll8") = false);
  m.def(
      "allreduce_ll128",
      [](SymmetricHeap& heap, uintptr_t in, uintptr_t out, uint64_t bytes, DataType dtype, ReduceOp op, uintptr_t scratch, uint64_t slotBytes,
         int nBlocks, int nThreads, uintptr_t stream) {
        CollArgs a = makeCollArgs(heap, in, out, bytes, kAllReduce, false);
        if (!heap.contains(reinterpret_cast<const void*>(scratch), ll128ScratchBytes(heap.world(), slotBytes)))
          throw Error("allreduce_ll128: the scratch must be symmetric-heap memory of 2 x world x slot_bytes", ErrorCode::InvalidUsage);
        a.ll128Scratch = reinterpret_cast<void*>(scratch);
        a.ll128SlotBytes = slotBytes;
        checkCuda(launchAllreduceLL128(a, dtype, op, nBlocks, nThreads, reinterpret_cast<cudaStream_t>(stream)), "allreduce_ll128");
      },
      py::arg("heap"), py::arg("input"), py::arg("output"), py::arg("bytes"), py::arg("dtype"), py::arg("op") = SUM, py::arg("scratch"),
      py::arg("slot_bytes"), py::arg("n_blocks") = 32, py::arg("n_threads") = 512, py::arg("stream") = 0);
  m.def(
      "allreduce_ll_rmsnorm",
      [](SymmetricHeap& heap, uintptr_t in, uintptr_t out, int rows, int hidden, DataType dtype, float eps,
         uintptr_t residualIn, uintptr_t residualOut, uintptr_t gamma, int nBlocks, int nThreads, uintptr_t stream,
         bool nvls) {
        const uint64_t bytes = static_cast<uint64_t>(rows) * hidden * dataTypeSize(dtype);
        CollArgs a = makeCollArgs(heap, in, out, bytes, kAllReduce, nvls);
        setNorm(a, rows, hidden, eps, residualIn, residualOut, gamma, false);
        checkCuda(launchAllreduceLL(a, dtype, SUM, nBlocks, nThreads, reinterpret_cast<cudaStream_t>(stream)),
                  "allreduce_ll_rmsnorm");
      },
      py::arg("heap"), py::arg("input"), py::arg("output"), py::arg("rows"), py::arg("hidden"), py::arg("dtype"),
      py::arg("eps"), py::arg("residual_in") = 0, py::arg("residual_out") = 0, py::arg("gamma") = 0,
      py::arg("n_blocks") = 8, py::arg("n_threads") = 1024, py::arg("stream") = 0, py::arg("nvls") = false);
  m.def(
      "two_shot",
      [](SymmetricHeap& heap, uintptr_t in, uintptr_t out, uint64_t bytes, DataType dtype, ReduceOp op, int mode,
         int nBlocks, int nThreads, uintptr_t stream, bool nvls, int root, int oneShot, uintptr_t stamps) {
        CollArgs a = makeCollArgs(heap, in, out, bytes, mode, nvls);
        a.root = root;
        a.oneShot = oneShot;
        a.stamps = reinterpret_cast<unsigned long long*>(stamps);
        checkCuda(launchTwoShot(a, dtype, op, nBlocks, nThreads, reinterpret_cast<cudaStream_t>(stream)), "two_shot");
      },
      py::arg("heap"), py::arg("input"), py::arg("output"), py::arg("bytes"), py::arg("dtype"), py::arg("op") = SUM,
      py::arg("mode") = 0, py::arg("n_blocks") = 32, py::arg("n_threads") = 512, py::arg("stream") = 0,
      py::arg("nvls") = false, py::arg("root") = 0, py::arg("one_shot") = 0, py::arg("stamps") = 0);
  m.def(
      "pipeline_allreduce",
      [](SymmetricHeap& heap, uintptr_t in, uintptr_t out, uint64_t bytes, DataType dtype, ReduceOp op, uintptr_t scratch, uint64_t sliceBytes,
         int nBlocks, int nThreads, uintptr_t stream, bool nvls, uint64_t emuStride) {
        if (nvls && !heap.nvls()) throw Error("NVLS requested but the heap has no multicast mapping", ErrorCode::InvalidUsage);
        if (!heap.contains(reinterpret_cast<const void*>(scratch), pipelineScratchBytes(nBlocks, sliceBytes)))
          throw Error("pipeline_allreduce: the scratch must be symmetric-heap memory of pipeline_scratch_bytes(n_blocks, slice_bytes)",
                      ErrorCode::InvalidUsage);
        PipeArgs a{};
        a.comm = heap.deviceComm();
        a.in = reinterpret_cast<const void*>(in);
        a.out = reinterpret_cast<void*>(out);
        a.bytes = bytes;
        a.scratch = reinterpret_cast<void*>(scratch);
        a.sliceBytes = sliceBytes;
        a.emuRanks = heap.emulated() ? heap.world() : 1;
        a.emuStride = heap.emulated() ? emuStride : 0;
        a.nvls = nvls ? 1 : 0;
        checkCuda(launchPipelineAllreduce(a, dtype, op, nBlocks, nThreads, reinterpret_cast<cudaStream_t>(stream)), "pipeline_allreduce");
      },
      py::arg("heap"), py::arg("input"), py::arg("output"), py::arg("bytes"), py::arg("dtype"), py::arg("op") = SUM, py::arg("scratch"),
      py::arg("slice_bytes"), py::arg("n_blocks") = 64, py::arg("n_threads") = 512, py::arg("stream") = 0, py::arg("nvls") = false,
      py::arg("emu_stride") = 0);
  m.def("pipeline_scratch_bytes", [](int nBlocks, uint64_t sliceBytes) { return pipelineScratchBytes(nBlocks, sliceBytes); },
        py::arg("n_blocks"), py::arg("slice_bytes"));
  m.def(
      "two_shot_rmsnorm",
      [](SymmetricHeap& heap, uintptr_t in, uintptr_t out, int rows, int hidden, DataType dtype, float eps,
         uintptr_t residualIn, uintptr_t residualOut, uintptr_t gamma, bool broadcastResidual, int nBlocks, int nThreads,
         uintptr_t stream, bool nvls) {
        const uint64_t bytes = static_cast<uint64_t>(rows) * hidden * dataTypeSize(dtype);
        CollArgs a = makeCollArgs(heap, in, out, bytes, kAllReduce, nvls);
        setNorm(a, rows, hidden, eps, residualIn, residualOut, gamma, broadcastResidual);
        checkCuda(launchTwoShot(a, dtype, SUM, nBlocks, nThreads, reinterpret_cast<cudaStream_t>(stream)),
                  "two_shot_rmsnorm");
      },
      py::arg("heap"), py::arg("input"), py::arg("output"), py::arg("rows"), py::arg("hidden"), py::arg("dtype"),
      py::arg("eps"), py::arg("residual_in") = 0, py::arg("residual_out") = 0, py::arg("gamma") = 0,
      py::arg("broadcast_residual") = true, py::arg("n_blocks") = 32, py::arg("n_threads") = 512, py::arg("stream") = 0,
      py::arg("nvls") = false);

  // ------------------------------------------------------------------ GEMM
  m.def(
      "gemm_bf16",
      [](uintptr_t A, uintptr_t B, uintptr_t D, int M, int N, int K, int ldd, int blockN, int numCtas, uintptr_t status,
         uintptr_t stream, int probe, int band) {
        checkCuda(gemm::gemmBf16(reinterpret_cast<const void*>(A), reinterpret_cast<const void*>(B),
                                 reinterpret_cast<void*>(D), M, N, K, ldd, blockN, numCtas,
                                 reinterpret_cast<DeviceStatus*>(status), reinterpret_cast<cudaStream_t>(stream), probe, band),
                  "gemm_bf16");
      },
      py::arg("a"), py::arg("b"), py::arg("d"), py::arg("m"), py::arg("n"), py::arg("k"), py::arg("ldd"),
      py::arg("block_n") = 256, py::arg("num_ctas") = 0, py::arg("status") = 0, py::arg("stream") = 0, py::arg("probe") = 0,
      py::arg("band") = 0);

  m.def(
      "gemm_bf16_two_sm",
      [](uintptr_t A, uintptr_t B, uintptr_t D, int M, int N, int K, int ldd, int numCtas, uintptr_t status, uintptr_t stream, int probe, int band) {
        checkCuda(gemm::gemmBf16TwoSm(reinterpret_cast<const void*>(A), reinterpret_cast<const void*>(B), reinterpret_cast<void*>(D), M, N,
                                      K, ldd, numCtas, reinterpret_cast<DeviceStatus*>(status), reinterpret_cast<cudaStream_t>(stream), probe, band),
                  "gemm_bf16_two_sm");
      },
      py::arg("a"), py::arg("b"), py::arg("d"), py::arg("m"), py::arg("n"), py::arg("k"), py::arg("ldd"), py::arg("num_ctas") = 0,
      py::arg("status") = 0, py::arg("stream") = 0, py::arg("probe") = 0, py::arg("band") = 0);

  registerCoreBindings(m);
  registerAlgorithmBindings(m);
  registerMoreBindings(m);
}
