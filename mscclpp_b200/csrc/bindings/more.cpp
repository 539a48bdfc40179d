// Bindings of components added after the first slice (fused layers, channels, executor, proxy, ...).
#include "bindings.hpp"

#include <pybind11/stl.h>

#include <mscclpp/errors.hpp>
#include <mscclpp/executor.hpp>
#include <mscclpp/symmetric_heap.hpp>

#include "../kernels/moe.cuh"
#include "../kernels/sp_fused.cuh"
#include "../kernels/tp_fused.cuh"

namespace py = pybind11;
using namespace mscclpp;

namespace {
void checkCudaMore(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw CudaError(std::string(what) + " failed", static_cast<int>(e));
}
}  // namespace

void registerMoreBindings(py::module_& m) {
  // ------------------------------------------------------------------ executor
  py::enum_<PacketType>(m, "PacketType").value("LL8", PacketType::LL8).value("LL16", PacketType::LL16);
  py::class_<ExecutionPlan>(m, "ExecutionPlan")
      .def(py::init<const std::string&, int>(), py::arg("plan_path"), py::arg("rank"))
      .def_static("from_string", &ExecutionPlan::fromString, py::arg("json_text"), py::arg("rank"))
      .def_property_readonly("name", &ExecutionPlan::name)
      .def_property_readonly("collective", &ExecutionPlan::collective)
      .def_property_readonly("protocol", &ExecutionPlan::protocol)
      .def_property_readonly("min_message_size", &ExecutionPlan::minMessageSize)
      .def_property_readonly("max_message_size", &ExecutionPlan::maxMessageSize)
      .def_property_readonly("is_in_place", &ExecutionPlan::isInPlace)
      .def_property_readonly("n_ranks", &ExecutionPlan::nRanks);
  py::class_<Executor, std::shared_ptr<Executor>>(m, "Executor")
      .def(py::init<std::shared_ptr<SymmetricHeap>>(), py::arg("heap"))
      .def(
          "execute",
          [](Executor& self, int rank, uintptr_t sendbuff, uintptr_t recvbuff, size_t sendBytes, size_t recvBytes,
             DataType dtype, const ExecutionPlan& plan, uintptr_t stream, PacketType packetType) {
            self.execute(rank, reinterpret_cast<void*>(sendbuff), reinterpret_cast<void*>(recvbuff), sendBytes, recvBytes, dtype,
                         plan, reinterpret_cast<cudaStream_t>(stream), packetType);
          },
          py::arg("rank"), py::arg("sendbuff"), py::arg("recvbuff"), py::arg("send_bytes"), py::arg("recv_bytes"),
          py::arg("dtype"), py::arg("plan"), py::arg("stream") = 0, py::arg("packet_type") = PacketType::LL16)
      .def("reset", &Executor::reset)
      .def("zero_copy_launches", &Executor::zeroCopyLaunches)
      .def("check_canaries", &Executor::checkCanaries)
      .def("canary_regions", [](const Executor& self) {
        std::vector<std::tuple<std::string, uint64_t, size_t>> out;
        for (const auto& r : self.canaryRegions()) out.emplace_back(r.label, r.address, r.bytes);
        return out;
      });

  m.def(
      "tp_fused",
      [](SymmetricHeap& heap, std::vector<uintptr_t> a, std::vector<uintptr_t> b, uintptr_t partial, uintptr_t residualIn,
         uintptr_t residualOut, uintptr_t out, uintptr_t gamma, uintptr_t rinv, int M, int N, int K, float eps, int blockN,
         int numGemmCtas, int numReducers, int rowsPerUnit, int mode, bool nvls, uintptr_t stream, uintptr_t timeline,
         int sysFence) {
        TpFusedArgs args{};
        args.sysFence = sysFence;
        args.comm = heap.deviceComm();
        args.shape.M = M;
        args.shape.N = N;
        args.shape.K = K;
        args.timeline = reinterpret_cast<unsigned long long*>(timeline);
        args.partial = reinterpret_cast<__nv_bfloat16*>(partial);
        args.residualIn = reinterpret_cast<const __nv_bfloat16*>(residualIn);
        args.residualOut = reinterpret_cast<__nv_bfloat16*>(residualOut);
        args.out = reinterpret_cast<__nv_bfloat16*>(out);
        args.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
        args.rinv = reinterpret_cast<float*>(rinv);
        args.eps = eps;
        args.blockN = blockN;
        args.numGemmCtas = numGemmCtas;
        args.rowsPerUnit = rowsPerUnit;
        args.mode = mode;
        args.nvls = nvls ? 1 : 0;
        args.emuRanks = heap.emulated() ? heap.world() : 1;
        const size_t need = heap.emulated() ? heap.world() : 1;
        if (a.size() != need || b.size() != need) throw Error("tp_fused: one A and one B pointer per (emulated) rank", ErrorCode::InvalidUsage);
        std::vector<const void*> ap, bp;
        for (auto v : a) ap.push_back(reinterpret_cast<const void*>(v));
        for (auto v : b) bp.push_back(reinterpret_cast<const void*>(v));
        checkCudaMore(launchTpFused(args, ap.data(), bp.data(), numReducers, reinterpret_cast<cudaStream_t>(stream)), "tp_fused");
      },
      py::arg("heap"), py::arg("a"), py::arg("b"), py::arg("partial"), py::arg("residual_in"), py::arg("residual_out"),
      py::arg("out"), py::arg("gamma"), py::arg("rinv"), py::arg("m"), py::arg("n"), py::arg("k"), py::arg("eps"),
      py::arg("block_n") = 256, py::arg("num_gemm_ctas") = 0, py::arg("num_reducers") = 0, py::arg("rows_per_unit") = 0,
      py::arg("mode") = 0, py::arg("nvls") = false, py::arg("stream") = 0, py::arg("timeline") = 0, py::arg("sys_fence") = -1);
  m.def(
      "all_gather_gemm",
      [](SymmetricHeap& heap, uintptr_t aLocal, uintptr_t aFull, std::vector<uintptr_t> b, uintptr_t d, int M, int N, int K, int blockN,
         int numGemmCtas, int numCopiers, int activation, uintptr_t stream) {
        AgGemmArgs args{};
        args.comm = heap.deviceComm();
        args.shape.M = M;
        args.shape.N = N;
        args.shape.K = K;
        args.aLocal = reinterpret_cast<const __nv_bfloat16*>(aLocal);
        args.aFull = reinterpret_cast<__nv_bfloat16*>(aFull);
        args.D = reinterpret_cast<__nv_bfloat16*>(d);
        args.blockN = blockN;
        args.numGemmCtas = numGemmCtas;
        args.activation = activation;
        args.emuRanks = heap.emulated() ? heap.world() : 1;
        const size_t need = heap.emulated() ? heap.world() : 1;
        if (b.size() != need) throw Error("all_gather_gemm: one B pointer per (emulated) rank", ErrorCode::InvalidUsage);
        for (uintptr_t p : {aLocal, aFull, d}) {
          if (!heap.contains(reinterpret_cast<const void*>(p))) throw Error("all_gather_gemm: a_local, a_full and d must be symmetric-heap memory", ErrorCode::InvalidUsage);
        }
        std::vector<const void*> bp;
        for (auto v : b) bp.push_back(reinterpret_cast<const void*>(v));
        checkCudaMore(launchAllGatherGemm(args, bp.data(), numCopiers, reinterpret_cast<cudaStream_t>(stream)), "all_gather_gemm");
      },
      py::arg("heap"), py::arg("a_local"), py::arg("a_full"), py::arg("b"), py::arg("d"), py::arg("m"), py::arg("n"), py::arg("k"),
      py::arg("block_n") = 256, py::arg("num_gemm_ctas") = 0, py::arg("num_copiers") = 0, py::arg("activation") = 0,
      py::arg("stream") = 0);
  m.def(
      "tp_reduce_norm",
      [](SymmetricHeap& heap, uintptr_t partial, uintptr_t residualIn, uintptr_t residualOut, uintptr_t out, uintptr_t gamma, uintptr_t rinv,
         int M, int N, float eps, int numCtas, int rowsPerUnit, int mode, bool nvls, uintptr_t stream) {
        TpFusedArgs args{};
        args.comm = heap.deviceComm();
        args.shape.M = M;
        args.shape.N = N;
        args.partial = reinterpret_cast<__nv_bfloat16*>(partial);
        args.residualIn = reinterpret_cast<const __nv_bfloat16*>(residualIn);
        args.residualOut = reinterpret_cast<__nv_bfloat16*>(residualOut);
        args.out = reinterpret_cast<__nv_bfloat16*>(out);
        args.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
        args.rinv = reinterpret_cast<float*>(rinv);
        args.eps = eps;
        args.rowsPerUnit = rowsPerUnit;
        args.mode = mode;
        args.nvls = nvls ? 1 : 0;
        args.emuRanks = heap.emulated() ? heap.world() : 1;
        checkCudaMore(launchTpReduceNorm(args, numCtas, reinterpret_cast<cudaStream_t>(stream)), "tp_reduce_norm");
      },
      py::arg("heap"), py::arg("partial"), py::arg("residual_in"), py::arg("residual_out"), py::arg("out"), py::arg("gamma"), py::arg("rinv"),
      py::arg("m"), py::arg("n"), py::arg("eps"), py::arg("num_ctas") = 0, py::arg("rows_per_unit") = 0, py::arg("mode") = 0,
      py::arg("nvls") = false, py::arg("stream") = 0);
  m.def(
      "gemm_residual_sumsq",
      [](uintptr_t a, uintptr_t b, uintptr_t residual, uintptr_t h, uintptr_t sumsq, int M, int N, int K, int blockN, bool twoSm,
         uintptr_t stream) {
        checkCudaMore(launchGemmResidualSumsq(reinterpret_cast<const void*>(a), reinterpret_cast<const void*>(b),
                                              reinterpret_cast<const void*>(residual), reinterpret_cast<void*>(h),
                                              reinterpret_cast<float*>(sumsq), M, N, K, blockN, twoSm, nullptr,
                                              reinterpret_cast<cudaStream_t>(stream)),
                      "gemm_residual_sumsq");
        return tpSumsqParts(N, blockN, twoSm);  // parts per row written to sumsq[part][row]
      },
      py::arg("a"), py::arg("b"), py::arg("residual"), py::arg("h"), py::arg("sumsq"), py::arg("m"), py::arg("n"), py::arg("k"),
      py::arg("block_n") = 256, py::arg("two_sm") = false, py::arg("stream") = 0);
  m.def(
      "tp_decode",
      [](SymmetricHeap& heap, std::vector<uintptr_t> x, std::vector<uintptr_t> w, uintptr_t residualIn, uintptr_t residualOut, uintptr_t out,
         uintptr_t gamma, int T, int N, int K, float eps, bool nvls, int numCtas, uintptr_t stream, uintptr_t stamps) {
        const size_t need = heap.emulated() ? static_cast<size_t>(heap.world()) : 1;
        if (x.size() != need || w.size() != need) throw Error("tp_decode: one x and one w pointer per (emulated) rank", ErrorCode::InvalidUsage);
        for (uintptr_t p : {residualOut, out}) {
          if (p != 0 && !heap.contains(reinterpret_cast<const void*>(p))) throw Error("tp_decode: out and residual_out must be symmetric-heap memory", ErrorCode::InvalidUsage);
        }
        if (residualIn != 0 && !heap.contains(reinterpret_cast<const void*>(residualIn))) throw Error("tp_decode: residual_in must be symmetric-heap memory", ErrorCode::InvalidUsage);
        if (nvls && !heap.nvls()) throw Error("NVLS requested but the heap has no multicast mapping", ErrorCode::InvalidUsage);
        TpDecodeArgs a{};
        a.comm = heap.deviceComm();
        for (size_t e = 0; e < need; e++) {
          a.x[e] = reinterpret_cast<const __nv_bfloat16*>(x[e]);
          a.w[e] = reinterpret_cast<const __nv_bfloat16*>(w[e]);
        }
        a.residualIn = reinterpret_cast<const __nv_bfloat16*>(residualIn);
        a.residualOut = reinterpret_cast<__nv_bfloat16*>(residualOut);
        a.out = reinterpret_cast<__nv_bfloat16*>(out);
        a.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
        a.T = T;
        a.N = N;
        a.K = K;
        a.eps = eps;
        a.nvls = nvls ? 1 : 0;
        a.emuRanks = heap.emulated() ? heap.world() : 1;
        a.numCtas = numCtas;
        a.stamps = reinterpret_cast<unsigned long long*>(stamps);
        checkCudaMore(launchTpDecode(a, reinterpret_cast<cudaStream_t>(stream)), "tp_decode");
      },
      py::arg("heap"), py::arg("x"), py::arg("w"), py::arg("residual_in"), py::arg("residual_out"), py::arg("out"), py::arg("gamma"),
      py::arg("t"), py::arg("n"), py::arg("k"), py::arg("eps") = 1e-5f, py::arg("nvls") = false, py::arg("num_ctas") = 0, py::arg("stream") = 0,
      py::arg("stamps") = 0);
  m.def("tp_local_fused_workspace_bytes", [](int M, int N) { return tpLocalFusedWorkspaceBytes(M, N); }, py::arg("m"), py::arg("n"));
  m.def(
      "tp_local_fused",
      [](uintptr_t a, uintptr_t b, uintptr_t residual, uintptr_t h, uintptr_t out, uintptr_t gamma, uintptr_t workspace, int M, int N, int K,
         float eps, int blockN, bool twoSm, uintptr_t status, uintptr_t stream, int probe, uintptr_t stamps) {
        checkCudaMore(launchTpLocalFused(reinterpret_cast<const void*>(a), reinterpret_cast<const void*>(b), reinterpret_cast<const void*>(residual),
                                         reinterpret_cast<void*>(h), reinterpret_cast<void*>(out), reinterpret_cast<const void*>(gamma),
                                         reinterpret_cast<void*>(workspace), M, N, K, eps, blockN, twoSm,
                                         reinterpret_cast<DeviceStatus*>(status), reinterpret_cast<cudaStream_t>(stream), probe,
                                         reinterpret_cast<unsigned long long*>(stamps)),
                      "tp_local_fused");
      },
      py::arg("a"), py::arg("b"), py::arg("residual"), py::arg("h"), py::arg("out"), py::arg("gamma"), py::arg("workspace"), py::arg("m"),
      py::arg("n"), py::arg("k"), py::arg("eps") = 1e-5f, py::arg("block_n") = 256, py::arg("two_sm") = false, py::arg("status") = 0,
      py::arg("stream") = 0, py::arg("probe") = 0, py::arg("stamps") = 0);
  m.def(
      "tp_scale_rows_from_sumsq",
      [](uintptr_t h, uintptr_t sumsq, int numParts, uintptr_t gamma, uintptr_t out, int M, int N, float eps, uintptr_t stream) {
        checkCudaMore(launchTpScaleRowsFromSumsq(reinterpret_cast<const void*>(h), reinterpret_cast<const float*>(sumsq), numParts,
                                                 reinterpret_cast<const void*>(gamma), reinterpret_cast<void*>(out), M, N, eps,
                                                 reinterpret_cast<cudaStream_t>(stream)),
                      "tp_scale_rows_from_sumsq");
      },
      py::arg("h"), py::arg("sumsq"), py::arg("num_parts"), py::arg("gamma"), py::arg("out"), py::arg("m"), py::arg("n"), py::arg("eps"),
      py::arg("stream") = 0);
  m.def("moe_workspace_bytes", [] { return moeWorkspaceBytes(); });
  m.def(
      "moe_dispatch",
      [](SymmetricHeap& heap, uintptr_t x, uintptr_t topkIdx, uintptr_t slotMap, uintptr_t recvX, uintptr_t recvScales, uintptr_t recvSrc,
         uintptr_t recvCounts, uintptr_t workspace, int tokens, int hidden, int topk, int numExperts, int capacity, bool fp8, int nBlocks,
         uintptr_t stream) {
        MoeDispatchArgs a{};
        a.comm = heap.deviceComm();
        a.tokens = tokens;
        a.hidden = hidden;
        a.topk = topk;
        a.numExperts = numExperts;
        a.capacity = capacity;
        a.fp8 = fp8 ? 1 : 0;
        a.x = reinterpret_cast<const __nv_bfloat16*>(x);
        a.topkIdx = reinterpret_cast<const int32_t*>(topkIdx);
        a.slotMap = reinterpret_cast<int32_t*>(slotMap);
        a.recvX = reinterpret_cast<void*>(recvX);
        a.recvScales = reinterpret_cast<float*>(recvScales);
        a.recvSrc = reinterpret_cast<int32_t*>(recvSrc);
        a.recvCounts = reinterpret_cast<int32_t*>(recvCounts);
        a.workspace = reinterpret_cast<uint32_t*>(workspace);
        a.emuRanks = heap.emulated() ? heap.world() : 1;
        for (uintptr_t p : {recvX, recvSrc, workspace}) {
          if (!heap.contains(reinterpret_cast<const void*>(p))) throw Error("moe_dispatch: receive buffers and workspace must be symmetric-heap memory", ErrorCode::InvalidUsage);
        }
        checkCudaMore(launchMoeDispatch(a, nBlocks, reinterpret_cast<cudaStream_t>(stream)), "moe_dispatch");
      },
      py::arg("heap"), py::arg("x"), py::arg("topk_idx"), py::arg("slot_map"), py::arg("recv_x"), py::arg("recv_scales"), py::arg("recv_src"),
      py::arg("recv_counts"), py::arg("workspace"), py::arg("tokens"), py::arg("hidden"), py::arg("topk"), py::arg("num_experts"),
      py::arg("capacity"), py::arg("fp8") = false, py::arg("n_blocks") = 0, py::arg("stream") = 0);
  m.def(
      "moe_combine",
      [](SymmetricHeap& heap, uintptr_t topkIdx, uintptr_t topkWeights, uintptr_t slotMap, uintptr_t expertOut, uintptr_t y, int tokens,
         int hidden, int topk, int numExperts, int nBlocks, uintptr_t stream, uintptr_t outScales) {
        MoeCombineArgs a{};
        a.fp8 = outScales != 0 ? 1 : 0;
        a.outScales = reinterpret_cast<const float*>(outScales);
        if (outScales != 0 && !heap.contains(reinterpret_cast<const void*>(outScales))) throw Error("moe_combine: out_scales must be symmetric-heap memory", ErrorCode::InvalidUsage);
        a.comm = heap.deviceComm();
        a.tokens = tokens;
        a.hidden = hidden;
        a.topk = topk;
        a.numExperts = numExperts;
        a.topkIdx = reinterpret_cast<const int32_t*>(topkIdx);
        a.topkWeights = reinterpret_cast<const float*>(topkWeights);
        a.slotMap = reinterpret_cast<const int32_t*>(slotMap);
        a.expertOut = reinterpret_cast<const void*>(expertOut);
        a.y = reinterpret_cast<__nv_bfloat16*>(y);
        a.emuRanks = heap.emulated() ? heap.world() : 1;
        if (!heap.contains(reinterpret_cast<const void*>(expertOut))) throw Error("moe_combine: expert_out must be symmetric-heap memory", ErrorCode::InvalidUsage);
        checkCudaMore(launchMoeCombine(a, nBlocks, reinterpret_cast<cudaStream_t>(stream)), "moe_combine");
      },
      py::arg("heap"), py::arg("topk_idx"), py::arg("topk_weights"), py::arg("slot_map"), py::arg("expert_out"), py::arg("y"), py::arg("tokens"),
      py::arg("hidden"), py::arg("topk"), py::arg("num_experts"), py::arg("n_blocks") = 0, py::arg("stream") = 0, py::arg("out_scales") = 0);
  m.def(
      "moe_quantize_rows",
      [](uintptr_t x, uintptr_t q, uintptr_t scales, int rows, int hidden, uintptr_t stream) {
        checkCudaMore(launchMoeQuantizeRows(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<void*>(q), reinterpret_cast<float*>(scales),
                                            rows, hidden, reinterpret_cast<cudaStream_t>(stream)),
                      "moe_quantize_rows");
      },
      py::arg("x"), py::arg("q"), py::arg("scales"), py::arg("rows"), py::arg("hidden"), py::arg("stream") = 0);
  m.def(
      "tp_scale_rows",
      [](uintptr_t h, uintptr_t rinv, uintptr_t gamma, uintptr_t out, int M, int N, uintptr_t stream) {
        checkCudaMore(launchTpScaleRows(reinterpret_cast<const void*>(h), reinterpret_cast<const float*>(rinv),
                                        reinterpret_cast<const void*>(gamma), reinterpret_cast<void*>(out), M, N,
                                        reinterpret_cast<cudaStream_t>(stream)),
                      "tp_scale_rows");
      },
      py::arg("h"), py::arg("rinv"), py::arg("gamma"), py::arg("out"), py::arg("m"), py::arg("n"), py::arg("stream") = 0);
}
