#include <mscclpp/algorithm.hpp>

#include <mscclpp/gpu_utils.hpp>

#include "logger.hpp"

namespace mscclpp {

NativeAlgorithm::NativeAlgorithm(std::string name, std::string collective, InitFunc init, KernelFunc kernel, size_t minMessageSize,
                                 size_t maxMessageSize, CollectiveBufferMode bufferMode,
                                 std::unordered_map<std::string, uint64_t> tags, Constraint constraint)
    : name_(std::move(name)),
      collective_(std::move(collective)),
      init_(std::move(init)),
      kernel_(std::move(kernel)),
      minSize_(minMessageSize),
      maxSize_(maxMessageSize),
      bufferMode_(bufferMode),
      tags_(std::move(tags)),
      constraint_(constraint) {}

CommResult NativeAlgorithm::execute(std::shared_ptr<Communicator> comm, const void* input, void* output, size_t inputSize,
                                    size_t outputSize, DataType dtype, ReduceOp op, cudaStream_t stream, std::shared_ptr<Executor>,
                                    int nBlocks, int nThreadsPerBlock, bool symmetricMemory,
                                    const std::unordered_map<std::string, uintptr_t>& extras, DataType) {
  if (!initialized_) {
    if (init_) init_(comm);
    initialized_ = true;
  }
  return kernel_(input, output, inputSize, outputSize, dtype, op, stream, nBlocks, nThreadsPerBlock, symmetricMemory, extras);
}

DslAlgorithm::DslAlgorithm(std::string id, ExecutionPlan plan, std::unordered_map<std::string, uint64_t> tags, Constraint constraint)
    : id_(std::move(id)), name_(plan.name()), collective_(plan.collective()), plan_(plan), tags_(std::move(tags)), constraint_(constraint) {}

CommResult DslAlgorithm::execute(std::shared_ptr<Communicator>, const void* input, void* output, size_t inputSize, size_t outputSize,
                                 DataType dtype, ReduceOp op, cudaStream_t stream, std::shared_ptr<Executor> executor, int, int, bool,
                                 const std::unordered_map<std::string, uintptr_t>&, DataType) {
  if (!executor) return CommResult::InvalidUsage;
  if (op != SUM) {
    LOG_WARN(LogSubsys::EXEC, "plan '", name_, "': execution plans reduce with SUM only");
    return CommResult::InvalidArgument;
  }
  try {
    executor->execute(executor->heap()->rank(), const_cast<void*>(input), output, inputSize, outputSize, dtype, plan_, stream);
  } catch (const Error& e) {
    LOG_ERROR(LogSubsys::EXEC, "plan '", name_, "' failed: ", e.what());
    return e.getErrorCode() == ErrorCode::Timeout ? CommResult::Timeout : CommResult::InternalError;
  } catch (const BaseError& e) {
    LOG_ERROR(LogSubsys::EXEC, "plan '", name_, "' failed: ", e.what());
    return CommResult::UnhandledCudaError;
  }
  return CommResult::Success;
}

std::shared_ptr<Algorithm> AlgorithmCollection::selectAlgorithm(const CollectiveRequest& request) const {
  std::shared_ptr<Algorithm> algo;
  if (selector_) algo = selector_(algoMap_, request);
  if (!algo && fallbackSelector_) algo = fallbackSelector_(algoMap_, request);
  if (algo) {
    LOG_DEBUG(LogSubsys::ALGO, request.collective, " ", request.messageSize, " bytes -> ", algo->name());
  } else {
    LOG_DEBUG(LogSubsys::ALGO, request.collective, " ", request.messageSize, " bytes -> no algorithm");
  }
  return algo;
}

void AlgorithmCollection::registerAlgorithm(const std::string& collective, const std::string& algoName, std::shared_ptr<Algorithm> algorithm) {
  algoMap_[collective][algoName] = std::move(algorithm);
}

std::unordered_map<std::string, std::shared_ptr<Algorithm>> AlgorithmCollection::getAlgorithmsByCollective(const std::string& collective) const {
  auto it = algoMap_.find(collective);
  if (it == algoMap_.end()) return {};
  return it->second;
}

std::vector<std::shared_ptr<Algorithm>> AlgorithmCollection::getAllAlgorithms() const {
  std::vector<std::shared_ptr<Algorithm>> out;
  for (auto& c : algoMap_)
    for (auto& a : c.second) out.push_back(a.second);
  return out;
}

void AlgorithmCollection::setSelectors(AlgoSelectFunc selector, AlgoSelectFunc fallbackSelector) {
  selector_ = std::move(selector);
  fallbackSelector_ = std::move(fallbackSelector);
}

void AlgorithmCollection::extend(const AlgorithmCollection& other) {
  for (auto& c : other.algoMap_)
    for (auto& a : c.second) algoMap_[c.first][a.first] = a.second;
}

std::pair<std::shared_ptr<void>, size_t> getFlagBuffer() {
  static std::shared_ptr<uint32_t> buffer;
  constexpr size_t kFlags = 128;
  if (!buffer) {
    buffer = gpuCallocShared<uint32_t>(kFlags);
    std::vector<uint32_t> ones(kFlags, 1u);
    gpuMemcpy(buffer.get(), ones.data(), kFlags * sizeof(uint32_t), cudaMemcpyHostToDevice);
  }
  return {std::static_pointer_cast<void>(buffer), kFlags * sizeof(uint32_t)};
}

}  // namespace mscclpp
