// Algorithm framework: a uniform interface over native (hand-written kernel) and DSL (execution plan)
// collective algorithms, a registry and a selector hook (reference: include/mscclpp/algorithm.hpp:20-379,
// src/core/algorithm.cc:13-268).
#pragma once

#include <cuda_runtime.h>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "core.hpp"
#include "executor.hpp"
#include "gpu_data_types.hpp"
#include "symmetric_heap.hpp"

namespace mscclpp {

enum class CollectiveBufferMode { Any = 0, InPlace, OutOfPlace };
enum class AlgorithmType { Native = 0, DSL };
enum class CommResult {
  Success = 0,
  UnhandledCudaError = 1,
  SystemError = 2,
  InternalError = 3,
  InvalidArgument = 4,
  InvalidUsage = 5,
  RemoteError = 6,
  InProgress = 7,
  Timeout = 8,
};

struct CollectiveRequest {
  int worldSize = 1;
  int nRanksPerNode = 1;
  int rank = 0;
  const void* inputBuffer = nullptr;
  void* outputBuffer = nullptr;
  size_t messageSize = 0;
  cudaStream_t stream = nullptr;
  std::string collective;
  DataType dtype = DataType::FLOAT32;
  ReduceOp op = SUM;
  bool symmetricMemory = false;  // both buffers live in the symmetric heap at equal offsets on all ranks
  bool inCapture = false;        // the stream is being captured into a CUDA graph
  std::unordered_map<std::string, std::vector<uint64_t>> hints;
  CollectiveBufferMode bufferMode() const {
    return inputBuffer == outputBuffer ? CollectiveBufferMode::InPlace : CollectiveBufferMode::OutOfPlace;
  }
};

class Algorithm {
 public:
  struct Constraint {
    int worldSize = 0;      // 0 = any
    int nRanksPerNode = 0;  // 0 = any
  };
  virtual ~Algorithm() = default;
  virtual const std::string& name() const = 0;
  virtual const std::string& collective() const = 0;
  virtual std::pair<size_t, size_t> messageRange() const = 0;
  virtual void setMessageSizeRange(size_t minMessageSize, size_t maxMessageSize) = 0;
  virtual const std::unordered_map<std::string, uint64_t>& tags() const = 0;
  virtual CollectiveBufferMode bufferMode() const = 0;
  virtual Constraint constraint() const = 0;
  virtual AlgorithmType type() const = 0;
  // inputSize / outputSize in bytes. nBlocks / nThreads = 0 lets the algorithm choose.
  virtual CommResult execute(std::shared_ptr<Communicator> comm, const void* input, void* output, size_t inputSize,
                             size_t outputSize, DataType dtype, ReduceOp op, cudaStream_t stream,
                             std::shared_ptr<Executor> executor, int nBlocks = 0, int nThreadsPerBlock = 0,
                             bool symmetricMemory = false,
                             const std::unordered_map<std::string, uintptr_t>& extras = {},
                             DataType accumDtype = DataType::AUTO) = 0;
  virtual void reset() = 0;
};

// A native algorithm is a kernel-launch closure plus optional one-time initialisation.
class NativeAlgorithm : public Algorithm {
 public:
  using InitFunc = std::function<void(std::shared_ptr<Communicator>)>;
  using KernelFunc = std::function<CommResult(const void* input, void* output, size_t inputSize, size_t outputSize, DataType dtype,
                                              ReduceOp op, cudaStream_t stream, int nBlocks, int nThreadsPerBlock,
                                              bool symmetricMemory, const std::unordered_map<std::string, uintptr_t>& extras)>;
  NativeAlgorithm(std::string name, std::string collective, InitFunc init, KernelFunc kernel, size_t minMessageSize = 0,
                  size_t maxMessageSize = UINT64_MAX, CollectiveBufferMode bufferMode = CollectiveBufferMode::Any,
                  std::unordered_map<std::string, uint64_t> tags = {}, Constraint constraint = {});
  const std::string& name() const override { return name_; }
  const std::string& collective() const override { return collective_; }
  std::pair<size_t, size_t> messageRange() const override { return {minSize_, maxSize_}; }
  void setMessageSizeRange(size_t minMessageSize, size_t maxMessageSize) override {
    minSize_ = minMessageSize;
    maxSize_ = maxMessageSize;
  }
  const std::unordered_map<std::string, uint64_t>& tags() const override { return tags_; }
  CollectiveBufferMode bufferMode() const override { return bufferMode_; }
  Constraint constraint() const override { return constraint_; }
  AlgorithmType type() const override { return AlgorithmType::Native; }
  CommResult execute(std::shared_ptr<Communicator> comm, const void* input, void* output, size_t inputSize, size_t outputSize,
                     DataType dtype, ReduceOp op, cudaStream_t stream, std::shared_ptr<Executor> executor, int nBlocks,
                     int nThreadsPerBlock, bool symmetricMemory, const std::unordered_map<std::string, uintptr_t>& extras,
                     DataType accumDtype) override;
  void reset() override { initialized_ = false; }

 private:
  std::string name_, collective_;
  InitFunc init_;
  KernelFunc kernel_;
  size_t minSize_, maxSize_;
  CollectiveBufferMode bufferMode_;
  std::unordered_map<std::string, uint64_t> tags_;
  Constraint constraint_;
  bool initialized_ = false;
};

// A DSL algorithm runs an execution plan through the Executor.
class DslAlgorithm : public Algorithm {
 public:
  DslAlgorithm(std::string id, ExecutionPlan plan, std::unordered_map<std::string, uint64_t> tags = {}, Constraint constraint = {});
  const std::string& name() const override { return name_; }
  const std::string& collective() const override { return collective_; }
  std::pair<size_t, size_t> messageRange() const override {
    return rangeSet_ ? std::make_pair(minSize_, maxSize_) : std::make_pair(plan_.minMessageSize(), plan_.maxMessageSize());
  }
  void setMessageSizeRange(size_t minMessageSize, size_t maxMessageSize) override {
    minSize_ = minMessageSize;
    maxSize_ = maxMessageSize;
    rangeSet_ = true;
  }
  const std::unordered_map<std::string, uint64_t>& tags() const override { return tags_; }
  CollectiveBufferMode bufferMode() const override {
    return plan_.isInPlace() ? CollectiveBufferMode::InPlace : CollectiveBufferMode::OutOfPlace;
  }
  Constraint constraint() const override { return constraint_; }
  AlgorithmType type() const override { return AlgorithmType::DSL; }
  CommResult execute(std::shared_ptr<Communicator> comm, const void* input, void* output, size_t inputSize, size_t outputSize,
                     DataType dtype, ReduceOp op, cudaStream_t stream, std::shared_ptr<Executor> executor, int nBlocks,
                     int nThreadsPerBlock, bool symmetricMemory, const std::unordered_map<std::string, uintptr_t>& extras,
                     DataType accumDtype) override;
  void reset() override {}
  const std::string& id() const { return id_; }

 private:
  std::string id_, name_, collective_;
  ExecutionPlan plan_;
  std::unordered_map<std::string, uint64_t> tags_;
  Constraint constraint_;
  size_t minSize_ = 0, maxSize_ = 0;
  bool rangeSet_ = false;
};

class AlgorithmBuilder {
 public:
  virtual ~AlgorithmBuilder() = default;
  virtual std::shared_ptr<Algorithm> build() = 0;
};

using AlgoSelectFunc = std::function<std::shared_ptr<Algorithm>(
    const std::unordered_map<std::string, std::unordered_map<std::string, std::shared_ptr<Algorithm>>>& algoMapByCollective,
    const CollectiveRequest& request)>;

class AlgorithmCollection {
 public:
  // User selector first, then the fallback selector; nullptr when neither picks anything.
  std::shared_ptr<Algorithm> selectAlgorithm(const CollectiveRequest& request) const;
  void registerAlgorithm(const std::string& collective, const std::string& algoName, std::shared_ptr<Algorithm> algorithm);
  std::unordered_map<std::string, std::shared_ptr<Algorithm>> getAlgorithmsByCollective(const std::string& collective) const;
  std::vector<std::shared_ptr<Algorithm>> getAllAlgorithms() const;
  void setSelectors(AlgoSelectFunc selector, AlgoSelectFunc fallbackSelector);
  void extend(const AlgorithmCollection& other);

 private:
  std::unordered_map<std::string, std::unordered_map<std::string, std::shared_ptr<Algorithm>>> algoMap_;
  AlgoSelectFunc selector_;
  AlgoSelectFunc fallbackSelector_;
};

// Process-wide buffer of 128 x uint32 flags, initialised to 1 (kept for plans and user kernels that
// expect it; the native kernels of this library keep their launch epoch in the symmetric heap).
std::pair<std::shared_ptr<void>, size_t> getFlagBuffer();

}  // namespace mscclpp
