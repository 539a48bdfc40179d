// Executor: runs a DSL-compiled JSON execution plan on the GPU (reference API:
// include/mscclpp/executor.hpp:25-99; semantics: src/core/executor/execution_plan.cc:478-668 and
// src/core/include/execution_kernel.hpp:46-798).
//
// B200-first difference: the executor works on the symmetric heap. Input, output and scratch buffers
// are heap ranges at equal offsets on all ranks, so "remote buffer" operands, channel semaphores and
// switch (multimem) operands are all plain arithmetic on peerBase / mcBase; nothing is connected or
// registered per plan. User buffers outside the heap are staged through heap buffers of the executor.
#pragma once

#include <memory>
#include <string>
#include <vector>

#include "core.hpp"
#include "gpu_data_types.hpp"
#include "symmetric_heap.hpp"

namespace mscclpp {

enum class PacketType { LL8, LL16 };

class ExecutionPlan {
 public:
  ExecutionPlan(const std::string& planPath, int rank);
  // Parse from JSON text instead of a file.
  static ExecutionPlan fromString(const std::string& jsonText, int rank);
  ~ExecutionPlan();
  ExecutionPlan(const ExecutionPlan&);
  ExecutionPlan& operator=(const ExecutionPlan&);

  std::string name() const;
  std::string collective() const;
  std::string protocol() const;
  size_t minMessageSize() const;
  size_t maxMessageSize() const;
  bool isInPlace() const;
  int nRanks() const;
  int nThreadsPerBlock() const;

  struct Impl;
  std::shared_ptr<Impl> impl_;

 private:
  ExecutionPlan() = default;
};

class Executor {
 public:
  explicit Executor(std::shared_ptr<SymmetricHeap> heap);
  // API-compatible form: builds a symmetric heap over the communicator's bootstrap.
  explicit Executor(std::shared_ptr<Communicator> comm, std::shared_ptr<char> defaultScratchBuffer = nullptr);
  ~Executor();

  // `rank` must be the heap's rank. Buffers inside the heap are used in place (they must sit at the same
  // heap offset on every rank); other buffers are copied through staging buffers on `stream`.
  void execute(int rank, void* sendbuff, void* recvbuff, size_t sendBuffSize, size_t recvBuffSize, DataType dataType,
               const ExecutionPlan& plan, cudaStream_t stream, PacketType packetType = PacketType::LL16);
  // Drops cached plan contexts (their heap allocations are returned).
  void reset();
  std::shared_ptr<SymmetricHeap> heap() const;
  // How many execute() calls so far ran directly on buffers outside the heap (mapped on every rank) instead of staging them.
  uint64_t zeroCopyLaunches() const;

  // Debugging aid, switched on with MSCCLPP_EXECUTOR_CANARY=1 when the executor is created: every buffer the executor
  // allocates for a plan (scratch, staging) gets a guard band of 256 bytes of 0xA5 on both sides. checkCanaries()
  // waits for the device, reads all bands back and throws an Error that names plan, buffer, side and the first
  // overwritten byte; it returns the number of bands it looked at (0 when the switch is off). Every rank's bands also
  // catch what a PEER wrote past the end of this rank's scratch. reset() runs the check before it frees the buffers.
  struct CanaryRegion {
    std::string label;  // "<plan>/<buffer>/<front|back>[/rank r]"
    uint64_t address;   // device address of the band
    size_t bytes;
  };
  std::vector<CanaryRegion> canaryRegions() const;
  size_t checkCanaries();

 private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
};

}  // namespace mscclpp
