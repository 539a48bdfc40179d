// Builder of the default native algorithm collection plus user-registered builders and selectors
// (reference: include/mscclpp/ext/collectives/algorithm_collection_builder.hpp:20-61).
#pragma once

#include <memory>
#include <vector>

#include "../../algorithm.hpp"

namespace mscclpp {
namespace collective {

class AlgorithmCollectionBuilder {
 public:
  static std::shared_ptr<AlgorithmCollectionBuilder> getInstance();
  static void reset();
  void addAlgorithmBuilder(std::shared_ptr<AlgorithmBuilder> builder);
  void setAlgorithmSelector(AlgoSelectFunc selector);
  void setFallbackAlgorithmSelector(AlgoSelectFunc selector);
  // Native algorithms of this library on `heap` (names default_allreduce_*, default_allgather_*,
  // default_reducescatter_*), user builders' algorithms and DSL plans found in <cache>/default/.
  AlgorithmCollection buildDefaultAlgorithms(std::shared_ptr<SymmetricHeap> heap);
  AlgorithmCollection build();

 private:
  std::vector<std::shared_ptr<AlgorithmBuilder>> builders_;
  AlgoSelectFunc selector_;
  AlgoSelectFunc fallbackSelector_;
};

// Size/placement based choice among the default algorithms, tuned on B200 (the reference's Blackwell
// table: src/ext/nccl/algorithm_selector.cc:52-89).
std::shared_ptr<Algorithm> selectDefaultAlgorithm(
    const std::unordered_map<std::string, std::unordered_map<std::string, std::shared_ptr<Algorithm>>>& algoMapByCollective,
    const CollectiveRequest& request);

}  // namespace collective
}  // namespace mscclpp
