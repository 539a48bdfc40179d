// Context internals: copy streams for CudaIpc connections and the token pool semaphores draw from.
#pragma once

#include <map>

#include <cuda_runtime.h>
#include <memory>
#include <mutex>
#include <vector>

#include <mscclpp/core.hpp>

#include "ib.hpp"

namespace mscclpp {

class IpcStream {
 public:
  explicit IpcStream(int deviceId);
  ~IpcStream();
  cudaStream_t stream();
  void markDirty() { dirty_ = true; }
  void sync();

 private:
  int deviceId_;
  cudaStream_t stream_ = nullptr;
  bool dirty_ = false;
};

// 8-byte device tokens for semaphores, carved from one allocation so that thousands of semaphores
// do not cost thousands of cudaMalloc calls (and, on the VMM path, stay multicast-bindable).
class TokenPool {
 public:
  explicit TokenPool(size_t nTokens);
  ~TokenPool();
  std::shared_ptr<uint64_t> getToken();
  void* base() const { return base_; }
  size_t bytes() const { return nTokens_ * sizeof(uint64_t); }

 private:
  size_t nTokens_;
  void* base_ = nullptr;
  bool physical_ = false;
  std::mutex mutex_;
  std::vector<uint32_t> freeList_;
};

struct Context::Impl {
  std::mutex mutex;
  std::vector<std::shared_ptr<IpcStream>> streams;
  std::map<int, std::shared_ptr<TokenPool>> tokenPools;  // one pool per GPU of this process
  std::map<Transport, std::shared_ptr<IbCtx>> ibContexts;  // opened on first use, one per IB device
  std::shared_ptr<IpcStream> ipcStream();
  std::shared_ptr<TokenPool> tokens();  // the pool of the current device
  IbCtx& ibContext(Transport ibTransport);
};

}  // namespace mscclpp
