// Process-wide, read-once configuration taken from MSCCLPP_* environment variables.
// Variable set mirrors the reference (include/mscclpp/env.hpp:20-126, src/core/env.cpp:48-70).
#pragma once

#include <memory>
#include <string>

namespace mscclpp {

class Env {
 public:
  const std::string debug;                // MSCCLPP_DEBUG (legacy level name)
  const std::string debugSubsys;          // MSCCLPP_DEBUG_SUBSYS
  const std::string debugFile;            // MSCCLPP_DEBUG_FILE
  const std::string logLevel;             // MSCCLPP_LOG_LEVEL: DEBUG|INFO|WARN|ERROR (default ERROR)
  const std::string logSubsys;            // MSCCLPP_LOG_SUBSYS: comma list of ENV,GPU,NET,CONN,EXEC,NCCL,ALGO; ^ inverts
  const std::string logFile;              // MSCCLPP_LOG_FILE
  const std::string hcaDevices;           // MSCCLPP_HCA_DEVICES
  const std::string ibvSo;                // MSCCLPP_IBV_SO
  const std::string ibvMode;              // MSCCLPP_IBV_MODE: host | host-no-atomic
  const std::string hostid;               // MSCCLPP_HOSTID: overrides the host identity (lets one box pose as many)
  const std::string socketFamily;         // MSCCLPP_SOCKET_FAMILY: AF_INET | AF_INET6
  const std::string socketIfname;         // MSCCLPP_SOCKET_IFNAME: interface name or prefix list
  const std::string commId;               // MSCCLPP_COMM_ID: "ip:port" rendezvous used by the NCCL shim
  const std::string cacheDir;             // MSCCLPP_CACHE_DIR (default ~/.cache/mscclpp)
  const std::string npkitDumpDir;         // MSCCLPP_NPKIT_DUMP_DIR
  const bool cudaIpcUseDefaultStream;     // MSCCLPP_CUDAIPC_USE_DEFAULT_STREAM
  const std::string ncclLibPath;          // MSCCLPP_NCCL_LIB_PATH: real NCCL to fall back to
  const std::string forceNcclFallbackOperation;  // MSCCLPP_FORCE_NCCL_FALLBACK_OPERATION: comma list or "all"
  const bool ncclSymmetricMemory;         // MSCCLPP_NCCL_SYMMETRIC_MEMORY
  const bool forceDisableNvls;            // MSCCLPP_FORCE_DISABLE_NVLS
  const bool forceDisableGdr;             // MSCCLPP_FORCE_DISABLE_GDR
  const int ibGidIndex;                   // MSCCLPP_IB_GID_INDEX (-1 = auto)
  const long deviceTimeoutMs;             // MSCCLPP_DEVICE_TIMEOUT_MS: budget of device-side waits (default 10000)
  const long heapBytes;                   // MSCCLPP_HEAP_BYTES: symmetric heap size per rank (default 2 GiB)

 private:
  Env();
  friend std::shared_ptr<Env> env();
};

// The singleton. First call reads the environment; later changes to the environment are ignored.
std::shared_ptr<Env> env();

}  // namespace mscclpp
