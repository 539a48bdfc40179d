#include <mscclpp/env.hpp>

#include <cstdlib>
#include <mutex>

#include "logger.hpp"

namespace mscclpp {

namespace {
std::string readStr(const char* name, const std::string& dflt = "") {
  const char* v = std::getenv(name);
  return v ? std::string(v) : dflt;
}
bool readBool(const char* name, bool dflt) {
  const char* v = std::getenv(name);
  if (!v) return dflt;
  std::string s(v);
  for (auto& ch : s) ch = static_cast<char>(std::tolower(ch));
  return !(s == "0" || s == "false" || s == "off" || s == "no" || s.empty());
}
long readLong(const char* name, long dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  char* end = nullptr;
  long r = std::strtol(v, &end, 0);
  if (end == v) return dflt;
  // accept K/M/G suffixes for sizes
  if (end && (*end == 'K' || *end == 'k')) r <<= 10;
  if (end && (*end == 'M' || *end == 'm')) r <<= 20;
  if (end && (*end == 'G' || *end == 'g')) r <<= 30;
  return r;
}
std::string defaultCacheDir() {
  const char* home = std::getenv("HOME");
  return std::string(home ? home : "/tmp") + "/.cache/mscclpp";
}
}  // namespace

Env::Env()
    : debug(readStr("MSCCLPP_DEBUG")),
      debugSubsys(readStr("MSCCLPP_DEBUG_SUBSYS")),
      debugFile(readStr("MSCCLPP_DEBUG_FILE")),
      logLevel(readStr("MSCCLPP_LOG_LEVEL", "ERROR")),
      logSubsys(readStr("MSCCLPP_LOG_SUBSYS", "ALL")),
      logFile(readStr("MSCCLPP_LOG_FILE")),
      hcaDevices(readStr("MSCCLPP_HCA_DEVICES")),
      ibvSo(readStr("MSCCLPP_IBV_SO")),
      ibvMode(readStr("MSCCLPP_IBV_MODE", "host")),
      hostid(readStr("MSCCLPP_HOSTID")),
      socketFamily(readStr("MSCCLPP_SOCKET_FAMILY")),
      socketIfname(readStr("MSCCLPP_SOCKET_IFNAME")),
      commId(readStr("MSCCLPP_COMM_ID")),
      cacheDir(readStr("MSCCLPP_CACHE_DIR", defaultCacheDir())),
      npkitDumpDir(readStr("MSCCLPP_NPKIT_DUMP_DIR")),
      cudaIpcUseDefaultStream(readBool("MSCCLPP_CUDAIPC_USE_DEFAULT_STREAM", false)),
      ncclLibPath(readStr("MSCCLPP_NCCL_LIB_PATH")),
      forceNcclFallbackOperation(readStr("MSCCLPP_FORCE_NCCL_FALLBACK_OPERATION")),
      ncclSymmetricMemory(readBool("MSCCLPP_NCCL_SYMMETRIC_MEMORY", false)),
      forceDisableNvls(readBool("MSCCLPP_FORCE_DISABLE_NVLS", false)),
      forceDisableGdr(readBool("MSCCLPP_FORCE_DISABLE_GDR", false)),
      ibGidIndex(static_cast<int>(readLong("MSCCLPP_IB_GID_INDEX", -1))),
      deviceTimeoutMs(readLong("MSCCLPP_DEVICE_TIMEOUT_MS", 10000)),
      heapBytes(readLong("MSCCLPP_HEAP_BYTES", 2L << 30)) {}

std::shared_ptr<Env> env() {
  static std::shared_ptr<Env> instance;
  static std::once_flag once;
  std::call_once(once, [] {
    instance = std::shared_ptr<Env>(new Env());
    LOG_INFO(LogSubsys::ENV, "MSCCLPP_LOG_LEVEL=", instance->logLevel, " MSCCLPP_LOG_SUBSYS=", instance->logSubsys,
             " MSCCLPP_HOSTID=", instance->hostid, " MSCCLPP_SOCKET_IFNAME=", instance->socketIfname,
             " MSCCLPP_CACHE_DIR=", instance->cacheDir, " MSCCLPP_FORCE_DISABLE_NVLS=", instance->forceDisableNvls,
             " MSCCLPP_DEVICE_TIMEOUT_MS=", instance->deviceTimeoutMs, " MSCCLPP_HEAP_BYTES=", instance->heapBytes);
  });
  return instance;
}

}  // namespace mscclpp
