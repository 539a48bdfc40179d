#include "gdr.hpp"

#include <dlfcn.h>
#include <unistd.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

#include <mscclpp/env.hpp>
#include <mscclpp/gpu_utils.hpp>

#include "logger.hpp"

namespace mscclpp {

namespace {

// the part of gdrapi.h that is used
struct GdrMh {
  unsigned long h;
};
struct GdrInfo {
  uint64_t va;
  uint64_t mappedSize;
  uint32_t pageSize;
  uint64_t tmCycles;
  uint32_t cyclesPerMs;
  unsigned mapped : 1;
  unsigned wcMapping : 1;
  int mappingType;
};

constexpr size_t kGpuPage = 64 * 1024;

struct GdrApi {
  void* lib = nullptr;
  void* ctx = nullptr;  // gdr_t
  GdrStatus status = GdrStatus::LibraryMissing;
  std::string detail;
  void* (*open)() = nullptr;
  int (*close)(void*) = nullptr;
  int (*pin)(void*, unsigned long, size_t, uint64_t, uint32_t, GdrMh*) = nullptr;
  int (*unpin)(void*, GdrMh) = nullptr;
  int (*map)(void*, GdrMh, void**, size_t) = nullptr;
  int (*unmap)(void*, GdrMh, void*, size_t) = nullptr;
  int (*getInfo)(void*, GdrMh, GdrInfo*) = nullptr;

  GdrApi() {
    if (env()->forceDisableGdr) {
      status = GdrStatus::Disabled;
      return;
    }
    const char* forced = std::getenv("MSCCLPP_GDRCOPY_SO");
    const char* names[] = {forced, "libgdrapi.so.2", "libgdrapi.so"};
    for (const char* n : names) {
      if (n == nullptr || n[0] == '\0') continue;
      lib = ::dlopen(n, RTLD_NOW | RTLD_LOCAL);
      if (lib != nullptr) break;
      detail = ::dlerror();
      if (n == forced) break;  // a named library that does not load is an answer
    }
    if (lib == nullptr) return;
    auto sym = [&](auto& slot, const char* name) {
      slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(::dlsym(lib, name));
      return slot != nullptr;
    };
    const bool ok = sym(open, "gdr_open") & sym(close, "gdr_close") & sym(pin, "gdr_pin_buffer") & sym(unpin, "gdr_unpin_buffer") &
                    sym(map, "gdr_map") & sym(unmap, "gdr_unmap") & sym(getInfo, "gdr_get_info");
    if (!ok) {
      detail = "libgdrapi lacks a required symbol";
      return;
    }
    // the stock library talks to /dev/gdrdrv; a library named explicitly may be a software stand-in without a driver
    if (forced == nullptr && ::access("/dev/gdrdrv", F_OK) != 0) {
      status = GdrStatus::DriverMissing;
      return;
    }
    ctx = open();
    status = ctx != nullptr ? GdrStatus::Ok : GdrStatus::OpenFailed;
  }
  ~GdrApi() {
    if (ctx != nullptr) (void)close(ctx);
  }
};

GdrApi& gdr() {
  static GdrApi api;
  return api;
}

}  // namespace

GdrStatus gdrStatus() { return gdr().status; }

std::string gdrStatusMessage() {
  switch (gdr().status) {
    case GdrStatus::Ok:
      return "GDRCopy is available";
    case GdrStatus::Disabled:
      return "GDRCopy is switched off by MSCCLPP_FORCE_DISABLE_GDR";
    case GdrStatus::LibraryMissing:
      return "libgdrapi could not be loaded (" + gdr().detail + ")";
    case GdrStatus::DriverMissing:
      return "the gdrdrv kernel module is not loaded (/dev/gdrdrv is absent)";
    case GdrStatus::OpenFailed:
      return "gdr_open() failed";
  }
  return "unknown";
}

GdrMap::GdrMap(void* deviceAddr, int deviceId) {
  GdrApi& g = gdr();
  if (g.status != GdrStatus::Ok || deviceAddr == nullptr) return;
  std::unique_ptr<CudaDeviceGuard> guard;
  if (deviceId >= 0) guard = std::make_unique<CudaDeviceGuard>(deviceId);
  const unsigned long addr = reinterpret_cast<unsigned long>(deviceAddr);
  const unsigned long page = addr & ~(kGpuPage - 1);
  GdrMh mh{};
  if (g.pin(g.ctx, page, kGpuPage, 0, 0, &mh) != 0) {
    LOG_WARN(LogSubsys::CONN, "gdr_pin_buffer failed for the GPU page at ", reinterpret_cast<void*>(page));
    return;
  }
  handle_ = mh.h;
  pinned_ = true;
  void* va = nullptr;
  if (g.map(g.ctx, mh, &va, kGpuPage) != 0 || va == nullptr) {
    LOG_WARN(LogSubsys::CONN, "gdr_map failed");
    return;
  }
  mapBase_ = va;
  mapBytes_ = kGpuPage;
  GdrInfo info{};
  uint64_t start = page;
  if (g.getInfo(g.ctx, mh, &info) == 0 && info.va != 0) start = info.va;  // the pinned range may begin below the page asked for
  hostPtr_ = reinterpret_cast<uint64_t*>(static_cast<char*>(va) + (addr - start));
}

GdrMap::~GdrMap() {
  GdrApi& g = gdr();
  GdrMh mh{handle_};
  if (mapBase_ != nullptr) (void)g.unmap(g.ctx, mh, mapBase_, mapBytes_);
  if (pinned_) (void)g.unpin(g.ctx, mh);
}

void GdrMap::store(uint64_t value) const {
  // BAR1 is mapped write-combining: the fence pushes the store out instead of leaving it in a combining buffer
  reinterpret_cast<std::atomic<uint64_t>*>(hostPtr_)->store(value, std::memory_order_release);
  std::atomic_thread_fence(std::memory_order_seq_cst);
}

uint64_t GdrMap::load() const { return reinterpret_cast<std::atomic<uint64_t>*>(hostPtr_)->load(std::memory_order_acquire); }

}  // namespace mscclpp
