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
  enum class State { Open, SwitchedOff, NoLibrary, NoDriver, OpenFailed };
  State state = State::NoLibrary;
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
      state = State::SwitchedOff;
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
      state = State::NoDriver;
      return;
    }
    ctx = open();
    state = ctx != nullptr ? State::Open : State::OpenFailed;
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

const GdrAvailability& gdrAvailability() {
  static const GdrAvailability answer = [] {
    GdrAvailability a;
    const GdrApi& g = gdr();
    a.usable = g.state == GdrApi::State::Open;
    switch (g.state) {
      case GdrApi::State::Open:
        a.reason = "GDRCopy is available";
        break;
      case GdrApi::State::SwitchedOff:
        a.reason = "GDRCopy is switched off by MSCCLPP_FORCE_DISABLE_GDR";
        break;
      case GdrApi::State::NoLibrary:
        a.reason = "libgdrapi could not be loaded (" + g.detail + ")";
        break;
      case GdrApi::State::NoDriver:
        a.reason = "the gdrdrv kernel module is not loaded (/dev/gdrdrv is absent)";
        break;
      case GdrApi::State::OpenFailed:
        a.reason = "gdr_open() failed";
        break;
    }
    return a;
  }();
  return answer;
}

std::unique_ptr<GdrWindow> GdrWindow::open(void* deviceAddr, int deviceId) {
  GdrApi& g = gdr();
  if (g.state != GdrApi::State::Open || deviceAddr == nullptr) return nullptr;
  std::unique_ptr<CudaDeviceGuard> guard;
  if (deviceId >= 0) guard = std::make_unique<CudaDeviceGuard>(deviceId);
  const unsigned long addr = reinterpret_cast<unsigned long>(deviceAddr);
  const unsigned long page = addr & ~(kGpuPage - 1);
  std::unique_ptr<GdrWindow> w(new GdrWindow());  // its destructor undoes whatever was done when a later step fails
  GdrMh mh{};
  if (g.pin(g.ctx, page, kGpuPage, 0, 0, &mh) != 0) {
    LOG_WARN(LogSubsys::CONN, "gdr_pin_buffer failed for the GPU page at ", reinterpret_cast<void*>(page));
    return nullptr;
  }
  w->pinHandle_ = mh.h;
  w->pinned_ = true;
  void* va = nullptr;
  if (g.map(g.ctx, mh, &va, kGpuPage) != 0 || va == nullptr) {
    LOG_WARN(LogSubsys::CONN, "gdr_map failed");
    return nullptr;
  }
  w->mapBase_ = va;
  w->mapBytes_ = kGpuPage;
  GdrInfo info{};
  uint64_t start = page;
  if (g.getInfo(g.ctx, mh, &info) == 0 && info.va != 0) start = info.va;  // the pinned range may begin below the page asked for
  w->word_ = reinterpret_cast<uint64_t*>(static_cast<char*>(va) + (addr - start));
  return w;
}

GdrWindow::~GdrWindow() {
  GdrApi& g = gdr();
  GdrMh mh{pinHandle_};
  if (mapBase_ != nullptr) (void)g.unmap(g.ctx, mh, mapBase_, mapBytes_);
  if (pinned_) (void)g.unpin(g.ctx, mh);
}

void GdrWindow::store(uint64_t value) const {
  // BAR1 is mapped write-combining: the fence pushes the store out instead of leaving it in a combining buffer
  reinterpret_cast<std::atomic<uint64_t>*>(word_)->store(value, std::memory_order_release);
  std::atomic_thread_fence(std::memory_order_seq_cst);
}

uint64_t GdrWindow::load() const { return reinterpret_cast<std::atomic<uint64_t>*>(word_)->load(std::memory_order_acquire); }

}  // namespace mscclpp
