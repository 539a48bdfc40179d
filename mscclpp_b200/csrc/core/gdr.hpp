// GDRCopy: a window onto one page of GPU memory through the GPU's BAR1, so that a CPU thread can store an 8-byte
// semaphore token into device memory with ordinary, ordered stores. Only the InfiniBand transport in its mode without
// RDMA atomics uses it (the receive thread forwards tokens that arrive as immediate data). Same role as the reference's
// GDRCopy wrapper (src/core/include/gdr.hpp:14-60, src/core/gdr.cc:83-194). libgdrapi is loaded with dlopen
// (MSCCLPP_GDRCOPY_SO, default libgdrapi.so.2), never linked.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>

namespace mscclpp {

// Whether this process can open BAR1 windows, and if not, why (library missing, kernel module missing, switched off
// with MSCCLPP_FORCE_DISABLE_GDR, gdr_open() failed). The library is opened on the first call.
struct GdrAvailability {
  bool usable = false;
  std::string reason;  // "GDRCopy is available" when usable
};
const GdrAvailability& gdrAvailability();

// The 64 KB GPU page around one device address, pinned and mapped for the CPU.
class GdrWindow {
 public:
  // nullptr when GDRCopy is not usable or the page cannot be pinned or mapped: the caller takes another route.
  static std::unique_ptr<GdrWindow> open(void* deviceAddr, int deviceId);
  ~GdrWindow();
  GdrWindow(const GdrWindow&) = delete;
  GdrWindow& operator=(const GdrWindow&) = delete;

  // the CPU's address of *deviceAddr
  uint64_t* word() const { return word_; }
  // ordered 8-byte store / load through the window
  void store(uint64_t value) const;
  uint64_t load() const;

 private:
  GdrWindow() = default;
  uint64_t* word_ = nullptr;
  void* mapBase_ = nullptr;
  size_t mapBytes_ = 0;
  unsigned long pinHandle_ = 0;
  bool pinned_ = false;
};

}  // namespace mscclpp
