// GDRCopy: a window onto one page of GPU memory through the GPU's BAR1, so that a CPU thread can store an 8-byte
// semaphore token into device memory with ordinary, ordered stores. Only the InfiniBand transport in its mode without
// RDMA atomics uses it (the receive thread forwards tokens that arrive as immediate data). Same role as the reference's
// GdrContext / GdrMap (src/core/include/gdr.hpp:14-60, src/core/gdr.cc:83-194). libgdrapi is loaded with dlopen
// (MSCCLPP_GDRCOPY_SO, default libgdrapi.so.2), never linked.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>

namespace mscclpp {

enum class GdrStatus {
  Ok,             // library loaded and gdr_open() succeeded
  Disabled,       // MSCCLPP_FORCE_DISABLE_GDR
  LibraryMissing, // libgdrapi could not be loaded
  DriverMissing,  // library present, /dev/gdrdrv absent
  OpenFailed,     // gdr_open() failed
};

// State of the process-wide GDRCopy context (opened on first use).
GdrStatus gdrStatus();
inline bool gdrEnabled() { return gdrStatus() == GdrStatus::Ok; }
std::string gdrStatusMessage();

// One pinned and mapped GPU page that contains `deviceAddr`. valid() is false when GDRCopy is not available or the
// page could not be pinned; then hostPtr() is null and the caller takes another route.
class GdrMap {
 public:
  GdrMap(void* deviceAddr, int deviceId);
  ~GdrMap();
  GdrMap(const GdrMap&) = delete;
  GdrMap& operator=(const GdrMap&) = delete;
  bool valid() const { return hostPtr_ != nullptr; }
  // the CPU's address of *deviceAddr
  uint64_t* hostPtr() const { return hostPtr_; }
  // ordered 8-byte store / load through the window
  void store(uint64_t value) const;
  uint64_t load() const;

 private:
  uint64_t* hostPtr_ = nullptr;
  void* mapBase_ = nullptr;
  size_t mapBytes_ = 0;
  unsigned long handle_ = 0;
  bool pinned_ = false;
};

}  // namespace mscclpp
