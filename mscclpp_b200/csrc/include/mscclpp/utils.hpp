// Small host utilities of the public API (reference: include/mscclpp/utils.hpp:10-58).
#pragma once

#include <functional>
#include <string>

#include "core.hpp"

namespace mscclpp {
namespace detail {
// Folds `value` into `seed` (the usual golden-ratio mix), for hashing aggregates.
template <typename T>
inline void hashCombine(std::size_t& seed, const T& value) {
  seed ^= std::hash<T>{}(value) + 0x9e3779b97f4a7c15ull + (seed << 6) + (seed >> 2);
}
}  // namespace detail

// Host name cut at `maxlen` characters and at the first `delim` (e.g. '.' to drop the domain). Throws SystemError.
std::string getHostName(int maxlen, const char delim);

// InfiniBand devices the kernel lists under /sys/class/infiniband (0 on machines without any; this build has no
// verbs transport, the functions exist so that portable set-up code keeps working).
int getIBDeviceCount();
// Name of the device behind Transport::IB<n> (honours MSCCLPP_HCA_DEVICES). Throws InvalidUsage when there is none.
std::string getIBDeviceName(Transport ibTransport);
// Inverse of getIBDeviceName.
Transport getIBTransportByDeviceName(const std::string& ibDeviceName);

// Whether this device can export memory as fabric handles (multi-node NVLink); false without a usable GPU.
bool isFabricMemHandleAvailable();

}  // namespace mscclpp
