#include <mscclpp/utils.hpp>

#include <dirent.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <sstream>
#include <vector>

#include <mscclpp/env.hpp>
#include <mscclpp/errors.hpp>

#include <cuda_runtime.h>

#include "ib.hpp"

namespace mscclpp {

std::string getHostName(int maxlen, const char delim) {
  char buf[1024] = {0};
  if (::gethostname(buf, sizeof(buf) - 1) != 0) throw SysError("gethostname", errno);
  std::string name(buf);
  const size_t cut = name.find(delim);
  if (cut != std::string::npos) name.resize(cut);
  if (maxlen >= 0 && static_cast<size_t>(maxlen) < name.size()) name.resize(maxlen);
  return name;
}

namespace {
// MSCCLPP_HCA_DEVICES ("mlx5_0,mlx5_2") when set, else what the kernel lists, sorted by name.
std::vector<std::string> ibDeviceNames() {
  std::vector<std::string> names;
  const std::string forced = env()->hcaDevices;
  if (!forced.empty()) {
    std::stringstream ss(forced);
    std::string item;
    while (std::getline(ss, item, ',')) {
      if (!item.empty()) names.push_back(item);
    }
    return names;
  }
  // what the loaded verbs library lists (a software provider has no sysfs entries), else what the kernel lists
  names = ibDeviceNamesFromLibrary();
  if (!names.empty()) return names;
  if (DIR* d = ::opendir("/sys/class/infiniband")) {
    while (dirent* e = ::readdir(d)) {
      const std::string n = e->d_name;
      if (n != "." && n != "..") names.push_back(n);
    }
    ::closedir(d);
  }
  std::sort(names.begin(), names.end());
  return names;
}

int ibIndex(Transport t) {
  const int i = static_cast<int>(t) - static_cast<int>(Transport::IB0);
  if (i < 0 || i > static_cast<int>(Transport::IB7) - static_cast<int>(Transport::IB0)) {
    throw Error("not an InfiniBand transport", ErrorCode::InvalidUsage);
  }
  return i;
}
}  // namespace

int getIBDeviceCount() { return static_cast<int>(ibDeviceNames().size()); }

std::string getIBDeviceName(Transport ibTransport) {
  const int i = ibIndex(ibTransport);
  const std::vector<std::string> names = ibDeviceNames();
  if (i >= static_cast<int>(names.size())) {
    throw Error("IB" + std::to_string(i) + " requested, " + std::to_string(names.size()) + " InfiniBand device(s) present", ErrorCode::InvalidUsage);
  }
  return names[i];
}

Transport getIBTransportByDeviceName(const std::string& ibDeviceName) {
  const std::vector<std::string> names = ibDeviceNames();
  for (size_t i = 0; i < names.size() && i < 8; i++) {
    if (names[i] == ibDeviceName) return static_cast<Transport>(static_cast<int>(Transport::IB0) + static_cast<int>(i));
  }
  throw Error("no InfiniBand device named '" + ibDeviceName + "'", ErrorCode::InvalidUsage);
}

bool isFabricMemHandleAvailable() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  int supported = 0;
#if CUDA_VERSION >= 12030
  if (cudaDeviceGetAttribute(&supported, cudaDevAttrHandleTypeFabricSupported, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
#endif
  return supported != 0;
}

}  // namespace mscclpp
