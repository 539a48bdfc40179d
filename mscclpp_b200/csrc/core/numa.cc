#include <mscclpp/numa.hpp>

#include <cuda_runtime.h>
#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cerrno>
#include <fstream>
#include <sstream>

#include <mscclpp/errors.hpp>
#include <mscclpp/gpu_utils.hpp>

namespace mscclpp {

std::vector<int> parseCpuList(const std::string& text) {
  std::vector<int> cpus;
  std::stringstream ss(text);
  std::string item;
  while (std::getline(ss, item, ',')) {
    item.erase(std::remove_if(item.begin(), item.end(), [](unsigned char c) { return std::isspace(c); }), item.end());
    if (item.empty()) continue;
    const size_t dash = item.find('-');
    try {
      size_t used = 0;
      if (dash == std::string::npos) {
        const int v = std::stoi(item, &used);
        if (used != item.size() || v < 0) throw std::invalid_argument(item);
        cpus.push_back(v);
      } else {
        const std::string a = item.substr(0, dash), b = item.substr(dash + 1);
        size_t ua = 0, ub = 0;
        const int lo = std::stoi(a, &ua), hi = std::stoi(b, &ub);
        if (ua != a.size() || ub != b.size() || lo < 0 || hi < lo) throw std::invalid_argument(item);
        for (int v = lo; v <= hi; v++) cpus.push_back(v);
      }
    } catch (const std::exception&) {
      throw Error("malformed CPU list: '" + text + "'", ErrorCode::InvalidUsage);
    }
  }
  return cpus;
}

int getDeviceNumaNode(int deviceId) {
  char busId[32] = {0};
  MSCCLPP_CUDATHROW(cudaDeviceGetPCIBusId(busId, sizeof(busId), deviceId));
  std::string id(busId);
  std::transform(id.begin(), id.end(), id.begin(), [](unsigned char c) { return static_cast<char>(std::tolower(c)); });
  const std::string path = "/sys/bus/pci/devices/" + id + "/numa_node";
  std::ifstream f(path);
  int node = -1;
  if (!f || !(f >> node)) throw Error("cannot read " + path, ErrorCode::SystemError);
  return node;
}

std::vector<int> getNumaNodeCpus(int node) {
  const std::string path = "/sys/devices/system/node/node" + std::to_string(node) + "/cpulist";
  std::ifstream f(path);
  std::string line;
  if (node < 0 || !f || !std::getline(f, line)) throw Error("NUMA node " + std::to_string(node) + " does not exist", ErrorCode::InvalidUsage);
  return parseCpuList(line);
}

void numaBind(int node) {
  if (node < 0) return;
  const std::vector<int> cpus = getNumaNodeCpus(node);
  cpu_set_t allowed;
  CPU_ZERO(&allowed);
  if (sched_getaffinity(0, sizeof(allowed), &allowed) != 0) throw SysError("sched_getaffinity", errno);
  cpu_set_t wanted;
  CPU_ZERO(&wanted);
  int n = 0;
  for (int c : cpus) {
    if (c < CPU_SETSIZE && CPU_ISSET(c, &allowed)) {
      CPU_SET(c, &wanted);
      n++;
    }
  }
  if (n == 0) throw Error("no CPU of NUMA node " + std::to_string(node) + " is available to this thread", ErrorCode::SystemError);
  if (sched_setaffinity(0, sizeof(wanted), &wanted) != 0) throw SysError("sched_setaffinity", errno);
#ifdef SYS_set_mempolicy
  // MPOL_PREFERRED (1): allocate on this node when possible, fall back elsewhere instead of failing. Best effort.
  if (node < 1024) {
    unsigned long mask[1024 / (8 * sizeof(unsigned long))] = {0};
    mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
    (void)syscall(SYS_set_mempolicy, 1, mask, 1024 + 1);
  }
#endif
}

}  // namespace mscclpp
