// NUMA placement helpers: which node a GPU hangs off, and binding the calling thread (CPUs and preferred memory) to a
// node. Implemented on sysfs and plain system calls, so libnuma is not needed (reference: include/mscclpp/numa.hpp:13-18,
// src/core/numa.cc, which wrap libnuma).
#pragma once

#include <string>
#include <vector>

namespace mscclpp {

// NUMA node of CUDA device `deviceId` as the kernel reports it for the device's PCI function; -1 when the platform
// does not say (single-node machines, some virtual machines). Throws when the device or its sysfs entry cannot be read.
int getDeviceNumaNode(int deviceId);

// CPUs of a node, from /sys/devices/system/node/node<N>/cpulist. Throws InvalidUsage for a node that does not exist.
std::vector<int> getNumaNodeCpus(int node);

// Restricts the calling thread to the CPUs of `node` and asks the kernel to prefer that node's memory for it.
// node < 0 is a no-op. CPUs outside the process's cpuset are dropped; throws SystemError when none is left.
void numaBind(int node);

// "0-3,8,10-11" -> {0,1,2,3,8,10,11}; throws InvalidUsage on malformed text.
std::vector<int> parseCpuList(const std::string& text);

}  // namespace mscclpp
