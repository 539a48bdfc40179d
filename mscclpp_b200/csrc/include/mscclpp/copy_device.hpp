// Cooperative memory copies executed by many threads, used by MemoryChannel::put/get and by the plan
// interpreter: 16-byte vector body with byte-granular head and tail, plus pack/unpack loops between
// plain data and LL packets (role of the reference's include/mscclpp/copy_device.hpp:68-232).
#pragma once

#include <cstdint>

#include "device/ptx.cuh"
#include "packet_device.hpp"

namespace mscclpp {

#if defined(__CUDACC__)

// Copy `bytes` from src to dst with threads `threadId` of `numThreads`. Any alignment; when src and
// dst are congruent modulo 16 the body moves 16 bytes per access, otherwise 4 or 1.
MSCCLPP_DEVICE_INLINE void copyBytes(void* dst, const void* src, uint64_t bytes, uint32_t threadId, uint32_t numThreads) {
  char* d = reinterpret_cast<char*>(dst);
  const char* s = reinterpret_cast<const char*>(src);
  const uintptr_t da = reinterpret_cast<uintptr_t>(d), sa = reinterpret_cast<uintptr_t>(s);
  if (((da ^ sa) & 15) == 0) {
    // head up to the first 16-byte boundary, vector body, tail
    uint64_t head = (16 - (da & 15)) & 15;
    if (head > bytes) head = bytes;
    for (uint64_t i = threadId; i < head; i += numThreads) d[i] = s[i];
    const uint64_t body = (bytes - head) / 16;
    const uint4* sv = reinterpret_cast<const uint4*>(s + head);
    uint4* dv = reinterpret_cast<uint4*>(d + head);
    for (uint64_t i = threadId; i < body; i += numThreads) ptx::st_na_v4(dv + i, ptx::ld_nc_na_v4(sv + i));
    const uint64_t done = head + body * 16;
    for (uint64_t i = done + threadId; i < bytes; i += numThreads) d[i] = s[i];
  } else if (((da | sa | bytes) & 3) == 0) {
    const uint32_t* sv = reinterpret_cast<const uint32_t*>(s);
    uint32_t* dv = reinterpret_cast<uint32_t*>(d);
    for (uint64_t i = threadId; i < bytes / 4; i += numThreads) dv[i] = sv[i];
  } else {
    for (uint64_t i = threadId; i < bytes; i += numThreads) d[i] = s[i];
  }
}

// The two `copy` overloads of the reference (include/mscclpp/copy_device.hpp:34-127). The byte form ignores its
// template parameters: copyBytes already picks the widest access the two addresses allow and always copies the tail.
template <typename T>
MSCCLPP_DEVICE_INLINE void copy(T* dst, T* src, uint64_t numElems, uint32_t threadId, uint32_t numThreads) {
  for (uint64_t i = threadId; i < numElems; i += numThreads) dst[i] = src[i];
}
template <int Alignment = 16, bool CopyRemainder = true>
MSCCLPP_DEVICE_INLINE void copy(void* dst, void* src, uint64_t bytes, uint32_t threadId, uint32_t numThreads) {
  copyBytes(dst, src, bytes, threadId, numThreads);
}

// Plain data -> packets. originBytes must be a multiple of the packet payload (8 for LL16, 4 for LL8).
template <typename PacketType>
MSCCLPP_DEVICE_INLINE void copyToPackets(void* packets, const void* origin, uint64_t originBytes, uint32_t threadId,
                                         uint32_t numThreads, uint32_t flag) {
  using Payload = typename PacketType::Payload;
  const Payload* src = reinterpret_cast<const Payload*>(origin);
  PacketType* dst = reinterpret_cast<PacketType*>(packets);
  const uint64_t n = originBytes / sizeof(Payload);
  for (uint64_t i = threadId; i < n; i += numThreads) dst[i].write(src[i], flag);
}

// Packets -> plain data; spins (bounded) on each packet's flag. Returns false if a packet never arrived.
template <typename PacketType>
MSCCLPP_DEVICE_INLINE bool copyFromPackets(void* origin, const void* packets, uint64_t originBytes, uint32_t threadId,
                                           uint32_t numThreads, uint32_t flag, DeviceStatus* status = nullptr,
                                           uint64_t timeoutNs = 10000000000ull) {
  using Payload = typename PacketType::Payload;
  Payload* dst = reinterpret_cast<Payload*>(origin);
  const PacketType* src = reinterpret_cast<const PacketType*>(packets);
  const uint64_t n = originBytes / sizeof(Payload);
  for (uint64_t i = threadId; i < n; i += numThreads) {
    Payload v;
    if (!src[i].read(flag, v, status, timeoutNs)) return false;
    dst[i] = v;
  }
  return true;
}

#endif  // __CUDACC__

}  // namespace mscclpp
