// Device handle of MemoryChannel: GPU threads copy to/from peer-mapped memory themselves and
// synchronise through a device-to-device semaphore (reference:
// include/mscclpp/memory_channel_device.hpp:15-224).
#pragma once

#include "copy_device.hpp"
#include "packet_device.hpp"
#include "semaphore_device.hpp"

namespace mscclpp {

struct BaseMemoryChannelDeviceHandle {
  MemoryDevice2DeviceSemaphoreDeviceHandle semaphore_;

#if defined(__CUDACC__)
  MSCCLPP_DEVICE_INLINE void signal() { semaphore_.signal(); }
  MSCCLPP_DEVICE_INLINE void relaxedSignal() { semaphore_.relaxedSignal(); }
  MSCCLPP_DEVICE_INLINE bool poll() { return semaphore_.poll(); }
  MSCCLPP_DEVICE_INLINE bool wait(uint64_t timeoutNs = 10000000000ull, DeviceStatus* st = nullptr) {
    return semaphore_.wait(timeoutNs, st);
  }
  MSCCLPP_DEVICE_INLINE bool relaxedWait(uint64_t timeoutNs = 10000000000ull, DeviceStatus* st = nullptr) {
    return semaphore_.relaxedWait(timeoutNs, st);
  }
#endif
};

struct MemoryChannelDeviceHandle : public BaseMemoryChannelDeviceHandle {
  void* dst_;           // peer's buffer, mapped here
  void* src_;           // local buffer
  void* packetBuffer_;  // local scratch that the peer fills with packets

#if defined(__CUDACC__)
  template <typename T>
  MSCCLPP_DEVICE_INLINE T read(uint64_t index) {
    return reinterpret_cast<T*>(dst_)[index];
  }
  template <typename T>
  MSCCLPP_DEVICE_INLINE void write(uint64_t index, const T& v) {
    reinterpret_cast<T*>(dst_)[index] = v;
  }
  // Collective over the calling threads: local src_ + srcOffset -> peer dst_ + dstOffset.
  MSCCLPP_DEVICE_INLINE void put(uint64_t dstOffset, uint64_t srcOffset, uint64_t bytes, uint32_t threadId,
                                 uint32_t numThreads) {
    copyBytes(static_cast<char*>(dst_) + dstOffset, static_cast<const char*>(src_) + srcOffset, bytes, threadId, numThreads);
  }
  MSCCLPP_DEVICE_INLINE void put(uint64_t offset, uint64_t bytes, uint32_t threadId, uint32_t numThreads) {
    put(offset, offset, bytes, threadId, numThreads);
  }
  // peer dst_ + dstOffset -> local src_ + srcOffset (argument names follow the reference: the first
  // offset addresses the peer buffer, the second the local one).
  MSCCLPP_DEVICE_INLINE void get(uint64_t dstOffset, uint64_t srcOffset, uint64_t bytes, uint32_t threadId,
                                 uint32_t numThreads) {
    copyBytes(static_cast<char*>(src_) + srcOffset, static_cast<const char*>(dst_) + dstOffset, bytes, threadId, numThreads);
  }
  MSCCLPP_DEVICE_INLINE void get(uint64_t offset, uint64_t bytes, uint32_t threadId, uint32_t numThreads) {
    get(offset, offset, bytes, threadId, numThreads);
  }
  // local src_ + srcOffset -> packets in the peer's dst_ + dstOffset (packet space).
  template <typename PacketType = LL16Packet>
  MSCCLPP_DEVICE_INLINE void putPackets(uint64_t dstOffset, uint64_t srcOffset, uint64_t bytes, uint32_t threadId,
                                        uint32_t numThreads, uint32_t flag) {
    copyToPackets<PacketType>(static_cast<char*>(dst_) + dstOffset, static_cast<const char*>(src_) + srcOffset, bytes, threadId,
                              numThreads, flag);
  }
  // packets in local packetBuffer_ + pktOffset -> local src_ + dstOffset. false = a packet never came.
  template <typename PacketType = LL16Packet>
  MSCCLPP_DEVICE_INLINE bool unpackPackets(uint64_t pktOffset, uint64_t dstOffset, uint64_t bytes, uint32_t threadId,
                                           uint32_t numThreads, uint32_t flag, DeviceStatus* st = nullptr,
                                           uint64_t timeoutNs = 10000000000ull) {
    return copyFromPackets<PacketType>(static_cast<char*>(src_) + dstOffset, static_cast<const char*>(packetBuffer_) + pktOffset,
                                       bytes, threadId, numThreads, flag, st, timeoutNs);
  }
  template <typename PacketType = LL16Packet>
  MSCCLPP_DEVICE_INLINE bool unpackPacket(uint64_t index, uint32_t flag, typename PacketType::Payload& out,
                                          DeviceStatus* st = nullptr, uint64_t timeoutNs = 10000000000ull) {
    return reinterpret_cast<const PacketType*>(packetBuffer_)[index].read(flag, out, st, timeoutNs);
  }
#endif
};

}  // namespace mscclpp
