// Device handle of PortChannel: the GPU asks a host proxy thread to move data (copy engine, TCP or,
// in builds that have it, RDMA) by pushing 16-byte requests into a FIFO
// (reference: include/mscclpp/port_channel_device.hpp:27-195).
#pragma once

#include "fifo_device.hpp"
#include "semaphore_device.hpp"

namespace mscclpp {

using SemaphoreId = uint32_t;
using MemoryId = uint32_t;

using TriggerType = uint64_t;
constexpr TriggerType TriggerData = 0x1;  // copy [srcMem + srcOffset, +size) to dstMem + dstOffset
constexpr TriggerType TriggerFlag = 0x2;  // signal the peer's semaphore
constexpr TriggerType TriggerSync = 0x4;  // flush: everything before this request is complete when it is consumed

// Request layout inside ProxyTrigger:
//   fst = size[0,32) | srcOffset[32,64)
//   snd = dstOffset[0,32) | srcMemoryId[32,41) | dstMemoryId[41,50) | type[50,53) | semaphoreId[53,63) | parity[63]
constexpr int kTriggerSizeBits = 32;
constexpr int kTriggerOffsetBits = 32;
constexpr int kTriggerMemIdBits = 9;
constexpr int kTriggerTypeBits = 3;
constexpr int kTriggerSemIdBits = 10;

MSCCLPP_HOST_DEVICE_INLINE ProxyTrigger makeTrigger(TriggerType type, MemoryId dst, uint64_t dstOffset, MemoryId src,
                                                   uint64_t srcOffset, uint64_t size, SemaphoreId semaphoreId) {
  ProxyTrigger t;
  t.fst = (size & 0xffffffffull) | ((srcOffset & 0xffffffffull) << 32);
  t.snd = (dstOffset & 0xffffffffull) | (static_cast<uint64_t>(src & 0x1ff) << 32) | (static_cast<uint64_t>(dst & 0x1ff) << 41) |
          ((type & 0x7) << 50) | (static_cast<uint64_t>(semaphoreId & 0x3ff) << 53);
  return t;
}

struct TriggerFields {
  uint64_t size, srcOffset, dstOffset;
  MemoryId srcMemoryId, dstMemoryId;
  TriggerType type;
  SemaphoreId semaphoreId;
};
MSCCLPP_HOST_DEVICE_INLINE TriggerFields decodeTrigger(const ProxyTrigger& t) {
  TriggerFields f;
  f.size = t.fst & 0xffffffffull;
  f.srcOffset = t.fst >> 32;
  f.dstOffset = t.snd & 0xffffffffull;
  f.srcMemoryId = static_cast<MemoryId>((t.snd >> 32) & 0x1ff);
  f.dstMemoryId = static_cast<MemoryId>((t.snd >> 41) & 0x1ff);
  f.type = (t.snd >> 50) & 0x7;
  f.semaphoreId = static_cast<SemaphoreId>((t.snd >> 53) & 0x3ff);
  return f;
}

struct BasePortChannelDeviceHandle {
  SemaphoreId semaphoreId_;
  Host2DeviceSemaphoreDeviceHandle semaphore_;
  FifoDeviceHandle fifo_;

#if defined(__CUDACC__)
  MSCCLPP_DEVICE_INLINE void put(MemoryId dst, uint64_t dstOffset, MemoryId src, uint64_t srcOffset, uint64_t size) {
    fifo_.push(makeTrigger(TriggerData, dst, dstOffset, src, srcOffset, size, semaphoreId_));
  }
  MSCCLPP_DEVICE_INLINE void signal() { fifo_.push(makeTrigger(TriggerFlag, 0, 0, 0, 0, 1, semaphoreId_)); }
  MSCCLPP_DEVICE_INLINE void putWithSignal(MemoryId dst, uint64_t dstOffset, MemoryId src, uint64_t srcOffset,
                                           uint64_t size) {
    fifo_.push(makeTrigger(TriggerData | TriggerFlag, dst, dstOffset, src, srcOffset, size, semaphoreId_));
  }
  // Returns false when the proxy did not confirm within the budget.
  MSCCLPP_DEVICE_INLINE bool putWithSignalAndFlush(MemoryId dst, uint64_t dstOffset, MemoryId src, uint64_t srcOffset,
                                                   uint64_t size, DeviceStatus* st = nullptr,
                                                   uint64_t timeoutNs = 10000000000ull) {
    uint64_t ticket = fifo_.push(makeTrigger(TriggerData | TriggerFlag | TriggerSync, dst, dstOffset, src, srcOffset, size,
                                             semaphoreId_), st, timeoutNs);
    return ticket != UINT64_MAX && fifo_.sync(ticket, st, timeoutNs);
  }
  MSCCLPP_DEVICE_INLINE bool flush(DeviceStatus* st = nullptr, uint64_t timeoutNs = 10000000000ull) {
    uint64_t ticket = fifo_.push(makeTrigger(TriggerSync, 0, 0, 0, 0, 1, semaphoreId_), st, timeoutNs);
    return ticket != UINT64_MAX && fifo_.sync(ticket, st, timeoutNs);
  }
  MSCCLPP_DEVICE_INLINE bool poll() { return semaphore_.poll(); }
  MSCCLPP_DEVICE_INLINE bool wait(uint64_t timeoutNs = 10000000000ull, DeviceStatus* st = nullptr) {
    return semaphore_.wait(timeoutNs, st);
  }
#endif
};

struct PortChannelDeviceHandle : public BasePortChannelDeviceHandle {
  MemoryId dst_;
  MemoryId src_;

#if defined(__CUDACC__)
  MSCCLPP_DEVICE_INLINE void put(uint64_t dstOffset, uint64_t srcOffset, uint64_t size) {
    BasePortChannelDeviceHandle::put(dst_, dstOffset, src_, srcOffset, size);
  }
  MSCCLPP_DEVICE_INLINE void put(uint64_t offset, uint64_t size) { put(offset, offset, size); }
  MSCCLPP_DEVICE_INLINE void putWithSignal(uint64_t dstOffset, uint64_t srcOffset, uint64_t size) {
    BasePortChannelDeviceHandle::putWithSignal(dst_, dstOffset, src_, srcOffset, size);
  }
  MSCCLPP_DEVICE_INLINE void putWithSignal(uint64_t offset, uint64_t size) { putWithSignal(offset, offset, size); }
  MSCCLPP_DEVICE_INLINE bool putWithSignalAndFlush(uint64_t dstOffset, uint64_t srcOffset, uint64_t size,
                                                   DeviceStatus* st = nullptr, uint64_t timeoutNs = 10000000000ull) {
    return BasePortChannelDeviceHandle::putWithSignalAndFlush(dst_, dstOffset, src_, srcOffset, size, st, timeoutNs);
  }
#endif
};

}  // namespace mscclpp
