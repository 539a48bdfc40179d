// Low-latency (LL) packets: data and a validity flag travel in one store, so the receiver needs
// no separate signal. Three formats:
//   LL16  : 16 B = {data0, flag, data1, flag}; one 16-byte volatile store, 8 B payload.
//   LL8   :  8 B = {data, flag};               one  8-byte volatile store, 4 B payload.
//   LL128 : 128 B line = 120 B payload + 8 B flag, written and read by 8 cooperating lanes with
//           16-byte accesses (lane 7 carries 8 B payload + the 8 B flag). This format does not
//           exist in the reference (it ships LL16/LL8 only: include/mscclpp/packet_device.hpp:19-158).
// The flag is the launch epoch, so scratch buffers are never cleared. All readers spin with a
// time budget and report through DeviceStatus instead of hanging.
#pragma once

#include <cstdint>

#include "device/ptx.cuh"
#include "poll_device.hpp"

namespace mscclpp {

union alignas(16) LL16Packet {
  struct {
    uint32_t data1;
    uint32_t flag1;
    uint32_t data2;
    uint32_t flag2;
  };
  uint4 raw;
  using Payload = uint2;

#if defined(__CUDACC__)
  MSCCLPP_DEVICE_INLINE LL16Packet() {}
  MSCCLPP_DEVICE_INLINE LL16Packet(uint2 v, uint32_t flag) : data1(v.x), flag1(flag), data2(v.y), flag2(flag) {}

  MSCCLPP_DEVICE_INLINE void write(uint32_t v1, uint32_t v2, uint32_t flag) {
    ptx::st_volatile_v4(this, make_uint4(v1, flag, v2, flag));
  }
  MSCCLPP_DEVICE_INLINE void write(uint2 v, uint32_t flag) { write(v.x, v.y, flag); }
  MSCCLPP_DEVICE_INLINE void write(uint64_t v, uint32_t flag) {
    write(static_cast<uint32_t>(v), static_cast<uint32_t>(v >> 32), flag);
  }
  // One probe. True when both flags carry `flag`; then `out` holds the payload.
  MSCCLPP_DEVICE_INLINE bool tryRead(uint32_t flag, uint2& out) const {
    uint4 r = ptx::ld_volatile_v4(this);
    out = make_uint2(r.x, r.z);
    return r.y == flag && r.w == flag;
  }
  // Name and sense of the reference (include/mscclpp/packet_device.hpp:66): true while the packet has NOT arrived.
  MSCCLPP_DEVICE_INLINE bool readOnce(uint32_t flag, uint2& data) const { return !tryRead(flag, data); }
  // Bounded blocking read. Returns false (payload undefined) when the budget ran out.
  MSCCLPP_DEVICE_INLINE bool read(uint32_t flag, uint2& out, DeviceStatus* st, uint64_t budgetNs, uint32_t rank = 0,
                                  uint32_t peer = 0) const {
    SpinGuard g(st, budgetNs);
    while (!tryRead(flag, out)) {
      if (!g.keepSpinning()) {
        g.report(kDevTimeoutPacket, rank, 16, peer, flag, flag1);
        return false;
      }
    }
    return true;
  }
  MSCCLPP_DEVICE_INLINE void clear() { ptx::st_volatile_v4(this, make_uint4(0, 0, 0, 0)); }
#endif
};

union alignas(8) LL8Packet {
  struct {
    uint32_t data;
    uint32_t flag;
  };
  uint64_t raw;
  using Payload = uint32_t;

#if defined(__CUDACC__)
  MSCCLPP_DEVICE_INLINE LL8Packet() {}
  MSCCLPP_DEVICE_INLINE LL8Packet(uint32_t v, uint32_t f) : data(v), flag(f) {}
  MSCCLPP_DEVICE_INLINE void write(uint32_t v, uint32_t f) { ptx::st_volatile_v2(this, make_uint2(v, f)); }
  MSCCLPP_DEVICE_INLINE bool tryRead(uint32_t f, uint32_t& out) const {
    uint2 r = ptx::ld_volatile_v2(this);
    out = r.x;
    return r.y == f;
  }
  MSCCLPP_DEVICE_INLINE bool readOnce(uint32_t f, uint32_t& data) const { return !tryRead(f, data); }
  MSCCLPP_DEVICE_INLINE bool read(uint32_t f, uint32_t& out, DeviceStatus* st, uint64_t budgetNs, uint32_t rank = 0,
                                  uint32_t peer = 0) const {
    SpinGuard g(st, budgetNs);
    while (!tryRead(f, out)) {
      if (!g.keepSpinning()) {
        g.report(kDevTimeoutPacket, rank, 8, peer, f, flag);
        return false;
      }
    }
    return true;
  }
  MSCCLPP_DEVICE_INLINE void clear() { ptx::st_volatile_v2(this, make_uint2(0, 0)); }
#endif
};

using LLPacket = LL16Packet;

// ---------------------------------------------------------------- LL128
// A line is 8 x 16 B. Lanes 0..6 of an 8-lane group carry 16 B of payload each, lane 7 carries
// 8 B of payload in .x/.y and the 64-bit flag in .z/.w. The writer issues the eight 16-byte
// stores from eight consecutive lanes of one warp so that they leave the SM as one 128-byte
// transaction; the reader accepts the line only when lane 7 sees the flag, then every lane
// re-reads its 16 B (the second read is ordered after the flag by the volatile semantics plus
// an explicit fence), so a line that was torn on the wire is never consumed half-old.
struct alignas(128) LL128Line {
  uint4 w[8];
};
constexpr int kLL128PayloadBytes = 120;

#if defined(__CUDACC__)

// Called by 8 consecutive lanes (sub = lane & 7). `payload` = this lane's 16 B (lane 7: only
// .x/.y are payload).
MSCCLPP_DEVICE_INLINE void ll128Write(LL128Line* line, uint32_t sub, uint4 payload, uint64_t flag) {
  if (sub == 7) {
    payload.z = static_cast<uint32_t>(flag);
    payload.w = static_cast<uint32_t>(flag >> 32);
  }
  ptx::st_volatile_v4(&line->w[sub], payload);
}

// Called by the same 8 lanes (mask = the 8-lane group's bits in the warp). Returns false on budget expiry.
MSCCLPP_DEVICE_INLINE bool ll128Read(const LL128Line* line, uint32_t sub, uint32_t groupMask, uint64_t flag,
                                     uint4& payload, DeviceStatus* st, uint64_t budgetNs, uint32_t rank = 0,
                                     uint32_t peer = 0) {
  SpinGuard g(st, budgetNs);
  bool alive = true;
  while (true) {
    uint4 v = ptx::ld_volatile_v4(&line->w[sub]);
    bool mine = true;
    if (sub == 7) mine = (v.z == static_cast<uint32_t>(flag)) && (v.w == static_cast<uint32_t>(flag >> 32));
    // every lane of the group learns whether lane 7 saw the flag
    uint32_t ok = __ballot_sync(groupMask, mine) & groupMask;
    if (ok == groupMask) {
      __threadfence_system();
      payload = ptx::ld_volatile_v4(&line->w[sub]);
      // the flag must still be there after the payload re-read (guards against a newer epoch racing in)
      bool still = true;
      if (sub == 7) still = (payload.z == static_cast<uint32_t>(flag)) && (payload.w == static_cast<uint32_t>(flag >> 32));
      if ((__ballot_sync(groupMask, still) & groupMask) == groupMask) return true;
    }
    if (alive && !g.keepSpinning()) {
      g.report(kDevTimeoutPacket, rank, 128, peer, flag, v.z);
      alive = false;
    }
    if ((__ballot_sync(groupMask, alive) & groupMask) != groupMask) return false;
  }
}

// The fast form, as NCCL's LL128 uses the format: ONE 16-byte load per lane, taken by the eight lanes in one warp
// instruction, and the line is accepted as loaded when lane 7's copy carries the flag. It rests on the property that makes
// the format worth having at all - the eight 16-byte stores of ll128Write leave as one 128-byte transaction and arrive as
// one, and the eight loads here are one transaction too, so flag and payload of a line are never from different writes.
// (That holds for GPUs connected by NVLink, where 128 bytes is the transfer unit end to end; ll128Read above makes no
// such assumption and pays a system-scope fence and a second read per line for it.) Returns false on budget expiry.
MSCCLPP_DEVICE_INLINE bool ll128ReadFast(const LL128Line* line, uint32_t sub, uint32_t groupMask, uint64_t flag, uint4& payload,
                                         DeviceStatus* st, uint64_t budgetNs, uint32_t rank = 0, uint32_t peer = 0) {
  uint4 v = ptx::ld_volatile_v4(&line->w[sub]);
  bool mine = sub != 7 || ((v.z == static_cast<uint32_t>(flag)) && (v.w == static_cast<uint32_t>(flag >> 32)));
  if ((__ballot_sync(groupMask, mine) & groupMask) == groupMask) {
    payload = v;
    return true;
  }
  SpinGuard g(st, budgetNs);
  bool alive = true;
  while (true) {
    v = ptx::ld_volatile_v4(&line->w[sub]);
    mine = sub != 7 || ((v.z == static_cast<uint32_t>(flag)) && (v.w == static_cast<uint32_t>(flag >> 32)));
    if ((__ballot_sync(groupMask, mine) & groupMask) == groupMask) {
      payload = v;
      return true;
    }
    if (alive && !g.keepSpinning()) {
      g.report(kDevTimeoutPacket, rank, 129, peer, flag, v.z);
      alive = false;
    }
    if ((__ballot_sync(groupMask, alive) & groupMask) != groupMask) return false;
  }
}

#endif  // __CUDACC__

}  // namespace mscclpp
