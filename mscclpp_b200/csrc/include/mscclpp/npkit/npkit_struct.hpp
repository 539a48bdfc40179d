// Trace event record and per-buffer write cursor. The 16-byte record (type:8, size:32, rsvd:24, timestamp:64)
// is the on-disk format too, so dumps stay readable by tools written for the reference's NPKit
// (include/mscclpp/npkit/npkit_struct.hpp:11-27).
#pragma once

#include <cstdint>

#pragma pack(push, 1)
union NpKitEvent {
  uint64_t bits[2];
  struct {
    uint64_t type : 8;
    uint64_t size : 32;
    uint64_t rsvd : 24;
    uint64_t timestamp;
  } fields;
};

struct NpKitEventCollectContext {
  NpKitEvent* event_buffer;
  uint64_t event_buffer_head;
};
#pragma pack(pop)

static_assert(sizeof(NpKitEvent) == 16, "event record is 16 bytes");
