// First-fit allocator over an abstract range [0, capacity) with a granule: used for the offsets of a multicast object,
// where bound ranges must be returned when their channel goes away (a pointer that only ever advances runs out after a
// few bind/unbind rounds of user buffers). Host-only, no CUDA. Role of the reference's range bookkeeping in
// src/core/switch_channel.cc:115-172.
#pragma once

#include <cstddef>
#include <map>
#include <stdexcept>

namespace mscclpp {

class RangeAllocator {
 public:
  RangeAllocator() = default;
  RangeAllocator(size_t capacity, size_t granule) { reset(capacity, granule); }

  void reset(size_t capacity, size_t granule) {
    if (granule == 0) throw std::invalid_argument("RangeAllocator: granule must be positive");
    granule_ = granule;
    capacity_ = capacity / granule * granule;
    free_.clear();
    used_.clear();
    if (capacity_ != 0) free_[0] = capacity_;
  }

  // Offset of a free range of `size` bytes (rounded up to the granule), lowest address first; npos when none fits.
  static constexpr size_t npos = static_cast<size_t>(-1);
  size_t allocate(size_t size) {
    if (size == 0) return npos;
    const size_t need = (size + granule_ - 1) / granule_ * granule_;
    for (auto it = free_.begin(); it != free_.end(); ++it) {
      if (it->second < need) continue;
      const size_t off = it->first, left = it->second - need;
      free_.erase(it);
      if (left != 0) free_[off + need] = left;
      used_[off] = need;
      return off;
    }
    return npos;
  }

  // Returns the range that starts at `offset`; neighbours that are free too are merged with it.
  void release(size_t offset) {
    auto it = used_.find(offset);
    if (it == used_.end()) throw std::invalid_argument("RangeAllocator: release of an offset that is not allocated");
    size_t begin = offset, size = it->second;
    used_.erase(it);
    auto next = free_.lower_bound(begin);
    if (next != free_.end() && next->first == begin + size) {
      size += next->second;
      next = free_.erase(next);
    }
    if (next != free_.begin()) {
      auto prev = std::prev(next);
      if (prev->first + prev->second == begin) {
        begin = prev->first;
        size += prev->second;
        free_.erase(prev);
      }
    }
    free_[begin] = size;
  }

  size_t capacity() const { return capacity_; }
  size_t bytesFree() const {
    size_t n = 0;
    for (auto& kv : free_) n += kv.second;
    return n;
  }
  size_t largestFree() const {
    size_t n = 0;
    for (auto& kv : free_) n = kv.second > n ? kv.second : n;
    return n;
  }
  size_t rangesInUse() const { return used_.size(); }

 private:
  size_t capacity_ = 0, granule_ = 1;
  std::map<size_t, size_t> free_;  // offset -> size
  std::map<size_t, size_t> used_;
};

}  // namespace mscclpp
