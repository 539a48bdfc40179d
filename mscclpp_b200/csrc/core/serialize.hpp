// Tiny byte-stream helpers for the objects that travel over the bootstrap.
#pragma once

#include <cstring>
#include <string>
#include <vector>

#include <mscclpp/errors.hpp>

namespace mscclpp {

struct Writer {
  std::vector<char> bytes;
  template <typename T>
  void put(const T& v) {
    const char* p = reinterpret_cast<const char*>(&v);
    bytes.insert(bytes.end(), p, p + sizeof(T));
  }
  void putRaw(const void* p, size_t n) {
    const char* c = static_cast<const char*>(p);
    bytes.insert(bytes.end(), c, c + n);
  }
  void putBlob(const std::vector<char>& b) {
    put<uint64_t>(b.size());
    bytes.insert(bytes.end(), b.begin(), b.end());
  }
};

struct Reader {
  const std::vector<char>& bytes;
  size_t pos = 0;
  explicit Reader(const std::vector<char>& b) : bytes(b) {}
  void need(size_t n) const {
    if (pos + n > bytes.size()) throw Error("truncated serialized object", ErrorCode::InvalidUsage);
  }
  template <typename T>
  T get() {
    need(sizeof(T));
    T v;
    std::memcpy(&v, bytes.data() + pos, sizeof(T));
    pos += sizeof(T);
    return v;
  }
  void getRaw(void* p, size_t n) {
    need(n);
    std::memcpy(p, bytes.data() + pos, n);
    pos += n;
  }
  std::vector<char> getBlob() {
    uint64_t n = get<uint64_t>();
    need(n);
    std::vector<char> out(bytes.begin() + pos, bytes.begin() + pos + n);
    pos += n;
    return out;
  }
  bool done() const { return pos == bytes.size(); }
};

}  // namespace mscclpp
