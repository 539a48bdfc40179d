// Minimal JSON reader for execution plans (objects, arrays, strings, integers up to 2^64-1, doubles,
// booleans, null). Values are immutable after parsing; lookups of missing keys throw ExecutorError so
// that malformed plans fail with a message instead of undefined behaviour.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include <mscclpp/errors.hpp>

namespace mscclpp {
namespace json {

class Value {
 public:
  enum class Kind { Null, Bool, Int, UInt, Double, String, Array, Object };
  Kind kind = Kind::Null;
  bool b = false;
  int64_t i = 0;
  uint64_t u = 0;
  double d = 0;
  std::string s;
  std::vector<Value> arr;
  std::vector<std::pair<std::string, Value>> obj;  // insertion order kept

  bool isNull() const { return kind == Kind::Null; }
  bool isObject() const { return kind == Kind::Object; }
  bool isArray() const { return kind == Kind::Array; }
  bool contains(const std::string& key) const {
    if (kind != Kind::Object) return false;
    for (auto& kv : obj)
      if (kv.first == key) return true;
    return false;
  }
  const Value& at(const std::string& key) const {
    if (kind != Kind::Object) throw Error("JSON: '" + key + "' looked up in a non-object", ErrorCode::ExecutorError);
    for (auto& kv : obj)
      if (kv.first == key) return kv.second;
    throw Error("JSON: missing key '" + key + "'", ErrorCode::ExecutorError);
  }
  const Value& at(size_t idx) const {
    if (kind != Kind::Array || idx >= arr.size()) throw Error("JSON: array index out of range", ErrorCode::ExecutorError);
    return arr[idx];
  }
  size_t size() const { return kind == Kind::Array ? arr.size() : (kind == Kind::Object ? obj.size() : 0); }
  int64_t asInt() const {
    if (kind == Kind::Int) return i;
    if (kind == Kind::UInt) return static_cast<int64_t>(u);
    if (kind == Kind::Double) return static_cast<int64_t>(d);
    throw Error("JSON: number expected", ErrorCode::ExecutorError);
  }
  uint64_t asUInt() const {
    if (kind == Kind::UInt) return u;
    if (kind == Kind::Int && i >= 0) return static_cast<uint64_t>(i);
    if (kind == Kind::Double && d >= 0) return static_cast<uint64_t>(d);
    throw Error("JSON: non-negative number expected", ErrorCode::ExecutorError);
  }
  bool asBool() const {
    if (kind != Kind::Bool) throw Error("JSON: boolean expected", ErrorCode::ExecutorError);
    return b;
  }
  const std::string& asString() const {
    if (kind != Kind::String) throw Error("JSON: string expected", ErrorCode::ExecutorError);
    return s;
  }
  int64_t intOr(const std::string& key, int64_t dflt) const { return contains(key) ? at(key).asInt() : dflt; }
  uint64_t uintOr(const std::string& key, uint64_t dflt) const { return contains(key) ? at(key).asUInt() : dflt; }
  bool boolOr(const std::string& key, bool dflt) const { return contains(key) ? at(key).asBool() : dflt; }
};

Value parse(const std::string& text);
Value parseFile(const std::string& path);

}  // namespace json
}  // namespace mscclpp
