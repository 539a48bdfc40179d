#include "json.hpp"

#include <cstdlib>
#include <fstream>
#include <sstream>

namespace mscclpp {
namespace json {

namespace {

struct Parser {
  const std::string& t;
  size_t p = 0;
  explicit Parser(const std::string& text) : t(text) {}

  [[noreturn]] void fail(const std::string& what) {
    throw Error("JSON parse error at byte " + std::to_string(p) + ": " + what, ErrorCode::ExecutorError);
  }
  void ws() {
    while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\t' || t[p] == '\r')) p++;
  }
  bool eat(char c) {
    ws();
    if (p < t.size() && t[p] == c) {
      p++;
      return true;
    }
    return false;
  }
  void expect(char c) {
    if (!eat(c)) fail(std::string("expected '") + c + "'");
  }
  Value value() {
    ws();
    if (p >= t.size()) fail("unexpected end");
    char c = t[p];
    if (c == '{') return object();
    if (c == '[') return array();
    if (c == '"') {
      Value v;
      v.kind = Value::Kind::String;
      v.s = string();
      return v;
    }
    if (c == 't' || c == 'f') {
      Value v;
      v.kind = Value::Kind::Bool;
      if (t.compare(p, 4, "true") == 0) {
        v.b = true;
        p += 4;
      } else if (t.compare(p, 5, "false") == 0) {
        v.b = false;
        p += 5;
      } else {
        fail("bad literal");
      }
      return v;
    }
    if (c == 'n') {
      if (t.compare(p, 4, "null") != 0) fail("bad literal");
      p += 4;
      return Value();
    }
    return number();
  }
  std::string string() {
    expect('"');
    std::string out;
    while (p < t.size() && t[p] != '"') {
      char c = t[p++];
      if (c == '\\') {
        if (p >= t.size()) fail("bad escape");
        char e = t[p++];
        switch (e) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {
            if (p + 4 > t.size()) fail("bad \\u escape");
            unsigned code = static_cast<unsigned>(std::strtoul(t.substr(p, 4).c_str(), nullptr, 16));
            p += 4;
            if (code < 0x80) out += static_cast<char>(code);
            else if (code < 0x800) {
              out += static_cast<char>(0xc0 | (code >> 6));
              out += static_cast<char>(0x80 | (code & 0x3f));
            } else {
              out += static_cast<char>(0xe0 | (code >> 12));
              out += static_cast<char>(0x80 | ((code >> 6) & 0x3f));
              out += static_cast<char>(0x80 | (code & 0x3f));
            }
            break;
          }
          default: out += e;
        }
      } else {
        out += c;
      }
    }
    if (p >= t.size()) fail("unterminated string");
    p++;
    return out;
  }
  Value number() {
    size_t start = p;
    bool isFloat = false;
    if (p < t.size() && (t[p] == '-' || t[p] == '+')) p++;
    while (p < t.size() && (std::isdigit(static_cast<unsigned char>(t[p])) || t[p] == '.' || t[p] == 'e' || t[p] == 'E' ||
                            t[p] == '-' || t[p] == '+')) {
      if (t[p] == '.' || t[p] == 'e' || t[p] == 'E') isFloat = true;
      p++;
    }
    if (p == start) fail("unexpected character");
    std::string tok = t.substr(start, p - start);
    Value v;
    if (isFloat) {
      v.kind = Value::Kind::Double;
      v.d = std::strtod(tok.c_str(), nullptr);
    } else if (tok[0] == '-') {
      v.kind = Value::Kind::Int;
      v.i = std::strtoll(tok.c_str(), nullptr, 10);
    } else {
      v.kind = Value::Kind::UInt;
      v.u = std::strtoull(tok.c_str(), nullptr, 10);
      if (v.u <= static_cast<uint64_t>(INT64_MAX)) {
        v.kind = Value::Kind::Int;
        v.i = static_cast<int64_t>(v.u);
      }
    }
    return v;
  }
  Value array() {
    expect('[');
    Value v;
    v.kind = Value::Kind::Array;
    if (eat(']')) return v;
    do {
      v.arr.push_back(value());
    } while (eat(','));
    expect(']');
    return v;
  }
  Value object() {
    expect('{');
    Value v;
    v.kind = Value::Kind::Object;
    if (eat('}')) return v;
    do {
      ws();
      std::string key = string();
      expect(':');
      v.obj.emplace_back(std::move(key), value());
    } while (eat(','));
    expect('}');
    return v;
  }
};

}  // namespace

Value parse(const std::string& text) {
  Parser p(text);
  Value v = p.value();
  p.ws();
  if (p.p != text.size()) p.fail("trailing characters");
  return v;
}

Value parseFile(const std::string& path) {
  std::ifstream in(path);
  if (!in) throw Error("cannot open execution plan '" + path + "'", ErrorCode::ExecutorError);
  std::stringstream ss;
  ss << in.rdbuf();
  return parse(ss.str());
}

}  // namespace json
}  // namespace mscclpp
