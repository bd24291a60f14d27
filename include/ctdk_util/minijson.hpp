// Minimal JSON reader / line writer for the command-line tools: the run config, the
// safetensors header and the loss.jsonl events (the reference uses nlohmann/json for these,
// emberlm tools/ctd_train/main.cpp:72-103, 377-389; src/core/safetensors.cpp:40-70).
// Numbers are kept as double (non-negative integer literals also exactly, as uint64, so that a
// 64-bit seed survives), objects keep their keys sorted (as nlohmann's default object does,
// which is what makes the written header and events come out in alphabetical key order).
#pragma once

#include <cctype>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace minijson {

struct Value;
using Object = std::map<std::string, Value>;
using Array = std::vector<Value>;

struct Value {
  enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
  bool b = false;
  double num = 0.0;
  uint64_t u64 = 0;        // exact value of a non-negative integer literal
  bool is_u64 = false;
  std::string str;
  std::shared_ptr<Array> arr;
  std::shared_ptr<Object> obj;

  bool is_object() const { return kind == kObject; }
  bool contains(const std::string& k) const { return kind == kObject && obj->count(k) != 0; }
  const Value& at(const std::string& k) const {
    if (kind != kObject) throw std::runtime_error("json: not an object while looking up '" + k + "'");
    auto it = obj->find(k);
    if (it == obj->end()) throw std::runtime_error("json: key '" + k + "' not found");
    return it->second;
  }
  double number() const {
    if (kind != kNumber) throw std::runtime_error("json: number expected");
    return num;
  }
  // A non-negative integer literal exactly (nlohmann's get<uint64_t>()); other numbers are truncated.
  uint64_t as_uint64() const {
    if (kind != kNumber) throw std::runtime_error("json: number expected");
    return is_u64 ? u64 : static_cast<uint64_t>(num);
  }
  const std::string& string() const {
    if (kind != kString) throw std::runtime_error("json: string expected");
    return str;
  }
  bool boolean() const {
    if (kind != kBool) throw std::runtime_error("json: boolean expected");
    return b;
  }
  const Array& array() const {
    if (kind != kArray) throw std::runtime_error("json: array expected");
    return *arr;
  }
  // value(key, default): the key's value if present, else the default (nlohmann's json::value)
  double value(const std::string& k, double d) const { return contains(k) ? at(k).number() : d; }
  bool value(const std::string& k, bool d) const { return contains(k) ? at(k).boolean() : d; }
  std::string value(const std::string& k, const std::string& d) const { return contains(k) ? at(k).string() : d; }
};

class Parser {
 public:
  explicit Parser(const std::string& text) : s_(text) {}
  Value parse() {
    Value v = parse_value();
    skip_ws();
    if (pos_ != s_.size()) fail("trailing characters");
    return v;
  }

 private:
  const std::string& s_;
  size_t pos_ = 0;

  [[noreturn]] void fail(const std::string& what) const {
    throw std::runtime_error("json: " + what + " at offset " + std::to_string(pos_));
  }
  void skip_ws() {
    while (pos_ < s_.size() && std::isspace(static_cast<unsigned char>(s_[pos_]))) ++pos_;
  }
  char peek() {
    skip_ws();
    if (pos_ >= s_.size()) fail("unexpected end");
    return s_[pos_];
  }
  void expect(char c) {
    if (peek() != c) fail(std::string("expected '") + c + "'");
    ++pos_;
  }
  Value parse_value() {
    const char c = peek();
    if (c == '{') return parse_object();
    if (c == '[') return parse_array();
    if (c == '"') {
      Value v;
      v.kind = Value::kString;
      v.str = parse_string();
      return v;
    }
    if (s_.compare(pos_, 4, "true") == 0) return literal(4, Value::kBool, true);
    if (s_.compare(pos_, 5, "false") == 0) return literal(5, Value::kBool, false);
    if (s_.compare(pos_, 4, "null") == 0) return literal(4, Value::kNull, false);
    return parse_number();
  }
  Value literal(size_t n, Value::Kind k, bool b) {
    pos_ += n;
    Value v;
    v.kind = k;
    v.b = b;
    return v;
  }
  Value parse_number() {
    const char* begin = s_.c_str() + pos_;
    char* end = nullptr;
    const double d = std::strtod(begin, &end);
    if (end == begin) fail("value expected");
    pos_ += static_cast<size_t>(end - begin);
    Value v;
    v.kind = Value::kNumber;
    v.num = d;
    bool digits = end > begin;
    for (const char* c = begin; c < end; ++c) digits = digits && *c >= '0' && *c <= '9';
    if (digits && end - begin <= 20) {
      errno = 0;
      const unsigned long long u = std::strtoull(begin, nullptr, 10);
      if (errno == 0) {
        v.u64 = u;
        v.is_u64 = true;
      }
    }
    return v;
  }
  std::string parse_string() {
    expect('"');
    std::string out;
    while (true) {
      if (pos_ >= s_.size()) fail("unterminated string");
      const char c = s_[pos_++];
      if (c == '"') break;
      if (c != '\\') {
        out.push_back(c);
        continue;
      }
      if (pos_ >= s_.size()) fail("bad escape");
      const char e = s_[pos_++];
      switch (e) {
        case 'n': out.push_back('\n'); break;
        case 't': out.push_back('\t'); break;
        case 'r': out.push_back('\r'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'u': {
          if (pos_ + 4 > s_.size()) fail("bad \\u escape");
          const unsigned cp = static_cast<unsigned>(std::strtoul(s_.substr(pos_, 4).c_str(), nullptr, 16));
          pos_ += 4;
          if (cp < 0x80) {
            out.push_back(static_cast<char>(cp));
          } else if (cp < 0x800) {
            out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
          } else {
            out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
            out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
            out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
          }
          break;
        }
        default: out.push_back(e);  // \" \\ \/
      }
    }
    return out;
  }
  Value parse_array() {
    expect('[');
    Value v;
    v.kind = Value::kArray;
    v.arr = std::make_shared<Array>();
    if (peek() == ']') {
      ++pos_;
      return v;
    }
    while (true) {
      v.arr->push_back(parse_value());
      if (peek() == ',') {
        ++pos_;
        continue;
      }
      expect(']');
      return v;
    }
  }
  Value parse_object() {
    expect('{');
    Value v;
    v.kind = Value::kObject;
    v.obj = std::make_shared<Object>();
    if (peek() == '}') {
      ++pos_;
      return v;
    }
    while (true) {
      if (peek() != '"') fail("key expected");
      std::string k = parse_string();
      expect(':');
      (*v.obj)[k] = parse_value();
      if (peek() == ',') {
        ++pos_;
        continue;
      }
      expect('}');
      return v;
    }
  }
};

inline Value parse(const std::string& text) { return Parser(text).parse(); }

inline std::string quote(const std::string& s) {
  std::string out = "\"";
  for (const char c : s) {
    if (c == '"' || c == '\\') {
      out.push_back('\\');
      out.push_back(c);
    } else if (static_cast<unsigned char>(c) < 0x20) {
      char buf[8];
      std::snprintf(buf, sizeof buf, "\\u%04x", c);
      out += buf;
    } else {
      out.push_back(c);
    }
  }
  out.push_back('"');
  return out;
}

// One flat event object per line: keys sorted, compact separators.
class Line {
 public:
  Line& add(const std::string& k, double v) {
    char buf[40];
    std::snprintf(buf, sizeof buf, "%.17g", v);
    items_[k] = buf;
    return *this;
  }
  Line& add(const std::string& k, float v) {
    char buf[40];
    std::snprintf(buf, sizeof buf, "%.9g", static_cast<double>(v));
    items_[k] = buf;
    return *this;
  }
  Line& add(const std::string& k, long long v) {
    items_[k] = std::to_string(v);
    return *this;
  }
  Line& add(const std::string& k, const std::string& v) {
    items_[k] = quote(v);
    return *this;
  }
  Line& add_bool(const std::string& k, bool v) {
    items_[k] = v ? "true" : "false";
    return *this;
  }
  std::string dump() const {
    std::string out = "{";
    bool first = true;
    for (const auto& kv : items_) {
      if (!first) out.push_back(',');
      first = false;
      out += quote(kv.first) + ":" + kv.second;
    }
    out.push_back('}');
    return out;
  }

 private:
  std::map<std::string, std::string> items_;
};

}  // namespace minijson
