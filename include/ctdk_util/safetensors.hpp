// Host-side reader / writer of the reference's safetensors files (weights and optimizer state),
// byte-compatible with emberlm src/core/safetensors.cpp:
//   8-byte little-endian header length | JSON header | raw little-endian tensor data
//   header: {"name": {"dtype": "F32", "shape": [...], "data_offsets": [begin, end]}, ...}
// The writer emits header keys in alphabetical order, data in the caller's order, and pads the
// header with spaces to a multiple of 8 bytes (safetensors.cpp:100-119). The reader accepts F32
// tensors and skips "__metadata__"; other dtypes are reported as unsupported when requested.
#pragma once

#include <cstdint>
#include <cstring>
#include <fstream>
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "minijson.hpp"

namespace st {

struct Entry {
  std::string dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;   // byte offsets inside the data section
  int64_t numel() const {
    int64_t n = 1;
    for (const int64_t d : shape) n *= d;
    return n;
  }
};

class File {
 public:
  explicit File(const std::string& path) : path_(path), in_(path, std::ios::binary) {
    if (!in_) throw std::runtime_error("cannot open " + path);
    unsigned char len8[8];
    if (!in_.read(reinterpret_cast<char*>(len8), 8)) throw std::runtime_error("safetensors: short read on header length: " + path);
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | len8[i];
    in_.seekg(0, std::ios::end);
    const uint64_t size = static_cast<uint64_t>(in_.tellg());
    if (8 + hlen > size) throw std::runtime_error("safetensors: short read on header: " + path);
    std::string text(hlen, '\0');
    in_.seekg(8, std::ios::beg);
    in_.read(text.data(), static_cast<std::streamsize>(hlen));
    origin_ = 8 + hlen;
    const minijson::Value h = minijson::parse(text);
    if (!h.is_object()) throw std::runtime_error("safetensors: header is not an object: " + path);
    for (const auto& kv : *h.obj) {
      if (kv.first == "__metadata__") continue;
      Entry e;
      e.dtype = kv.second.at("dtype").string();
      for (const auto& d : kv.second.at("shape").array()) e.shape.push_back(static_cast<int64_t>(d.number()));
      const auto& off = kv.second.at("data_offsets").array();
      if (off.size() != 2) throw std::runtime_error("safetensors: bad data_offsets for " + kv.first);
      e.begin = static_cast<uint64_t>(off[0].number());
      e.end = static_cast<uint64_t>(off[1].number());
      if (e.end < e.begin || origin_ + e.end > size) throw std::runtime_error("safetensors: data of " + kv.first + " lies outside the file");
      entries_[kv.first] = std::move(e);
    }
  }

  const std::map<std::string, Entry>& entries() const { return entries_; }
  uint64_t data_origin() const { return origin_; }   // file offset of the data section
  bool has(const std::string& name) const { return entries_.count(name) != 0; }
  const Entry& entry(const std::string& name) const {
    auto it = entries_.find(name);
    if (it == entries_.end()) throw std::runtime_error("safetensors: missing tensor " + name + " in " + path_);
    return it->second;
  }
  // Reads an F32 tensor of exactly `numel` elements into dst.
  void read_f32(const std::string& name, float* dst, int64_t numel) {
    const Entry& e = entry(name);
    if (e.dtype != "F32") throw std::runtime_error("safetensors: " + name + " has dtype " + e.dtype + ", F32 expected");
    if (e.numel() != numel || static_cast<int64_t>(e.end - e.begin) != numel * 4)
      throw std::runtime_error("safetensors: shape mismatch for " + name);
    in_.clear();
    in_.seekg(static_cast<std::streamoff>(origin_ + e.begin), std::ios::beg);
    if (!in_.read(reinterpret_cast<char*>(dst), static_cast<std::streamsize>(numel * 4)))
      throw std::runtime_error("safetensors: short read on " + name);
  }

 private:
  std::string path_;
  std::ifstream in_;
  uint64_t origin_ = 0;
  std::map<std::string, Entry> entries_;
};

struct Item {
  std::string name;
  std::vector<int64_t> shape;
  const float* data;   // host pointer, numel floats
};

// The 8-byte length and the JSON header text of a file holding `items` in this order.
inline std::string header_bytes(const std::vector<Item>& items) {
  std::map<std::string, std::string> header;   // sorted by name
  uint64_t running = 0;
  for (const Item& it : items) {
    int64_t n = 1;
    std::string shape = "[";
    for (size_t i = 0; i < it.shape.size(); ++i) {
      n *= it.shape[i];
      shape += (i ? "," : "") + std::to_string(it.shape[i]);
    }
    shape += "]";
    const uint64_t bytes = static_cast<uint64_t>(n) * 4;
    header[it.name] = "{\"data_offsets\":[" + std::to_string(running) + "," + std::to_string(running + bytes) +
                      "],\"dtype\":\"F32\",\"shape\":" + shape + "}";
    running += bytes;
  }
  std::string text = "{";
  bool first = true;
  for (const auto& kv : header) {
    if (!first) text.push_back(',');
    first = false;
    text += minijson::quote(kv.first) + ":" + kv.second;
  }
  text.push_back('}');
  while (text.size() % 8 != 0) text.push_back(' ');
  std::string out(8, '\0');
  const uint64_t hlen = text.size();
  for (int i = 0; i < 8; ++i) out[i] = static_cast<char>((hlen >> (8 * i)) & 0xFF);
  return out + text;
}

inline void save(const std::vector<Item>& items, const std::string& path) {
  const std::string head = header_bytes(items);
  std::ofstream out(path, std::ios::binary | std::ios::trunc);
  if (!out) throw std::runtime_error("cannot open " + path + " for writing");
  out.write(head.data(), static_cast<std::streamsize>(head.size()));
  for (const Item& it : items) {
    int64_t n = 1;
    for (const int64_t d : it.shape) n *= d;
    out.write(reinterpret_cast<const char*>(it.data), static_cast<std::streamsize>(n * 4));
  }
  if (!out) throw std::runtime_error("short write on " + path);
}

}  // namespace st
