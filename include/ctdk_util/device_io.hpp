// Checkpoint I/O between safetensors files and device memory through two pinned staging buffers.
//
// The reference stages every tensor through a pageable std::vector and a blocking cudaMemcpy
// (emberlm src/core/safetensors.cpp:78-91 on load, 131-144 on save), so the disk and the PCIe
// link take turns. Here the two overlap: while chunk k is written to (read from) the file, chunk
// k+1 is already moving over PCIe with cudaMemcpyAsync. The file format is unchanged
// (safetensors.hpp).
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "safetensors.hpp"

namespace st {

class PinnedPipe {
 public:
  explicit PinnedPipe(size_t chunk_bytes = size_t{32} << 20) : chunk_(chunk_bytes) {
    for (int i = 0; i < 2; ++i) {
      if (cudaMallocHost(reinterpret_cast<void**>(&buf_[i]), chunk_) != cudaSuccess ||
          cudaEventCreateWithFlags(&done_[i], cudaEventDisableTiming) != cudaSuccess)
        throw std::runtime_error("PinnedPipe: pinned staging buffers unavailable");
    }
    if (cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking) != cudaSuccess)
      throw std::runtime_error("PinnedPipe: stream creation failed");
  }
  PinnedPipe(const PinnedPipe&) = delete;
  PinnedPipe& operator=(const PinnedPipe&) = delete;
  ~PinnedPipe() {
    for (int i = 0; i < 2; ++i) {
      if (done_[i]) cudaEventDestroy(done_[i]);
      if (buf_[i]) cudaFreeHost(buf_[i]);
    }
    if (stream_) cudaStreamDestroy(stream_);
  }

  // Device -> file. `after` (optional) is an event the device data must wait for.
  void write_from_device(std::FILE* f, const float* dev, size_t bytes, cudaEvent_t after = nullptr) {
    if (after) check(cudaStreamWaitEvent(stream_, after, 0), "wait");
    const char* src = reinterpret_cast<const char*>(dev);
    const size_t n = (bytes + chunk_ - 1) / chunk_;
    auto fetch = [&](size_t k) {
      const size_t off = k * chunk_, len = std::min(chunk_, bytes - off);
      check(cudaMemcpyAsync(buf_[k & 1], src + off, len, cudaMemcpyDeviceToHost, stream_), "D2H");
      check(cudaEventRecord(done_[k & 1], stream_), "record");
    };
    if (n > 0) fetch(0);
    for (size_t k = 0; k < n; ++k) {
      if (k + 1 < n) fetch(k + 1);   // in flight while chunk k goes to the file
      check(cudaEventSynchronize(done_[k & 1]), "sync");
      const size_t len = std::min(chunk_, bytes - k * chunk_);
      if (std::fwrite(buf_[k & 1], 1, len, f) != len) throw std::runtime_error("short write");
    }
  }

  // File -> device. Returns with the last copies possibly still in flight on stream(); record an
  // event there or synchronise before the data is used.
  void read_to_device(std::FILE* f, float* dev, size_t bytes) {
    char* dst = reinterpret_cast<char*>(dev);
    const size_t n = (bytes + chunk_ - 1) / chunk_;
    for (size_t k = 0; k < n; ++k) {
      const size_t off = k * chunk_, len = std::min(chunk_, bytes - off);
      check(cudaEventSynchronize(done_[k & 1]), "sync");   // the buffer's previous copy has left it
      if (std::fread(buf_[k & 1], 1, len, f) != len) throw std::runtime_error("short read");
      check(cudaMemcpyAsync(dst + off, buf_[k & 1], len, cudaMemcpyHostToDevice, stream_), "H2D");
      check(cudaEventRecord(done_[k & 1], stream_), "record");
    }
  }

  cudaStream_t stream() const { return stream_; }
  void synchronize() { check(cudaStreamSynchronize(stream_), "sync"); }

 private:
  static void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("PinnedPipe ") + what + ": " + cudaGetErrorString(e));
  }
  size_t chunk_;
  char* buf_[2] = {nullptr, nullptr};
  cudaEvent_t done_[2] = {nullptr, nullptr};
  cudaStream_t stream_ = nullptr;
};

// Writes a safetensors file whose tensors live in device memory: the header for all of `items`
// first, then the data appended tensor by tensor in the same order (so the caller may refill a
// staging area between appends). The file is the one st::save() would write from host copies.
class DeviceWriter {
 public:
  DeviceWriter(const std::string& path, const std::vector<Item>& items, PinnedPipe& pipe)
      : path_(path), items_(items), pipe_(pipe) {
    const std::string head = header_bytes(items_);
    f_ = std::fopen(path.c_str(), "wb");
    if (!f_) throw std::runtime_error("cannot open " + path + " for writing");
    if (std::fwrite(head.data(), 1, head.size(), f_) != head.size()) fail("short write on ");
  }
  DeviceWriter(const DeviceWriter&) = delete;
  DeviceWriter& operator=(const DeviceWriter&) = delete;
  ~DeviceWriter() {
    if (f_) std::fclose(f_);
  }
  // The next tensor of the list, from device memory (after `after`, if given) or from the host.
  void append_device(const float* dev, cudaEvent_t after = nullptr) {
    pipe_.write_from_device(f_, dev, next_bytes(), after);
  }
  void append_host(const void* host) {
    const size_t n = next_bytes();
    if (std::fwrite(host, 1, n, f_) != n) fail("short write on ");
  }
  void close() {
    if (next_ != items_.size()) fail("not every tensor was appended to ");
    std::FILE* f = f_;
    f_ = nullptr;
    if (std::fclose(f) != 0) fail("short write on ");
  }

 private:
  size_t next_bytes() {
    if (next_ >= items_.size()) fail("too many tensors appended to ");
    int64_t n = 1;
    for (const int64_t d : items_[next_].shape) n *= d;
    ++next_;
    return static_cast<size_t>(n) * 4;
  }
  [[noreturn]] void fail(const char* what) { throw std::runtime_error(what + path_); }
  std::string path_;
  std::vector<Item> items_;
  PinnedPipe& pipe_;
  std::FILE* f_ = nullptr;
  size_t next_ = 0;
};

// Reads the F32 tensor `name` of `file` (opened at `path`) into device memory.
inline void read_f32_to_device(const File& file, const std::string& path, std::FILE* f, const std::string& name,
                               float* dev, int64_t numel, PinnedPipe& pipe) {
  const Entry& e = file.entry(name);
  if (e.dtype != "F32") throw std::runtime_error("safetensors: " + name + " has dtype " + e.dtype + ", F32 expected");
  if (e.numel() != numel || static_cast<int64_t>(e.end - e.begin) != numel * 4)
    throw std::runtime_error("safetensors: shape mismatch for " + name + " in " + path);
  if (fseeko(f, static_cast<off_t>(file.data_origin() + e.begin), SEEK_SET) != 0)
    throw std::runtime_error("safetensors: seek failed in " + path);
  pipe.read_to_device(f, dev, static_cast<size_t>(numel) * 4);
}

}  // namespace st
