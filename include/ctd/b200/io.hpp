// ctd::load_safetensors / save_safetensors / sample with the reference's signatures
// (emberlm include/ctd/safetensors.h, include/ctd/sampling.h) on this tree's reader / writer
// (ctdk_util/safetensors.hpp, device_io.hpp): tensors stream between the file and device memory
// through two pinned buffers instead of one pageable vector per tensor.
#pragma once

#include <filesystem>
#include <random>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../ctdk_util/device_io.hpp"
#include "core.hpp"

namespace ctd {

using TensorDict = std::unordered_map<std::string, Tensor>;

inline TensorDict load_safetensors(const std::filesystem::path& path, Device device) {
  if (device.is_cuda()) CTD_CUDA_CHECK(cudaDeviceSynchronize());   // the copies below run on a stream of their own
  st::File file(path.string());
  std::FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) throw std::runtime_error("safetensors: cannot open " + path.string());
  TensorDict out;
  try {
    std::unique_ptr<st::PinnedPipe> pipe;
    if (device.is_cuda()) pipe = std::make_unique<st::PinnedPipe>();
    for (const auto& kv : file.entries()) {
      const st::Entry& e = kv.second;
      DType dt;
      if (e.dtype == "F32") dt = DType::kFloat32;
      else if (e.dtype == "I64") dt = DType::kInt64;
      else if (e.dtype == "I32") dt = DType::kInt32;
      else throw std::runtime_error("safetensors: " + kv.first + " has dtype " + e.dtype + " (only F32 / I64 / I32 are supported)");
      Tensor t = Tensor::empty(e.shape, dt, device);
      if (t.nbytes() != e.end - e.begin) throw std::runtime_error("safetensors: size mismatch for " + kv.first);
      if (t.nbytes() == 0) {
        out.emplace(kv.first, std::move(t));
        continue;
      }
      if (fseeko(f, static_cast<off_t>(file.data_origin() + e.begin), SEEK_SET) != 0)
        throw std::runtime_error("safetensors: seek failed for " + kv.first);
      if (device.is_cuda()) {
        pipe->read_to_device(f, static_cast<float*>(t.data_ptr()), t.nbytes());
      } else if (std::fread(t.data_ptr(), 1, t.nbytes(), f) != t.nbytes()) {
        throw std::runtime_error("safetensors: short read for tensor " + kv.first);
      }
      out.emplace(kv.first, std::move(t));
    }
    if (pipe) pipe->synchronize();
  } catch (...) {
    std::fclose(f);
    throw;
  }
  std::fclose(f);
  return out;
}

inline void save_safetensors(const std::vector<std::pair<std::string, Tensor>>& named_tensors, const std::filesystem::path& path) {
  std::vector<st::Item> items;
  for (const auto& kv : named_tensors) {
    if (kv.second.dtype() != DType::kFloat32) throw std::runtime_error("save_safetensors: only fp32 supported, got " + kv.first);
    if (!kv.second.is_contiguous()) throw std::runtime_error("save_safetensors: non-contiguous tensor " + kv.first);
    items.push_back({kv.first, kv.second.shape(), nullptr});
  }
  CTD_CUDA_CHECK(cudaStreamSynchronize(nullptr));   // the tensors' producers ran on the default stream
  st::PinnedPipe pipe;
  st::DeviceWriter w(path.string(), items, pipe);
  for (const auto& kv : named_tensors) {
    if (kv.second.device().is_cuda()) w.append_device(static_cast<const float*>(kv.second.data_ptr()));
    else w.append_host(kv.second.data_ptr());
  }
  w.close();
}

// ---- sampling.h -----------------------------------------------------------------------------
struct SamplerConfig {
  float temperature = 1.0f;   // <= 0: greedy (argmax)
  int top_k = 0;              // 0: off
  float top_p = 0.0f;         // 0: off
};

// One token per batch row from logits_last fp32 [B, 1, V]; returns the ids on the host. The
// selection runs on the device (ctdk_sample): only the uniform draws go there (one per row, in row
// order, as the reference draws them) and only the ids come back.
inline std::vector<int64_t> sample(const Tensor& logits_last, const SamplerConfig& cfg, std::mt19937_64& rng) {
  if (logits_last.dtype() != DType::kFloat32) throw std::runtime_error("sample: fp32 logits only");
  if (logits_last.dim() != 3 || logits_last.shape()[1] != 1) throw std::runtime_error("sample: expected logits shape [B, 1, V]");
  const int64_t B = logits_last.shape()[0], V = logits_last.shape()[2];
  Tensor logits = logits_last;
  if (!logits.device().is_cuda()) {
    std::vector<float> host(static_cast<size_t>(logits.numel()));
    logits.copy_to_host(host.data());
    logits = Tensor::from_host(host.data(), logits_last.shape(), DType::kFloat32, kCUDA0);
  }
  const bool greedy = cfg.temperature <= 0.0f;
  std::vector<double> u(static_cast<size_t>(B), 0.0);
  if (!greedy) {
    std::uniform_real_distribution<double> dist(0.0, 1.0);
    for (int64_t b = 0; b < B; ++b) u[static_cast<size_t>(b)] = dist(rng);
  }
  Tensor d_u = Tensor::from_host(u.data(), {2 * B}, DType::kInt32, kCUDA0);   // B doubles as raw bytes
  Tensor d_out = Tensor::empty({B}, DType::kInt64, kCUDA0);
  Tensor work = Tensor::empty({greedy ? 1 : ctdk_sample_workspace_bytes(B, V) / 4}, DType::kFloat32, kCUDA0);
  detail::ctdk_ok(ctdk_sample(static_cast<const float*>(logits.data_ptr()), B, V, cfg.temperature, cfg.top_k, cfg.top_p,
                              static_cast<const double*>(d_u.data_ptr()), work.data_ptr(), static_cast<int64_t*>(d_out.data_ptr()), nullptr));
  std::vector<int64_t> out(static_cast<size_t>(B));
  d_out.copy_to_host(out.data());
  return out;
}

}  // namespace ctd
