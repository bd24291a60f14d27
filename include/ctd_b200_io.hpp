// ctd::load_safetensors / ctd::save_safetensors with the reference's signatures
// (include/ctd/safetensors.h:14-20) over the reader / writer the command-line tools use. fp32
// tensors only, which is what the training path stores (weights, and the optimizer's m / v / step,
// tools/ctd_train/main.cpp:208-234); another dtype in a file throws.
#pragma once

#include <filesystem>
#include <string>
#include <utility>
#include <vector>

#include "ctd_b200_nn.hpp"
#include "ctdk_util/safetensors.hpp"

namespace ctd {

inline TensorDict load_safetensors(const std::filesystem::path& path, Device device) {
  st::File file(path.string());
  TensorDict out;
  std::vector<float> buf;
  for (const auto& kv : file.entries()) {
    const int64_t n = kv.second.numel();
    buf.resize(static_cast<size_t>(n > 0 ? n : 1));
    file.read_f32(kv.first, buf.data(), n);
    out[kv.first] = Tensor::from_host(buf.data(), kv.second.shape, DType::kFloat32, device);
  }
  return out;
}

inline void save_safetensors(const std::vector<std::pair<std::string, Tensor>>& named_tensors, const std::filesystem::path& path) {
  std::vector<std::vector<float>> host(named_tensors.size());
  std::vector<st::Item> items;
  for (size_t i = 0; i < named_tensors.size(); ++i) {
    const Tensor& t = named_tensors[i].second;
    detail::require(t.defined() && t.dtype() == DType::kFloat32, "save_safetensors: fp32 tensors only");
    host[i].resize(static_cast<size_t>(t.numel() > 0 ? t.numel() : 1));
    t.copy_to_host(host[i].data());
    items.push_back(st::Item{named_tensors[i].first, t.shape(), host[i].data()});
  }
  st::save(items, path.string());
}

}  // namespace ctd
