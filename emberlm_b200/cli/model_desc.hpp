// Model description shared by the command-line tools: the architecture presets the reference
// detects from the embedding's shape (emberlm include/ctd/nn/model.h:39-141), the HF parameter
// names in Model::collect_parameters order (src/nn/model.cpp:78-98) with their shapes, and the
// parameter arena (ctdk_model_layout) they live in on the device.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/ctdk.h"

namespace cli {

inline ctdk_model_config preset(int vocab, int hid, int inter, int layers, int heads, int kv_heads, int head_dim,
                                float eps, float theta, int qk_norm) {
  ctdk_model_config c{};
  c.vocab_size = vocab;
  c.hidden_size = hid;
  c.intermediate_size = inter;
  c.num_hidden_layers = layers;
  c.num_attention_heads = heads;
  c.num_key_value_heads = kv_heads;
  c.head_dim = head_dim;
  c.rms_norm_eps = eps;
  c.rope_theta = theta;
  c.qk_norm = qk_norm;
  c.rope_scaling_factor = 0.0f;
  c.rope_scaling_low_freq_factor = 1.0f;
  c.rope_scaling_high_freq_factor = 4.0f;
  c.rope_scaling_original_max_pos = 8192;
  c.gradient_checkpointing = 0;
  c.precision = CTDK_GEMM_TF32;
  return c;
}

// The five architectures, chosen by (hidden_size, vocab_size) of model.embed_tokens.weight.
inline ctdk_model_config autodetect_config(int64_t vocab, int64_t hidden) {
  if (hidden == 576) return preset(49152, 576, 1536, 30, 9, 3, 64, 1e-5f, 100000.0f, 0);
  if (hidden == 960) return preset(49152, 960, 2560, 32, 15, 5, 64, 1e-5f, 100000.0f, 0);
  if (hidden == 1024 && vocab == 151936) return preset(151936, 1024, 3072, 28, 16, 8, 128, 1e-6f, 1000000.0f, 1);
  if (hidden == 2048 && vocab == 151936) return preset(151936, 2048, 6144, 28, 16, 8, 128, 1e-6f, 1000000.0f, 1);
  if (hidden == 2048 && vocab == 128256) {
    ctdk_model_config c = preset(128256, 2048, 8192, 16, 32, 8, 64, 1e-5f, 500000.0f, 0);
    c.rope_scaling_factor = 32.0f;
    return c;
  }
  throw std::runtime_error("autodetect_config: unsupported hidden_size=" + std::to_string(hidden) +
                           " vocab_size=" + std::to_string(vocab));
}

struct ParamDesc {
  std::string name;
  std::vector<int64_t> shape;
  int64_t offset = 0, numel = 0;   // floats, inside the arena
  bool decay = false;
};

inline std::vector<ParamDesc> describe_parameters(const ctdk_model_config& c, int64_t* arena_floats) {
  const int64_t hid = c.hidden_size, I = c.intermediate_size, D = c.head_dim;
  const int64_t H = c.num_attention_heads, Hk = c.num_key_value_heads;
  std::vector<ParamDesc> out;
  auto add = [&](const std::string& n, std::vector<int64_t> shape) {
    ParamDesc p;
    p.name = n;
    p.shape = std::move(shape);
    out.push_back(std::move(p));
  };
  add("model.embed_tokens.weight", {c.vocab_size, hid});
  for (int l = 0; l < c.num_hidden_layers; ++l) {
    const std::string p = "model.layers." + std::to_string(l) + ".";
    add(p + "input_layernorm.weight", {hid});
    add(p + "self_attn.q_proj.weight", {H * D, hid});
    add(p + "self_attn.k_proj.weight", {Hk * D, hid});
    add(p + "self_attn.v_proj.weight", {Hk * D, hid});
    add(p + "self_attn.o_proj.weight", {hid, H * D});
    if (c.qk_norm) {
      add(p + "self_attn.q_norm.weight", {D});
      add(p + "self_attn.k_norm.weight", {D});
    }
    add(p + "post_attention_layernorm.weight", {hid});
    add(p + "mlp.gate_proj.weight", {I, hid});
    add(p + "mlp.up_proj.weight", {I, hid});
    add(p + "mlp.down_proj.weight", {hid, I});
  }
  add("model.norm.weight", {hid});
  const int64_t n = ctdk_model_num_tensors(&c);
  if (n != static_cast<int64_t>(out.size())) throw std::runtime_error(std::string("model layout: ") + ctdk_last_error());
  std::vector<int64_t> off(n), num(n);
  std::vector<int> dec(n);
  int64_t total = 0;
  if (ctdk_model_layout(&c, off.data(), num.data(), dec.data(), &total) != CTDK_OK)
    throw std::runtime_error(std::string("model layout: ") + ctdk_last_error());
  for (int64_t i = 0; i < n; ++i) {
    int64_t k = 1;
    for (const int64_t d : out[i].shape) k *= d;
    if (k != num[i]) throw std::runtime_error("model layout: size mismatch for " + out[i].name);
    out[i].offset = off[i];
    out[i].numel = num[i];
    out[i].decay = dec[i] != 0;
  }
  *arena_floats = total;
  return out;
}

}  // namespace cli
