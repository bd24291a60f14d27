// C++ mirror of the reference's model-level API for the training loop, on top of the step engine in
// ctdk.h: ctd::nn::LlamaConfig, ctd::nn::Model with collect_parameters() and forward_train_masked(),
// ctd::nn::build_model(), ctd::TensorDict — same names and member meaning as emberlm's
// include/ctd/nn/model.h:19-220 and include/ctd/safetensors.h:14 — so that the loop of
// tools/ctd_train/main.cpp:346-373
//
//     Tensor loss = model.forward_train_masked(ids, targets, loss_mask);
//     ops::mul_scalar(loss, 1.0f / accum).backward();
//     ... optim::clip_grad_norm_(all_params, c);  opt.step();  opt.zero_grad();
//
// compiles and runs against this build. The model is not a tree of layer objects here: its
// parameters live in one arena in collect_parameters order and the forward + backward of a
// micro-batch is ONE fused pass of the engine, started by backward() on the loss (or by reading the
// loss, for a pass without gradients). Gradients accumulate over micro-batches until the
// optimizer's zero_grad(), as with the reference's AccumulateGrad nodes. Header-only.
#pragma once

#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "ctd_b200.hpp"

namespace ctd {

using TensorDict = std::unordered_map<std::string, Tensor>;

namespace nn {

struct LlamaConfig {
  int vocab_size;
  int hidden_size;
  int intermediate_size;
  int num_hidden_layers;
  int num_attention_heads;
  int num_key_value_heads;
  int head_dim;
  int max_position_embeddings;
  float rms_norm_eps;
  float rope_theta;
  bool tie_word_embeddings;
  bool qk_norm = false;
  float rope_scaling_factor = 0.0f;
  float rope_scaling_low_freq_factor = 1.0f;
  float rope_scaling_high_freq_factor = 4.0f;
  int rope_scaling_original_max_pos = 8192;
};

namespace detail {

inline ctdk_model_config to_ctdk(const LlamaConfig& c, bool checkpointing) {
  ctdk_model_config k{};
  k.vocab_size = c.vocab_size;
  k.hidden_size = c.hidden_size;
  k.intermediate_size = c.intermediate_size;
  k.num_hidden_layers = c.num_hidden_layers;
  k.num_attention_heads = c.num_attention_heads;
  k.num_key_value_heads = c.num_key_value_heads;
  k.head_dim = c.head_dim;
  k.rms_norm_eps = c.rms_norm_eps;
  k.rope_theta = c.rope_theta;
  k.qk_norm = c.qk_norm ? 1 : 0;
  k.rope_scaling_factor = c.rope_scaling_factor;
  k.rope_scaling_low_freq_factor = c.rope_scaling_low_freq_factor;
  k.rope_scaling_high_freq_factor = c.rope_scaling_high_freq_factor;
  k.rope_scaling_original_max_pos = c.rope_scaling_original_max_pos;
  k.gradient_checkpointing = checkpointing ? 1 : 0;
  k.precision = CTDK_GEMM_TF32;
  return k;
}

struct ParamInfo {
  std::string name;
  std::vector<int64_t> shape;
  int64_t offset = 0, numel = 0;
  bool decay = false;
};

// Names and shapes in Model::collect_parameters order (src/nn/model.cpp:78-98), offsets and decay
// flags from the engine's own layout.
inline std::vector<ParamInfo> parameter_table(const ctdk_model_config& c, int64_t* arena_floats) {
  const int64_t hid = c.hidden_size, I = c.intermediate_size, D = c.head_dim;
  const int64_t H = c.num_attention_heads, Hk = c.num_key_value_heads;
  std::vector<ParamInfo> out;
  auto add = [&](const std::string& n, std::vector<int64_t> shape) {
    ParamInfo p;
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
  ctd::detail::require(n == static_cast<int64_t>(out.size()), "model layout: tensor count differs from the engine's");
  std::vector<int64_t> off(static_cast<size_t>(n)), num(static_cast<size_t>(n));
  std::vector<int> dec(static_cast<size_t>(n));
  ctd::detail::ctdk_ok(ctdk_model_layout(&c, off.data(), num.data(), dec.data(), arena_floats));
  for (size_t i = 0; i < out.size(); ++i) {
    int64_t k = 1;
    for (const int64_t d : out[i].shape) k *= d;
    ctd::detail::require(k == num[i], "model layout: tensor size differs from the engine's");
    out[i].offset = off[i];
    out[i].numel = num[i];
    out[i].decay = dec[i] != 0;
  }
  return out;
}

}  // namespace detail

struct Model {
  LlamaConfig config{};
  bool gradient_checkpointing = false;

  struct NamedParameters {
    std::vector<std::pair<std::string, Tensor>> all;
    std::vector<Tensor> decay;
    std::vector<Tensor> no_decay;
    std::vector<std::string> decay_names;
    std::vector<std::string> no_decay_names;
  };

  // Handles onto the parameter arena, in the reference's order; decay = embedding and linear
  // weights, no_decay = every norm weight (src/nn/model.cpp:78-98).
  NamedParameters collect_parameters() {
    ctd::detail::require(state != nullptr, "collect_parameters: model not built (use build_model)");
    NamedParameters out;
    for (size_t i = 0; i < state->table.size(); ++i) {
      const detail::ParamInfo& p = state->table[i];
      out.all.emplace_back(p.name, state->tensors[i]);
      (p.decay ? out.decay : out.no_decay).push_back(state->tensors[i]);
      (p.decay ? out.decay_names : out.no_decay_names).push_back(p.name);
    }
    return out;
  }

  // The masked mean cross-entropy of the batch as a [1] tensor (include/ctd/nn/model.h:196-206).
  // Nothing runs yet: backward() on the result (or on ops::mul_scalar of it) runs forward and
  // backward in one fused pass; copy_to_host() before any backward() runs the forward alone.
  Tensor forward_train_masked(const Tensor& input_ids, const Tensor& targets, const Tensor& loss_mask) const {
    ctd::detail::require(state != nullptr, "forward_train_masked: model not built (use build_model)");
    ctd::detail::require(input_ids.dim() == 2 && input_ids.dtype() == DType::kInt64 && input_ids.device().is_cuda(),
                         "forward_train_masked: input_ids must be int64 [B, T] on CUDA");
    ctd::detail::require(targets.dtype() == DType::kInt64 && targets.numel() == input_ids.numel() && targets.device().is_cuda(),
                         "forward_train_masked: targets must be int64 with input_ids' element count, on CUDA");
    ctd::detail::require(loss_mask.dtype() == DType::kFloat32 && loss_mask.numel() == input_ids.numel() && loss_mask.device().is_cuda(),
                         "forward_train_masked: loss_mask must be fp32 with input_ids' element count, on CUDA");
    const int64_t B = input_ids.shape()[0], T = input_ids.shape()[1];
    std::shared_ptr<State> st = state;
    const bool ckpt = gradient_checkpointing;
    auto node = std::make_shared<ctd::detail::LossNode>();
    ctd::detail::LossNode* raw = node.get();   // the closures live inside the node: no owning capture of it
    node->forward = [st, ckpt, input_ids, targets, loss_mask, B, T, raw]() {
      st->ensure_engine(B, T, ckpt);
      float* sums = st->loss_sums();
      ctd::detail::cuda_ok(cudaMemset(sums, 0, 2 * sizeof(float)), "forward_train_masked: cudaMemset");
      ctd::detail::ctdk_ok(ctdk_engine_forward_loss(st->engine, static_cast<const int64_t*>(input_ids.data_ptr()),
                                                    static_cast<const int64_t*>(targets.data_ptr()),
                                                    static_cast<const float*>(loss_mask.data_ptr()), B, T, sums, nullptr));
      raw->value = st->read_loss();
      raw->have_value = true;
    };
    node->backward = [st, ckpt, input_ids, targets, loss_mask, B, T, raw](float dy) {
      // row weight = mask * dy / sum(mask): the factor of CrossEntropyMaskedBackward (src/ops/loss.cu:388-411)
      std::vector<float> m(static_cast<size_t>(B * T));
      loss_mask.copy_to_host(m.data());
      double sm = 0.0;
      for (const float v : m) sm += v;
      if (sm <= 0.0) throw std::runtime_error("cross_entropy_masked backward: sum(loss_mask) == 0");
      for (auto& v : m) v = static_cast<float>(v * dy / sm);
      Tensor rw = Tensor::from_host(m.data(), {B * T}, DType::kFloat32, loss_mask.device());
      st->ensure_engine(B, T, ckpt);
      const int accumulate = st->tensors.front().grad().defined() ? 1 : 0;   // until the optimizer's zero_grad()
      float* sums = st->loss_sums();
      ctd::detail::cuda_ok(cudaMemset(sums, 0, 2 * sizeof(float)), "backward: cudaMemset");
      ctd::detail::ctdk_ok(ctdk_engine_forward_backward(st->engine, static_cast<const int64_t*>(input_ids.data_ptr()),
                                                        static_cast<const int64_t*>(targets.data_ptr()),
                                                        static_cast<const float*>(loss_mask.data_ptr()),
                                                        static_cast<const float*>(rw.data_ptr()), B, T, accumulate, sums, nullptr));
      raw->value = st->read_loss();   // blocking: rw stays alive until the pass has finished
      raw->have_value = true;
      if (!accumulate)
        for (size_t i = 0; i < st->table.size(); ++i)
          st->tensors[i].set_grad(Tensor::view(st->grads, static_cast<float*>(st->grads.get()) + st->table[i].offset,
                                               st->table[i].shape, DType::kFloat32, kCUDA0));
    };
    return Tensor::loss_of(std::move(node), 1.0f, kCUDA0);
  }

  // Everything a built model owns on the device; copies of a Model share it.
  struct State {
    ctdk_model_config kcfg{};
    std::vector<detail::ParamInfo> table;
    std::vector<Tensor> tensors;   // views of `params`
    int64_t total = 0;
    std::shared_ptr<void> params, grads, workspace, scalars;
    void* engine = nullptr;
    int64_t eng_B = 0, eng_T = 0;
    ~State() {
      if (engine != nullptr) ctdk_engine_destroy(engine);
    }
    static std::shared_ptr<void> device_alloc(size_t bytes, const char* what) {
      void* p = nullptr;
      ctd::detail::cuda_ok(cudaMalloc(&p, bytes), what);
      return std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
    }
    float* loss_sums() { return static_cast<float*>(scalars.get()); }
    float read_loss() {
      float h[2];
      ctd::detail::cuda_ok(cudaMemcpy(h, scalars.get(), sizeof h, cudaMemcpyDeviceToHost), "read loss");
      return h[1] > 0.0f ? h[0] / h[1] : 0.0f;
    }
    // (Re)creates the engine when the batch outgrows its workspace or checkpointing was switched.
    void ensure_engine(int64_t B, int64_t T, bool ckpt) {
      if (engine != nullptr && B <= eng_B && T <= eng_T && (kcfg.gradient_checkpointing != 0) == ckpt) return;
      if (engine != nullptr) {
        ctd::detail::cuda_ok(cudaDeviceSynchronize(), "ensure_engine: synchronize");
        ctdk_engine_destroy(engine);
        engine = nullptr;
        workspace.reset();
      }
      kcfg.gradient_checkpointing = ckpt ? 1 : 0;
      const int64_t nb = B > eng_B ? B : eng_B, nt = T > eng_T ? T : eng_T;
      const int64_t bytes = ctdk_engine_workspace_bytes(&kcfg, nb, nt);
      if (bytes < 0) throw std::runtime_error(ctdk_last_error());
      workspace = device_alloc(static_cast<size_t>(bytes), "ensure_engine: workspace");
      ctd::detail::ctdk_ok(ctdk_engine_create(&kcfg, static_cast<float*>(params.get()), static_cast<float*>(grads.get()),
                                              workspace.get(), bytes, nb, nt, &engine));
      eng_B = nb;
      eng_T = nt;
    }
  };
  std::shared_ptr<State> state;
};

// Lays the named tensors of `w` (fp32, on the host or the device) out in the parameter arena.
// A missing or mis-sized tensor throws, as the reference's build_model does (src/nn/model.cpp:24-76).
inline Model build_model(const TensorDict& w, const LlamaConfig& cfg) {
  ctd::detail::require(cfg.tie_word_embeddings, "build_model: untied output embeddings are not supported by the engine");
  Model m;
  m.config = cfg;
  auto st = std::make_shared<Model::State>();
  st->kcfg = detail::to_ctdk(cfg, false);
  st->table = detail::parameter_table(st->kcfg, &st->total);
  const size_t bytes = static_cast<size_t>(st->total) * sizeof(float);
  st->params = Model::State::device_alloc(bytes, "build_model: parameter arena");
  st->grads = Model::State::device_alloc(bytes, "build_model: gradient arena");
  st->scalars = Model::State::device_alloc(64, "build_model: scalars");
  ctd::detail::cuda_ok(cudaMemset(st->params.get(), 0, bytes), "build_model: cudaMemset");
  ctd::detail::cuda_ok(cudaMemset(st->grads.get(), 0, bytes), "build_model: cudaMemset");
  for (const detail::ParamInfo& p : st->table) {
    auto it = w.find(p.name);
    if (it == w.end()) throw std::runtime_error("build_model: missing tensor " + p.name);
    const Tensor& src = it->second;
    if (src.dtype() != DType::kFloat32 || src.numel() != p.numel)
      throw std::runtime_error("build_model: tensor " + p.name + " has the wrong type or size");
    float* dst = static_cast<float*>(st->params.get()) + p.offset;
    ctd::detail::cuda_ok(cudaMemcpy(dst, src.data_ptr(), src.nbytes(),
                                    src.device().is_cuda() ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice),
                         "build_model: copy");
    st->tensors.push_back(Tensor::view(st->params, dst, p.shape, DType::kFloat32, kCUDA0));
  }
  m.state = std::move(st);
  return m;
}

}  // namespace nn
}  // namespace ctd
