// ctd::nn — the reference's layer and model API (emberlm include/ctd/nn/*.h, src/nn/model.cpp) on
// the ctdk kernels. The aggregates keep the reference's member names and order (its tests build them
// with designated initialisers), the functions their signatures and error behaviour.
//
// What runs underneath is not the reference's op-by-op chain:
//   - Attention::forward_train is ONE tape node around the fused kernels (q/k/v projections into a
//     packed buffer, per-head QK-Norm + RoPE in one kernel, flash-style causal GQA attention that
//     never materialises the [B*H, T, T] scores, and their fused backward);
//   - MLP::forward is ONE tape node that uses the SwiGLU GEMM epilogues when gate_proj and up_proj
//     are adjacent in memory (they are in a built model);
//   - build_model lays every parameter out in one arena, and the training entry points of a built
//     model (forward_train, forward_train_masked) return a loss whose backward() is ONE pass of the
//     step engine (ctdk_engine_forward_backward): forward, masked CE and backward fused, with the
//     gradients written into a gradient arena that the parameters' grad() are views of.
// Header-only.
#pragma once

#include <cmath>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "ops.hpp"

namespace ctd {

using TensorDict = std::unordered_map<std::string, Tensor>;

namespace nn {

namespace detail {
using ::ctd::detail::ctdk_ok;
using ::ctd::detail::require;
using ::ctd::ops::detail::f;
using ::ctd::ops::detail::Grads;
// b directly follows a in the same storage.
inline bool adjacent(const Tensor& a, const Tensor& b) {
  return a.storage() && a.storage() == b.storage() && b.storage_offset() == a.storage_offset() + a.numel();
}
inline int64_t rows_of(const Tensor& x) { return x.numel() / x.shape().back(); }
inline std::vector<int64_t> with_last(const Tensor& x, int64_t last) {
  std::vector<int64_t> s = x.shape();
  s.back() = last;
  return s;
}
inline void gemm(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                 int ta, int tb, int epilogue = CTDK_EPI_STORE) {
  ctdk_ok(ctdk_gemm(A, B, C, M, N, K, lda, ldb, ldc, ta, tb, ::ctd::detail::matmul_precision(), epilogue, nullptr, nullptr));
}
}  // namespace detail

// ---- linear.h / rms_norm.h / embedding.h ------------------------------------------------------
struct Linear {
  Tensor weight;   // [out, in]; y = x W^T over any leading shape
  Tensor forward(const Tensor& x) const {
    const int64_t in = weight.shape()[1];
    if (x.shape().back() != in) throw std::runtime_error("Linear: in_features mismatch");
    Tensor y = ops::matmul(x.reshape({x.numel() / in, in}), weight, false, true);
    return y.reshape(detail::with_last(x, weight.shape()[0]));
  }
};

struct RMSNorm {
  Tensor weight;   // [hidden]
  float eps = 1e-5f;
  Tensor forward(const Tensor& x) const { return ops::rms_norm(x, weight, eps); }
};

struct Embedding {
  Tensor weight;   // [vocab, hidden]
  Tensor forward(const Tensor& ids) const { return ops::embedding(ids, weight); }
};

// ---- mlp.h ----------------------------------------------------------------------------------
struct MLP {
  Linear gate_proj;
  Linear up_proj;
  Linear down_proj;

  // y = down(silu(gate(x)) * up(x))
  Tensor forward(const Tensor& x) const {
    const Tensor &wg = gate_proj.weight, &wu = up_proj.weight, &wd = down_proj.weight;
    const int64_t hid = wg.shape()[1], I = wg.shape()[0], M = detail::rows_of(x);
    if (x.shape().back() != hid) throw std::runtime_error("Linear: in_features mismatch");
    if (!detail::adjacent(wg, wu) || wu.shape() != wg.shape()) {
      Tensor h = ops::mul(ops::silu(gate_proj.forward(x)), up_proj.forward(x));
      return down_proj.forward(h);
    }
    // gate | up from one GEMM over the stacked [2I, hid] weight, SwiGLU in its epilogue
    Tensor gu = Tensor::empty({M, 2 * I}, DType::kFloat32, x.device());
    Tensor act = Tensor::empty({M, I}, DType::kFloat32, x.device());
    detail::ctdk_ok(ctdk_gemm_swiglu(detail::f(x), detail::f(wg), detail::f(gu), detail::f(act), M, I, hid, CTDK_GEMM_TF32, nullptr));
    const int64_t out = wd.shape()[0];
    Tensor y = Tensor::empty(detail::with_last(x, out), DType::kFloat32, x.device());
    detail::gemm(detail::f(act), detail::f(wd), detail::f(y), M, out, I, I, I, out, 0, 1);
    Tensor sx = x.detach(), swg = wg.detach(), swd = wd.detach();
    autograd::detail::record(y, {x, wg, wu, wd}, "FusedMlpBackward", [=](const detail::Grads& g) {
      const Tensor& dy = g.at(0);
      Tensor dgu = Tensor::empty({M, 2 * I}, DType::kFloat32, dy.device());
      Tensor dact = Tensor::empty({M, I}, DType::kFloat32, dy.device());
      // d(act) = dy Wd with MulBackward / SiluBackward in the epilogue (dact is scratch for shapes
      // the fused kernel does not take)
      detail::ctdk_ok(ctdk_gemm_swiglu_bwd(detail::f(dy), detail::f(swd), detail::f(gu), detail::f(dgu), detail::f(dact), M, I, out,
                                           CTDK_GEMM_TF32, nullptr));
      Tensor dwd = Tensor::empty({out, I}, DType::kFloat32, dy.device());
      detail::gemm(detail::f(dy), detail::f(act), detail::f(dwd), out, I, M, out, I, I, 1, 0);
      Tensor dx = Tensor::empty(sx.shape(), DType::kFloat32, dy.device());
      detail::gemm(detail::f(dgu), detail::f(swg), detail::f(dx), M, hid, 2 * I, 2 * I, hid, hid, 0, 0);
      StoragePtr both = make_storage(static_cast<size_t>(2 * I * hid) * 4, cuda_allocator());
      Tensor dwg = Tensor::view_of(both, 0, {I, hid}, DType::kFloat32), dwu = Tensor::view_of(both, I * hid, {I, hid}, DType::kFloat32);
      detail::gemm(detail::f(dgu), detail::f(sx), detail::f(dwg), 2 * I, hid, M, 2 * I, hid, hid, 1, 0);
      return detail::Grads{dx, dwg, dwu, dwd};
    });
    return y;
  }
};

// ---- kv_cache.h -----------------------------------------------------------------------------
struct KVLayer {
  Tensor k;   // [B, H_kv, max_seq_len, D]
  Tensor v;
};

struct KVCache {
  std::vector<KVLayer> layers;
  int64_t current_len = 0;
  int64_t max_seq_len = 0;
  int64_t batch = 0;

  static KVCache allocate(int num_layers, int num_kv_heads, int head_dim, int64_t batch, int64_t max_seq, Device device) {
    KVCache c;
    c.batch = batch;
    c.max_seq_len = max_seq;
    for (int i = 0; i < num_layers; ++i)
      c.layers.push_back({Tensor::zeros({batch, num_kv_heads, max_seq, head_dim}, DType::kFloat32, device),
                          Tensor::zeros({batch, num_kv_heads, max_seq, head_dim}, DType::kFloat32, device)});
    return c;
  }
  void reset() { current_len = 0; }
};

// ---- attention.h ----------------------------------------------------------------------------
struct Attention {
  Linear q_proj;
  Linear k_proj;
  Linear v_proj;
  Linear o_proj;
  int num_heads = 0;
  int num_kv_heads = 0;
  int head_dim = 0;
  float rope_theta = 100000.0f;
  ops::RopeScaling rope_scaling{};
  RMSNorm q_norm{Tensor{}, 0.0f};   // Qwen3 QK-Norm: per-head RMSNorm on q and k before RoPE;
  RMSNorm k_norm{Tensor{}, 0.0f};   // absent (no storage) in models without it

  bool has_qk_norm() const { return q_norm.weight.storage() != nullptr; }
  int group() const { return num_heads / num_kv_heads; }
  int hidden_size() const { return num_heads * head_dim; }

  // Inference. With a cache: K / V of the T new positions are written at position_start and the
  // queries attend over cache[0 : position_start + T].
  Tensor forward(const Tensor& x, KVLayer* kv = nullptr, int position_start = 0) const {
    const int64_t B = x.shape()[0], T = x.shape()[1];
    const int H = num_heads, Hk = num_kv_heads, D = head_dim;
    Tensor q = q_proj.forward(x).reshape({B, T, H, D});
    Tensor k = k_proj.forward(x).reshape({B, T, Hk, D});
    Tensor v = v_proj.forward(x).reshape({B, T, Hk, D});
    if (has_qk_norm()) {
      q = q_norm.forward(q);
      k = k_norm.forward(k);
    }
    ops::apply_rope_inplace(q, position_start, rope_theta, rope_scaling);
    ops::apply_rope_inplace(k, position_start, rope_theta, rope_scaling);
    int64_t L = T;
    Tensor keys, values;   // [B, H, L, D]
    if (kv != nullptr) {
      ops::write_kv_inplace(kv->k, k, position_start);
      ops::write_kv_inplace(kv->v, v, position_start);
      L = position_start + T;
      keys = ops::read_kv_expanded(kv->k, static_cast<int>(L), group());
      values = ops::read_kv_expanded(kv->v, static_cast<int>(L), group());
    } else {
      keys = ops::permute(ops::repeat_kv_heads(k, group()), {0, 2, 1, 3});
      values = ops::permute(ops::repeat_kv_heads(v, group()), {0, 2, 1, 3});
    }
    Tensor q3 = ops::permute(q, {0, 2, 1, 3}).reshape({B * H, T, D});
    Tensor scores = ops::bmm(q3, keys.reshape({B * H, L, D}), false, true);   // [B*H, T, L]
    scores = ops::mul_scalar(scores, 1.0f / std::sqrt(static_cast<float>(D)));
    ops::apply_causal_mask_inplace(scores, position_start);
    Tensor ctx = ops::bmm(ops::softmax(scores), values.reshape({B * H, L, D}), false, false);   // [B*H, T, D]
    ctx = ops::permute(ctx.reshape({B, H, T, D}), {0, 2, 1, 3}).reshape({B, T, static_cast<int64_t>(H) * D});
    return o_proj.forward(ctx);
  }

  // Training (autograd-aware, no cache).
  Tensor forward_train(const Tensor& x) const {
    const int D = head_dim;
    if ((D != 64 && D != 128) || x.dtype() != DType::kFloat32 || !x.device().is_cuda()) return forward_train_chain(x);
    return o_proj.forward(fused_attention(x));
  }

 private:
  // The reference's op chain on the tape (bmm -> scale -> mask -> softmax -> bmm), for head sizes
  // the fused kernels do not take.
  Tensor forward_train_chain(const Tensor& x) const {
    const int64_t B = x.shape()[0], T = x.shape()[1];
    const int H = num_heads, Hk = num_kv_heads, D = head_dim;
    Tensor q = q_proj.forward(x).reshape({B, T, H, D});
    Tensor k = k_proj.forward(x).reshape({B, T, Hk, D});
    Tensor v = v_proj.forward(x).reshape({B, T, Hk, D});
    if (has_qk_norm()) {
      q = q_norm.forward(q);
      k = k_norm.forward(k);
    }
    q = ops::rope(q, 0, rope_theta, rope_scaling);
    k = ops::rope(k, 0, rope_theta, rope_scaling);
    Tensor keys = ops::permute(ops::repeat_kv_heads(k, group()), {0, 2, 1, 3}).reshape({B * H, T, D});
    Tensor values = ops::permute(ops::repeat_kv_heads(v, group()), {0, 2, 1, 3}).reshape({B * H, T, D});
    Tensor q3 = ops::permute(q, {0, 2, 1, 3}).reshape({B * H, T, D});
    Tensor scores = ops::mul_scalar(ops::bmm(q3, keys, false, true), 1.0f / std::sqrt(static_cast<float>(D)));
    Tensor probs = ops::softmax(ops::apply_causal_mask(scores, 0));
    Tensor ctx = ops::bmm(probs, values, false, false).reshape({B, H, T, D});
    return o_proj.forward(ops::permute(ctx, {0, 2, 1, 3}).reshape({B, T, static_cast<int64_t>(H) * D}));
  }

  // x [B, T, hid] -> attention output [B, T, H*D] (before o_proj) as one tape node.
  Tensor fused_attention(const Tensor& x) const {
    const int64_t B = x.shape()[0], T = x.shape()[1], rows = B * T;
    const int H = num_heads, Hk = num_kv_heads, D = head_dim;
    const int64_t hid = x.shape()[2], QN = static_cast<int64_t>(H + 2 * Hk) * D, HD = static_cast<int64_t>(H) * D, KD = static_cast<int64_t>(Hk) * D;
    const Tensor &wq = q_proj.weight, &wk = k_proj.weight, &wv = v_proj.weight;
    if (wq.shape()[1] != hid) throw std::runtime_error("Linear: in_features mismatch");
    const bool stacked = detail::adjacent(wq, wk) && detail::adjacent(wk, wv);
    const bool norm = has_qk_norm();
    const float eps = q_norm.eps;
    const Device dev = x.device();
    Tensor qkv_pre = Tensor::empty({rows, QN}, DType::kFloat32, dev);
    if (stacked) {
      detail::gemm(detail::f(x), detail::f(wq), detail::f(qkv_pre), rows, QN, hid, hid, hid, QN, 0, 1);
    } else {
      detail::gemm(detail::f(x), detail::f(wq), detail::f(qkv_pre), rows, HD, hid, hid, hid, QN, 0, 1);
      detail::gemm(detail::f(x), detail::f(wk), detail::f(qkv_pre) + HD, rows, KD, hid, hid, hid, QN, 0, 1);
      detail::gemm(detail::f(x), detail::f(wv), detail::f(qkv_pre) + HD + KD, rows, KD, hid, hid, hid, QN, 0, 1);
    }
    ctdk_rope_params rp;
    rp.theta = rope_theta;
    rp.scaling_factor = rope_scaling.enabled() ? rope_scaling.factor : 0.0f;
    rp.low_freq_wavelen = rope_scaling.low_freq_wavelen();
    rp.high_freq_wavelen = rope_scaling.high_freq_wavelen();
    Tensor table = Tensor::empty({T, D}, DType::kFloat32, dev);
    detail::ctdk_ok(ctdk_rope_table(detail::f(table), T, D, 0, &rp, nullptr));
    Tensor qkv = norm ? Tensor::empty({rows, QN}, DType::kFloat32, dev) : qkv_pre;
    Tensor rstd_q = norm ? Tensor::empty({rows * H}, DType::kFloat32, dev) : Tensor{};
    Tensor rstd_k = norm ? Tensor::empty({rows * Hk}, DType::kFloat32, dev) : Tensor{};
    Tensor wqn = norm ? q_norm.weight.detach() : Tensor{}, wkn = norm ? k_norm.weight.detach() : Tensor{};
    detail::ctdk_ok(ctdk_qk_norm_rope_fwd(detail::f(qkv_pre), detail::f(qkv), norm ? detail::f(wqn) : nullptr, norm ? detail::f(wkn) : nullptr,
                                          norm ? detail::f(rstd_q) : nullptr, norm ? detail::f(rstd_k) : nullptr, detail::f(table), B, T, H,
                                          Hk, D, eps, nullptr));
    Tensor out = Tensor::empty({B, T, HD}, DType::kFloat32, dev);
    Tensor lse = Tensor::empty({B, H, T}, DType::kFloat32, dev);
    detail::ctdk_ok(ctdk_attn_fwd(detail::f(qkv), detail::f(out), detail::f(lse), B, T, H, Hk, D, nullptr));

    std::vector<Tensor> inputs{x, wq, wk, wv};
    if (norm) {
      inputs.push_back(q_norm.weight);
      inputs.push_back(k_norm.weight);
    }
    Tensor sx = x.detach(), swq = wq.detach(), swk = wk.detach(), swv = wv.detach(), sout = out.detach();
    autograd::detail::record(out, inputs, "FusedAttentionBackward", [=](const detail::Grads& g) {
      const Tensor& dout = g.at(0);
      Tensor dqkv = Tensor::empty({rows, QN}, DType::kFloat32, dev);
      Tensor delta = Tensor::empty({B, H, T}, DType::kFloat32, dev);
      detail::ctdk_ok(ctdk_attn_bwd(detail::f(qkv), detail::f(sout), detail::f(dout), detail::f(lse), detail::f(delta), detail::f(dqkv), B, T,
                                    H, Hk, D, nullptr));
      Tensor dwqn, dwkn, scratch;
      if (norm) {
        dwqn = Tensor::empty({D}, DType::kFloat32, dev);
        dwkn = Tensor::empty({D}, DType::kFloat32, dev);
        scratch = Tensor::empty({ctdk_qk_norm_rope_bwd_scratch_floats(D)}, DType::kFloat32, dev);
      }
      detail::ctdk_ok(ctdk_qk_norm_rope_bwd(detail::f(dqkv), detail::f(qkv_pre), norm ? detail::f(wqn) : nullptr, norm ? detail::f(wkn) : nullptr,
                                            norm ? detail::f(rstd_q) : nullptr, norm ? detail::f(rstd_k) : nullptr,
                                            norm ? detail::f(dwqn) : nullptr, norm ? detail::f(dwkn) : nullptr,
                                            norm ? detail::f(scratch) : nullptr, detail::f(table), B, T, H, Hk, D, 0, nullptr));
      // dx = dq Wq + dk Wk + dv Wv;  dW = d(slice)^T x
      Tensor dx = Tensor::empty(sx.shape(), DType::kFloat32, dev);
      StoragePtr wgrad = make_storage(static_cast<size_t>(QN * hid) * 4, cuda_allocator());
      Tensor dwq = Tensor::view_of(wgrad, 0, {HD, hid}, DType::kFloat32), dwk = Tensor::view_of(wgrad, HD * hid, {KD, hid}, DType::kFloat32),
             dwv = Tensor::view_of(wgrad, (HD + KD) * hid, {KD, hid}, DType::kFloat32);
      const float* dq = detail::f(dqkv);
      if (stacked) {
        detail::gemm(dq, detail::f(swq), detail::f(dx), rows, hid, QN, QN, hid, hid, 0, 0);
      } else {
        detail::gemm(dq, detail::f(swq), detail::f(dx), rows, hid, HD, QN, hid, hid, 0, 0);
        detail::gemm(dq + HD, detail::f(swk), detail::f(dx), rows, hid, KD, QN, hid, hid, 0, 0, CTDK_EPI_ACCUMULATE);
        detail::gemm(dq + HD + KD, detail::f(swv), detail::f(dx), rows, hid, KD, QN, hid, hid, 0, 0, CTDK_EPI_ACCUMULATE);
      }
      detail::gemm(dq, detail::f(sx), detail::f(dwq), QN, hid, rows, QN, hid, hid, 1, 0);   // the three dW stacked: one GEMM
      detail::Grads r{dx, dwq, dwk, dwv};
      if (norm) {
        r.push_back(dwqn);
        r.push_back(dwkn);
      }
      return r;
    });
    return out;
  }
};

// ---- transformer_block.h ----------------------------------------------------------------------
struct TransformerBlock {
  RMSNorm input_layernorm;
  RMSNorm post_attention_layernorm;
  Attention self_attn;
  MLP mlp;

  // h = x + attn(norm(x));  y = h + mlp(norm(h))
  Tensor forward(const Tensor& x, KVLayer* kv = nullptr, int position_start = 0) const {
    Tensor h = ops::add(x, self_attn.forward(input_layernorm.forward(x), kv, position_start));
    return ops::add(h, mlp.forward(post_attention_layernorm.forward(h)));
  }
  Tensor forward_train(const Tensor& x) const {
    Tensor h = ops::add(x, self_attn.forward_train(input_layernorm.forward(x)));
    return ops::add(h, mlp.forward(post_attention_layernorm.forward(h)));
  }
};

// ---- model.h --------------------------------------------------------------------------------
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
  float rope_scaling_factor = 0.0f;   // LLaMA 3 RoPE scaling; 0 = off
  float rope_scaling_low_freq_factor = 1.0f;
  float rope_scaling_high_freq_factor = 4.0f;
  int rope_scaling_original_max_pos = 8192;
};

namespace detail {
constexpr LlamaConfig preset(int vocab, int hid, int inter, int layers, int heads, int kv_heads, int head_dim, int max_pos, float eps,
                             float theta, bool qk_norm, float rope_factor) {
  LlamaConfig c{};
  c.vocab_size = vocab;
  c.hidden_size = hid;
  c.intermediate_size = inter;
  c.num_hidden_layers = layers;
  c.num_attention_heads = heads;
  c.num_key_value_heads = kv_heads;
  c.head_dim = head_dim;
  c.max_position_embeddings = max_pos;
  c.rms_norm_eps = eps;
  c.rope_theta = theta;
  c.tie_word_embeddings = true;
  c.qk_norm = qk_norm;
  c.rope_scaling_factor = rope_factor;
  c.rope_scaling_low_freq_factor = 1.0f;
  c.rope_scaling_high_freq_factor = 4.0f;
  c.rope_scaling_original_max_pos = 8192;
  return c;
}
}  // namespace detail

// The five architectures of include/ctd/nn/model.h:39-124.
constexpr LlamaConfig smollm2_135m_config() { return detail::preset(49152, 576, 1536, 30, 9, 3, 64, 8192, 1e-5f, 100000.0f, false, 0.0f); }
constexpr LlamaConfig smollm2_360m_config() { return detail::preset(49152, 960, 2560, 32, 15, 5, 64, 8192, 1e-5f, 100000.0f, false, 0.0f); }
constexpr LlamaConfig qwen3_0_6b_config() { return detail::preset(151936, 1024, 3072, 28, 16, 8, 128, 40960, 1e-6f, 1000000.0f, true, 0.0f); }
constexpr LlamaConfig qwen3_1_7b_config() { return detail::preset(151936, 2048, 6144, 28, 16, 8, 128, 40960, 1e-6f, 1000000.0f, true, 0.0f); }
constexpr LlamaConfig llama3_2_1b_config() { return detail::preset(128256, 2048, 8192, 16, 32, 8, 64, 131072, 1e-5f, 500000.0f, false, 32.0f); }

// Architecture from the shape of model.embed_tokens.weight.
inline LlamaConfig autodetect_config(const TensorDict& w) {
  auto it = w.find("model.embed_tokens.weight");
  if (it == w.end()) throw std::runtime_error("autodetect_config: missing model.embed_tokens.weight");
  const int64_t vocab = it->second.shape().at(0), hidden = it->second.shape().at(1);
  if (hidden == 576) return smollm2_135m_config();
  if (hidden == 960) return smollm2_360m_config();
  if (hidden == 1024 && vocab == 151936) return qwen3_0_6b_config();
  if (hidden == 2048 && vocab == 151936) return qwen3_1_7b_config();
  if (hidden == 2048 && vocab == 128256) return llama3_2_1b_config();
  throw std::runtime_error("autodetect_config: unsupported hidden_size=" + std::to_string(hidden) + " vocab_size=" + std::to_string(vocab));
}
inline LlamaConfig autodetect_smollm2_config(const TensorDict& w) { return autodetect_config(w); }

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

// What a built model owns besides its layer objects: the two arenas (parameters in
// collect_parameters order, gradients in the same layout) and the step engine over them.
struct FusedState {
  ctdk_model_config kcfg{};
  StoragePtr params, grads, workspace, scalars;
  std::vector<int64_t> offsets, numels;
  std::vector<std::vector<int64_t>> shapes;
  std::vector<std::shared_ptr<autograd::AutogradMeta>> metas;   // of the parameter tensors, once collected
  int64_t total = 0;
  void* engine = nullptr;
  int64_t eng_B = 0, eng_T = 0;
  ~FusedState() {
    if (engine != nullptr) ctdk_engine_destroy(engine);
  }
  float* sums() { return static_cast<float*>(scalars->data()); }
  // (Re)creates the engine when the batch outgrows its workspace or checkpointing was switched.
  void ensure_engine(int64_t B, int64_t T, bool ckpt) {
    if (engine != nullptr && B <= eng_B && T <= eng_T && (kcfg.gradient_checkpointing != 0) == ckpt) return;
    if (engine != nullptr) {
      CTD_CUDA_CHECK(cudaDeviceSynchronize());
      ctdk_engine_destroy(engine);
      engine = nullptr;
      workspace.reset();
    }
    kcfg.gradient_checkpointing = ckpt ? 1 : 0;
    const int64_t nb = B > eng_B ? B : eng_B, nt = T > eng_T ? T : eng_T;
    const int64_t bytes = ctdk_engine_workspace_bytes(&kcfg, nb, nt);
    if (bytes < 0) throw std::runtime_error(ctdk_last_error());
    workspace = make_storage(static_cast<size_t>(bytes), cuda_allocator());
    ctdk_ok(ctdk_engine_create(&kcfg, static_cast<float*>(params->data()), static_cast<float*>(grads->data()), workspace->data(), bytes, nb,
                               nt, &engine));
    eng_B = nb;
    eng_T = nt;
  }
};

}  // namespace detail

struct Model {
  LlamaConfig config{};
  Embedding embed_tokens;
  std::vector<TransformerBlock> layers;
  RMSNorm norm;
  bool gradient_checkpointing = false;

  // input_ids int64 [B, T] -> logits fp32 [B, T, vocab]. With a cache the new positions are
  // appended at position_start.
  Tensor forward(const Tensor& input_ids, KVCache* cache = nullptr, int position_start = 0) const {
    Tensor h = embed_tokens.forward(input_ids);
    for (size_t i = 0; i < layers.size(); ++i) h = layers[i].forward(h, cache ? &cache->layers[i] : nullptr, position_start);
    if (cache) cache->current_len = position_start + input_ids.shape()[input_ids.dim() - 1];
    return Linear{embed_tokens.weight}.forward(norm.forward(h));   // tied LM head
  }

  Tensor forward_train_logits(const Tensor& input_ids) const {
    Tensor h = embed_tokens.forward(input_ids);
    for (const TransformerBlock& layer : layers)
      h = gradient_checkpointing ? autograd::checkpoint([&layer](const Tensor& x) { return layer.forward_train(x); }, h) : layer.forward_train(h);
    return Linear{embed_tokens.weight}.forward(norm.forward(h));
  }

  // Mean cross-entropy over all positions, shape [1].
  Tensor forward_train(const Tensor& input_ids, const Tensor& targets) const {
    if (fused) {
      std::vector<float> ones(static_cast<size_t>(input_ids.numel()), 1.0f);
      return fused_loss(input_ids, targets, Tensor::from_host(ones.data(), input_ids.shape(), DType::kFloat32, input_ids.device()), false);
    }
    const int64_t n = input_ids.numel();
    Tensor logits = forward_train_logits(input_ids);
    return ops::cross_entropy(logits.reshape({n, logits.shape().back()}), targets.reshape({n}));
  }

  // SFT loss: loss_mask fp32 [B, T], 1 at supervised positions; sum(mask * nll) / sum(mask).
  Tensor forward_train_masked(const Tensor& input_ids, const Tensor& targets, const Tensor& loss_mask) const {
    if (fused) return fused_loss(input_ids, targets, loss_mask, true);
    const int64_t n = input_ids.numel();
    Tensor logits = forward_train_logits(input_ids);
    return ops::cross_entropy_masked(logits.reshape({n, logits.shape().back()}), targets.reshape({n}), loss_mask.reshape({n}));
  }

  struct NamedParameters {
    std::vector<std::pair<std::string, Tensor>> all;
    std::vector<Tensor> decay;
    std::vector<Tensor> no_decay;
    std::vector<std::string> decay_names;
    std::vector<std::string> no_decay_names;
  };

  // Every parameter once (the tied LM head is the embedding), marked as requiring a gradient;
  // decay = embedding and linear weights, no_decay = every norm weight.
  NamedParameters collect_parameters() {
    NamedParameters out;
    auto add = [&](const std::string& name, Tensor& t, bool decay) {
      t.requires_grad_(true);
      out.all.emplace_back(name, t);
      (decay ? out.decay : out.no_decay).push_back(t);
      (decay ? out.decay_names : out.no_decay_names).push_back(name);
    };
    add("model.embed_tokens.weight", embed_tokens.weight, true);
    for (size_t i = 0; i < layers.size(); ++i) {
      const std::string p = "model.layers." + std::to_string(i) + ".";
      TransformerBlock& b = layers[i];
      add(p + "input_layernorm.weight", b.input_layernorm.weight, false);
      add(p + "self_attn.q_proj.weight", b.self_attn.q_proj.weight, true);
      add(p + "self_attn.k_proj.weight", b.self_attn.k_proj.weight, true);
      add(p + "self_attn.v_proj.weight", b.self_attn.v_proj.weight, true);
      add(p + "self_attn.o_proj.weight", b.self_attn.o_proj.weight, true);
      if (b.self_attn.has_qk_norm()) {
        add(p + "self_attn.q_norm.weight", b.self_attn.q_norm.weight, false);
        add(p + "self_attn.k_norm.weight", b.self_attn.k_norm.weight, false);
      }
      add(p + "post_attention_layernorm.weight", b.post_attention_layernorm.weight, false);
      add(p + "mlp.gate_proj.weight", b.mlp.gate_proj.weight, true);
      add(p + "mlp.up_proj.weight", b.mlp.up_proj.weight, true);
      add(p + "mlp.down_proj.weight", b.mlp.down_proj.weight, true);
    }
    add("model.norm.weight", norm.weight, false);
    if (fused) {
      fused->metas.clear();
      for (auto& kv : out.all) fused->metas.push_back(kv.second.autograd_meta());
    }
    return out;
  }

  // Set by build_model (copies of a Model share it). A model assembled by hand from layer objects
  // has none and trains through the per-layer tape nodes.
  std::shared_ptr<detail::FusedState> fused;

 private:
  // The loss as a deferred [1] tensor: reading it runs the forward pass alone; backward() runs ONE
  // fused forward + backward pass of the step engine with the incoming gradient folded into the
  // per-row weights, and leaves the loss value behind as well. Gradients accumulate over calls
  // until the parameters' zero_grad_() (the optimizer's zero_grad()), as AccumulateGrad would.
  Tensor fused_loss(const Tensor& input_ids, const Tensor& targets, const Tensor& loss_mask, bool masked) const {
    using ::ctd::detail::require;
    require(input_ids.dim() == 2 && input_ids.dtype() == DType::kInt64 && input_ids.device().is_cuda(),
            "forward_train: input_ids must be int64 [B, T] on CUDA");
    require(targets.dtype() == DType::kInt64 && targets.numel() == input_ids.numel() && targets.device().is_cuda(),
            "forward_train: targets must be int64 with input_ids' element count, on CUDA");
    require(loss_mask.dtype() == DType::kFloat32 && loss_mask.numel() == input_ids.numel() && loss_mask.device().is_cuda(),
            "forward_train_masked: loss_mask must be fp32 with input_ids' element count, on CUDA");
    const int64_t B = input_ids.shape()[0], T = input_ids.shape()[1];
    std::shared_ptr<detail::FusedState> st = fused;
    const bool ckpt = gradient_checkpointing;
    Tensor loss = Tensor::empty({1}, DType::kFloat32, input_ids.device());
    float* loss_ptr = static_cast<float*>(loss.storage()->data());
    StoragePtr loss_keep = loss.storage();
    auto deferred = std::make_shared<::ctd::detail::Deferred>();
    deferred->compute = [st, ckpt, input_ids, targets, loss_mask, B, T, loss_ptr, loss_keep]() {
      st->ensure_engine(B, T, ckpt);
      CTD_CUDA_CHECK(cudaMemsetAsync(st->sums(), 0, 2 * sizeof(float), nullptr));
      detail::ctdk_ok(ctdk_engine_forward_loss(st->engine, ops::detail::i64(input_ids), ops::detail::i64(targets), detail::f(loss_mask), B, T,
                                               st->sums(), nullptr));
      detail::ctdk_ok(ctdk_loss_ratio(st->sums(), loss_ptr, nullptr));
    };
    loss.set_deferred(deferred);
    if (!autograd::is_grad_enabled()) return loss;
    std::weak_ptr<::ctd::detail::Deferred> value = deferred;
    auto node = std::make_shared<autograd::detail::FnNode>(
        "FusedModelBackward", [st, ckpt, input_ids, targets, loss_mask, B, T, loss_ptr, loss_keep, value, masked](const detail::Grads& g) {
          const int64_t n = B * T;
          const Device dev = input_ids.device();
          // row weight = mask * dy / sum(mask): the factor of CrossEntropy(Masked)Backward
          Tensor msum = Tensor::zeros({1}, DType::kFloat32, dev);
          detail::ctdk_ok(ctdk_sumsq(detail::f(loss_mask), n, detail::f(msum), nullptr));   // 0 / 1 values: sum of squares = sum
          float h = 0.0f;
          msum.copy_to_host(&h);
          if (h <= 0.0f) throw std::runtime_error(std::string(masked ? "cross_entropy_masked" : "cross_entropy") + " backward: sum(loss_mask) == 0");
          Tensor w = Tensor::empty({n}, DType::kFloat32, dev);
          detail::ctdk_ok(ctdk_ce_row_weight(detail::f(loss_mask), detail::f(g.at(0)), detail::f(msum), n, detail::f(w), nullptr));
          st->ensure_engine(B, T, ckpt);
          const bool accumulate = !st->metas.empty() && st->metas.front() && st->metas.front()->grad.storage() != nullptr;
          CTD_CUDA_CHECK(cudaMemsetAsync(st->sums(), 0, 2 * sizeof(float), nullptr));
          detail::ctdk_ok(ctdk_engine_forward_backward(st->engine, ops::detail::i64(input_ids), ops::detail::i64(targets), detail::f(loss_mask),
                                                       detail::f(w), B, T, accumulate ? 1 : 0, st->sums(), nullptr));
          detail::ctdk_ok(ctdk_loss_ratio(st->sums(), loss_ptr, nullptr));
          if (auto d = value.lock()) d->done = true;   // the loss value is in place: no separate forward pass
          if (!accumulate)
            for (size_t i = 0; i < st->metas.size(); ++i)
              if (st->metas[i]) st->metas[i]->grad = Tensor::view_of(st->grads, st->offsets[i], st->shapes[i], DType::kFloat32);
          return detail::Grads{};
        });
    autograd::set_history(loss, std::move(node));
    return loss;
  }
};

// Lays the named fp32 tensors of `w` out in one parameter arena (Model::collect_parameters order,
// each tensor on a 256-byte boundary, q/k/v and gate/up adjacent) and builds the layer objects as
// views of it. A missing weight throws; q_norm / k_norm are optional (Qwen3).
inline Model build_model(const TensorDict& w, const LlamaConfig& cfg) {
  auto must = [&](const std::string& key) -> const Tensor& {
    auto it = w.find(key);
    if (it == w.end()) throw std::runtime_error("build_model: missing weight '" + key + "'");
    return it->second;
  };
  Model m;
  m.config = cfg;
  const bool has_norms = w.find("model.layers.0.self_attn.q_norm.weight") != w.end();
  auto st = std::make_shared<detail::FusedState>();
  st->kcfg = detail::to_ctdk(cfg, false);
  st->kcfg.qk_norm = has_norms ? 1 : 0;
  // A shape the step engine does not take (head size other than 64 / 128, untied output embedding,
  // sizes that break its alignment rules) is built from the given tensors as they are and trains
  // through the per-layer tape nodes.
  const int64_t n = cfg.tie_word_embeddings ? ctdk_model_num_tensors(&st->kcfg) : -1;
  const bool arena = n > 0;
  if (arena) {
    st->offsets.resize(static_cast<size_t>(n));
    st->numels.resize(static_cast<size_t>(n));
    std::vector<int> decay(static_cast<size_t>(n));
    detail::ctdk_ok(ctdk_model_layout(&st->kcfg, st->offsets.data(), st->numels.data(), decay.data(), &st->total));
    st->params = make_storage(static_cast<size_t>(st->total) * 4, cuda_allocator());
    st->grads = make_storage(static_cast<size_t>(st->total) * 4, cuda_allocator());
    st->scalars = make_storage(64, cuda_allocator());
    CTD_CUDA_CHECK(cudaMemsetAsync(st->params->data(), 0, static_cast<size_t>(st->total) * 4, nullptr));
    CTD_CUDA_CHECK(cudaMemsetAsync(st->grads->data(), 0, static_cast<size_t>(st->total) * 4, nullptr));
  }
  size_t next = 0;
  // copies one named tensor into its arena slot and returns the view
  auto place = [&](const std::string& key) -> Tensor {
    const Tensor& src = must(key);
    if (!arena) return src;
    if (next >= st->offsets.size()) throw std::runtime_error("build_model: more tensors than the layout holds");
    if (src.dtype() != DType::kFloat32 || src.numel() != st->numels[next])
      throw std::runtime_error("build_model: weight '" + key + "' has the wrong type or size");
    Tensor view = Tensor::view_of(st->params, st->offsets[next], src.shape(), DType::kFloat32);
    CTD_CUDA_CHECK(cudaMemcpy(view.data_ptr(), src.data_ptr(), src.nbytes(), src.device().is_cuda() ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
    st->shapes.push_back(src.shape());
    ++next;
    return view;
  };
  m.embed_tokens = Embedding{place("model.embed_tokens.weight")};
  m.layers.reserve(static_cast<size_t>(cfg.num_hidden_layers));
  for (int i = 0; i < cfg.num_hidden_layers; ++i) {
    const std::string p = "model.layers." + std::to_string(i) + ".";
    TransformerBlock b;
    b.input_layernorm = RMSNorm{place(p + "input_layernorm.weight"), cfg.rms_norm_eps};
    Attention& a = b.self_attn;
    a.q_proj = Linear{place(p + "self_attn.q_proj.weight")};
    a.k_proj = Linear{place(p + "self_attn.k_proj.weight")};
    a.v_proj = Linear{place(p + "self_attn.v_proj.weight")};
    a.o_proj = Linear{place(p + "self_attn.o_proj.weight")};
    a.num_heads = cfg.num_attention_heads;
    a.num_kv_heads = cfg.num_key_value_heads;
    a.head_dim = cfg.head_dim;
    a.rope_theta = cfg.rope_theta;
    a.rope_scaling = ops::RopeScaling{cfg.rope_scaling_factor, cfg.rope_scaling_low_freq_factor, cfg.rope_scaling_high_freq_factor,
                                      cfg.rope_scaling_original_max_pos};
    if (has_norms) {
      a.q_norm = RMSNorm{place(p + "self_attn.q_norm.weight"), cfg.rms_norm_eps};
      a.k_norm = RMSNorm{place(p + "self_attn.k_norm.weight"), cfg.rms_norm_eps};
    } else {
      a.q_norm = RMSNorm{Tensor{}, cfg.rms_norm_eps};
      a.k_norm = RMSNorm{Tensor{}, cfg.rms_norm_eps};
    }
    b.post_attention_layernorm = RMSNorm{place(p + "post_attention_layernorm.weight"), cfg.rms_norm_eps};
    b.mlp.gate_proj = Linear{place(p + "mlp.gate_proj.weight")};
    b.mlp.up_proj = Linear{place(p + "mlp.up_proj.weight")};
    b.mlp.down_proj = Linear{place(p + "mlp.down_proj.weight")};
    m.layers.push_back(std::move(b));
  }
  m.norm = RMSNorm{place("model.norm.weight"), cfg.rms_norm_eps};
  if (arena) m.fused = std::move(st);
  return m;
}

}  // namespace nn
}  // namespace ctd
