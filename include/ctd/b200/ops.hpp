// ctd::ops — the reference's per-op API (emberlm include/ctd/ops/*.h) on the ctdk kernels.
// `*_impl` functions compute; the un-suffixed functions also record the op on the autograd tape
// (core.hpp) when an input requires a gradient. Preconditions throw std::runtime_error as the
// reference's do. Everything runs on the legacy default stream.
#pragma once

#include <cfloat>
#include <cmath>

#include "core.hpp"

namespace ctd::ops {

namespace detail {
using ::ctd::detail::ctdk_ok;
using ::ctd::detail::require;
using ::ctd::autograd::detail::record;

inline const float* f(const Tensor& t) { return static_cast<const float*>(t.data_ptr()); }
inline float* f(Tensor& t) { return static_cast<float*>(t.data_ptr()); }
inline const int64_t* i64(const Tensor& t) { return static_cast<const int64_t*>(t.data_ptr()); }
inline void need_f32_cuda(const Tensor& t, const char* op) {
  if (t.dtype() != DType::kFloat32 || !t.device().is_cuda() || !t.is_contiguous())
    throw std::runtime_error(std::string(op) + ": only fp32 / contiguous / CUDA supported");
}
inline void same_shape(const Tensor& a, const Tensor& b, const char* op) {
  if (a.shape() != b.shape()) throw std::runtime_error(std::string(op) + ": shape mismatch");
}
inline Tensor like(const Tensor& x) { return Tensor::empty(x.shape(), DType::kFloat32, x.device()); }
using Grads = std::vector<Tensor>;
}  // namespace detail

// ---- elementwise.h --------------------------------------------------------------------------
inline Tensor add_impl(const Tensor& a, const Tensor& b) {
  detail::need_f32_cuda(a, "add");
  detail::need_f32_cuda(b, "add");
  detail::same_shape(a, b, "add");
  Tensor out = detail::like(a);
  detail::ctdk_ok(ctdk_add(detail::f(a), detail::f(b), detail::f(out), a.numel(), nullptr));
  return out;
}
inline Tensor sub_impl(const Tensor& a, const Tensor& b) {
  detail::need_f32_cuda(a, "sub");
  detail::need_f32_cuda(b, "sub");
  detail::same_shape(a, b, "sub");
  Tensor out = detail::like(a);
  detail::ctdk_ok(ctdk_sub(detail::f(a), detail::f(b), detail::f(out), a.numel(), nullptr));
  return out;
}
inline Tensor mul_impl(const Tensor& a, const Tensor& b) {
  detail::need_f32_cuda(a, "mul");
  detail::need_f32_cuda(b, "mul");
  detail::same_shape(a, b, "mul");
  Tensor out = detail::like(a);
  detail::ctdk_ok(ctdk_mul(detail::f(a), detail::f(b), detail::f(out), a.numel(), nullptr));
  return out;
}
inline Tensor scale_impl(const Tensor& x, float alpha) {
  detail::need_f32_cuda(x, "scale");
  Tensor out = detail::like(x);
  detail::ctdk_ok(ctdk_scale(detail::f(x), alpha, detail::f(out), x.numel(), nullptr));
  return out;
}
inline Tensor silu_impl(const Tensor& x) {
  detail::need_f32_cuda(x, "silu");
  Tensor out = detail::like(x);
  detail::ctdk_ok(ctdk_silu(detail::f(x), detail::f(out), x.numel(), nullptr));
  return out;
}
inline Tensor silu_backward_impl(const Tensor& x, const Tensor& g) {
  detail::need_f32_cuda(x, "silu_backward");
  detail::need_f32_cuda(g, "silu_backward");
  detail::same_shape(x, g, "silu_backward");
  Tensor out = detail::like(x);
  detail::ctdk_ok(ctdk_silu_bwd(detail::f(x), detail::f(g), detail::f(out), x.numel(), nullptr));
  return out;
}
inline Tensor add(const Tensor& a, const Tensor& b) {
  Tensor out = add_impl(a, b);
  detail::record(out, {a, b}, "AddBackward", [](const detail::Grads& g) { return detail::Grads{g.at(0), g.at(0)}; });
  return out;
}
inline Tensor mul(const Tensor& a, const Tensor& b) {
  Tensor out = mul_impl(a, b);
  Tensor sa = a.detach(), sb = b.detach();
  detail::record(out, {a, b}, "MulBackward",
                 [sa, sb](const detail::Grads& g) { return detail::Grads{mul_impl(g.at(0), sb), mul_impl(g.at(0), sa)}; });
  return out;
}
inline Tensor silu(const Tensor& x) {
  Tensor out = silu_impl(x);
  Tensor sx = x.detach();
  detail::record(out, {x}, "SiluBackward", [sx](const detail::Grads& g) { return detail::Grads{silu_backward_impl(sx, g.at(0))}; });
  return out;
}

// ---- repeat_kv.h ----------------------------------------------------------------------------
inline Tensor mul_scalar_impl(const Tensor& x, float c) { return scale_impl(x, c); }
inline Tensor mul_scalar(const Tensor& x, float c) {
  Tensor out;
  if (x.deferred() && !x.deferred()->done) {
    // A loss whose fused model pass has not run yet: the product is deferred too, so that
    // backward() still finds one fused forward + backward pass to run.
    out = detail::like(x);
    auto d = std::make_shared<::ctd::detail::Deferred>();
    Tensor src = x, dst = out;   // handles onto the same storages (dst without the hook)
    d->compute = [src, dst, c]() mutable {
      detail::ctdk_ok(ctdk_scale(detail::f(src), c, static_cast<float*>(dst.storage()->data()), src.numel(), nullptr));
    };
    out.set_deferred(std::move(d));
  } else {
    out = mul_scalar_impl(x, c);
  }
  detail::record(out, {x}, "MulScalarBackward", [c](const detail::Grads& g) { return detail::Grads{scale_impl(g.at(0), c)}; });
  return out;
}
inline Tensor repeat_kv_heads_impl(const Tensor& x, int group) {
  detail::need_f32_cuda(x, "repeat_kv_heads");
  detail::require(x.dim() == 4, "repeat_kv_heads: expected [B, T, H_kv, D]");
  detail::require(group > 0, "repeat_kv_heads: group must be > 0");
  const int64_t B = x.shape()[0], T = x.shape()[1], Hk = x.shape()[2], D = x.shape()[3];
  Tensor out = Tensor::empty({B, T, Hk * group, D}, DType::kFloat32, x.device());
  detail::ctdk_ok(ctdk_repeat_kv(detail::f(x), detail::f(out), B * T, static_cast<int>(Hk), static_cast<int>(D), group, nullptr));
  return out;
}
inline Tensor repeat_kv_sum_impl(const Tensor& y, int group) {
  detail::need_f32_cuda(y, "repeat_kv_sum");
  detail::require(y.dim() == 4 && group > 0 && y.shape()[2] % group == 0, "repeat_kv_sum: expected [B, T, H_kv*group, D]");
  const int64_t B = y.shape()[0], T = y.shape()[1], Hk = y.shape()[2] / group, D = y.shape()[3];
  Tensor out = Tensor::empty({B, T, Hk, D}, DType::kFloat32, y.device());
  detail::ctdk_ok(ctdk_repeat_kv_sum(detail::f(y), detail::f(out), B * T, static_cast<int>(Hk), static_cast<int>(D), group, nullptr));
  return out;
}
inline Tensor repeat_kv_heads(const Tensor& x, int group) {
  Tensor out = repeat_kv_heads_impl(x, group);
  detail::record(out, {x}, "RepeatKvBackward", [group](const detail::Grads& g) { return detail::Grads{repeat_kv_sum_impl(g.at(0), group)}; });
  return out;
}

// ---- matmul.h (semantics src/ops/matmul.cpp:13-118) -------------------------------------------
inline Tensor matmul_impl(const Tensor& a, const Tensor& b, bool transa, bool transb) {
  detail::need_f32_cuda(a, "matmul");
  detail::need_f32_cuda(b, "matmul");
  detail::require(a.dim() == 2 && b.dim() == 2, "matmul: expected 2D tensors");
  const int64_t M = transa ? a.shape()[1] : a.shape()[0], K = transa ? a.shape()[0] : a.shape()[1];
  const int64_t Kb = transb ? b.shape()[1] : b.shape()[0], N = transb ? b.shape()[0] : b.shape()[1];
  detail::require(K == Kb, "matmul: inner dims disagree");
  Tensor out = Tensor::empty({M, N}, DType::kFloat32, a.device());
  detail::ctdk_ok(ctdk_gemm(detail::f(a), detail::f(b), detail::f(out), M, N, K, a.shape()[1], b.shape()[1], N, transa ? 1 : 0,
                            transb ? 1 : 0, ::ctd::detail::matmul_precision(), CTDK_EPI_STORE, nullptr, nullptr));
  return out;
}
inline Tensor bmm_impl(const Tensor& a, const Tensor& b, bool transa, bool transb) {
  detail::need_f32_cuda(a, "bmm");
  detail::need_f32_cuda(b, "bmm");
  detail::require(a.dim() == 3 && b.dim() == 3 && a.shape()[0] == b.shape()[0], "bmm: expected 3D tensors with equal batch");
  const int64_t Bt = a.shape()[0];
  const int64_t M = transa ? a.shape()[2] : a.shape()[1], K = transa ? a.shape()[1] : a.shape()[2];
  const int64_t Kb = transb ? b.shape()[2] : b.shape()[1], N = transb ? b.shape()[1] : b.shape()[2];
  detail::require(K == Kb, "bmm: inner dims disagree");
  Tensor out = Tensor::empty({Bt, M, N}, DType::kFloat32, a.device());
  detail::ctdk_ok(ctdk_bmm(detail::f(a), detail::f(b), detail::f(out), Bt, M, N, K, transa ? 1 : 0, transb ? 1 : 0, ::ctd::detail::matmul_precision(),
                           nullptr));
  return out;
}
namespace detail {
// Gradients of C = op(A) op(B) for a product function mm(a, b, ta, tb):
//   dA = g op(B)^T (or its transpose when A is stored transposed), dB likewise.
template <typename MM>
inline Grads product_backward(const Tensor& g, const Tensor& a, const Tensor& b, bool ta, bool tb, MM mm) {
  Tensor da = ta ? mm(b, g, tb, true) : mm(g, b, false, !tb);
  Tensor db = tb ? mm(g, a, true, ta) : mm(a, g, !ta, false);
  return Grads{da, db};
}
}  // namespace detail
inline Tensor matmul(const Tensor& a, const Tensor& b, bool transa = false, bool transb = false) {
  Tensor out = matmul_impl(a, b, transa, transb);
  Tensor sa = a.detach(), sb = b.detach();
  detail::record(out, {a, b}, "MatmulBackward", [sa, sb, transa, transb](const detail::Grads& g) {
    return detail::product_backward(g.at(0), sa, sb, transa, transb, matmul_impl);
  });
  return out;
}
inline Tensor bmm(const Tensor& a, const Tensor& b, bool transa = false, bool transb = false) {
  Tensor out = bmm_impl(a, b, transa, transb);
  Tensor sa = a.detach(), sb = b.detach();
  detail::record(out, {a, b}, "BmmBackward", [sa, sb, transa, transb](const detail::Grads& g) {
    return detail::product_backward(g.at(0), sa, sb, transa, transb, bmm_impl);
  });
  return out;
}

// ---- norm.h ---------------------------------------------------------------------------------
inline Tensor rms_norm_impl(const Tensor& x, const Tensor& weight, float eps) {
  detail::need_f32_cuda(x, "rms_norm");
  detail::need_f32_cuda(weight, "rms_norm");
  detail::require(x.dim() >= 1 && weight.dim() == 1 && weight.shape()[0] == x.shape().back(), "rms_norm: weight must be [H]");
  const int H = static_cast<int>(x.shape().back());
  Tensor y = detail::like(x);
  detail::ctdk_ok(ctdk_rmsnorm_fwd(detail::f(x), detail::f(weight), detail::f(y), nullptr, x.numel() / H, H, eps, nullptr));
  return y;
}
inline std::pair<Tensor, Tensor> rms_norm_backward_impl(const Tensor& dy, const Tensor& x, const Tensor& weight, float eps) {
  detail::need_f32_cuda(dy, "rms_norm_backward");
  detail::need_f32_cuda(x, "rms_norm_backward");
  detail::same_shape(dy, x, "rms_norm_backward");
  const int H = static_cast<int>(x.shape().back());
  detail::require(weight.dim() == 1 && weight.shape()[0] == H, "rms_norm_backward: weight must be [H]");
  Tensor dx = detail::like(x), dw = Tensor::empty({H}, DType::kFloat32, x.device());
  Tensor scratch = Tensor::empty({ctdk_rmsnorm_bwd_scratch_floats(H)}, DType::kFloat32, x.device());
  detail::ctdk_ok(ctdk_rmsnorm_bwd(detail::f(dy), detail::f(x), detail::f(weight), detail::f(dx), detail::f(dw), detail::f(scratch),
                                   x.numel() / H, H, eps, 0, 0, nullptr));
  return {dx, dw};
}
inline Tensor rms_norm(const Tensor& x, const Tensor& weight, float eps) {
  Tensor out = rms_norm_impl(x, weight, eps);
  Tensor sx = x.detach(), sw = weight.detach();
  detail::record(out, {x, weight}, "RmsNormBackward", [sx, sw, eps](const detail::Grads& g) {
    auto r = rms_norm_backward_impl(g.at(0), sx, sw, eps);
    return detail::Grads{r.first, r.second};
  });
  return out;
}

// ---- rope.h ---------------------------------------------------------------------------------
struct RopeScaling {
  float factor = 0.0f;   // <= 1: plain RoPE; 32 for LLaMA 3
  float low_freq_factor = 1.0f;
  float high_freq_factor = 4.0f;
  int original_max_pos = 8192;
  bool enabled() const { return factor > 1.0f; }
  float low_freq_wavelen() const { return static_cast<float>(original_max_pos) / low_freq_factor; }
  float high_freq_wavelen() const { return static_cast<float>(original_max_pos) / high_freq_factor; }
};
namespace detail {
inline void rope_call(const Tensor& x, Tensor& out, int position_start, float theta, const RopeScaling& sc, float sin_sign) {
  need_f32_cuda(x, "rope");
  require(x.dim() == 4, "rope: expected [B, T, H, D]");
  require(x.shape()[3] % 2 == 0, "rope: head_dim must be even");
  ctdk_rope_params p;
  p.theta = theta;
  p.scaling_factor = sc.enabled() ? sc.factor : 0.0f;
  p.low_freq_wavelen = sc.low_freq_wavelen();
  p.high_freq_wavelen = sc.high_freq_wavelen();
  const int H = static_cast<int>(x.shape()[2]), D = static_cast<int>(x.shape()[3]);
  ctdk_ok(ctdk_rope(f(x), f(out), x.shape()[0], x.shape()[1], H, D, static_cast<int64_t>(H) * D, position_start, &p, sin_sign, nullptr));
}
}  // namespace detail
inline void apply_rope_inplace(Tensor& x, int position_start, float theta, const RopeScaling& scaling = {}) {
  detail::rope_call(x, x, position_start, theta, scaling, 1.0f);
}
inline Tensor rope_impl(const Tensor& x, int position_start, float theta, const RopeScaling& scaling = {}) {
  Tensor out = detail::like(x);
  detail::rope_call(x, out, position_start, theta, scaling, 1.0f);
  return out;
}
inline Tensor rope_transpose_impl(const Tensor& x, int position_start, float theta, const RopeScaling& scaling = {}) {
  Tensor out = detail::like(x);
  detail::rope_call(x, out, position_start, theta, scaling, -1.0f);
  return out;
}
inline Tensor rope(const Tensor& x, int position_start, float theta, const RopeScaling& scaling = {}) {
  Tensor out = rope_impl(x, position_start, theta, scaling);
  detail::record(out, {x}, "RopeBackward", [position_start, theta, scaling](const detail::Grads& g) {
    return detail::Grads{rope_transpose_impl(g.at(0), position_start, theta, scaling)};
  });
  return out;
}

// ---- embedding.h ----------------------------------------------------------------------------
inline Tensor embedding_impl(const Tensor& ids, const Tensor& weight) {
  detail::need_f32_cuda(weight, "embedding");
  detail::require(ids.dtype() == DType::kInt64 && ids.device().is_cuda(), "embedding: ids must be int64 on CUDA");
  detail::require(weight.dim() == 2, "embedding: weight must be [V, H]");
  std::vector<int64_t> shape = ids.shape();
  shape.push_back(weight.shape()[1]);
  Tensor out = Tensor::empty(shape, DType::kFloat32, weight.device());
  detail::ctdk_ok(ctdk_embedding_fwd(detail::i64(ids), detail::f(weight), detail::f(out), ids.numel(), static_cast<int>(weight.shape()[1]),
                                     weight.shape()[0], nullptr));
  return out;
}
inline Tensor embedding_backward_impl(const Tensor& ids, const Tensor& dy, int64_t vocab) {
  detail::need_f32_cuda(dy, "embedding_backward");
  detail::require(ids.dtype() == DType::kInt64 && ids.device().is_cuda(), "embedding_backward: ids must be int64 on CUDA");
  const int H = static_cast<int>(dy.shape().back());
  Tensor dw = Tensor::zeros({vocab, H}, DType::kFloat32, dy.device());
  detail::ctdk_ok(ctdk_embedding_bwd(detail::i64(ids), detail::f(dy), detail::f(dw), ids.numel(), H, vocab, nullptr));
  return dw;
}
inline Tensor embedding(const Tensor& ids, const Tensor& weight) {
  Tensor out = embedding_impl(ids, weight);
  const int64_t vocab = weight.shape()[0];
  Tensor sid = ids;
  detail::record(out, {weight}, "EmbeddingBackward",
                 [sid, vocab](const detail::Grads& g) { return detail::Grads{embedding_backward_impl(sid, g.at(0), vocab)}; });
  return out;
}

// ---- softmax.h ------------------------------------------------------------------------------
inline Tensor softmax_impl(const Tensor& x) {
  detail::need_f32_cuda(x, "softmax");
  detail::require(x.dim() >= 1, "softmax: expected at least 1D");
  const int64_t W = x.shape().back();
  Tensor y = detail::like(x);
  if (x.numel() > 0) detail::ctdk_ok(ctdk_softmax_fwd(detail::f(x), detail::f(y), x.numel() / W, W, nullptr));
  return y;
}
inline Tensor softmax_backward_impl(const Tensor& y, const Tensor& g) {
  detail::need_f32_cuda(y, "softmax_backward");
  detail::need_f32_cuda(g, "softmax_backward");
  detail::same_shape(y, g, "softmax_backward");
  const int64_t W = y.shape().back();
  Tensor dx = detail::like(y);
  if (y.numel() > 0) detail::ctdk_ok(ctdk_softmax_bwd(detail::f(y), detail::f(g), detail::f(dx), y.numel() / W, W, nullptr));
  return dx;
}
inline Tensor softmax(const Tensor& x) {
  Tensor out = softmax_impl(x);
  Tensor sy = out.detach();
  detail::record(out, {x}, "SoftmaxBackward", [sy](const detail::Grads& g) { return detail::Grads{softmax_backward_impl(sy, g.at(0))}; });
  return out;
}

// ---- permute.h ------------------------------------------------------------------------------
inline Tensor permute_impl(const Tensor& x, const std::vector<int>& perm) {
  detail::need_f32_cuda(x, "permute");
  detail::require(static_cast<int64_t>(perm.size()) == x.dim(), "permute: perm size must match tensor rank");
  detail::require(x.dim() >= 1 && x.dim() <= 6, "permute: 1 to 6 dimensions supported");
  std::vector<int64_t> out_shape(perm.size());
  std::vector<bool> seen(perm.size(), false);
  for (size_t i = 0; i < perm.size(); ++i) {
    detail::require(perm[i] >= 0 && perm[i] < static_cast<int>(perm.size()) && !seen[perm[i]], "permute: invalid permutation");
    seen[perm[i]] = true;
    out_shape[i] = x.shape()[perm[i]];
  }
  Tensor out = Tensor::empty(out_shape, DType::kFloat32, x.device());
  detail::ctdk_ok(ctdk_permute(detail::f(x), detail::f(out), static_cast<int>(perm.size()), x.shape().data(), perm.data(), nullptr));
  return out;
}
inline Tensor permute(const Tensor& x, const std::vector<int>& perm) {
  Tensor out = permute_impl(x, perm);
  std::vector<int> inv(perm.size());
  for (size_t i = 0; i < perm.size(); ++i) inv[perm[i]] = static_cast<int>(i);
  detail::record(out, {x}, "PermuteBackward", [inv](const detail::Grads& g) { return detail::Grads{permute_impl(g.at(0), inv)}; });
  return out;
}

// ---- mask.h ---------------------------------------------------------------------------------
namespace detail {
inline void mask_call(const Tensor& in, Tensor& out, int q_pos_start, float fill, const char* op) {
  need_f32_cuda(in, op);
  require(in.dim() >= 2, "causal_mask: expected at least 2D scores");
  const int64_t Tk = in.shape()[in.dim() - 1], Tq = in.shape()[in.dim() - 2];
  const int64_t mats = (Tq * Tk) > 0 ? in.numel() / (Tq * Tk) : 0;
  ctdk_ok(ctdk_causal_mask(f(in), f(out), mats, Tq, Tk, q_pos_start, fill, nullptr));
}
}  // namespace detail
inline void apply_causal_mask_inplace(Tensor& scores, int q_pos_start = 0) {
  detail::mask_call(scores, scores, q_pos_start, -FLT_MAX, "apply_causal_mask");
}
inline Tensor apply_causal_mask_impl(const Tensor& scores, int q_pos_start) {
  Tensor out = detail::like(scores);
  detail::mask_call(scores, out, q_pos_start, -FLT_MAX, "apply_causal_mask");
  return out;
}
inline Tensor causal_mask_backward_impl(const Tensor& g, int q_pos_start) {
  Tensor out = detail::like(g);
  detail::mask_call(g, out, q_pos_start, 0.0f, "causal_mask_backward");
  return out;
}
inline Tensor apply_causal_mask(const Tensor& scores, int q_pos_start = 0) {
  Tensor out = apply_causal_mask_impl(scores, q_pos_start);
  detail::record(out, {scores}, "CausalMaskBackward",
                 [q_pos_start](const detail::Grads& g) { return detail::Grads{causal_mask_backward_impl(g.at(0), q_pos_start)}; });
  return out;
}

// ---- kv_cache.h -----------------------------------------------------------------------------
inline void write_kv_inplace(Tensor& cache, const Tensor& src, int pos) {
  if (cache.dtype() != DType::kFloat32 || src.dtype() != DType::kFloat32) throw std::runtime_error("write_kv: fp32 only");
  if (!cache.device().is_cuda() || !src.device().is_cuda()) throw std::runtime_error("write_kv: CUDA only");
  if (!cache.is_contiguous() || !src.is_contiguous()) throw std::runtime_error("write_kv: contiguous only");
  if (cache.dim() != 4 || src.dim() != 4) throw std::runtime_error("write_kv: expected 4D inputs");
  const int64_t B = src.shape()[0], T = src.shape()[1], H = src.shape()[2], D = src.shape()[3];
  if (cache.shape()[0] != B || cache.shape()[1] != H || cache.shape()[3] != D) throw std::runtime_error("write_kv: cache / src dim mismatch");
  detail::ctdk_ok(ctdk_kv_write(detail::f(src), detail::f(cache), B, T, static_cast<int>(H), static_cast<int>(D), cache.shape()[2], pos, nullptr));
}
inline Tensor read_kv_expanded(const Tensor& cache, int valid_len, int group) {
  if (cache.dtype() != DType::kFloat32 || !cache.device().is_cuda() || !cache.is_contiguous())
    throw std::runtime_error("read_kv_expanded: fp32/contig/CUDA only");
  if (cache.dim() != 4) throw std::runtime_error("read_kv_expanded: 4D cache required");
  const int64_t B = cache.shape()[0], Hk = cache.shape()[1], max_seq = cache.shape()[2], D = cache.shape()[3];
  if (valid_len < 0 || valid_len > max_seq) throw std::runtime_error("read_kv_expanded: valid_len out of range");
  if (group <= 0) throw std::runtime_error("read_kv_expanded: group must be > 0");
  Tensor out = Tensor::empty({B, Hk * group, valid_len, D}, DType::kFloat32, cache.device());
  detail::ctdk_ok(ctdk_kv_read_expanded(detail::f(cache), detail::f(out), B, static_cast<int>(Hk), group, valid_len, static_cast<int>(D),
                                        max_seq, nullptr));
  return out;
}

// ---- loss.h ---------------------------------------------------------------------------------
inline Tensor mse_loss_impl(const Tensor& pred, const Tensor& target) {
  detail::need_f32_cuda(pred, "mse_loss");
  detail::need_f32_cuda(target, "mse_loss");
  detail::same_shape(pred, target, "mse_loss");
  detail::require(pred.numel() > 0, "mse_loss: empty input");
  Tensor loss = Tensor::empty({1}, DType::kFloat32, pred.device());
  detail::ctdk_ok(ctdk_mse_fwd(detail::f(pred), detail::f(target), pred.numel(), detail::f(loss), nullptr));
  return loss;
}
inline Tensor mse_loss(const Tensor& pred, const Tensor& target) {
  Tensor out = mse_loss_impl(pred, target);
  Tensor sp = pred.detach(), st = target.detach();
  detail::record(out, {pred}, "MseLossBackward", [sp, st](const detail::Grads& g) {
    Tensor dp = detail::like(sp);
    detail::ctdk_ok(ctdk_mse_bwd(detail::f(sp), detail::f(st), detail::f(g.at(0)), detail::f(dp), sp.numel(), nullptr));
    return detail::Grads{dp};
  });
  return out;
}

namespace detail {
inline void check_ce(const Tensor& logits, const Tensor& targets, const Tensor* mask, const char* op) {
  need_f32_cuda(logits, op);
  require(logits.dim() == 2, std::string(op) + ": logits must be [N, V]");
  require(targets.dtype() == DType::kInt64 && targets.device().is_cuda() && targets.numel() == logits.shape()[0],
          std::string(op) + ": targets must be int64 [N] on CUDA");
  if (mask != nullptr) {
    need_f32_cuda(*mask, op);
    require(mask->numel() == logits.shape()[0], std::string(op) + ": loss_mask must be [N]");
  }
}
// loss = sum(mask * (lse - z_target)) / sum(mask) (mask == nullptr: all ones); 0 for an empty mask.
inline Tensor ce_forward(const Tensor& logits, const Tensor& targets, const Tensor* mask) {
  Tensor sums = Tensor::zeros({2}, DType::kFloat32, logits.device());
  ctdk_ok(ctdk_ce_masked(const_cast<float*>(f(logits)), i64(targets), mask ? f(*mask) : nullptr, nullptr, f(sums), nullptr,
                         logits.shape()[0], logits.shape()[1], 0, nullptr));
  Tensor loss = Tensor::empty({1}, DType::kFloat32, logits.device());
  ctdk_ok(ctdk_loss_ratio(f(sums), f(loss), nullptr));
  return loss;
}
// dlogits = dy / sum(mask) * mask_i * (softmax(z_i) - onehot(t_i)); throws when the mask is empty
// (CrossEntropyMaskedBackward, src/ops/loss.cu:388-411).
inline Tensor ce_backward(const Tensor& logits, const Tensor& targets, const Tensor* mask, const Tensor& dy, const char* op) {
  const int64_t N = logits.shape()[0];
  Tensor msum = Tensor::zeros({1}, DType::kFloat32, logits.device());
  if (mask != nullptr) {
    ctdk_ok(ctdk_sumsq(f(*mask), N, f(msum), nullptr));   // the mask holds 0 / 1: sum of squares = sum
    float h = 0.0f;
    msum.copy_to_host(&h);
    if (h <= 0.0f) throw std::runtime_error(std::string(op) + " backward: sum(loss_mask) == 0");
  }
  Tensor w = Tensor::empty({N}, DType::kFloat32, logits.device());
  ctdk_ok(ctdk_ce_row_weight(mask ? f(*mask) : nullptr, f(dy), f(msum), N, f(w), nullptr));
  Tensor dlogits = like(logits);
  CTD_CUDA_CHECK(cudaMemcpyAsync(dlogits.data_ptr(), logits.data_ptr(), logits.nbytes(), cudaMemcpyDeviceToDevice, nullptr));
  Tensor sums = Tensor::zeros({2}, DType::kFloat32, logits.device());
  ctdk_ok(ctdk_ce_masked(f(dlogits), i64(targets), mask ? f(*mask) : nullptr, f(w), f(sums), nullptr, N, logits.shape()[1], 1, nullptr));
  return dlogits;
}
}  // namespace detail
inline Tensor cross_entropy_impl(const Tensor& logits, const Tensor& targets) {
  detail::check_ce(logits, targets, nullptr, "cross_entropy");
  return detail::ce_forward(logits, targets, nullptr);
}
inline Tensor cross_entropy(const Tensor& logits, const Tensor& targets) {
  Tensor out = cross_entropy_impl(logits, targets);
  Tensor sl = logits.detach(), st = targets;
  detail::record(out, {logits}, "CrossEntropyBackward",
                 [sl, st](const detail::Grads& g) { return detail::Grads{detail::ce_backward(sl, st, nullptr, g.at(0), "cross_entropy")}; });
  return out;
}
inline Tensor cross_entropy_masked_impl(const Tensor& logits, const Tensor& targets, const Tensor& loss_mask) {
  detail::check_ce(logits, targets, &loss_mask, "cross_entropy_masked");
  return detail::ce_forward(logits, targets, &loss_mask);
}
inline Tensor cross_entropy_masked(const Tensor& logits, const Tensor& targets, const Tensor& loss_mask) {
  Tensor out = cross_entropy_masked_impl(logits, targets, loss_mask);
  Tensor sl = logits.detach(), st = targets, sm = loss_mask.detach();
  detail::record(out, {logits}, "CrossEntropyMaskedBackward", [sl, st, sm](const detail::Grads& g) {
    return detail::Grads{detail::ce_backward(sl, st, &sm, g.at(0), "cross_entropy_masked")};
  });
  return out;
}

}  // namespace ctd::ops
