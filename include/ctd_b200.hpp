// C++ mirror of the reference's public op API for the decoder training path, on top of the C-ABI in
// ctdk.h: same namespaces, names, argument order and error behaviour (precondition violations and
// failed launches throw std::runtime_error with a message) as emberlm's include/ctd/tensor.h,
// include/ctd/ops/*.h and include/ctd/optim.h, so code and tests written against `ctd::ops::*_impl`,
// `ctd::optim::AdamW` and `ctd::optim::clip_grad_norm_` compile against this header unchanged.
//
// What it is not: there is no general autograd tape here. The un-suffixed functions (ops::matmul,
// ops::add, ...) are the forward computations only; training runs through the step engine
// (ctdk_engine_*), which owns the fixed forward / backward schedule of the decoder. The one graph
// this layer does record is the one the reference's training loop builds
// (tools/ctd_train/main.cpp:359-361): the loss of nn::Model::forward_train_masked (ctd_b200_nn.hpp),
// optionally scaled by ops::mul_scalar, then backward(). Elsewhere gradients are attached with
// Tensor::set_grad. Every op allocates its output with cudaMalloc, as the reference's
// allocator does (src/core/allocator.cpp:14-30); this layer is the compatibility surface, not the
// hot path. Header-only; link with -lctdk -lcudart.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include <cuda_runtime.h>

#include "ctdk.h"

namespace ctd {

enum class DeviceType : uint8_t { kCPU = 0, kCUDA = 1 };
struct Device {
  DeviceType type = DeviceType::kCPU;
  int index = 0;
  constexpr Device() = default;
  constexpr Device(DeviceType t, int i = 0) : type(t), index(i) {}
  bool is_cpu() const { return type == DeviceType::kCPU; }
  bool is_cuda() const { return type == DeviceType::kCUDA; }
  bool operator==(const Device& o) const { return type == o.type && index == o.index; }
  bool operator!=(const Device& o) const { return !(*this == o); }
};
constexpr Device kCPU{DeviceType::kCPU, 0};
constexpr Device kCUDA0{DeviceType::kCUDA, 0};

enum class DType : uint8_t { kFloat32 = 0, kFloat16 = 1, kBFloat16 = 2, kInt32 = 3, kInt64 = 4 };
constexpr size_t dtype_size(DType dt) {
  return dt == DType::kFloat32 || dt == DType::kInt32 ? 4 : (dt == DType::kInt64 ? 8 : 2);
}

class Tensor;

namespace detail {
// The deferred model pass behind a loss tensor: backward(dy) runs forward + backward in one fused
// pass of the step engine and leaves the loss in `value`; forward() runs the loss alone, for a
// caller that reads the loss without ever calling backward().
struct LossNode {
  std::function<void(float)> backward;
  std::function<void()> forward;
  float value = 0.0f;
  bool have_value = false, backward_done = false;
};
inline void cuda_ok(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
inline void ctdk_ok(int rc) {
  if (rc != CTDK_OK) throw std::runtime_error(ctdk_last_error());
}
inline void require(bool ok, const char* msg) {
  if (!ok) throw std::runtime_error(msg);
}
}  // namespace detail

// Contiguous row-major device (or host) buffer with a shape. Copies of a Tensor are handles to one
// shared object (storage, shape and gradient slot), as with the reference's TensorImpl
// (include/ctd/tensor.h:20-60): a gradient attached through one handle is seen through all.
class Tensor {
 public:
  Tensor() = default;
  static Tensor empty(std::vector<int64_t> shape, DType dtype, Device device) {
    Tensor t;
    t.impl_ = std::make_shared<Impl>();
    t.impl_->shape = std::move(shape);
    t.impl_->dtype = dtype;
    t.impl_->device = device;
    const size_t bytes = t.nbytes() ? t.nbytes() : 1;
    void* p = nullptr;
    if (device.is_cuda()) {
      detail::cuda_ok(cudaMalloc(&p, bytes), "Tensor::empty: cudaMalloc");
      t.impl_->storage = std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
    } else {
      p = ::operator new(bytes);
      t.impl_->storage = std::shared_ptr<void>(p, [](void* q) { ::operator delete(q); });
    }
    return t;
  }
  static Tensor zeros(std::vector<int64_t> shape, DType dtype, Device device) {
    Tensor t = empty(std::move(shape), dtype, device);
    if (device.is_cuda()) detail::cuda_ok(cudaMemset(t.data_ptr(), 0, t.nbytes()), "Tensor::zeros: cudaMemset");
    else std::memset(t.data_ptr(), 0, t.nbytes());
    return t;
  }
  static Tensor from_host(const void* host, std::vector<int64_t> shape, DType dtype, Device device) {
    Tensor t = empty(std::move(shape), dtype, device);
    if (device.is_cuda()) detail::cuda_ok(cudaMemcpy(t.data_ptr(), host, t.nbytes(), cudaMemcpyHostToDevice), "Tensor::from_host");
    else std::memcpy(t.data_ptr(), host, t.nbytes());
    return t;
  }
  // A tensor over memory owned by `owner` (a slice of a larger allocation).
  static Tensor view(std::shared_ptr<void> owner, void* ptr, std::vector<int64_t> shape, DType dtype, Device device) {
    Tensor t;
    t.impl_ = std::make_shared<Impl>();
    t.impl_->storage = std::shared_ptr<void>(std::move(owner), ptr);
    t.impl_->shape = std::move(shape);
    t.impl_->dtype = dtype;
    t.impl_->device = device;
    return t;
  }
  void copy_to_host(void* dst) const {   // blocking, like the reference's (tensor.cpp:132-142)
    if (impl_->node) {   // a loss (times a constant) whose model pass may not have run yet
      if (!impl_->node->have_value) impl_->node->forward();
      const float v = impl_->node->value * impl_->node_scale;
      std::memcpy(dst, &v, sizeof v);
      return;
    }
    if (device().is_cuda()) detail::cuda_ok(cudaMemcpy(dst, data_ptr(), nbytes(), cudaMemcpyDeviceToHost), "Tensor::copy_to_host");
    else std::memcpy(dst, data_ptr(), nbytes());
  }
  // A new tensor object over the same storage (no gradient slot of its own yet).
  Tensor reshape(std::vector<int64_t> new_shape) const {
    Tensor t;
    t.impl_ = std::make_shared<Impl>();
    t.impl_->storage = impl_->storage;
    t.impl_->shape = std::move(new_shape);
    t.impl_->dtype = impl_->dtype;
    t.impl_->device = impl_->device;
    detail::require(t.numel() == numel(), "reshape: element count differs");
    return t;
  }
  const std::vector<int64_t>& shape() const { return impl_->shape; }
  int64_t dim() const { return static_cast<int64_t>(impl_->shape.size()); }
  int64_t numel() const {
    int64_t n = 1;
    for (const int64_t d : impl_->shape) n *= d;
    return n;
  }
  size_t nbytes() const { return static_cast<size_t>(numel()) * dtype_size(impl_->dtype); }
  DType dtype() const { return impl_->dtype; }
  const Device& device() const { return impl_->device; }
  bool is_contiguous() const { return true; }
  void* data_ptr() { return impl_->storage.get(); }
  const void* data_ptr() const { return impl_->storage.get(); }
  bool defined() const { return impl_ != nullptr; }
  // Gradient slot read by the optimizer. There is no tape in this layer: the caller attaches it.
  Tensor grad() const { return impl_ && impl_->grad ? *impl_->grad : Tensor(); }
  void set_grad(const Tensor& g) { impl_->grad = std::make_shared<Tensor>(g); }
  void zero_grad_() { impl_->grad.reset(); }

  // Loss tensors only (the reference's Tensor::backward walks a tape, src/core/autograd.cu:158-237;
  // here the only recorded graph is model loss x constant). Runs the fused forward + backward pass
  // with this tensor's scale as the upstream gradient; the parameters' grad() then point into the
  // model's gradient arena. Like the reference's tape, a graph can be walked once.
  void backward() {
    detail::require(impl_ && impl_->node, "backward: this build records no graph for this tensor (only model losses)");
    detail::require(!impl_->node->backward_done, "backward: the graph of this loss has already been consumed");
    impl_->node->backward_done = true;
    impl_->node->backward(impl_->node_scale);
  }
  bool has_loss_node() const { return impl_ && impl_->node; }
  static Tensor loss_of(std::shared_ptr<detail::LossNode> node, float scale, Device device) {
    Tensor t = empty({1}, DType::kFloat32, device);
    t.impl_->node = std::move(node);
    t.impl_->node_scale = scale;
    return t;
  }
  Tensor scaled_loss(float c) const { return loss_of(impl_->node, impl_->node_scale * c, impl_->device); }

 private:
  struct Impl {
    std::shared_ptr<void> storage;
    std::vector<int64_t> shape;
    DType dtype = DType::kFloat32;
    Device device{};
    std::shared_ptr<Tensor> grad;
    std::shared_ptr<detail::LossNode> node;   // set for model losses only
    float node_scale = 1.0f;
  };
  std::shared_ptr<Impl> impl_;
};

namespace ops {

namespace detail2 {
inline const float* f(const Tensor& t) { return static_cast<const float*>(t.data_ptr()); }
inline float* f(Tensor& t) { return static_cast<float*>(t.data_ptr()); }
inline void need_f32_cuda(const Tensor& t, const char* op) {
  if (!t.device().is_cuda()) throw std::runtime_error(std::string(op) + ": CUDA tensors only");
  if (t.dtype() != DType::kFloat32) throw std::runtime_error(std::string(op) + ": fp32 only");
}
inline void same_shape(const Tensor& a, const Tensor& b, const char* op) {
  if (a.shape() != b.shape()) throw std::runtime_error(std::string(op) + ": shape mismatch");
}
inline Tensor like(const Tensor& x) { return Tensor::empty(x.shape(), DType::kFloat32, x.device()); }
}  // namespace detail2

// ---- elementwise (include/ctd/ops/elementwise.h, repeat_kv.h:16-17) ----
#define CTD_B200_BINARY(NAME, ENTRY)                                                          \
  inline Tensor NAME##_impl(const Tensor& a, const Tensor& b) {                               \
    detail2::need_f32_cuda(a, #NAME);                                                         \
    detail2::need_f32_cuda(b, #NAME);                                                         \
    detail2::same_shape(a, b, #NAME);                                                         \
    Tensor out = detail2::like(a);                                                            \
    detail::ctdk_ok(ENTRY(detail2::f(a), detail2::f(b), detail2::f(out), a.numel(), nullptr)); \
    return out;                                                                               \
  }
CTD_B200_BINARY(add, ctdk_add)
CTD_B200_BINARY(sub, ctdk_sub)
CTD_B200_BINARY(mul, ctdk_mul)
#undef CTD_B200_BINARY
inline Tensor scale_impl(const Tensor& x, float alpha) {
  detail2::need_f32_cuda(x, "scale");
  Tensor out = detail2::like(x);
  detail::ctdk_ok(ctdk_scale(detail2::f(x), alpha, detail2::f(out), x.numel(), nullptr));
  return out;
}
inline Tensor mul_scalar_impl(const Tensor& x, float c) { return scale_impl(x, c); }
inline Tensor silu_impl(const Tensor& x) {
  detail2::need_f32_cuda(x, "silu");
  Tensor out = detail2::like(x);
  detail::ctdk_ok(ctdk_silu(detail2::f(x), detail2::f(out), x.numel(), nullptr));
  return out;
}
inline Tensor silu_backward_impl(const Tensor& x, const Tensor& g) {
  detail2::need_f32_cuda(x, "silu_backward");
  detail2::need_f32_cuda(g, "silu_backward");
  detail2::same_shape(x, g, "silu_backward");
  Tensor out = detail2::like(x);
  detail::ctdk_ok(ctdk_silu_bwd(detail2::f(x), detail2::f(g), detail2::f(out), x.numel(), nullptr));
  return out;
}
inline Tensor add(const Tensor& a, const Tensor& b) { return add_impl(a, b); }
inline Tensor mul(const Tensor& a, const Tensor& b) { return mul_impl(a, b); }
inline Tensor silu(const Tensor& x) { return silu_impl(x); }
inline Tensor mul_scalar(const Tensor& x, float c) { return x.has_loss_node() ? x.scaled_loss(c) : mul_scalar_impl(x, c); }

// ---- matmul / bmm (include/ctd/ops/matmul.h; semantics src/ops/matmul.cpp:13-49) ----
inline Tensor matmul_impl(const Tensor& a, const Tensor& b, bool transa, bool transb) {
  detail2::need_f32_cuda(a, "matmul");
  detail2::need_f32_cuda(b, "matmul");
  detail::require(a.dim() == 2 && b.dim() == 2, "matmul: expected 2D tensors");
  const int64_t M = transa ? a.shape()[1] : a.shape()[0], K = transa ? a.shape()[0] : a.shape()[1];
  const int64_t Kb = transb ? b.shape()[1] : b.shape()[0], N = transb ? b.shape()[0] : b.shape()[1];
  detail::require(K == Kb, "matmul: inner dims disagree");
  Tensor out = Tensor::empty({M, N}, DType::kFloat32, a.device());
  detail::ctdk_ok(ctdk_gemm(detail2::f(a), detail2::f(b), detail2::f(out), M, N, K, a.shape()[1], b.shape()[1], N, transa ? 1 : 0,
                            transb ? 1 : 0, CTDK_GEMM_TF32, CTDK_EPI_STORE, nullptr, nullptr));
  return out;
}
inline Tensor matmul(const Tensor& a, const Tensor& b, bool transa = false, bool transb = false) {
  return matmul_impl(a, b, transa, transb);
}
inline Tensor bmm_impl(const Tensor& a, const Tensor& b, bool transa, bool transb) {
  detail2::need_f32_cuda(a, "bmm");
  detail2::need_f32_cuda(b, "bmm");
  detail::require(a.dim() == 3 && b.dim() == 3 && a.shape()[0] == b.shape()[0], "bmm: expected 3D tensors with equal batch");
  const int64_t Bt = a.shape()[0];
  const int64_t M = transa ? a.shape()[2] : a.shape()[1], K = transa ? a.shape()[1] : a.shape()[2];
  const int64_t Kb = transb ? b.shape()[2] : b.shape()[1], N = transb ? b.shape()[1] : b.shape()[2];
  detail::require(K == Kb, "bmm: inner dims disagree");
  Tensor out = Tensor::empty({Bt, M, N}, DType::kFloat32, a.device());
  detail::ctdk_ok(ctdk_bmm(detail2::f(a), detail2::f(b), detail2::f(out), Bt, M, N, K, transa ? 1 : 0, transb ? 1 : 0,
                           CTDK_GEMM_TF32, nullptr));
  return out;
}
inline Tensor bmm(const Tensor& a, const Tensor& b, bool transa = false, bool transb = false) {
  return bmm_impl(a, b, transa, transb);
}

// ---- RMSNorm (include/ctd/ops/norm.h) ----
inline Tensor rms_norm_impl(const Tensor& x, const Tensor& weight, float eps) {
  detail2::need_f32_cuda(x, "rms_norm");
  detail2::need_f32_cuda(weight, "rms_norm");
  detail::require(x.dim() >= 1 && weight.dim() == 1 && weight.shape()[0] == x.shape().back(), "rms_norm: weight must be [H]");
  const int H = static_cast<int>(x.shape().back());
  Tensor y = detail2::like(x);
  detail::ctdk_ok(ctdk_rmsnorm_fwd(detail2::f(x), detail2::f(weight), detail2::f(y), nullptr, x.numel() / H, H, eps, nullptr));
  return y;
}
inline Tensor rms_norm(const Tensor& x, const Tensor& weight, float eps) { return rms_norm_impl(x, weight, eps); }
inline std::pair<Tensor, Tensor> rms_norm_backward_impl(const Tensor& dy, const Tensor& x, const Tensor& w, float eps) {
  detail2::need_f32_cuda(dy, "rms_norm_backward");
  detail2::need_f32_cuda(x, "rms_norm_backward");
  detail2::same_shape(dy, x, "rms_norm_backward");
  const int H = static_cast<int>(x.shape().back());
  detail::require(w.dim() == 1 && w.shape()[0] == H, "rms_norm_backward: weight must be [H]");
  Tensor dx = detail2::like(x), dw = Tensor::empty({H}, DType::kFloat32, x.device());
  Tensor scratch = Tensor::empty({ctdk_rmsnorm_bwd_scratch_floats(H)}, DType::kFloat32, x.device());
  detail::ctdk_ok(ctdk_rmsnorm_bwd(detail2::f(dy), detail2::f(x), detail2::f(w), detail2::f(dx), detail2::f(dw), detail2::f(scratch),
                                   x.numel() / H, H, eps, 0, 0, nullptr));
  return {dx, dw};
}

// ---- RoPE (include/ctd/ops/rope.h) ----
struct RopeScaling {
  float factor = 0.0f;
  float low_freq_factor = 1.0f;
  float high_freq_factor = 4.0f;
  int original_max_pos = 8192;
  bool enabled() const { return factor > 1.0f; }
  float low_freq_wavelen() const { return static_cast<float>(original_max_pos) / low_freq_factor; }
  float high_freq_wavelen() const { return static_cast<float>(original_max_pos) / high_freq_factor; }
};
namespace detail2 {
inline void rope_call(const Tensor& x, Tensor& out, int position_start, float theta, const RopeScaling& sc, float sin_sign) {
  need_f32_cuda(x, "rope");
  detail::require(x.dim() == 4 && x.shape()[3] % 2 == 0, "rope: expected [B, T, H, D] with even D");
  ctdk_rope_params p;
  p.theta = theta;
  p.scaling_factor = sc.enabled() ? sc.factor : 0.0f;
  p.low_freq_wavelen = sc.low_freq_wavelen();
  p.high_freq_wavelen = sc.high_freq_wavelen();
  const int H = static_cast<int>(x.shape()[2]), D = static_cast<int>(x.shape()[3]);
  detail::ctdk_ok(ctdk_rope(f(x), f(out), x.shape()[0], x.shape()[1], H, D, static_cast<int64_t>(H) * D, position_start, &p, sin_sign,
                            nullptr));
}
}  // namespace detail2
inline Tensor rope_impl(const Tensor& x, int position_start, float theta, const RopeScaling& scaling = {}) {
  Tensor out = detail2::like(x);
  detail2::rope_call(x, out, position_start, theta, scaling, 1.0f);
  return out;
}
inline Tensor rope(const Tensor& x, int position_start, float theta, const RopeScaling& scaling = {}) {
  return rope_impl(x, position_start, theta, scaling);
}
// The backward of rope: the rotation by the negative angle (src/ops/rope.cu:100-145).
inline Tensor rope_transpose_impl(const Tensor& x, int position_start, float theta, const RopeScaling& scaling = {}) {
  Tensor out = detail2::like(x);
  detail2::rope_call(x, out, position_start, theta, scaling, -1.0f);
  return out;
}
inline void apply_rope_inplace(Tensor& x, int position_start, float theta, const RopeScaling& scaling = {}) {
  detail2::rope_call(x, x, position_start, theta, scaling, 1.0f);
}

// ---- embedding (include/ctd/ops/embedding.h) ----
inline Tensor embedding_impl(const Tensor& ids, const Tensor& weight) {
  detail2::need_f32_cuda(weight, "embedding");
  detail::require(ids.dtype() == DType::kInt64 && ids.device().is_cuda(), "embedding: ids must be int64 on CUDA");
  detail::require(weight.dim() == 2, "embedding: weight must be [V, H]");
  std::vector<int64_t> shape = ids.shape();
  shape.push_back(weight.shape()[1]);
  Tensor out = Tensor::empty(shape, DType::kFloat32, weight.device());
  detail::ctdk_ok(ctdk_embedding_fwd(static_cast<const int64_t*>(ids.data_ptr()), detail2::f(weight), detail2::f(out), ids.numel(),
                                     static_cast<int>(weight.shape()[1]), weight.shape()[0], nullptr));
  return out;
}
inline Tensor embedding(const Tensor& ids, const Tensor& weight) { return embedding_impl(ids, weight); }
inline Tensor embedding_backward_impl(const Tensor& ids, const Tensor& dy, int64_t vocab) {
  detail2::need_f32_cuda(dy, "embedding_backward");
  detail::require(ids.dtype() == DType::kInt64, "embedding_backward: ids must be int64");
  const int H = static_cast<int>(dy.shape().back());
  Tensor dw = Tensor::zeros({vocab, H}, DType::kFloat32, dy.device());
  detail::ctdk_ok(ctdk_embedding_bwd(static_cast<const int64_t*>(ids.data_ptr()), detail2::f(dy), detail2::f(dw), ids.numel(), H, vocab,
                                     nullptr));
  return dw;
}

// ---- masked cross-entropy (include/ctd/ops/loss.h:17-26; src/ops/loss.cu:254-429) ----
// logits fp32 [N, V], targets int64 [N], loss_mask fp32 [N]; returns the scalar [1] loss
// sum(mask * (lse - z_target)) / sum(mask) (0 when the mask is empty, as the forward there).
inline Tensor cross_entropy_masked_impl(const Tensor& logits, const Tensor& targets, const Tensor& loss_mask) {
  detail2::need_f32_cuda(logits, "cross_entropy_masked");
  detail2::need_f32_cuda(loss_mask, "cross_entropy_masked");
  detail::require(logits.dim() == 2, "cross_entropy_masked: logits must be [N, V]");
  detail::require(targets.dtype() == DType::kInt64 && targets.numel() == logits.shape()[0], "cross_entropy_masked: targets must be int64 [N]");
  detail::require(loss_mask.numel() == logits.shape()[0], "cross_entropy_masked: loss_mask must be [N]");
  Tensor sums = Tensor::zeros({2}, DType::kFloat32, logits.device());
  // forward only (last flag 0): the logits are read, never written
  detail::ctdk_ok(ctdk_ce_masked(const_cast<float*>(detail2::f(logits)), static_cast<const int64_t*>(targets.data_ptr()),
                                 detail2::f(loss_mask), nullptr, detail2::f(sums), nullptr, logits.shape()[0], logits.shape()[1], 0,
                                 nullptr));
  float h[2];
  sums.copy_to_host(h);
  const float loss = h[1] > 0.0f ? h[0] / h[1] : 0.0f;
  return Tensor::from_host(&loss, {1}, DType::kFloat32, logits.device());
}
inline Tensor cross_entropy_masked(const Tensor& logits, const Tensor& targets, const Tensor& loss_mask) {
  return cross_entropy_masked_impl(logits, targets, loss_mask);
}
// d(loss)/d(logits) for the upstream scalar gradient dy (CrossEntropyMaskedBackward, loss.cu:388-411):
// dy / sum(mask) * mask_i * (softmax(z_i) - onehot(t_i)). Throws when the mask is empty.
inline Tensor cross_entropy_masked_backward_impl(const Tensor& logits, const Tensor& targets, const Tensor& loss_mask, float dy) {
  detail2::need_f32_cuda(logits, "cross_entropy_masked_backward");
  const int64_t N = logits.shape()[0];
  std::vector<float> m(static_cast<size_t>(N));
  loss_mask.copy_to_host(m.data());
  double sm = 0.0;
  for (const float v : m) sm += v;
  if (sm <= 0.0) throw std::runtime_error("cross_entropy_masked backward: sum(loss_mask) == 0");
  for (auto& v : m) v = static_cast<float>(v * dy / sm);
  Tensor w = Tensor::from_host(m.data(), {N}, DType::kFloat32, logits.device());
  Tensor dlogits = detail2::like(logits);
  detail::cuda_ok(cudaMemcpy(dlogits.data_ptr(), logits.data_ptr(), logits.nbytes(), cudaMemcpyDeviceToDevice), "cross_entropy_masked_backward: copy");
  Tensor sums = Tensor::zeros({2}, DType::kFloat32, logits.device());
  detail::ctdk_ok(ctdk_ce_masked(detail2::f(dlogits), static_cast<const int64_t*>(targets.data_ptr()), detail2::f(loss_mask), detail2::f(w),
                                 detail2::f(sums), nullptr, N, logits.shape()[1], 1, nullptr));
  return dlogits;
}

}  // namespace ops

namespace optim {

// Global L2 norm of the parameters' gradients; scales them by max_norm / (norm + eps) when the
// norm exceeds max_norm; returns the norm before clipping (src/core/optim.cu:248-293).
inline float clip_grad_norm_(const std::vector<Tensor>& params, float max_norm, float eps = 1e-6f) {
  Tensor acc = Tensor::zeros({4}, DType::kFloat32, kCUDA0);
  float* a = static_cast<float*>(acc.data_ptr());
  for (const Tensor& p : params) {
    Tensor g = p.grad();
    if (!g.defined()) continue;
    detail::ctdk_ok(ctdk_sumsq(static_cast<const float*>(g.data_ptr()), g.numel(), a, nullptr));
  }
  detail::ctdk_ok(ctdk_clip_scale(a, max_norm, eps, a + 1, a + 2, nullptr));
  float h[4];
  acc.copy_to_host(h);
  if (h[1] != 1.0f) {
    for (const Tensor& p : params) {
      Tensor g = p.grad();
      if (!g.defined()) continue;
      float* gp = static_cast<float*>(g.data_ptr());
      detail::ctdk_ok(ctdk_scale(gp, h[1], gp, g.numel(), nullptr));
    }
  }
  return h[2];
}

struct ParamGroup {
  std::vector<Tensor> params;
  float lr;
  float weight_decay;
};

// AdamW with decoupled weight decay and the reference's fp32 bias corrections
// (include/ctd/optim.h:38-94, src/core/optim.cu:54-73, 132-168). Moments live on the device.
class AdamW {
 public:
  AdamW(std::vector<Tensor> params, float lr, float weight_decay = 0.0f, float beta1 = 0.9f, float beta2 = 0.95f, float eps = 1e-8f)
      : AdamW(std::vector<ParamGroup>{ParamGroup{std::move(params), lr, weight_decay}}, beta1, beta2, eps) {}
  AdamW(std::vector<ParamGroup> groups, float beta1 = 0.9f, float beta2 = 0.95f, float eps = 1e-8f, bool offload = false)
      : groups_(std::move(groups)), beta1_(beta1), beta2_(beta2), eps_(eps) {
    (void)offload;   // moments always stay in HBM here
    for (const auto& g : groups_) {
      state_.emplace_back();
      for (const Tensor& p : g.params) {
        State st;
        st.m = Tensor::zeros(p.shape(), DType::kFloat32, p.device());
        st.v = Tensor::zeros(p.shape(), DType::kFloat32, p.device());
        state_.back().push_back(st);
      }
    }
  }
  void step() {
    ++step_;
    const float t = static_cast<float>(step_);
    for (size_t gi = 0; gi < groups_.size(); ++gi) {
      ParamGroup& g = groups_[gi];
      ctdk_adamw_params hp{g.lr, beta1_, beta2_, eps_, g.weight_decay, 1.0f - std::pow(beta1_, t), 1.0f - std::pow(beta2_, t)};
      for (size_t pi = 0; pi < g.params.size(); ++pi) {
        Tensor& p = g.params[pi];
        Tensor gr = p.grad();
        if (!gr.defined()) continue;
        detail::ctdk_ok(ctdk_adamw(static_cast<float*>(p.data_ptr()), static_cast<const float*>(gr.data_ptr()),
                                   static_cast<float*>(state_[gi][pi].m.data_ptr()), static_cast<float*>(state_[gi][pi].v.data_ptr()),
                                   p.numel(), &hp, nullptr, nullptr, nullptr, 0, nullptr));
      }
    }
  }
  void zero_grad() {
    for (auto& g : groups_)
      for (auto& p : g.params) p.zero_grad_();
  }
  int64_t step_count() const { return step_; }
  void set_step_count(int64_t s) { step_ = s; }
  void set_lr(float lr) {
    for (auto& g : groups_) g.lr = lr;
  }
  float lr() const { return groups_.empty() ? 0.0f : groups_.front().lr; }
  size_t num_groups() const { return groups_.size(); }
  size_t num_params(size_t gi) const { return groups_.at(gi).params.size(); }
  Tensor& m_tensor(size_t gi, size_t pi) { return state_.at(gi).at(pi).m; }
  Tensor& v_tensor(size_t gi, size_t pi) { return state_.at(gi).at(pi).v; }
  bool is_offloaded() const { return false; }

 private:
  struct State {
    Tensor m, v;
  };
  std::vector<ParamGroup> groups_;
  std::vector<std::vector<State>> state_;
  float beta1_, beta2_, eps_;
  int64_t step_ = 0;
};

}  // namespace optim
}  // namespace ctd
