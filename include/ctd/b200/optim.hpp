// ctd::optim — SGD, AdamW and clip_grad_norm_ with the reference's interface and arithmetic
// (emberlm include/ctd/optim.h, src/core/optim.cu:54-73, 132-168, 248-293).
//
// When every parameter is a view into one arena and every gradient a view at the same offset of a
// second arena (the parameters of a built nn::Model), the norm is ONE sum-of-squares launch over
// the gradient arena and the update ONE fused AdamW launch over the parameter arena with a
// per-range weight-decay table; m and v are arenas of the same layout and m_tensor / v_tensor views
// of them. Any other set of tensors is handled tensor by tensor. AdamW's moments always stay in
// HBM: `offload` is accepted and ignored (a multi-GPU run shards them instead, ctdk_trainer_*).
#pragma once

#include <algorithm>
#include <cmath>

#include "core.hpp"

namespace ctd::optim {

namespace detail {
using ::ctd::detail::ctdk_ok;
inline float* f(const Tensor& t) { return static_cast<float*>(const_cast<void*>(t.data_ptr())); }

// The arena range [lo, hi) (in floats) that the tensors cover if they all live in one storage.
struct Span {
  StoragePtr storage;
  int64_t lo = 0, hi = 0;
  bool ok = false;
};
inline Span span_of(const std::vector<Tensor>& ts) {
  Span s;
  for (const Tensor& t : ts) {
    if (!t.storage() || t.dtype() != DType::kFloat32 || !t.is_contiguous() || !t.device().is_cuda()) return Span{};
    if (!s.storage) {
      s.storage = t.storage();
      s.lo = t.storage_offset();
      s.hi = s.lo + t.numel();
    } else if (t.storage() != s.storage) {
      return Span{};
    } else {
      s.lo = std::min(s.lo, t.storage_offset());
      s.hi = std::max(s.hi, t.storage_offset() + t.numel());
    }
  }
  s.ok = s.storage != nullptr && s.lo % 4 == 0;
  return s;
}
}  // namespace detail

class SGD {
 public:
  explicit SGD(std::vector<Tensor> params, float lr) : params_(std::move(params)), lr_(lr) {}
  // p <- p - lr * g
  void step() {
    for (Tensor& p : params_) {
      Tensor g = p.grad();
      if (!g.storage()) continue;
      Tensor scaled = Tensor::empty(g.shape(), DType::kFloat32, g.device());
      detail::ctdk_ok(ctdk_scale(detail::f(g), lr_, detail::f(scaled), g.numel(), nullptr));
      detail::ctdk_ok(ctdk_sub(detail::f(p), detail::f(scaled), detail::f(p), p.numel(), nullptr));
    }
  }
  void zero_grad() {
    for (Tensor& p : params_) p.zero_grad_();
  }

 private:
  std::vector<Tensor> params_;
  float lr_;
};

struct ParamGroup {
  std::vector<Tensor> params;
  float lr;
  float weight_decay;
};

class AdamW {
 public:
  AdamW(std::vector<Tensor> params, float lr, float weight_decay = 0.0f, float beta1 = 0.9f, float beta2 = 0.95f, float eps = 1e-8f,
        bool offload = false)
      : AdamW(std::vector<ParamGroup>{ParamGroup{std::move(params), lr, weight_decay}}, beta1, beta2, eps, offload) {}
  AdamW(std::vector<ParamGroup> groups, float beta1 = 0.9f, float beta2 = 0.95f, float eps = 1e-8f, bool offload = false)
      : groups_(std::move(groups)), beta1_(beta1), beta2_(beta2), eps_(eps), offload_(offload) {}
  ~AdamW() = default;

  void step() {
    ensure_state_initialized();
    ++step_;
    const float t = static_cast<float>(step_);
    const float bc1 = 1.0f - std::pow(beta1_, t), bc2 = 1.0f - std::pow(beta2_, t);
    if (arena_.ok && fused_step(bc1, bc2)) return;
    for (size_t gi = 0; gi < groups_.size(); ++gi) {
      const ParamGroup& g = groups_[gi];
      const ctdk_adamw_params hp{g.lr, beta1_, beta2_, eps_, g.weight_decay, bc1, bc2};
      for (size_t pi = 0; pi < g.params.size(); ++pi) {
        const Tensor& p = g.params[pi];
        Tensor gr = p.grad();
        if (!gr.storage()) continue;
        detail::ctdk_ok(ctdk_adamw(detail::f(p), detail::f(gr), detail::f(state_[gi][pi].m), detail::f(state_[gi][pi].v), p.numel(), &hp,
                                   nullptr, nullptr, nullptr, 0, nullptr));
      }
    }
  }
  void zero_grad() {
    for (ParamGroup& g : groups_)
      for (Tensor& p : g.params) p.zero_grad_();
  }
  int64_t step_count() const { return step_; }
  bool is_offloaded() const { return offload_; }
  void set_lr(float lr) {
    for (ParamGroup& g : groups_) g.lr = lr;
  }
  float lr() const { return groups_.empty() ? 0.0f : groups_.front().lr; }
  // Allocates (zeroed) m / v on first use: before step(), or before state is loaded at resume.
  void ensure_state_initialized() {
    if (!state_.empty()) return;
    std::vector<Tensor> all;
    for (const ParamGroup& g : groups_) all.insert(all.end(), g.params.begin(), g.params.end());
    arena_ = detail::span_of(all);
    if (arena_.ok) {
      const size_t bytes = static_cast<size_t>(arena_.hi - arena_.lo) * 4;
      m_arena_ = make_storage(bytes, cuda_allocator());
      v_arena_ = make_storage(bytes, cuda_allocator());
      CTD_CUDA_CHECK(cudaMemsetAsync(m_arena_->data(), 0, bytes, nullptr));
      CTD_CUDA_CHECK(cudaMemsetAsync(v_arena_->data(), 0, bytes, nullptr));
    }
    for (const ParamGroup& g : groups_) {
      state_.emplace_back();
      for (const Tensor& p : g.params) {
        State st;
        if (arena_.ok) {
          st.m = Tensor::view_of(m_arena_, p.storage_offset() - arena_.lo, p.shape(), DType::kFloat32);
          st.v = Tensor::view_of(v_arena_, p.storage_offset() - arena_.lo, p.shape(), DType::kFloat32);
        } else {
          st.m = Tensor::zeros(p.shape(), DType::kFloat32, p.device());
          st.v = Tensor::zeros(p.shape(), DType::kFloat32, p.device());
        }
        state_.back().push_back(std::move(st));
      }
    }
  }
  void set_step_count(int64_t s) { step_ = s; }
  size_t num_groups() const { return groups_.size(); }
  size_t num_params(size_t gi) const { return groups_.at(gi).params.size(); }
  Tensor& m_tensor(size_t gi, size_t pi) { return state_.at(gi).at(pi).m; }
  Tensor& v_tensor(size_t gi, size_t pi) { return state_.at(gi).at(pi).v; }

 private:
  struct State {
    Tensor m;
    Tensor v;
  };

  // One launch over the arena. Needs one learning rate, every gradient present and laid out like
  // the parameters in one gradient arena; returns false (nothing done) otherwise.
  bool fused_step(float bc1, float bc2) {
    std::vector<Tensor> grads;
    for (const ParamGroup& g : groups_) {
      if (g.lr != groups_.front().lr) return false;
      for (const Tensor& p : g.params) {
        Tensor gr = p.grad();
        if (!gr.storage() || gr.storage_offset() != p.storage_offset() || gr.numel() != p.numel()) return false;
        grads.push_back(std::move(gr));
      }
    }
    const detail::Span gs = detail::span_of(grads);
    if (!gs.ok || gs.lo != arena_.lo || gs.hi != arena_.hi) return false;
    if (!seg_end_.storage()) {
      // weight-decay ranges: tensors in arena order, a tensor's range runs to the start of the next
      struct Item {
        int64_t off;
        float wd;
      };
      std::vector<Item> items;
      for (const ParamGroup& g : groups_)
        for (const Tensor& p : g.params) items.push_back({p.storage_offset() - arena_.lo, g.weight_decay});
      std::sort(items.begin(), items.end(), [](const Item& a, const Item& b) { return a.off < b.off; });
      std::vector<int64_t> ends;
      std::vector<float> wds;
      for (size_t i = 0; i < items.size(); ++i) {
        const int64_t end = i + 1 < items.size() ? items[i + 1].off : arena_.hi - arena_.lo;
        if (end % 4 != 0) return false;
        if (!wds.empty() && wds.back() == items[i].wd) ends.back() = end;
        else {
          ends.push_back(end);
          wds.push_back(items[i].wd);
        }
      }
      if (ends.size() > 2048) return false;
      seg_end_ = Tensor::from_host(ends.data(), {static_cast<int64_t>(ends.size())}, DType::kInt64, kCUDA0);
      seg_wd_ = Tensor::from_host(wds.data(), {static_cast<int64_t>(wds.size())}, DType::kFloat32, kCUDA0);
    }
    const ctdk_adamw_params hp{groups_.front().lr, beta1_, beta2_, eps_, 0.0f, bc1, bc2};
    float* p0 = static_cast<float*>(arena_.storage->data()) + arena_.lo;
    const float* g0 = static_cast<const float*>(gs.storage->data()) + gs.lo;
    detail::ctdk_ok(ctdk_adamw(p0, g0, static_cast<float*>(m_arena_->data()), static_cast<float*>(v_arena_->data()), arena_.hi - arena_.lo,
                               &hp, nullptr, static_cast<const int64_t*>(seg_end_.data_ptr()), static_cast<const float*>(seg_wd_.data_ptr()),
                               static_cast<int>(seg_end_.numel()), nullptr));
    return true;
  }

  std::vector<ParamGroup> groups_;
  std::vector<std::vector<State>> state_;
  float beta1_, beta2_, eps_;
  int64_t step_ = 0;
  bool offload_ = false;
  detail::Span arena_;
  StoragePtr m_arena_, v_arena_;
  Tensor seg_end_, seg_wd_;
};

// Global L2 norm of the parameters' gradients; scales them in place by max_norm / (norm + eps)
// when the norm exceeds max_norm; returns the norm before clipping.
inline float clip_grad_norm_(const std::vector<Tensor>& params, float max_norm, float eps = 1e-6f) {
  std::vector<Tensor> grads;
  for (const Tensor& p : params) {
    Tensor g = p.grad();
    if (g.storage()) grads.push_back(std::move(g));
  }
  if (grads.empty()) return 0.0f;
  Tensor acc = Tensor::zeros({4}, DType::kFloat32, kCUDA0);
  float* a = static_cast<float*>(acc.data_ptr());
  const detail::Span gs = detail::span_of(grads);
  int64_t covered = 0;
  for (const Tensor& g : grads) covered += (g.numel() + 63) / 64 * 64;
  // one launch when the gradients tile one arena (the gaps are padding, which holds zeros)
  const bool whole = gs.ok && covered >= gs.hi - gs.lo;
  if (whole) {
    detail::ctdk_ok(ctdk_sumsq(static_cast<const float*>(gs.storage->data()) + gs.lo, gs.hi - gs.lo, a, nullptr));
  } else {
    for (const Tensor& g : grads) detail::ctdk_ok(ctdk_sumsq(detail::f(g), g.numel(), a, nullptr));
  }
  detail::ctdk_ok(ctdk_clip_scale(a, max_norm, eps, a + 1, a + 2, nullptr));
  float h[4];
  acc.copy_to_host(h);
  if (h[1] != 1.0f) {
    if (whole) {
      float* g0 = static_cast<float*>(gs.storage->data()) + gs.lo;
      detail::ctdk_ok(ctdk_scale(g0, h[1], g0, gs.hi - gs.lo, nullptr));
    } else {
      for (const Tensor& g : grads) detail::ctdk_ok(ctdk_scale(detail::f(g), h[1], detail::f(g), g.numel(), nullptr));
    }
  }
  return h[2];
}

}  // namespace ctd::optim
