// The general part of the C++ `ctd::` surface (include/ctd/*.h): the autograd tape on arbitrary
// graphs, the stand-alone ops (softmax, permute, repeat_kv, causal mask, mse / cross-entropy, KV
// cache copies), the layer objects (nn::Linear ... nn::TransformerBlock, nn::KVCache), the three
// ways a model trains (per-layer tape nodes, with activation checkpointing, the fused step engine
// of a built model), cached inference, SGD and the device sampler. Shaped after the reference's
// gtest cases (emberlm tests/test_autograd.cpp, test_softmax.cpp, test_permute.cpp, test_mask.cpp,
// test_kv_cache.cpp, test_train_forward.cpp, test_sampling.cpp) with CPU loops as the oracle; a few
// macros stand in for gtest. Prints one "[ OK ]"/"[FAIL]" line per case; exit code 1 if any failed.
// Needs a B200; built and run by tests/test_cpp_api.py.
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstdio>
#include <functional>
#include <numeric>
#include <random>
#include <string>
#include <vector>

#include "ctd/autograd.h"
#include "ctd/nn/kv_cache.h"
#include "ctd/nn/model.h"
#include "ctd/ops/elementwise.h"
#include "ctd/ops/kv_cache.h"
#include "ctd/ops/loss.h"
#include "ctd/ops/mask.h"
#include "ctd/ops/matmul.h"
#include "ctd/ops/norm.h"
#include "ctd/ops/permute.h"
#include "ctd/ops/repeat_kv.h"
#include "ctd/ops/rope.h"
#include "ctd/ops/softmax.h"
#include "ctd/optim.h"
#include "ctd/sampling.h"
#include "ctd/tensor.h"

using namespace ctd;

namespace {

struct Case {
  const char* name;
  std::function<void()> fn;
};
std::vector<Case>& cases() {
  static std::vector<Case> c;
  return c;
}
struct Reg {
  Reg(const char* n, std::function<void()> f) { cases().push_back({n, std::move(f)}); }
};
int g_fail = 0;
#define CASE(NAME)                           \
  static void case_##NAME();                 \
  static Reg reg_##NAME(#NAME, case_##NAME); \
  static void case_##NAME()
#define CHECK(COND)                                                            \
  do {                                                                         \
    if (!(COND)) {                                                             \
      std::printf("    %s:%d: CHECK(%s) failed\n", __FILE__, __LINE__, #COND); \
      ++g_fail;                                                                \
    }                                                                          \
  } while (0)
#define CHECK_NEAR(A, B, TOL)                                                                 \
  do {                                                                                        \
    const double a_ = (A), b_ = (B);                                                          \
    if (!(std::fabs(a_ - b_) <= (TOL))) {                                                     \
      std::printf("    %s:%d: |%g - %g| > %g\n", __FILE__, __LINE__, a_, b_, (double)(TOL)); \
      ++g_fail;                                                                               \
    }                                                                                         \
  } while (0)
#define CHECK_THROWS(EXPR)                                                 \
  do {                                                                     \
    bool threw_ = false;                                                   \
    try {                                                                  \
      (void)(EXPR);                                                        \
    } catch (const std::runtime_error&) {                                  \
      threw_ = true;                                                       \
    }                                                                      \
    if (!threw_) {                                                         \
      std::printf("    %s:%d: no throw: %s\n", __FILE__, __LINE__, #EXPR); \
      ++g_fail;                                                            \
    }                                                                      \
  } while (0)

std::vector<float> randn(size_t n, unsigned seed, float lo = -1.0f, float hi = 1.0f) {
  std::mt19937 rng(seed);
  std::uniform_real_distribution<float> d(lo, hi);
  std::vector<float> v(n);
  for (auto& x : v) x = d(rng);
  return v;
}
Tensor dev(const std::vector<float>& h, std::vector<int64_t> shape) { return Tensor::from_host(h.data(), std::move(shape), DType::kFloat32, kCUDA0); }
Tensor dev_i64(const std::vector<int64_t>& h, std::vector<int64_t> shape) { return Tensor::from_host(h.data(), std::move(shape), DType::kInt64, kCUDA0); }
std::vector<float> host(const Tensor& t) {
  std::vector<float> h(static_cast<size_t>(t.numel()));
  t.copy_to_host(h.data());
  return h;
}
double rel_max(const std::vector<float>& a, const std::vector<float>& b) {
  double d = 0.0, s = 1e-30;
  for (size_t i = 0; i < a.size(); ++i) {
    d = std::max(d, std::fabs(static_cast<double>(a[i]) - b[i]));
    s = std::max(s, std::fabs(static_cast<double>(b[i])));
  }
  return d / s;
}

// d(loss)/dx by central differences of a scalar-valued function of one device tensor.
std::vector<float> finite_diff(const std::vector<float>& x0, std::vector<int64_t> shape, const std::function<float(const Tensor&)>& loss,
                               float h, const std::vector<size_t>& probes) {
  std::vector<float> g(probes.size());
  for (size_t k = 0; k < probes.size(); ++k) {
    auto xp = x0, xm = x0;
    xp[probes[k]] += h;
    xm[probes[k]] -= h;
    g[k] = (loss(dev(xp, shape)) - loss(dev(xm, shape))) / (2 * h);
  }
  return g;
}

nn::LlamaConfig tiny_config(bool qk_norm, int head_dim) {
  nn::LlamaConfig c{};
  c.vocab_size = 320;
  c.hidden_size = 128;
  c.intermediate_size = 256;
  c.num_hidden_layers = 2;
  c.num_attention_heads = 128 / head_dim * 2;
  c.num_key_value_heads = 128 / head_dim;
  c.head_dim = head_dim;
  c.max_position_embeddings = 2048;
  c.rms_norm_eps = 1e-5f;
  c.rope_theta = 10000.0f;
  c.tie_word_embeddings = true;
  c.qk_norm = qk_norm;
  return c;
}
TensorDict random_weights(const nn::LlamaConfig& c, unsigned seed) {
  std::mt19937 rng(seed);
  std::normal_distribution<float> nd(0.0f, 0.05f);
  std::uniform_real_distribution<float> un(0.8f, 1.2f);
  TensorDict w;
  auto mat = [&](const std::string& name, int64_t r, int64_t k) {
    std::vector<float> h(static_cast<size_t>(r * k));
    for (auto& v : h) v = nd(rng);
    w[name] = Tensor::from_host(h.data(), {r, k}, DType::kFloat32, kCUDA0);
  };
  auto vec = [&](const std::string& name, int64_t n) {
    std::vector<float> h(static_cast<size_t>(n));
    for (auto& v : h) v = un(rng);
    w[name] = Tensor::from_host(h.data(), {n}, DType::kFloat32, kCUDA0);
  };
  const int64_t hid = c.hidden_size, I = c.intermediate_size, D = c.head_dim, H = c.num_attention_heads, Hk = c.num_key_value_heads;
  mat("model.embed_tokens.weight", c.vocab_size, hid);
  for (int l = 0; l < c.num_hidden_layers; ++l) {
    const std::string p = "model.layers." + std::to_string(l) + ".";
    vec(p + "input_layernorm.weight", hid);
    mat(p + "self_attn.q_proj.weight", H * D, hid);
    mat(p + "self_attn.k_proj.weight", Hk * D, hid);
    mat(p + "self_attn.v_proj.weight", Hk * D, hid);
    mat(p + "self_attn.o_proj.weight", hid, H * D);
    if (c.qk_norm) {
      vec(p + "self_attn.q_norm.weight", D);
      vec(p + "self_attn.k_norm.weight", D);
    }
    vec(p + "post_attention_layernorm.weight", hid);
    mat(p + "mlp.gate_proj.weight", I, hid);
    mat(p + "mlp.up_proj.weight", I, hid);
    mat(p + "mlp.down_proj.weight", hid, I);
  }
  vec("model.norm.weight", hid);
  return w;
}

}  // namespace

// ---------------------------------------------------------------- stand-alone ops
CASE(Softmax_MatchesCpuAndSurvivesExtremes) {
  const int R = 37, W = 301;
  auto x = randn(static_cast<size_t>(R) * W, 1, -6.0f, 6.0f);
  for (int j = 0; j < W; ++j) x[j] = (j == 5) ? 1e4f : -1e4f;            // one huge entry: p = onehot, no NaN
  for (int j = 0; j < W; ++j) x[W + j] = -FLT_MAX;                         // a fully masked row: uniform
  auto y = host(ops::softmax(dev(x, {R, W})));
  for (int r = 0; r < R; ++r) {
    double mx = -1e300, s = 0.0;
    for (int j = 0; j < W; ++j) mx = std::max<double>(mx, x[r * W + j]);
    for (int j = 0; j < W; ++j) s += std::exp(x[r * W + j] - mx);
    for (int j = 0; j < W; j += 17) CHECK_NEAR(y[r * W + j], std::exp(x[r * W + j] - mx) / s, 2e-6);
  }
  CHECK(y[5] == 1.0f && y[4] == 0.0f);
  CHECK_NEAR(y[W + 3], 1.0 / W, 1e-7);
}
CASE(Permute_IndexMapAndInverse) {
  const std::vector<int64_t> shape = {2, 3, 4, 5};
  std::vector<float> x(120);
  std::iota(x.begin(), x.end(), 0.0f);
  Tensor X = dev(x, shape);
  auto y = host(ops::permute(X, {0, 2, 1, 3}));
  for (int a = 0; a < 2; ++a)
    for (int c = 0; c < 4; ++c)
      for (int b = 0; b < 3; ++b)
        for (int d = 0; d < 5; ++d) CHECK(y[((a * 4 + c) * 3 + b) * 5 + d] == x[((a * 3 + b) * 4 + c) * 5 + d]);
  Tensor P = ops::permute(X, {3, 1, 0, 2});
  CHECK(P.shape() == (std::vector<int64_t>{5, 3, 2, 4}));
  CHECK(host(ops::permute(P, {2, 1, 3, 0})) == x);   // the inverse permutation restores the input
  CHECK_THROWS(ops::permute(X, {0, 1, 2}));
  CHECK_THROWS(ops::permute(X, {0, 1, 1, 3}));
}
CASE(RepeatKv_ExpandsAndSumsBack) {
  const int B = 2, T = 3, Hk = 2, D = 8, G = 3;
  auto x = randn(static_cast<size_t>(B) * T * Hk * D, 2);
  Tensor Y = ops::repeat_kv_heads(dev(x, {B, T, Hk, D}), G);
  CHECK(Y.shape() == (std::vector<int64_t>{B, T, Hk * G, D}));
  auto y = host(Y);
  for (int r = 0; r < B * T; ++r)
    for (int h = 0; h < Hk * G; ++h)
      for (int d = 0; d < D; ++d) CHECK(y[(r * Hk * G + h) * D + d] == x[(r * Hk + h / G) * D + d]);
  auto s = host(ops::repeat_kv_sum_impl(Y, G));
  for (size_t i = 0; i < x.size(); ++i) CHECK_NEAR(s[i], 3.0 * x[i], 1e-6);
}
CASE(CausalMask_PatternsWithOffset) {
  const int M = 3, Tq = 4, Tk = 7;
  auto x = randn(static_cast<size_t>(M) * Tq * Tk, 3);
  for (int start : {0, 3}) {
    auto y = host(ops::apply_causal_mask(dev(x, {M, Tq, Tk}), start));
    auto g = host(ops::causal_mask_backward_impl(dev(x, {M, Tq, Tk}), start));
    for (int m = 0; m < M; ++m)
      for (int i = 0; i < Tq; ++i)
        for (int j = 0; j < Tk; ++j) {
          const size_t k = (static_cast<size_t>(m) * Tq + i) * Tk + j;
          const bool dead = j > start + i;
          CHECK(y[k] == (dead ? -FLT_MAX : x[k]));
          CHECK(g[k] == (dead ? 0.0f : x[k]));
        }
  }
  Tensor S = dev(x, {M, Tq, Tk});
  ops::apply_causal_mask_inplace(S, 1);
  CHECK(host(S)[3] == -FLT_MAX && host(S)[1] == x[1]);
}
CASE(KvCache_WriteThenReadExpanded) {
  const int B = 2, H = 2, D = 4, MAXS = 6, G = 2;
  Tensor cache = Tensor::zeros({B, H, MAXS, D}, DType::kFloat32, kCUDA0);
  auto a = randn(static_cast<size_t>(B) * 3 * H * D, 4), b = randn(static_cast<size_t>(B) * 1 * H * D, 5);
  ops::write_kv_inplace(cache, dev(a, {B, 3, H, D}), 0);
  ops::write_kv_inplace(cache, dev(b, {B, 1, H, D}), 3);
  Tensor R = ops::read_kv_expanded(cache, 4, G);
  CHECK(R.shape() == (std::vector<int64_t>{B, H * G, 4, D}));
  auto r = host(R);
  for (int bb = 0; bb < B; ++bb)
    for (int ho = 0; ho < H * G; ++ho)
      for (int t = 0; t < 4; ++t)
        for (int d = 0; d < D; ++d) {
          const int h = ho / G;
          const float want = t < 3 ? a[((bb * 3 + t) * H + h) * D + d] : b[(bb * H + h) * D + d];
          CHECK(r[((bb * H * G + ho) * 4 + t) * D + d] == want);
        }
  CHECK_THROWS(ops::write_kv_inplace(cache, dev(a, {B, 3, H, D}), 4));   // 4 + 3 > 6
  CHECK_THROWS(ops::read_kv_expanded(cache, 7, G));
  CHECK_THROWS(ops::read_kv_expanded(cache, 2, 0));
}
CASE(Losses_MseAndCrossEntropyMatchCpu) {
  const int N = 11, V = 57;
  auto p = randn(N * V, 6), t = randn(N * V, 7);
  double mse = 0.0;
  for (int i = 0; i < N * V; ++i) mse += (static_cast<double>(p[i]) - t[i]) * (p[i] - t[i]);
  CHECK_NEAR(host(ops::mse_loss(dev(p, {N, V}), dev(t, {N, V})))[0], mse / (N * V), 1e-6);
  std::vector<int64_t> tg(N);
  for (int i = 0; i < N; ++i) tg[i] = (i * 13 + 2) % V;
  double ce = 0.0;
  for (int i = 0; i < N; ++i) {
    double mx = -1e300, s = 0.0;
    for (int j = 0; j < V; ++j) mx = std::max<double>(mx, p[i * V + j]);
    for (int j = 0; j < V; ++j) s += std::exp(p[i * V + j] - mx);
    ce += mx + std::log(s) - p[i * V + tg[i]];
  }
  CHECK_NEAR(host(ops::cross_entropy(dev(p, {N, V}), dev_i64(tg, {N})))[0], ce / N, 2e-6);
}

// ---------------------------------------------------------------- tape
CASE(Autograd_LeafRulesAndNoGrad) {
  Tensor a = dev(randn(6, 8), {2, 3}), b = dev(randn(6, 9), {2, 3});
  a.requires_grad_(true);
  Tensor c = ops::mul(a, b);
  CHECK(c.requires_grad() && c.autograd_meta()->grad_fn != nullptr && std::string(c.autograd_meta()->grad_fn->name()) == "MulBackward");
  CHECK_THROWS(c.requires_grad_(true));    // not a leaf
  CHECK_THROWS(c.backward());              // not a scalar
  CHECK_THROWS(b.backward());              // no grad_fn
  {
    autograd::NoGradGuard ng;
    CHECK(!autograd::is_grad_enabled());
    CHECK(!ops::mul(a, b).requires_grad());
  }
  CHECK(autograd::is_grad_enabled());
  Tensor d = a.detach();
  CHECK(!d.requires_grad() && d.data_ptr() == a.data_ptr());
  Tensor x = dev(randn(6, 10), {6}), y = dev(randn(5, 11), {5});
  CHECK_THROWS(autograd::accumulate_inplace(x, y));
}
CASE(Autograd_FanOutAccumulatesAndSecondBackwardAdds) {
  // loss = mse(a*a + a, 0): a reaches the loss through three edges
  auto a0 = randn(64, 12);
  Tensor a = dev(a0, {8, 8});
  a.requires_grad_(true);
  Tensor zero = Tensor::zeros({8, 8}, DType::kFloat32, kCUDA0);
  auto run = [&]() { ops::mse_loss(ops::add(ops::mul(a, a), a), zero).backward(); };
  run();
  auto g1 = host(a.grad());
  for (int i = 0; i < 64; ++i) {
    const double v = a0[i], f = v * v + v;
    CHECK_NEAR(g1[i], 2.0 * f * (2 * v + 1) / 64.0, 1e-6);
  }
  run();   // gradients accumulate until zero_grad_
  auto g2 = host(a.grad());
  for (int i = 0; i < 64; ++i) CHECK_NEAR(g2[i], 2.0 * g1[i], 1e-6);
  a.zero_grad_();
  CHECK(a.grad().storage() == nullptr);
}
CASE(Autograd_OpGradientsMatchFiniteDifferences) {
  // y = softmax(mask(scale * bmm(permute(rope(rms_norm(x W^T))), K^T))) V, loss = mse(y, target):
  // every stand-alone op of the attention chain on one tape, against central differences
  const int B = 2, T = 6, H = 2, D = 8, HID = 16;
  auto x0 = randn(static_cast<size_t>(B) * T * HID, 13);
  auto w0 = randn(static_cast<size_t>(H) * D * HID, 14, -0.5f, 0.5f);
  auto nw0 = randn(D, 15, 0.5f, 1.5f);
  auto k0 = randn(static_cast<size_t>(B) * H * T * D, 16), v0 = randn(static_cast<size_t>(B) * H * T * D, 17);
  auto tg0 = randn(static_cast<size_t>(B) * H * T * D, 18);
  Tensor K = dev(k0, {B * H, T, D}), V = dev(v0, {B * H, T, D}), TG = dev(tg0, {B * H, T, D});
  auto forward = [&](const Tensor& x, const Tensor& w, const Tensor& nw) {
    Tensor q = ops::matmul(x.reshape({B * T, HID}), w, false, true).reshape({B, T, H, D});
    q = ops::rope(ops::rms_norm(q, nw, 1e-5f), 0, 10000.0f);
    Tensor q3 = ops::permute(q, {0, 2, 1, 3}).reshape({B * H, T, D});
    Tensor s = ops::mul_scalar(ops::bmm(q3, K, false, true), 1.0f / std::sqrt(static_cast<float>(D)));
    Tensor y = ops::bmm(ops::softmax(ops::apply_causal_mask(s, 0)), V, false, false);
    return ops::mse_loss(ops::silu(y), TG);
  };
  Tensor x = dev(x0, {B, T, HID}), w = dev(w0, {H * D, HID}), nw = dev(nw0, {D});
  x.requires_grad_(true);
  w.requires_grad_(true);
  nw.requires_grad_(true);
  forward(x, w, nw).backward();
  auto gx = host(x.grad()), gw = host(w.grad()), gn = host(nw.grad());
  const std::vector<size_t> px = {0, 17, 95, 191}, pw = {3, 100, 255}, pn = {0, 5, 7};
  // TF32 products: a coarse step keeps the difference quotient above the rounding of the loss
  auto fx = finite_diff(x0, {B, T, HID}, [&](const Tensor& t) { return host(forward(t, w.detach(), nw.detach()))[0]; }, 5e-2f, px);
  auto fw = finite_diff(w0, {H * D, HID}, [&](const Tensor& t) { return host(forward(x.detach(), t, nw.detach()))[0]; }, 5e-2f, pw);
  auto fn = finite_diff(nw0, {D}, [&](const Tensor& t) { return host(forward(x.detach(), w.detach(), t))[0]; }, 5e-2f, pn);
  double scale = 0.0;
  for (float g : gx) scale = std::max<double>(scale, std::fabs(g));
  for (size_t i = 0; i < px.size(); ++i) CHECK_NEAR(gx[px[i]], fx[i], 0.05 * scale + 2e-4);
  scale = 0.0;
  for (float g : gw) scale = std::max<double>(scale, std::fabs(g));
  for (size_t i = 0; i < pw.size(); ++i) CHECK_NEAR(gw[pw[i]], fw[i], 0.05 * scale + 2e-4);
  scale = 0.0;
  for (float g : gn) scale = std::max<double>(scale, std::fabs(g));
  for (size_t i = 0; i < pn.size(); ++i) CHECK_NEAR(gn[pn[i]], fn[i], 0.05 * scale + 2e-4);
}
CASE(Autograd_EmbeddingRepeatKvAndTransposedProducts) {
  // rows of the table used twice get both contributions; the four transpose cases of matmul backward
  const int V = 10, H = 6;
  auto e0 = randn(V * H, 19);
  Tensor E = dev(e0, {V, H});
  E.requires_grad_(true);
  Tensor ids = dev_i64({3, 7, 3, 0}, {4});
  Tensor tgt = Tensor::zeros({4, H}, DType::kFloat32, kCUDA0);
  ops::mse_loss(ops::embedding(ids, E), tgt).backward();
  auto g = host(E.grad());
  for (int j = 0; j < H; ++j) {
    CHECK_NEAR(g[3 * H + j], 2.0 * 2.0 * e0[3 * H + j] / (4 * H), 1e-6);
    CHECK_NEAR(g[7 * H + j], 2.0 * e0[7 * H + j] / (4 * H), 1e-6);
    CHECK(g[5 * H + j] == 0.0f);
  }
  const int M = 5, N = 4, K = 3;
  for (int ta = 0; ta < 2; ++ta)
    for (int tb = 0; tb < 2; ++tb) {
      auto a0 = randn(M * K, 20 + ta), b0 = randn(K * N, 30 + tb);
      Tensor A = dev(a0, ta ? std::vector<int64_t>{K, M} : std::vector<int64_t>{M, K});
      Tensor Bm = dev(b0, tb ? std::vector<int64_t>{N, K} : std::vector<int64_t>{K, N});
      A.requires_grad_(true);
      Bm.requires_grad_(true);
      Tensor C = ops::matmul(A, Bm, ta != 0, tb != 0);
      ops::mse_loss(C, Tensor::zeros({M, N}, DType::kFloat32, kCUDA0)).backward();
      auto c = host(C), ga = host(A.grad());
      // dL/dC = 2 C / (M N); dA[i,k] = sum_j dC[i,j] op(B)[k,j]
      for (int i = 0; i < M; ++i)
        for (int k = 0; k < K; ++k) {
          double want = 0.0;
          for (int j = 0; j < N; ++j) want += 2.0 * c[i * N + j] / (M * N) * (tb ? b0[j * K + k] : b0[k * N + j]);
          CHECK_NEAR(ga[ta ? k * M + i : i * K + k], want, 2e-3);
        }
    }
}
CASE(Autograd_CheckpointEqualsPlain) {
  const int R = 9, HID = 32;
  auto x0 = randn(R * HID, 40), w0 = randn(HID * HID, 41, -0.3f, 0.3f);
  Tensor tgt = Tensor::zeros({R, HID}, DType::kFloat32, kCUDA0);
  std::vector<float> gx[2], gw[2];
  for (int mode = 0; mode < 2; ++mode) {
    Tensor x = dev(x0, {R, HID}), w = dev(w0, {HID, HID});
    x.requires_grad_(true);
    w.requires_grad_(true);
    auto block = [w](const Tensor& t) { return ops::silu(ops::matmul(t, w, false, true)); };
    Tensor h = ops::add(x, x);
    Tensor y = mode ? autograd::checkpoint(block, h) : block(h);
    ops::mse_loss(y, tgt).backward();
    gx[mode] = host(x.grad());
    gw[mode] = host(w.grad());
  }
  CHECK(gx[0] == gx[1] && gw[0] == gw[1]);   // the same kernels on the same values
}

// ---------------------------------------------------------------- layers and models
CASE(Model_ThreeTrainingPathsAgree) {
  for (int variant = 0; variant < 2; ++variant) {
    const nn::LlamaConfig c = tiny_config(variant == 1, variant == 1 ? 128 : 64);
    const int64_t B = 2, T = 40;
    TensorDict w = random_weights(c, 50 + variant);
    std::mt19937 rng(51);
    std::uniform_int_distribution<int> tok(0, c.vocab_size - 1);
    std::vector<int64_t> ids(B * T), tg(B * T);
    std::vector<float> mk(B * T);
    for (int64_t i = 0; i < B * T; ++i) {
      ids[i] = tok(rng);
      tg[i] = tok(rng);
      mk[i] = (i % T) >= 10 && (i % T) < 30 ? 1.0f : 0.0f;
    }
    Tensor I = dev_i64(ids, {B, T}), TG = dev_i64(tg, {B, T}), MK = dev(mk, {B, T});
    std::vector<std::vector<std::vector<float>>> grads;
    std::vector<float> losses;
    for (int path = 0; path < 3; ++path) {   // 0: fused step engine, 1: per-layer tape nodes, 2: those + checkpointing
      nn::Model m = nn::build_model(w, c);
      CHECK(m.fused != nullptr);
      if (path > 0) m.fused.reset();
      m.gradient_checkpointing = path == 2;
      auto named = m.collect_parameters();
      Tensor loss = m.forward_train_masked(I, TG, MK);
      ops::mul_scalar(loss, 0.5f).backward();
      float l = 0.0f;
      loss.copy_to_host(&l);
      losses.push_back(l);
      grads.emplace_back();
      for (auto& kv : named.all) {
        CHECK(kv.second.grad().storage() != nullptr);
        grads.back().push_back(host(kv.second.grad()));
      }
    }
    CHECK_NEAR(losses[1], losses[0], 2e-4 * losses[0]);
    CHECK_NEAR(losses[2], losses[1], 1e-6 * losses[1]);
    for (size_t i = 0; i < grads[0].size(); ++i) {
      const double e01 = rel_max(grads[1][i], grads[0][i]), e12 = rel_max(grads[2][i], grads[1][i]);
      if (e01 > 1e-2 || e12 > 1e-5) {
        std::printf("    variant %d tensor %zu: tape vs engine %g, checkpointed vs plain %g\n", variant, i, e01, e12);
        ++g_fail;
      }
    }
  }
}
CASE(Model_UnmaskedLossEqualsAllOnesMask) {
  const nn::LlamaConfig c = tiny_config(false, 64);
  nn::Model m = nn::build_model(random_weights(c, 60), c);
  std::vector<int64_t> ids(2 * 24), tg(2 * 24);
  for (size_t i = 0; i < ids.size(); ++i) {
    ids[i] = (i * 7) % c.vocab_size;
    tg[i] = (i * 11 + 3) % c.vocab_size;
  }
  Tensor I = dev_i64(ids, {2, 24}), TG = dev_i64(tg, {2, 24});
  Tensor ones = dev(std::vector<float>(48, 1.0f), {2, 24});
  autograd::NoGradGuard ng;
  const float a = host(m.forward_train(I, TG))[0], b = host(m.forward_train_masked(I, TG, ones))[0];
  CHECK_NEAR(a, b, 1e-6 * b);
  nn::Model plain = m;
  plain.fused.reset();
  CHECK_NEAR(host(plain.forward_train(I, TG))[0], a, 2e-4 * a);
}
CASE(Model_CachedDecodingEqualsFullForward) {
  for (int variant = 0; variant < 2; ++variant) {
    const nn::LlamaConfig c = tiny_config(variant == 1, 64);
    nn::Model m = nn::build_model(random_weights(c, 70 + variant), c);
    autograd::NoGradGuard ng;
    const int64_t T = 9;
    std::vector<int64_t> ids(T + 2);
    for (size_t i = 0; i < ids.size(); ++i) ids[i] = (i * 37 + 11) % c.vocab_size;
    Tensor full = m.forward(dev_i64(ids, {1, T + 2}));   // [1, T+2, V]
    CHECK(full.shape() == (std::vector<int64_t>{1, T + 2, c.vocab_size}));
    auto f = host(full);
    nn::KVCache cache = nn::KVCache::allocate(c.num_hidden_layers, c.num_key_value_heads, c.head_dim, 1, 16, kCUDA0);
    auto pre = host(m.forward(dev_i64(std::vector<int64_t>(ids.begin(), ids.begin() + T), {1, T}), &cache, 0));
    CHECK(cache.current_len == T);
    const int V = c.vocab_size;
    std::vector<float> want_pre(f.begin(), f.begin() + T * V);
    CHECK(rel_max(pre, want_pre) < 2e-3);
    for (int step = 0; step < 2; ++step) {
      auto one = host(m.forward(dev_i64({ids[T + step]}, {1, 1}), &cache, static_cast<int>(T + step)));
      std::vector<float> want(f.begin() + (T + step) * V, f.begin() + (T + step + 1) * V);
      CHECK(rel_max(one, want) < 2e-3);
    }
    CHECK(cache.current_len == T + 2);
    // training-time logits are the same function
    CHECK(rel_max(host(m.forward_train_logits(dev_i64(ids, {1, T + 2}))), f) < 2e-3);
  }
}
CASE(Model_AutodetectAndPresets) {
  TensorDict w;
  w["model.embed_tokens.weight"] = Tensor::empty({49152, 960}, DType::kFloat32, kCPU);
  CHECK(nn::autodetect_config(w).num_hidden_layers == 32 && nn::autodetect_smollm2_config(w).num_attention_heads == 15);
  w["model.embed_tokens.weight"] = Tensor::empty({128256, 2048}, DType::kFloat32, kCPU);
  CHECK(nn::autodetect_config(w).rope_scaling_factor == 32.0f && nn::autodetect_config(w).intermediate_size == 8192);
  w["model.embed_tokens.weight"] = Tensor::empty({151936, 1024}, DType::kFloat32, kCPU);
  CHECK(nn::autodetect_config(w).qk_norm && nn::autodetect_config(w).head_dim == 128);
  w["model.embed_tokens.weight"] = Tensor::empty({10, 7}, DType::kFloat32, kCPU);
  CHECK_THROWS(nn::autodetect_config(w));
  CHECK_THROWS(nn::autodetect_config(TensorDict{}));
  CHECK(nn::qwen3_1_7b_config().intermediate_size == 6144 && nn::smollm2_135m_config().num_key_value_heads == 3);
}

// ---------------------------------------------------------------- optimizers, allocator, sampler
CASE(Sgd_StepAndFusedAdamWOnAnArena) {
  auto p0 = randn(12, 80), g0 = randn(12, 81);
  Tensor p = dev(p0, {12});
  p.requires_grad_(true);
  p.mutable_autograd_meta()->grad = dev(g0, {12});
  optim::SGD sgd({p}, 0.1f);
  sgd.step();
  auto p1 = host(p);
  for (int i = 0; i < 12; ++i) CHECK_NEAR(p1[i], p0[i] - 0.1f * g0[i], 1e-7);
  sgd.zero_grad();
  CHECK(p.grad().storage() == nullptr);
  // a built model's parameters: one launch over the arena must equal tensor-by-tensor updates
  const nn::LlamaConfig c = tiny_config(true, 64);
  TensorDict w = random_weights(c, 82);
  std::vector<std::vector<float>> after[2];
  for (int mode = 0; mode < 2; ++mode) {
    nn::Model m = nn::build_model(w, c);
    auto named = m.collect_parameters();
    std::vector<Tensor> all;
    for (auto& kv : named.all) all.push_back(kv.second);
    std::vector<int64_t> ids(2 * 20), tg(2 * 20);
    for (size_t i = 0; i < ids.size(); ++i) {
      ids[i] = (i * 5) % c.vocab_size;
      tg[i] = (i * 3 + 1) % c.vocab_size;
    }
    m.forward_train(dev_i64(ids, {2, 20}), dev_i64(tg, {2, 20})).backward();
    if (mode == 1)   // break the arena layout of the gradients: forces the tensor-by-tensor path
      for (Tensor& t : all) t.mutable_autograd_meta()->grad = dev(host(t.grad()), t.shape());
    const float norm = optim::clip_grad_norm_(all, 0.5f);
    CHECK(norm > 0.5f);
    optim::AdamW opt(std::vector<optim::ParamGroup>{{named.decay, 1e-2f, 0.1f}, {named.no_decay, 1e-2f, 0.0f}}, 0.9f, 0.999f, 1e-8f, false);
    opt.step();
    opt.step();
    CHECK(opt.step_count() == 2 && opt.num_groups() == 2 && opt.m_tensor(0, 0).shape() == named.decay[0].shape());
    for (Tensor& t : all) after[mode].push_back(host(t));
  }
  for (size_t i = 0; i < after[0].size(); ++i) CHECK(rel_max(after[0][i], after[1][i]) < 1e-6);
}
CASE(Allocator_BlocksAreReused) {
  Tensor a = dev(randn(4096, 90), {4096}), b = dev(randn(4096, 91), {4096});
  for (int i = 0; i < 3; ++i) (void)ops::add(ops::mul(a, b), a);
  const size_t before = cuda_arena().reserved_bytes();
  for (int i = 0; i < 50; ++i) (void)ops::add(ops::mul(a, b), a);
  CHECK(cuda_arena().reserved_bytes() == before);   // steady state takes nothing more from the driver
}
namespace {
// The reference sampler on the host (src/core/sampling.cpp:32-93), as the oracle.
int64_t sample_cpu(const std::vector<float>& row, float temperature, int top_k, float top_p, double r) {
  const int64_t V = static_cast<int64_t>(row.size());
  if (temperature <= 0.0f) return std::max_element(row.begin(), row.end()) - row.begin();
  std::vector<float> l(row);
  for (auto& v : l) v *= 1.0f / temperature;
  if (top_k > 0 && top_k < V) {
    std::vector<float> s(l);
    std::nth_element(s.begin(), s.begin() + (top_k - 1), s.end(), std::greater<float>());
    const float th = s[top_k - 1];
    for (auto& v : l) if (v < th) v = -INFINITY;
  }
  const float m = *std::max_element(l.begin(), l.end());
  double sum = 0.0;
  for (auto& v : l) {
    v = std::exp(v - m);
    sum += v;
  }
  const float inv = static_cast<float>(1.0 / sum);
  for (auto& v : l) v *= inv;
  if (top_p > 0.0f && top_p < 1.0f) {
    std::vector<int64_t> idx(V);
    std::iota(idx.begin(), idx.end(), 0);
    std::stable_sort(idx.begin(), idx.end(), [&](int64_t a, int64_t b) { return l[a] > l[b]; });
    std::vector<char> keep(V, 0);
    double cum = 0.0;
    for (int64_t i = 0; i < V; ++i) {
      cum += l[idx[i]];
      keep[idx[i]] = 1;
      if (cum >= top_p) break;
    }
    double s2 = 0.0;
    for (int64_t i = 0; i < V; ++i) {
      if (!keep[i]) l[i] = 0.0f;
      s2 += l[i];
    }
    if (s2 > 0.0) {
      const float inv2 = static_cast<float>(1.0 / s2);
      for (auto& v : l) v *= inv2;
    }
  }
  double c = 0.0;
  for (int64_t i = 0; i < V; ++i) {
    c += l[i];
    if (r < c) return i;
  }
  return V - 1;
}
}  // namespace
CASE(Sampler_MatchesHostReferenceDrawForDraw) {
  const int64_t B = 3, V = 5003;
  auto logits = randn(static_cast<size_t>(B) * V, 95, -4.0f, 4.0f);
  logits[17] = logits[4000] = 9.5f;   // a tie for the maximum: the first index wins
  Tensor L = dev(logits, {B, 1, V});
  std::mt19937_64 unused(0);
  auto greedy = sample(L, SamplerConfig{0.0f, 0, 0.0f}, unused);
  CHECK(greedy[0] == 17);
  for (int64_t b = 0; b < B; ++b) {
    std::vector<float> row(logits.begin() + b * V, logits.begin() + (b + 1) * V);
    CHECK(greedy[b] == sample_cpu(row, 0.0f, 0, 0.0f, 0.0));
  }
  const SamplerConfig cfgs[] = {{1.0f, 0, 0.0f}, {0.7f, 50, 0.0f}, {1.3f, 0, 0.9f}, {0.8f, 40, 0.95f}, {1.0f, 1, 0.0f}, {2.0f, 0, 0.3f}};
  int mismatches = 0, total = 0;
  for (const SamplerConfig& cfg : cfgs)
    for (uint64_t seed = 1; seed <= 12; ++seed) {
      std::mt19937_64 dev_rng(seed), host_rng(seed);
      auto got = sample(L, cfg, dev_rng);
      std::uniform_real_distribution<double> U(0.0, 1.0);
      for (int64_t b = 0; b < B; ++b) {
        std::vector<float> row(logits.begin() + b * V, logits.begin() + (b + 1) * V);
        const int64_t want = sample_cpu(row, cfg.temperature, cfg.top_k, cfg.top_p, U(host_rng));
        mismatches += got[b] != want;
        ++total;
      }
      CHECK(dev_rng == host_rng);   // the same number of draws was taken
    }
  std::printf("    sampler: %d of %d draws differ from the host reference\n", mismatches, total);
  CHECK(mismatches == 0);
  CHECK_THROWS(sample(dev(logits, {B, V}), SamplerConfig{}, unused));
}

int main() {
  int failed_cases = 0;
  for (const Case& c : cases()) {
    const int before = g_fail;
    try {
      c.fn();
    } catch (const std::exception& e) {
      std::printf("    exception: %s\n", e.what());
      ++g_fail;
    }
    const bool ok = g_fail == before;
    std::printf("%s %s\n", ok ? "[ OK ]" : "[FAIL]", c.name);
    failed_cases += ok ? 0 : 1;
  }
  std::printf("%zu cases, %d failed\n", cases().size(), failed_cases);
  return failed_cases ? 1 : 0;
}
