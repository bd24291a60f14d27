// Checks of the C++ `ctd::` surface (include/ctd/*.h) against plain CPU loops, shaped after
// the reference's own gtest cases for these ops (tests/test_matmul.cpp, test_bmm.cpp, test_norm.cpp,
// test_rope.cpp, test_elementwise.cpp, test_activations.cpp, test_embedding.cpp, test_tensor.cpp and
// the AdamW / ClipGradNorm / CrossEntropyMasked cases of tests/test_autograd.cpp). There is no gtest
// in this build, so a few macros stand in for it. Prints one "[ OK ]"/"[FAIL]" line per case and
// exits non-zero when any case failed. Needs a B200; built and run by tests/test_cpp_api_gpu.py.
#include <cmath>
#include <cstdio>
#include <functional>
#include <random>
#include <string>
#include <vector>

#include "ctd/autograd.h"
#include "ctd/ops/elementwise.h"
#include "ctd/ops/embedding.h"
#include "ctd/ops/loss.h"
#include "ctd/ops/matmul.h"
#include "ctd/ops/norm.h"
#include "ctd/ops/repeat_kv.h"
#include "ctd/ops/rope.h"
#include "ctd/optim.h"
#include "ctd/tensor.h"

using namespace ctd;

// Attaches a gradient to a leaf the way the tape would (AccumulateGrad stores the first one).
static void set_grad(Tensor& p, const Tensor& g) {
  p.requires_grad_(true);
  p.mutable_autograd_meta()->grad = g;
}

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
#define CASE(NAME)                         \
  static void case_##NAME();               \
  static Reg reg_##NAME(#NAME, case_##NAME); \
  static void case_##NAME()
#define CHECK(COND)                                                   \
  do {                                                                \
    if (!(COND)) {                                                    \
      std::printf("    %s:%d: CHECK(%s) failed\n", __FILE__, __LINE__, #COND); \
      ++g_fail;                                                       \
    }                                                                 \
  } while (0)
#define CHECK_NEAR(A, B, TOL)                                                          \
  do {                                                                                 \
    const double a_ = (A), b_ = (B);                                                   \
    if (!(std::fabs(a_ - b_) <= (TOL))) {                                              \
      std::printf("    %s:%d: |%g - %g| > %g\n", __FILE__, __LINE__, a_, b_, (double)(TOL)); \
      ++g_fail;                                                                        \
    }                                                                                  \
  } while (0)
#define CHECK_THROWS(EXPR)                                          \
  do {                                                              \
    bool threw_ = false;                                            \
    try {                                                           \
      (void)(EXPR);                                                 \
    } catch (const std::runtime_error&) {                           \
      threw_ = true;                                                \
    }                                                               \
    if (!threw_) {                                                  \
      std::printf("    %s:%d: no throw: %s\n", __FILE__, __LINE__, #EXPR); \
      ++g_fail;                                                     \
    }                                                               \
  } while (0)

std::vector<float> randn(size_t n, unsigned seed, float lo = -1.0f, float hi = 1.0f) {
  std::mt19937 rng(seed);
  std::uniform_real_distribution<float> d(lo, hi);
  std::vector<float> v(n);
  for (auto& x : v) x = d(rng);
  return v;
}
Tensor dev(const std::vector<float>& h, std::vector<int64_t> shape) {
  return Tensor::from_host(h.data(), std::move(shape), DType::kFloat32, kCUDA0);
}
Tensor dev_i64(const std::vector<int64_t>& h, std::vector<int64_t> shape) {
  return Tensor::from_host(h.data(), std::move(shape), DType::kInt64, kCUDA0);
}
std::vector<float> host(const Tensor& t) {
  std::vector<float> h(static_cast<size_t>(t.numel()));
  t.copy_to_host(h.data());
  return h;
}
double max_abs_diff(const std::vector<float>& a, const std::vector<double>& b) {
  double m = 0.0;
  for (size_t i = 0; i < a.size(); ++i) m = std::max(m, std::fabs(a[i] - b[i]));
  return m;
}
// C[M,N] = op(A) op(B) in double
std::vector<double> mm_cpu(const std::vector<float>& A, const std::vector<float>& B, int M, int N, int K, bool ta, bool tb) {
  std::vector<double> C(static_cast<size_t>(M) * N, 0.0);
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      double acc = 0.0;
      for (int k = 0; k < K; ++k) acc += static_cast<double>(ta ? A[k * M + i] : A[i * K + k]) * (tb ? B[j * K + k] : B[k * N + j]);
      C[static_cast<size_t>(i) * N + j] = acc;
    }
  return C;
}

}  // namespace

// ---------------------------------------------------------------- Tensor
CASE(Tensor_HostRoundTrip) {
  auto h = randn(3 * 5, 1);
  auto t = dev(h, {3, 5});
  CHECK(t.dim() == 2 && t.numel() == 15 && t.nbytes() == 60 && t.device() == kCUDA0 && t.dtype() == DType::kFloat32);
  CHECK(host(t) == h);
  auto r = t.reshape({5, 3});
  CHECK(r.data_ptr() == t.data_ptr() && r.shape()[0] == 5);
  CHECK_THROWS(t.reshape({4, 4}));
}
CASE(Tensor_ZerosIsZero) {
  auto z = host(Tensor::zeros({7, 9}, DType::kFloat32, kCUDA0));
  for (float v : z) CHECK(v == 0.0f);
}

// ---------------------------------------------------------------- elementwise
CASE(Elementwise_AddSubMulScaleMatchCpu) {
  const size_t n = 1000003;   // odd length: the vector body and the scalar tail both run
  auto a = randn(n, 2), b = randn(n, 3);
  auto A = dev(a, {static_cast<int64_t>(n)}), B = dev(b, {static_cast<int64_t>(n)});
  auto s = host(ops::add(A, B)), d = host(ops::sub_impl(A, B)), m = host(ops::mul(A, B)), c = host(ops::mul_scalar(A, 0.125f));
  bool ok = true;
  for (size_t i = 0; i < n; ++i) ok = ok && s[i] == a[i] + b[i] && d[i] == a[i] - b[i] && m[i] == a[i] * b[i] && c[i] == a[i] * 0.125f;
  CHECK(ok);   // one rounding each: bit-exact
}
CASE(Elementwise_AddRejectsShapeMismatch) {
  auto A = Tensor::zeros({4, 4}, DType::kFloat32, kCUDA0), B = Tensor::zeros({4, 5}, DType::kFloat32, kCUDA0);
  CHECK_THROWS(ops::add(A, B));
  CHECK_THROWS(ops::mul(A, B));
}
CASE(Elementwise_SiluAndBackwardMatchCpu) {
  const size_t n = 4099;
  auto x = randn(n, 4, -6.0f, 6.0f), g = randn(n, 5);
  auto X = dev(x, {static_cast<int64_t>(n)}), G = dev(g, {static_cast<int64_t>(n)});
  auto y = host(ops::silu(X)), dx = host(ops::silu_backward_impl(X, G));
  for (size_t i = 0; i < n; ++i) {
    const double s = 1.0 / (1.0 + std::exp(-static_cast<double>(x[i])));
    CHECK_NEAR(y[i], x[i] * s, 2e-6);
    CHECK_NEAR(dx[i], g[i] * s * (1.0 + x[i] * (1.0 - s)), 2e-6);
    if (g_fail) break;
  }
}

// ---------------------------------------------------------------- matmul / bmm
CASE(Matmul_AllTransposesMatchCpu) {
  const int M = 96, N = 80, K = 72;   // small, off the 128-tile grid: the general path
  auto a = randn(static_cast<size_t>(M) * K, 6), b = randn(static_cast<size_t>(K) * N, 7);
  for (int ta = 0; ta < 2; ++ta)
    for (int tb = 0; tb < 2; ++tb) {
      auto A = ta ? dev(a, {K, M}) : dev(a, {M, K});
      auto B = tb ? dev(b, {N, K}) : dev(b, {K, N});
      auto C = ops::matmul(A, B, ta, tb);
      CHECK(C.shape()[0] == M && C.shape()[1] == N);
      CHECK(max_abs_diff(host(C), mm_cpu(a, b, M, N, K, ta, tb)) < 2e-2);   // TF32 operands, K = 72
    }
}
CASE(Matmul_TensorCoreShapeMatchesCpu) {
  const int M = 256, N = 384, K = 320;
  auto a = randn(static_cast<size_t>(M) * K, 8), b = randn(static_cast<size_t>(N) * K, 9);
  auto C = ops::matmul(dev(a, {M, K}), dev(b, {N, K}), false, true);   // y = x W^T, the Linear layout
  CHECK(max_abs_diff(host(C), mm_cpu(a, b, M, N, K, false, true)) < 4e-2);
}
CASE(Matmul_RejectsInnerDimMismatch) {
  auto A = Tensor::zeros({4, 6}, DType::kFloat32, kCUDA0), B = Tensor::zeros({5, 3}, DType::kFloat32, kCUDA0);
  CHECK_THROWS(ops::matmul(A, B));
}
CASE(Bmm_NoTransposeAndTransposeB) {
  const int Bt = 3, M = 17, N = 19, K = 23;
  auto a = randn(static_cast<size_t>(Bt) * M * K, 10), b = randn(static_cast<size_t>(Bt) * K * N, 11);
  for (int tb = 0; tb < 2; ++tb) {
    auto A = dev(a, {Bt, M, K});
    auto B = tb ? dev(b, {Bt, N, K}) : dev(b, {Bt, K, N});
    auto c = host(ops::bmm(A, B, false, tb));
    for (int i = 0; i < Bt; ++i) {
      std::vector<float> ai(a.begin() + i * M * K, a.begin() + (i + 1) * M * K), bi(b.begin() + i * K * N, b.begin() + (i + 1) * K * N);
      std::vector<float> ci(c.begin() + i * M * N, c.begin() + (i + 1) * M * N);
      CHECK(max_abs_diff(ci, mm_cpu(ai, bi, M, N, K, false, tb)) < 1e-2);
    }
  }
}

// ---------------------------------------------------------------- RMSNorm
CASE(RmsNorm_MatchesCpu) {
  const int rows = 5, H = 576;
  auto x = randn(static_cast<size_t>(rows) * H, 12, -2.0f, 2.0f), w = randn(H, 13, -2.0f, 2.0f);
  auto y = host(ops::rms_norm(dev(x, {1, rows, H}), dev(w, {H}), 1e-5f));
  for (int r = 0; r < rows; ++r) {
    double ss = 0.0;
    for (int i = 0; i < H; ++i) ss += static_cast<double>(x[r * H + i]) * x[r * H + i];
    const double rs = 1.0 / std::sqrt(ss / H + 1e-5);
    for (int i = 0; i < H; ++i) CHECK_NEAR(y[r * H + i], x[r * H + i] * rs * w[i], 1e-4);
  }
}
CASE(RmsNorm_ShapeMismatchThrows) {
  auto x = Tensor::zeros({2, 8}, DType::kFloat32, kCUDA0), w = Tensor::zeros({4}, DType::kFloat32, kCUDA0);
  CHECK_THROWS(ops::rms_norm(x, w, 1e-5f));
}
CASE(RmsNorm_BackwardMatchesCpu) {
  const int rows = 37, H = 192;
  const double eps = 1e-5;
  auto x = randn(static_cast<size_t>(rows) * H, 14), w = randn(H, 15), dy = randn(static_cast<size_t>(rows) * H, 16);
  auto res = ops::rms_norm_backward_impl(dev(dy, {rows, H}), dev(x, {rows, H}), dev(w, {H}), static_cast<float>(eps));
  auto dx = host(res.first), dw = host(res.second);
  std::vector<double> dwr(H, 0.0);
  for (int r = 0; r < rows; ++r) {
    double ss = 0.0, dot = 0.0;
    for (int i = 0; i < H; ++i) ss += static_cast<double>(x[r * H + i]) * x[r * H + i];
    const double rs = 1.0 / std::sqrt(ss / H + eps);
    for (int i = 0; i < H; ++i) dot += static_cast<double>(dy[r * H + i]) * w[i] * x[r * H + i];
    for (int i = 0; i < H; ++i) {
      const double want = rs * dy[r * H + i] * w[i] - x[r * H + i] * rs * rs * rs * dot / H;
      CHECK_NEAR(dx[r * H + i], want, 1e-4);
      dwr[i] += static_cast<double>(dy[r * H + i]) * x[r * H + i] * rs;
    }
  }
  for (int i = 0; i < H; ++i) CHECK_NEAR(dw[i], dwr[i], 1e-4);
}

// ---------------------------------------------------------------- RoPE
namespace {
void rope_cpu(const std::vector<float>& x, std::vector<double>& y, int B, int T, int H, int D, int pos0, float theta, double sign) {
  y.assign(x.size(), 0.0);
  const int half = D / 2;
  for (int b = 0; b < B; ++b)
    for (int t = 0; t < T; ++t)
      for (int h = 0; h < H; ++h)
        for (int i = 0; i < half; ++i) {
          const size_t o = ((static_cast<size_t>(b) * T + t) * H + h) * D;
          const float freq = std::pow(theta, -2.0f * i / D);
          const float ang = static_cast<float>(pos0 + t) * freq;
          const double c = std::cos(ang), s = sign * std::sin(ang);
          y[o + i] = x[o + i] * c - x[o + i + half] * s;
          y[o + i + half] = x[o + i + half] * c + x[o + i] * s;
        }
}
}  // namespace
CASE(Rope_MatchesCpuAndRespectsPositionOffset) {
  const int B = 2, T = 7, H = 3, D = 64;
  auto x = randn(static_cast<size_t>(B) * T * H * D, 17);
  std::vector<double> want;
  for (int pos0 : {0, 11}) {
    rope_cpu(x, want, B, T, H, D, pos0, 10000.0f, 1.0);
    CHECK(max_abs_diff(host(ops::rope(dev(x, {B, T, H, D}), pos0, 10000.0f)), want) < 2e-5);
  }
  auto X = dev(x, {B, T, H, D});
  ops::apply_rope_inplace(X, 11, 10000.0f);
  CHECK(max_abs_diff(host(X), want) < 2e-5);
  // the transpose undoes the rotation
  auto back = host(ops::rope_transpose_impl(X, 11, 10000.0f));
  std::vector<double> xd(x.begin(), x.end());
  CHECK(max_abs_diff(back, xd) < 2e-5);
}
CASE(Rope_ScalingLeavesHighFrequenciesAlone) {
  const int B = 1, T = 4, H = 1, D = 64;
  auto x = randn(static_cast<size_t>(B) * T * H * D, 18);
  ops::RopeScaling sc;
  sc.factor = 32.0f;
  auto plain = host(ops::rope(dev(x, {B, T, H, D}), 100, 500000.0f)), scaled = host(ops::rope(dev(x, {B, T, H, D}), 100, 500000.0f, sc));
  // pair 0 has wavelength 2*pi, far below original_max_pos / high_freq_factor: unchanged;
  // the last pair's wavelength is far above original_max_pos / low_freq_factor: angle divided by 32
  bool first_same = true, last_differs = false;
  for (int t = 0; t < T; ++t) {
    first_same = first_same && plain[t * D] == scaled[t * D];
    last_differs = last_differs || plain[t * D + 31] != scaled[t * D + 31];
  }
  CHECK(first_same);
  CHECK(last_differs);
}

// ---------------------------------------------------------------- embedding
CASE(Embedding_GathersRowsAndBackwardScatters) {
  const int V = 50, H = 48;
  auto w = randn(static_cast<size_t>(V) * H, 19);
  std::vector<int64_t> ids = {3, 49, 0, 3, 17, 3};
  auto I = dev_i64(ids, {2, 3});
  auto out = ops::embedding(I, dev(w, {V, H}));
  CHECK(out.dim() == 3 && out.shape()[2] == H);
  auto o = host(out);
  for (size_t r = 0; r < ids.size(); ++r)
    for (int i = 0; i < H; ++i) CHECK(o[r * H + i] == w[ids[r] * H + i]);
  auto dy = randn(ids.size() * H, 20);
  auto dw = host(ops::embedding_backward_impl(I, dev(dy, {2, 3, H}), V));
  std::vector<double> want(static_cast<size_t>(V) * H, 0.0);
  for (size_t r = 0; r < ids.size(); ++r)
    for (int i = 0; i < H; ++i) want[ids[r] * H + i] += dy[r * H + i];
  CHECK(max_abs_diff(dw, want) < 1e-6);
}

// ---------------------------------------------------------------- masked cross-entropy
namespace {
double ce_cpu(const std::vector<float>& z, const std::vector<int64_t>& t, const std::vector<float>& m, int N, int V) {
  double num = 0.0, den = 0.0;
  for (int i = 0; i < N; ++i) {
    double mx = -1e30, s = 0.0;
    for (int j = 0; j < V; ++j) mx = std::max<double>(mx, z[i * V + j]);
    for (int j = 0; j < V; ++j) s += std::exp(z[i * V + j] - mx);
    num += m[i] * (mx + std::log(s) - z[i * V + t[i]]);
    den += m[i];
  }
  return den > 0 ? num / den : 0.0;
}
}  // namespace
CASE(CrossEntropyMasked_ForwardAndGradientMatchCpu) {
  const int N = 9, V = 131;
  auto z = randn(static_cast<size_t>(N) * V, 21, -3.0f, 3.0f);
  std::vector<int64_t> t(N);
  std::vector<float> m(N);
  for (int i = 0; i < N; ++i) {
    t[i] = (i * 37 + 5) % V;
    m[i] = (i % 3 != 1) ? 1.0f : 0.0f;
  }
  auto Z = dev(z, {N, V});
  auto T = dev_i64(t, {N});
  auto Mk = dev(m, {N});
  const float loss = host(ops::cross_entropy_masked(Z, T, Mk))[0];
  CHECK_NEAR(loss, ce_cpu(z, t, m, N, V), 1e-5);
  CHECK(host(Z) == z);   // the forward leaves the logits alone
  // all-ones mask equals the plain mean over rows; a half mask equals the mean over the kept rows
  std::vector<float> ones(N, 1.0f);
  CHECK_NEAR(host(ops::cross_entropy_masked(Z, T, dev(ones, {N})))[0], ce_cpu(z, t, ones, N, V), 1e-5);
  // gradient against central differences of the CPU loss
  Z.requires_grad_(true);
  ops::cross_entropy_masked(Z, T, Mk).backward();
  auto g = host(Z.grad());
  for (int probe : {0, 57, 2 * V + 3, 4 * V + static_cast<int>(t[4]), 8 * V + 130}) {
    auto zp = z, zm = z;
    zp[probe] += 1e-2f;
    zm[probe] -= 1e-2f;
    const double fd = (ce_cpu(zp, t, m, N, V) - ce_cpu(zm, t, m, N, V)) / 2e-2;
    CHECK_NEAR(g[probe], fd, 1e-4);
  }
  for (int j = 0; j < V; ++j) CHECK(g[1 * V + j] == 0.0f);   // a masked-out row gets exactly zero
}
CASE(CrossEntropyMasked_ZeroSumThrows) {
  const int N = 4, V = 16;
  auto Z = dev(randn(N * V, 22), {N, V});
  auto T = dev_i64(std::vector<int64_t>(N, 1), {N});
  auto Mk = Tensor::zeros({N}, DType::kFloat32, kCUDA0);
  CHECK(host(ops::cross_entropy_masked(Z, T, Mk))[0] == 0.0f);
  Z.requires_grad_(true);
  CHECK_THROWS(ops::cross_entropy_masked(Z, T, Mk).backward());
}

// ---------------------------------------------------------------- optimizer
CASE(AdamW_SingleElementMatchesClosedForm) {
  const float lr = 0.1f, b1 = 0.9f, b2 = 0.95f, eps = 1e-8f, wd = 0.01f;
  float p0 = 1.5f;
  Tensor p = Tensor::from_host(&p0, {1}, DType::kFloat32, kCUDA0);
  p.requires_grad_(true);   // before the optimizer copies the handle: copies share the gradient slot from here on
  optim::AdamW opt({p}, lr, wd, b1, b2, eps);
  double pr = p0, m = 0.0, v = 0.0;
  const float grads[3] = {0.5f, -0.25f, 2.0f};
  for (int s = 1; s <= 3; ++s) {
    set_grad(p, Tensor::from_host(&grads[s - 1], {1}, DType::kFloat32, kCUDA0));
    m = b1 * m + (1 - b1) * grads[s - 1];
    v = b2 * v + (1 - b2) * grads[s - 1] * grads[s - 1];
    const double mh = m / (1 - std::pow(b1, s)), vh = v / (1 - std::pow(b2, s));
    pr = pr - lr * (mh / (std::sqrt(vh) + eps) + wd * pr);
    opt.step();
    CHECK_NEAR(host(p)[0], pr, 2e-6);
  }
  CHECK(opt.step_count() == 3);
}
CASE(AdamW_DecoupledWeightDecayWithZeroGrad) {
  auto h = std::vector<float>(8, 2.0f);
  Tensor p = dev(h, {8});
  p.requires_grad_(true);
  optim::AdamW opt({p}, 0.5f, 0.1f);
  set_grad(p, Tensor::zeros({8}, DType::kFloat32, kCUDA0));   // seen by the optimizer's handle too
  opt.step();
  for (float v : host(p)) CHECK_NEAR(v, 2.0f - 0.5f * 0.1f * 2.0f, 1e-6);   // only the decay term moves it
}
CASE(ClipGradNorm_ScalesDownToMaxAndNoOpUnderMax) {
  std::vector<float> g1 = {3.0f, 0.0f, 0.0f}, g2 = {0.0f, 4.0f};
  Tensor p1 = Tensor::zeros({3}, DType::kFloat32, kCUDA0), p2 = Tensor::zeros({2}, DType::kFloat32, kCUDA0);
  set_grad(p1, dev(g1, {3}));
  set_grad(p2, dev(g2, {2}));
  const float norm = optim::clip_grad_norm_({p1, p2}, 1.0f);
  CHECK_NEAR(norm, 5.0f, 1e-6);
  auto a = host(p1.grad()), b = host(p2.grad());
  CHECK_NEAR(std::sqrt(a[0] * a[0] + b[1] * b[1]), 1.0, 1e-5);
  CHECK_NEAR(a[0] / b[1], 0.75, 1e-6);
  const float norm2 = optim::clip_grad_norm_({p1, p2}, 10.0f);
  CHECK_NEAR(norm2, 1.0f, 1e-5);
  CHECK(host(p1.grad()) == a && host(p2.grad()) == b);   // untouched when under the limit
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
