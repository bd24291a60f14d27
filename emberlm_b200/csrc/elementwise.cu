// HBM-bound elementwise kernels: 128-bit loads/stores, grid sized in multiples of the SM
// count, grid-stride loops. Arithmetic follows the reference's elementwise kernels
// (src/ops/elementwise.cu:15-69 in emberlm): silu forward uses the fast __expf, the silu
// derivative uses expf, exactly as there.
#include "common.cuh"

namespace ctdk {
namespace {

enum class Bin { Add, Sub, Mul };

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + __expf(-v)); }
__device__ __forceinline__ float dsilu_f(float v) {
  float s = 1.0f / (1.0f + expf(-v));
  return s + v * s * (1.0f - s);
}

template <Bin OP>
__device__ __forceinline__ float bin(float a, float b) {
  if (OP == Bin::Add) return a + b;
  if (OP == Bin::Sub) return a - b;
  return a * b;
}

template <Bin OP>
__global__ void __launch_bounds__(256) binary_kernel(const float* __restrict__ a,
                                                     const float* __restrict__ b,
                                                     float* __restrict__ out, int64_t n,
                                                     int vec_ok) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (vec_ok) {
    const int64_t n4 = n >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (int64_t i = tid; i < n4; i += stride) {
      float4 x = a4[i], y = b4[i], r;
      r.x = bin<OP>(x.x, y.x);
      r.y = bin<OP>(x.y, y.y);
      r.z = bin<OP>(x.z, y.z);
      r.w = bin<OP>(x.w, y.w);
      o4[i] = r;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) out[i] = bin<OP>(a[i], b[i]);
  } else {
    for (int64_t i = tid; i < n; i += stride) out[i] = bin<OP>(a[i], b[i]);
  }
}

enum class Un { Scale, Silu };

template <Un OP>
__global__ void __launch_bounds__(256) unary_kernel(const float* __restrict__ x, float alpha,
                                                    float* __restrict__ out, int64_t n,
                                                    int vec_ok) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  auto f = [alpha](float v) { return OP == Un::Scale ? alpha * v : silu_f(v); };
  if (vec_ok) {
    const int64_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (int64_t i = tid; i < n4; i += stride) {
      float4 v = x4[i], r;
      r.x = f(v.x);
      r.y = f(v.y);
      r.z = f(v.z);
      r.w = f(v.w);
      o4[i] = r;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) out[i] = f(x[i]);
  } else {
    for (int64_t i = tid; i < n; i += stride) out[i] = f(x[i]);
  }
}

__global__ void __launch_bounds__(256) silu_bwd_kernel(const float* __restrict__ x,
                                                       const float* __restrict__ g,
                                                       float* __restrict__ out, int64_t n,
                                                       int vec_ok) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (vec_ok) {
    const int64_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const float4* g4 = reinterpret_cast<const float4*>(g);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (int64_t i = tid; i < n4; i += stride) {
      float4 v = x4[i], d = g4[i], r;
      r.x = d.x * dsilu_f(v.x);
      r.y = d.y * dsilu_f(v.y);
      r.z = d.z * dsilu_f(v.z);
      r.w = d.w * dsilu_f(v.w);
      o4[i] = r;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) out[i] = g[i] * dsilu_f(x[i]);
  } else {
    for (int64_t i = tid; i < n; i += stride) out[i] = g[i] * dsilu_f(x[i]);
  }
}

// gu is [rows, 2I]: gate in columns [0,I), up in [I,2I). One float4 of act per thread-iter.
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const float* __restrict__ gu,
                                                         float* __restrict__ act, int64_t rows,
                                                         int I4) {
  const int64_t total = rows * I4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const float4* gu4 = reinterpret_cast<const float4*>(gu);
  float4* act4 = reinterpret_cast<float4*>(act);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int64_t r = i / I4;
    const int c = static_cast<int>(i - r * I4);
    const float4 g = gu4[r * 2 * I4 + c];
    const float4 u = gu4[r * 2 * I4 + I4 + c];
    float4 o;
    o.x = silu_f(g.x) * u.x;
    o.y = silu_f(g.y) * u.y;
    o.z = silu_f(g.z) * u.z;
    o.w = silu_f(g.w) * u.w;
    act4[i] = o;
  }
}

// d(gate) = dact * up * silu'(gate);  d(up) = dact * silu(gate)   (MulBackward then
// SiluBackward of the reference: src/ops/elementwise.cu:58-69,206-238).
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const float* __restrict__ gu,
                                                         const float* __restrict__ dact,
                                                         float* __restrict__ dgu, int64_t rows,
                                                         int I4) {
  const int64_t total = rows * I4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const float4* gu4 = reinterpret_cast<const float4*>(gu);
  const float4* da4 = reinterpret_cast<const float4*>(dact);
  float4* dgu4 = reinterpret_cast<float4*>(dgu);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int64_t r = i / I4;
    const int c = static_cast<int>(i - r * I4);
    const float4 g = gu4[r * 2 * I4 + c];
    const float4 u = gu4[r * 2 * I4 + I4 + c];
    const float4 d = da4[i];
    float4 dg, du;
    swiglu_bwd_elem(d.x, g.x, u.x, dg.x, du.x);
    swiglu_bwd_elem(d.y, g.y, u.y, dg.y, du.y);
    swiglu_bwd_elem(d.z, g.z, u.z, dg.z, du.z);
    swiglu_bwd_elem(d.w, g.w, u.w, dg.w, du.w);
    dgu4[r * 2 * I4 + c] = dg;
    dgu4[r * 2 * I4 + I4 + c] = du;
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int grid_for(int64_t work_items, int threads, int ctas_per_sm) {
  int64_t need = (work_items + threads - 1) / threads;
  int64_t cap = static_cast<int64_t>(sm_count()) * ctas_per_sm;
  if (need < 1) need = 1;
  return static_cast<int>(need < cap ? need : cap);
}

template <Bin OP>
int launch_binary(const float* a, const float* b, float* out, int64_t n, void* stream,
                  const char* name) {
  CTDK_REQUIRE(n >= 0, "%s: negative size", name);
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(a && b && out, "%s: null pointer", name);
  const int vec = aligned16(a) && aligned16(b) && aligned16(out);
  binary_kernel<OP><<<grid_for(vec ? n / 4 + 1 : n, 256, 8), 256, 0,
                      static_cast<cudaStream_t>(stream)>>>(a, b, out, n, vec);
  return check_launch(name);
}

}  // namespace
}  // namespace ctdk

using namespace ctdk;

extern "C" {

int ctdk_add(const float* a, const float* b, float* out, int64_t n, void* stream) {
  return launch_binary<Bin::Add>(a, b, out, n, stream, "ctdk_add");
}
int ctdk_sub(const float* a, const float* b, float* out, int64_t n, void* stream) {
  return launch_binary<Bin::Sub>(a, b, out, n, stream, "ctdk_sub");
}
int ctdk_mul(const float* a, const float* b, float* out, int64_t n, void* stream) {
  return launch_binary<Bin::Mul>(a, b, out, n, stream, "ctdk_mul");
}

int ctdk_scale(const float* x, float alpha, float* out, int64_t n, void* stream) {
  CTDK_REQUIRE(n >= 0, "ctdk_scale: negative size");
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(x && out, "ctdk_scale: null pointer");
  const int vec = aligned16(x) && aligned16(out);
  unary_kernel<Un::Scale><<<grid_for(vec ? n / 4 + 1 : n, 256, 8), 256, 0,
                            static_cast<cudaStream_t>(stream)>>>(x, alpha, out, n, vec);
  return check_launch("ctdk_scale");
}

int ctdk_silu(const float* x, float* out, int64_t n, void* stream) {
  CTDK_REQUIRE(n >= 0, "ctdk_silu: negative size");
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(x && out, "ctdk_silu: null pointer");
  const int vec = aligned16(x) && aligned16(out);
  unary_kernel<Un::Silu><<<grid_for(vec ? n / 4 + 1 : n, 256, 8), 256, 0,
                           static_cast<cudaStream_t>(stream)>>>(x, 0.0f, out, n, vec);
  return check_launch("ctdk_silu");
}

int ctdk_silu_bwd(const float* x, const float* g, float* out, int64_t n, void* stream) {
  CTDK_REQUIRE(n >= 0, "ctdk_silu_bwd: negative size");
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(x && g && out, "ctdk_silu_bwd: null pointer");
  const int vec = aligned16(x) && aligned16(g) && aligned16(out);
  silu_bwd_kernel<<<grid_for(vec ? n / 4 + 1 : n, 256, 8), 256, 0,
                    static_cast<cudaStream_t>(stream)>>>(x, g, out, n, vec);
  return check_launch("ctdk_silu_bwd");
}

int ctdk_swiglu_fwd(const float* gu, float* act, int64_t rows, int I, void* stream) {
  CTDK_REQUIRE(rows >= 0 && I > 0, "ctdk_swiglu_fwd: bad shape");
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(gu && act, "ctdk_swiglu_fwd: null pointer");
  CTDK_REQUIRE(I % 4 == 0 && aligned16(gu) && aligned16(act),
               "ctdk_swiglu_fwd: I must be a multiple of 4 and pointers 16-byte aligned");
  swiglu_fwd_kernel<<<grid_for(rows * (I / 4), 256, 8), 256, 0,
                      static_cast<cudaStream_t>(stream)>>>(gu, act, rows, I / 4);
  return check_launch("ctdk_swiglu_fwd");
}

int ctdk_swiglu_bwd(const float* gu, const float* dact, float* dgu, int64_t rows, int I,
                    void* stream) {
  CTDK_REQUIRE(rows >= 0 && I > 0, "ctdk_swiglu_bwd: bad shape");
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(gu && dact && dgu, "ctdk_swiglu_bwd: null pointer");
  CTDK_REQUIRE(I % 4 == 0 && aligned16(gu) && aligned16(dact) && aligned16(dgu),
               "ctdk_swiglu_bwd: I must be a multiple of 4 and pointers 16-byte aligned");
  swiglu_bwd_kernel<<<grid_for(rows * (I / 4), 256, 8), 256, 0,
                      static_cast<cudaStream_t>(stream)>>>(gu, dact, dgu, rows, I / 4);
  return check_launch("ctdk_swiglu_bwd");
}

}  // extern "C"
