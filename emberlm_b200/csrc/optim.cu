// Fused AdamW over a flat parameter range, gradient sum of squares and the clip scale.
//
// Arithmetic follows the reference optimizer (emberlm src/core/optim.cu:54-73 for the
// update, 221-293 for clip_grad_norm_): one rounding chain per element,
//   m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g
//   p = p - lr*((m/bc1)/(sqrtf(v/bc2)+eps) + wd*p)
// with the clip scale applied to g first (the reference scales the gradient in place before
// the step). One launch covers every tensor of the range; 128-bit accesses throughout.
#include "common.cuh"

namespace ctdk {
namespace {

constexpr int kMaxSegs = 2048;

__device__ __forceinline__ void adamw_one(float& p, float g, float& m, float& v,
                                          const ctdk_adamw_params& hp, float wd) {
  const float mi = hp.beta1 * m + (1.0f - hp.beta1) * g;
  const float vi = hp.beta2 * v + (1.0f - hp.beta2) * g * g;
  m = mi;
  v = vi;
  const float m_hat = mi / hp.bc1;
  const float v_hat = vi / hp.bc2;
  const float update = m_hat / (sqrtf(v_hat) + hp.eps);
  p = p - hp.lr * (update + wd * p);
}

// seg_end/seg_wd live in shared memory; a float4 never straddles a segment because every
// segment boundary is a multiple of 4 floats.
__global__ void __launch_bounds__(256)
    adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                 float* __restrict__ v, int64_t n, ctdk_adamw_params hp,
                 const float* __restrict__ grad_scale, const int64_t* __restrict__ seg_end,
                 const float* __restrict__ seg_wd, int nseg) {
  extern __shared__ unsigned char smem_raw[];
  int64_t* s_end = reinterpret_cast<int64_t*>(smem_raw);
  float* s_wd = reinterpret_cast<float*>(s_end + nseg);
  for (int i = threadIdx.x; i < nseg; i += blockDim.x) {
    s_end[i] = seg_end[i];
    s_wd[i] = seg_wd[i];
  }
  __syncthreads();
  const float gs = (grad_scale != nullptr) ? *grad_scale : 1.0f;
  const int64_t n4 = n >> 2;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  float4* p4 = reinterpret_cast<float4*>(p);
  const float4* g4 = reinterpret_cast<const float4*>(g);
  float4* m4 = reinterpret_cast<float4*>(m);
  float4* v4 = reinterpret_cast<float4*>(v);
  int seg = 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += stride) {
    float wd = hp.wd;
    if (nseg > 0) {
      const int64_t e = i << 2;
      // Offsets only grow along the grid-stride loop: resume from the previous segment when
      // it still holds, otherwise binary-search the remainder.
      if (!(e < s_end[seg] && (seg == 0 || e >= s_end[seg - 1]))) {
        int lo = seg, hi = nseg - 1;
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (e < s_end[mid]) hi = mid; else lo = mid + 1;
        }
        seg = lo;
      }
      wd = s_wd[seg];
    }
    float4 pv = p4[i], gv = g4[i], mv = m4[i], vv = v4[i];
    adamw_one(pv.x, gv.x * gs, mv.x, vv.x, hp, wd);
    adamw_one(pv.y, gv.y * gs, mv.y, vv.y, hp, wd);
    adamw_one(pv.z, gv.z * gs, mv.z, vv.z, hp, wd);
    adamw_one(pv.w, gv.w * gs, mv.w, vv.w, hp, wd);
    p4[i] = pv;
    m4[i] = mv;
    v4[i] = vv;
  }
  // Scalar tail (n not a multiple of 4): belongs to the last segment.
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const int64_t e = (n4 << 2) + threadIdx.x;
    const float wd = nseg > 0 ? s_wd[nseg - 1] : hp.wd;
    adamw_one(p[e], g[e] * gs, m[e], v[e], hp, wd);
  }
}

// Unaligned fallback, one element per thread-iteration.
__global__ void __launch_bounds__(256)
    adamw_scalar_kernel(float* __restrict__ p, const float* __restrict__ g,
                        float* __restrict__ m, float* __restrict__ v, int64_t n,
                        ctdk_adamw_params hp, const float* __restrict__ grad_scale,
                        const int64_t* __restrict__ seg_end, const float* __restrict__ seg_wd,
                        int nseg) {
  const float gs = (grad_scale != nullptr) ? *grad_scale : 1.0f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    float wd = hp.wd;
    if (nseg > 0) {
      int lo = 0, hi = nseg - 1;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (i < seg_end[mid]) hi = mid; else lo = mid + 1;
      }
      wd = seg_wd[lo];
    }
    adamw_one(p[i], g[i] * gs, m[i], v[i], hp, wd);
  }
}

__global__ void __launch_bounds__(256) sumsq_kernel(const float* __restrict__ g, int64_t n,
                                                    float* __restrict__ out, int vec_ok) {
  __shared__ float red[32];
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  float acc = 0.0f;
  if (vec_ok) {
    const int64_t n4 = n >> 2;
    const float4* g4 = reinterpret_cast<const float4*>(g);
    for (int64_t i = tid; i < n4; i += stride) {
      const float4 x = g4[i];
      acc += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) acc += g[i] * g[i];
  } else {
    for (int64_t i = tid; i < n; i += stride) acc += g[i] * g[i];
  }
  acc = warp_sum(acc);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) red[wid] = acc;
  __syncthreads();
  if (wid == 0) {
    float t = (lane < (blockDim.x >> 5)) ? red[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) atomicAdd(out, t);
  }
}

__global__ void clip_scale_kernel(const float* __restrict__ sumsq, float max_norm, float eps,
                                  float* __restrict__ scale_out, float* __restrict__ norm_out) {
  const float total = sqrtf(*sumsq);
  if (norm_out != nullptr) *norm_out = total;
  if (scale_out != nullptr) *scale_out = (total > max_norm) ? max_norm / (total + eps) : 1.0f;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace ctdk

using namespace ctdk;

extern "C" {

int ctdk_sumsq(const float* g, int64_t n, float* out, void* stream) {
  CTDK_REQUIRE(n >= 0, "ctdk_sumsq: negative size");
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(g && out, "ctdk_sumsq: null pointer");
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int64_t need = (n / 4 + 255) / 256 + 1;
  sumsq_kernel<<<static_cast<int>(need < cap ? need : cap), 256, 0,
                 static_cast<cudaStream_t>(stream)>>>(g, n, out, aligned16(g) ? 1 : 0);
  return check_launch("ctdk_sumsq");
}

int ctdk_clip_scale(const float* sumsq, float max_norm, float eps, float* scale_out,
                    float* norm_out, void* stream) {
  CTDK_REQUIRE(sumsq != nullptr, "ctdk_clip_scale: null pointer");
  clip_scale_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(sumsq, max_norm, eps,
                                                                    scale_out, norm_out);
  return check_launch("ctdk_clip_scale");
}

int ctdk_adamw(float* p, const float* g, float* m, float* v, int64_t n,
               const ctdk_adamw_params* hp, const float* grad_scale, const int64_t* seg_end,
               const float* seg_wd, int nseg, void* stream) {
  CTDK_REQUIRE(n >= 0, "ctdk_adamw: negative size");
  CTDK_REQUIRE(hp != nullptr, "ctdk_adamw: null hyper-parameters");
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(p && g && m && v, "ctdk_adamw: null pointer");
  CTDK_REQUIRE(nseg >= 0 && nseg <= kMaxSegs, "ctdk_adamw: nseg must be in [0, %d]", kMaxSegs);
  CTDK_REQUIRE(nseg == 0 || (seg_end && seg_wd), "ctdk_adamw: null segment table");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  void* tok = prof_begin(CTDK_PROF_ADAMW, 28.0 * static_cast<double>(n), s);
  if (aligned16(p) && aligned16(g) && aligned16(m) && aligned16(v)) {
    const int64_t need = (n / 4 + 255) / 256 + 1;
    const size_t smem = static_cast<size_t>(nseg) * (sizeof(int64_t) + sizeof(float));
    adamw_kernel<<<static_cast<int>(need < cap ? need : cap), 256, smem, s>>>(
        p, g, m, v, n, *hp, grad_scale, seg_end, seg_wd, nseg);
  } else {
    const int64_t need = (n + 255) / 256;
    adamw_scalar_kernel<<<static_cast<int>(need < cap ? need : cap), 256, 0, s>>>(
        p, g, m, v, n, *hp, grad_scale, seg_end, seg_wd, nseg);
  }
  prof_end(tok, s);
  return check_launch("ctdk_adamw");
}

}  // extern "C"
