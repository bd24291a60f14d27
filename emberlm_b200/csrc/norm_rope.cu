// RMSNorm forward/backward, RoPE, and the fused per-head QK-Norm + RoPE kernels.
//
// Arithmetic follows the reference (emberlm src/ops/norm.cu:18-106, src/ops/rope.cu:17-56):
//   scale = rsqrtf(sum(x^2)/H + eps);  y = x*scale*w
//   dx = s*(dy*w - x*s*s*c/H), c = sum(dy*w*x);  dw = sum_rows dy*x*s
//   rope: pairs (i, i+D/2), angle = float(pos)*freq_i, freq_i = theta^(-2i/D) with the
//   llama3 wavelength branches; backward = same rotation with sin negated.
// Differences are in the execution only: one CTA per row with 128-bit accesses and
// warp-shuffle reductions, dw reduced through per-CTA partial rows instead of one atomic per
// element, cos/sin from libm-accurate functions instead of the fast intrinsics.
#include <mutex>

#include "common.cuh"

namespace ctdk {
namespace {

constexpr int kMaxPartialRows = 512;    // QK-Norm backward
constexpr int kNormPartialRows = 2048;  // RMSNorm backward: up to 8 CTAs per SM keep HBM busy

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Block-wide sum of up to two values; `slot` toggles between two smem buffers so that one
// __syncthreads per reduction is enough.
template <int N>
__device__ __forceinline__ void block_sum(float (&v)[N], float* smem /* [2][N][32] */,
                                          int slot) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int k = 0; k < N; ++k) v[k] = warp_sum(v[k]);
  float* s = smem + slot * N * 32;
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < N; ++k) s[k * 32 + wid] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < N; ++k) {
    float t = (lane < nw) ? s[k * 32 + lane] : 0.0f;
    v[k] = warp_sum(t);
  }
}

// ---------------------------------------------------------------------------------------
// RMSNorm forward: one CTA per row (grid-stride), NV float4 per thread kept in registers.
// ---------------------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const float* __restrict__ x,
                                                          const float* __restrict__ w,
                                                          float* __restrict__ y,
                                                          float* __restrict__ rstd,
                                                          int64_t rows, int H4, float inv_H,
                                                          float eps) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[2 * 1 * 32];
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 wv[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    wv[j] = (c < H4) ? w4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // The next row is fetched before the current one is reduced, so a CTA always has two rows of loads
  // in flight across the block-wide reduction (at the SM clock a power-capped step runs at, one row
  // per CTA in flight leaves the kernel latency-bound).
  float4 xn[NV];
  auto fetch = [&](int64_t row) {
    const float4* x4 = reinterpret_cast<const float4*>(x) + row * H4;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = threadIdx.x + j * blockDim.x;
      xn[j] = (c < H4 && row < rows) ? __ldcs(x4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  fetch(blockIdx.x);
  int slot = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, slot ^= 1) {
    float4* y4 = reinterpret_cast<float4*>(y) + row * H4;
    float4 xv[NV];
    float acc[1] = {0.0f};
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      xv[j] = xn[j];
      acc[0] += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
    }
    fetch(row + gridDim.x);
    block_sum<1>(acc, red, slot);
    const float s = rsqrtf(acc[0] * inv_H + eps);
    if (rstd != nullptr && threadIdx.x == 0) rstd[row] = s;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = threadIdx.x + j * blockDim.x;
      if (c < H4) {
        float4 o;
        o.x = xv[j].x * s * wv[j].x;
        o.y = xv[j].y * s * wv[j].y;
        o.z = xv[j].z * s * wv[j].z;
        o.w = xv[j].w * s * wv[j].w;
        y4[c] = o;
      }
    }
  }
}

// Any H / any alignment: scalar loads, row re-read from cache for the second pass.
__global__ void __launch_bounds__(256) rmsnorm_fwd_generic_kernel(const float* __restrict__ x,
                                                                  const float* __restrict__ w,
                                                                  float* __restrict__ y,
                                                                  float* __restrict__ rstd,
                                                                  int64_t rows, int H,
                                                                  float eps) {
  __shared__ float red[2 * 1 * 32];
  int slot = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, slot ^= 1) {
    const float* xr = x + row * H;
    float acc[1] = {0.0f};
    for (int i = threadIdx.x; i < H; i += blockDim.x) acc[0] += xr[i] * xr[i];
    block_sum<1>(acc, red, slot);
    const float s = rsqrtf(acc[0] / static_cast<float>(H) + eps);
    if (rstd != nullptr && threadIdx.x == 0) rstd[row] = s;
    for (int i = threadIdx.x; i < H; i += blockDim.x) y[row * H + i] = xr[i] * s * w[i];
  }
}

// ---------------------------------------------------------------------------------------
// RMSNorm backward. dw partial sums stay in registers across the rows of a CTA and are
// written once per CTA to partial[blockIdx.x][H]; rmsnorm_dw_finalize sums the partial rows.
// ---------------------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(256)
    rmsnorm_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                       const float* __restrict__ w, float* __restrict__ dx,
                       float* __restrict__ partial, int64_t rows, int H4, float inv_H,
                       float eps, int add_to_dx) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[2 * 2 * 32];
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 wv[NV], dwv[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    wv[j] = (c < H4) ? w4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    dwv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // The next row's x and dy are fetched before the current row is reduced, so a CTA always has
  // two rows of loads in flight across the block-wide reductions.
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 xn[NV], gn[NV], pn[NV];
  auto fetch = [&](int64_t row) {
    const float4* x4 = reinterpret_cast<const float4*>(x) + row * H4;
    const float4* g4 = reinterpret_cast<const float4*>(dy) + row * H4;
    const float4* p4 = reinterpret_cast<const float4*>(dx) + row * H4;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = threadIdx.x + j * blockDim.x;
      const bool in = c < H4 && row < rows;
      xn[j] = in ? __ldcs(x4 + c) : zero4;
      gn[j] = in ? __ldcs(g4 + c) : zero4;
      pn[j] = (in && add_to_dx) ? p4[c] : zero4;
    }
  };
  fetch(blockIdx.x);
  int slot = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, slot ^= 1) {
    float4* dx4 = reinterpret_cast<float4*>(dx) + row * H4;
    float4 xv[NV], gv[NV], pv[NV];
    float acc[2] = {0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      xv[j] = xn[j];
      gv[j] = gn[j];
      pv[j] = pn[j];
    }
    fetch(row + gridDim.x);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      acc[0] += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
      acc[1] += gv[j].x * wv[j].x * xv[j].x + gv[j].y * wv[j].y * xv[j].y +
                gv[j].z * wv[j].z * xv[j].z + gv[j].w * wv[j].w * xv[j].w;
    }
    block_sum<2>(acc, red, slot);
    const float s = rsqrtf(acc[0] * inv_H + eps);
    const float k = s * s * acc[1] * inv_H;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = threadIdx.x + j * blockDim.x;
      if (c < H4) {
        float4 o;
        o.x = s * (gv[j].x * wv[j].x - xv[j].x * k);
        o.y = s * (gv[j].y * wv[j].y - xv[j].y * k);
        o.z = s * (gv[j].z * wv[j].z - xv[j].z * k);
        o.w = s * (gv[j].w * wv[j].w - xv[j].w * k);
        o.x += pv[j].x;   // zero unless add_to_dx
        o.y += pv[j].y;
        o.z += pv[j].z;
        o.w += pv[j].w;
        dx4[c] = o;
        dwv[j].x += gv[j].x * xv[j].x * s;
        dwv[j].y += gv[j].y * xv[j].y * s;
        dwv[j].z += gv[j].z * xv[j].z * s;
        dwv[j].w += gv[j].w * xv[j].w * s;
      }
    }
  }
  float4* p4 = reinterpret_cast<float4*>(partial) + static_cast<int64_t>(blockIdx.x) * H4;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < H4) p4[c] = dwv[j];
  }
}

// RMSNorm backward, one WARP per row (H <= 1024): a row is NF float4 per lane, both reductions are
// warp shuffles, so the eight rows of a CTA proceed independently and nothing waits on a block-wide
// barrier between a row's loads and its stores. The CTA-per-row kernel above keeps one row plus one
// prefetched row in flight per CTA and measured 0.70 of the copy bandwidth whatever the SM clock:
// it is bound by bytes in flight. dw: each warp adds into its own row of shared memory, the eight
// rows are summed in a fixed order at the end, one partial row per CTA (grid <= 2 per SM, so the
// finalize pass reads a quarter of the partial rows the other kernel leaves).
template <int NF>
__global__ void __launch_bounds__(256, 2)
    rmsnorm_bwd_rows_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                            const float* __restrict__ w, float* __restrict__ dx,
                            float* __restrict__ partial, int64_t rows, int H4, float inv_H,
                            float eps, int add_to_dx) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float4 sdw4[];   // [8][H4]: each warp's running dw (its own row of shared memory, no atomics)
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4* mydw = sdw4 + wid * H4;
#pragma unroll
  for (int j = 0; j < NF; ++j) {
    const int c = lane + 32 * j;
    if (c < H4) mydw[c] = zero4;
  }
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 8;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + wid; row < rows; row += stride) {
    const float4* x4 = reinterpret_cast<const float4*>(x) + row * H4;
    const float4* g4 = reinterpret_cast<const float4*>(dy) + row * H4;
    float4* dx4 = reinterpret_cast<float4*>(dx) + row * H4;
    float4 xv[NF], gv[NF], pv[NF];   // all of a row's loads are issued before anything waits on them
#pragma unroll
    for (int j = 0; j < NF; ++j) {
      const int c = lane + 32 * j;
      xv[j] = c < H4 ? __ldcs(x4 + c) : zero4;
      gv[j] = c < H4 ? __ldcs(g4 + c) : zero4;
      pv[j] = (c < H4 && add_to_dx) ? dx4[c] : zero4;
    }
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int j = 0; j < NF; ++j) {
      const int c = lane + 32 * j;
      const float4 wv = c < H4 ? __ldg(w4 + c) : zero4;
      a0 += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
      a1 += gv[j].x * wv.x * xv[j].x + gv[j].y * wv.y * xv[j].y + gv[j].z * wv.z * xv[j].z + gv[j].w * wv.w * xv[j].w;
    }
    a0 = warp_sum(a0);
    a1 = warp_sum(a1);
    const float s = rsqrtf(a0 * inv_H + eps);
    const float k = s * s * a1 * inv_H;
#pragma unroll
    for (int j = 0; j < NF; ++j) {
      const int c = lane + 32 * j;
      if (c < H4) {
        const float4 wv = __ldg(w4 + c);
        float4 o;
        o.x = s * (gv[j].x * wv.x - xv[j].x * k) + pv[j].x;   // pv is zero unless add_to_dx
        o.y = s * (gv[j].y * wv.y - xv[j].y * k) + pv[j].y;
        o.z = s * (gv[j].z * wv.z - xv[j].z * k) + pv[j].z;
        o.w = s * (gv[j].w * wv.w - xv[j].w * k) + pv[j].w;
        dx4[c] = o;
        float4 d = mydw[c];
        d.x += gv[j].x * xv[j].x * s;
        d.y += gv[j].y * xv[j].y * s;
        d.z += gv[j].z * xv[j].z * s;
        d.w += gv[j].w * xv[j].w * s;
        mydw[c] = d;
      }
    }
  }
  __syncthreads();
  float4* p4 = reinterpret_cast<float4*>(partial) + static_cast<int64_t>(blockIdx.x) * H4;
  for (int c = threadIdx.x; c < H4; c += blockDim.x) {
    float4 t = sdw4[c];
#pragma unroll
    for (int k2 = 1; k2 < 8; ++k2) {
      const float4 u = sdw4[k2 * H4 + c];
      t.x += u.x;
      t.y += u.y;
      t.z += u.z;
      t.w += u.w;
    }
    p4[c] = t;
  }
}

// Generic backward (any H): partial sums accumulated in the CTA's own partial row in global
// memory (each element is owned by one thread, so no atomics are needed).
__global__ void __launch_bounds__(256)
    rmsnorm_bwd_generic_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                               const float* __restrict__ w, float* __restrict__ dx,
                               float* __restrict__ partial, int64_t rows, int H, float eps,
                               int add_to_dx) {
  __shared__ float red[2 * 2 * 32];
  float* prow = partial + static_cast<int64_t>(blockIdx.x) * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) prow[i] = 0.0f;
  int slot = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, slot ^= 1) {
    const float* xr = x + row * H;
    const float* gr = dy + row * H;
    float acc[2] = {0.0f, 0.0f};
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      acc[0] += xr[i] * xr[i];
      acc[1] += gr[i] * w[i] * xr[i];
    }
    block_sum<2>(acc, red, slot);
    const float inv_H = 1.0f / static_cast<float>(H);
    const float s = rsqrtf(acc[0] * inv_H + eps);
    const float k = s * s * acc[1] * inv_H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float o = s * (gr[i] * w[i] - xr[i] * k);
      if (add_to_dx) o += dx[row * H + i];
      dx[row * H + i] = o;
      prow[i] += gr[i] * xr[i] * s;
    }
  }
}

// dw[c] (+)= sum_p partial[p][c]; one thread per column, coalesced across the CTA.
__global__ void __launch_bounds__(128) dw_finalize_kernel(const float* __restrict__ partial,
                                                          float* __restrict__ dw, int nparts,
                                                          int H, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float acc = 0.0f;
  for (int p = 0; p < nparts; ++p) acc += partial[static_cast<int64_t>(p) * H + c];
  dw[c] = accumulate ? dw[c] + acc : acc;
}

// Same column sum for many partial rows: 1024 threads = 32 row groups x 32 columns per CTA. The pass
// is latency-bound (a few MB read by H / 32 CTAs), so each thread issues sixteen independent loads
// before it adds them; the order of the additions is fixed. Columns below `split` go to dw0, the
// rest to dw1 (the QK-Norm pair keeps its two weight gradients in separate tensors).
__global__ void __launch_bounds__(1024) dw_finalize_wide_kernel(const float* __restrict__ partial,
                                                                float* __restrict__ dw0, float* __restrict__ dw1,
                                                                int split, int nparts, int H, int accumulate) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32][33];
  const int cl = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cl;
  float acc = 0.0f;
  if (c < H) {
    const float* src = partial + c;
    for (int base = rg; base < nparts; base += 32 * 16) {
      float v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int p = base + 32 * u;
        v[u] = p < nparts ? src[static_cast<int64_t>(p) * H] : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < 16; u += 4) acc += (v[u] + v[u + 1]) + (v[u + 2] + v[u + 3]);
    }
  }
  red[rg][cl] = acc;
  __syncthreads();
  if (rg == 0 && c < H) {
    float t = 0.0f;
#pragma unroll
    for (int r = 0; r < 32; ++r) t += red[r][cl];
    float* dst = c < split ? dw0 + c : dw1 + (c - split);
    *dst = accumulate ? *dst + t : t;
  }
}

// ---------------------------------------------------------------------------------------
// RoPE
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float rope_freq(int i, int D, const ctdk_rope_params& p) {
  const float base_freq = powf(p.theta, -(2.0f * i) / static_cast<float>(D));
  float freq = base_freq;
  if (p.scaling_factor > 1.0f) {
    const float wavelen = 6.2831853f / base_freq;
    if (wavelen > p.low_freq_wavelen) {
      freq = base_freq / p.scaling_factor;
    } else if (wavelen > p.high_freq_wavelen) {
      const float smooth =
          (wavelen - p.high_freq_wavelen) / (p.low_freq_wavelen - p.high_freq_wavelen);
      freq = (1.0f - smooth) * base_freq + smooth * (base_freq / p.scaling_factor);
    }
  }
  return freq;
}

// table[t][i] = (cos, sin) of float(position_start+t)*freq_i, i < D/2.
__global__ void rope_table_kernel(float2* __restrict__ table, int64_t T, int D,
                                  int position_start, ctdk_rope_params p) {
  const int Dh = D / 2;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * Dh) return;
  const int64_t t = idx / Dh;
  const int i = static_cast<int>(idx - t * Dh);
  const float angle = static_cast<float>(position_start + t) * rope_freq(i, D, p);
  float s, c;
  sincosf(angle, &s, &c);
  table[idx] = make_float2(c, s);
}

// One warp per (b,t,h) slot.
__global__ void __launch_bounds__(256)
    rope_kernel(const float* __restrict__ x_in, float* __restrict__ x_out, int64_t slots,
                int64_t T, int H, int D, int64_t row_stride, int position_start,
                ctdk_rope_params p, float sin_sign) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int Dh = D / 2;
  for (int64_t slot = warp0; slot < slots; slot += nwarps) {
    const int64_t bt = slot / H;
    const int h = static_cast<int>(slot - bt * H);
    const int64_t t = bt % T;
    const float* xr = x_in + bt * row_stride + static_cast<int64_t>(h) * D;
    float* yr = x_out + bt * row_stride + static_cast<int64_t>(h) * D;
    for (int i = lane; i < Dh; i += 32) {
      const float angle = static_cast<float>(position_start + t) * rope_freq(i, D, p);
      float s, c;
      sincosf(angle, &s, &c);
      s *= sin_sign;
      const float a = xr[i], b = xr[i + Dh];
      yr[i] = a * c - b * s;
      yr[i + Dh] = a * s + b * c;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Fused QK-Norm + RoPE over the packed qkv buffer. A group of D/8 threads owns one (row, head)
// slot: thread j of the group holds the float4 at [4j, 4j+3] and its rotation partners at
// [D/2+4j, D/2+4j+3], so every access is 128 bits and a warp covers 4 (D=64) or 2 (D=128)
// heads per iteration. NP = D/64.
// ---------------------------------------------------------------------------------------
template <int NP>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = 4 * NP; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void rot4(float4& a, float4& b, const float4 cs0, const float4 cs1,
                                     float sin_sign) {
  // cs0 = (c0,s0,c1,s1), cs1 = (c2,s2,c3,s3)
  float4 ra, rb;
  ra.x = a.x * cs0.x - b.x * cs0.y * sin_sign;  rb.x = a.x * cs0.y * sin_sign + b.x * cs0.x;
  ra.y = a.y * cs0.z - b.y * cs0.w * sin_sign;  rb.y = a.y * cs0.w * sin_sign + b.y * cs0.z;
  ra.z = a.z * cs1.x - b.z * cs1.y * sin_sign;  rb.z = a.z * cs1.y * sin_sign + b.z * cs1.x;
  ra.w = a.w * cs1.z - b.w * cs1.w * sin_sign;  rb.w = a.w * cs1.w * sin_sign + b.w * cs1.z;
  a = ra;
  b = rb;
}

template <int NP>
__global__ void __launch_bounds__(256)
    qk_norm_rope_fwd_kernel(const float* __restrict__ qkv, float* __restrict__ out,
                            const float* __restrict__ wq, const float* __restrict__ wk,
                            float* __restrict__ rstd_q, float* __restrict__ rstd_k,
                            const float2* __restrict__ table, int64_t rows, int64_t T, int H,
                            int Hk, float eps) {
  pdl_launch();
  pdl_wait();
  constexpr int D = 64 * NP, Dh = 32 * NP, TPH = 8 * NP;  // threads per head slot
  const int HT = H + 2 * Hk;
  const bool copy_v = (out != qkv);
  const bool has_norm = (wq != nullptr);
  const int HS = copy_v ? HT : H + Hk;   // head slots of a row this launch touches: in place, v is neither read nor written
  const int64_t items = rows * HS;
  const int j = threadIdx.x % TPH;
  const int64_t g0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / TPH;
  const int64_t ng = (static_cast<int64_t>(gridDim.x) * blockDim.x) / TPH;
  const int64_t iters = (items + ng - 1) / ng;  // every lane runs the same number of shuffles
  for (int64_t k = 0; k < iters; ++k) {
    const int64_t it = g0 + k * ng;
    const bool live = it < items;
    const int64_t row = live ? it / HS : 0;
    const int h = live ? static_cast<int>(it - row * HS) : 0;
    const bool is_v = h >= H + Hk, is_q = h < H;
    const int64_t off = (row * HT + h) * D;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (live) {
      a = *reinterpret_cast<const float4*>(qkv + off + 4 * j);
      b = *reinterpret_cast<const float4*>(qkv + off + Dh + 4 * j);
    }
    if (has_norm) {
      float ss = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y +
                 b.z * b.z + b.w * b.w;
      ss = group_sum<NP>(ss);
      if (live && !is_v) {
        const float s = rsqrtf(ss / static_cast<float>(D) + eps);
        if (j == 0) {
          if (is_q) rstd_q[row * H + h] = s;
          else rstd_k[row * Hk + (h - H)] = s;
        }
        const float* w = is_q ? wq : wk;
        const float4 wa = *reinterpret_cast<const float4*>(w + 4 * j);
        const float4 wb = *reinterpret_cast<const float4*>(w + Dh + 4 * j);
        a.x = a.x * s * wa.x;  a.y = a.y * s * wa.y;  a.z = a.z * s * wa.z;  a.w = a.w * s * wa.w;
        b.x = b.x * s * wb.x;  b.y = b.y * s * wb.y;  b.z = b.z * s * wb.z;  b.w = b.w * s * wb.w;
      }
    }
    if (!live) continue;
    if (!is_v) {
      const int64_t t = row % T;
      const float4* tb = reinterpret_cast<const float4*>(table + t * Dh + 4 * j);
      rot4(a, b, tb[0], tb[1], 1.0f);
    }
    *reinterpret_cast<float4*>(out + off + 4 * j) = a;
    *reinterpret_cast<float4*>(out + off + Dh + 4 * j) = b;
  }
}

// Backward, in place on dqkv: un-rotate (R(-theta)), then the RMSNorm backward per head.
// dw partials: registers -> shared-memory atomics -> partial[blockIdx.x][2][D].
template <int NP>
__global__ void __launch_bounds__(256)
    qk_norm_rope_bwd_kernel(float* __restrict__ dqkv, const float* __restrict__ qkv_pre,
                            const float* __restrict__ wq, const float* __restrict__ wk,
                            const float* __restrict__ rstd_q, const float* __restrict__ rstd_k,
                            float* __restrict__ partial, const float2* __restrict__ table,
                            int64_t rows, int64_t T, int H, int Hk) {
  pdl_launch();
  pdl_wait();
  constexpr int D = 64 * NP, Dh = 32 * NP, TPH = 8 * NP;
  __shared__ float sdw[2][D];
  const int HT = H + 2 * Hk, HQK = H + Hk;
  const int64_t items = rows * HQK;
  const int j = threadIdx.x % TPH;
  const int64_t g0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / TPH;
  const int64_t ng = (static_cast<int64_t>(gridDim.x) * blockDim.x) / TPH;
  const bool has_norm = (wq != nullptr);
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) sdw[i / D][i % D] = 0.0f;
  __syncthreads();
  float4 dwa[2], dwb[2];
  dwa[0] = dwa[1] = dwb[0] = dwb[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  const int64_t iters = (items + ng - 1) / ng;
  for (int64_t k = 0; k < iters; ++k) {
    const int64_t it = g0 + k * ng;
    const bool live = it < items;
    const int64_t row = live ? it / HQK : 0;
    const int h = live ? static_cast<int>(it - row * HQK) : 0;
    const bool is_q = h < H;
    const int64_t off = (row * HT + h) * D;
    float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), gb = ga;
    if (live) {
      ga = *reinterpret_cast<const float4*>(dqkv + off + 4 * j);
      gb = *reinterpret_cast<const float4*>(dqkv + off + Dh + 4 * j);
      const int64_t t = row % T;
      const float4* tb = reinterpret_cast<const float4*>(table + t * Dh + 4 * j);
      rot4(ga, gb, tb[0], tb[1], -1.0f);
    }
    if (has_norm) {
      float4 xa = make_float4(0.f, 0.f, 0.f, 0.f), xb = xa, wa = xa, wb = xa;
      float s = 0.0f;
      if (live) {
        const float* w = is_q ? wq : wk;
        xa = *reinterpret_cast<const float4*>(qkv_pre + off + 4 * j);
        xb = *reinterpret_cast<const float4*>(qkv_pre + off + Dh + 4 * j);
        wa = *reinterpret_cast<const float4*>(w + 4 * j);
        wb = *reinterpret_cast<const float4*>(w + Dh + 4 * j);
        s = is_q ? rstd_q[row * H + h] : rstd_k[row * Hk + (h - H)];
      }
      float c = ga.x * wa.x * xa.x + ga.y * wa.y * xa.y + ga.z * wa.z * xa.z + ga.w * wa.w * xa.w +
                gb.x * wb.x * xb.x + gb.y * wb.y * xb.y + gb.z * wb.z * xb.z + gb.w * wb.w * xb.w;
      c = group_sum<NP>(c);
      const float kk = s * s * c / static_cast<float>(D);
      const int sel = is_q ? 0 : 1;
      if (live) {
        dwa[sel].x += ga.x * xa.x * s;  dwa[sel].y += ga.y * xa.y * s;
        dwa[sel].z += ga.z * xa.z * s;  dwa[sel].w += ga.w * xa.w * s;
        dwb[sel].x += gb.x * xb.x * s;  dwb[sel].y += gb.y * xb.y * s;
        dwb[sel].z += gb.z * xb.z * s;  dwb[sel].w += gb.w * xb.w * s;
      }
      ga.x = s * (ga.x * wa.x - xa.x * kk);  ga.y = s * (ga.y * wa.y - xa.y * kk);
      ga.z = s * (ga.z * wa.z - xa.z * kk);  ga.w = s * (ga.w * wa.w - xa.w * kk);
      gb.x = s * (gb.x * wb.x - xb.x * kk);  gb.y = s * (gb.y * wb.y - xb.y * kk);
      gb.z = s * (gb.z * wb.z - xb.z * kk);  gb.w = s * (gb.w * wb.w - xb.w * kk);
    }
    if (live) {
      *reinterpret_cast<float4*>(dqkv + off + 4 * j) = ga;
      *reinterpret_cast<float4*>(dqkv + off + Dh + 4 * j) = gb;
    }
  }
  if (has_norm) {
#pragma unroll
    for (int sel = 0; sel < 2; ++sel) {
      atomicAdd(&sdw[sel][4 * j + 0], dwa[sel].x);
      atomicAdd(&sdw[sel][4 * j + 1], dwa[sel].y);
      atomicAdd(&sdw[sel][4 * j + 2], dwa[sel].z);
      atomicAdd(&sdw[sel][4 * j + 3], dwa[sel].w);
      atomicAdd(&sdw[sel][Dh + 4 * j + 0], dwb[sel].x);
      atomicAdd(&sdw[sel][Dh + 4 * j + 1], dwb[sel].y);
      atomicAdd(&sdw[sel][Dh + 4 * j + 2], dwb[sel].z);
      atomicAdd(&sdw[sel][Dh + 4 * j + 3], dwb[sel].w);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x)
      partial[static_cast<int64_t>(blockIdx.x) * 2 * D + i] = sdw[i / D][i % D];
  }
}

template <int NV>
void launch_rmsnorm_fwd(const float* x, const float* w, float* y, float* rstd, int64_t rows,
                        int H, float eps, int threads, int grid, cudaStream_t s) {
  launch_pdl(rmsnorm_fwd_kernel<NV>, dim3(grid), dim3(threads), 0, s, x, w, y, rstd, rows, H / 4,
             1.0f / static_cast<float>(H), eps);
}
template <int NV>
void launch_rmsnorm_bwd(const float* dy, const float* x, const float* w, float* dx,
                        float* partial, int64_t rows, int H, float eps, int add, int threads,
                        int grid, cudaStream_t s) {
  launch_pdl(rmsnorm_bwd_kernel<NV>, dim3(grid), dim3(threads), 0, s, dy, x, w, dx, partial, rows, H / 4,
             1.0f / static_cast<float>(H), eps, add);
}

}  // namespace
}  // namespace ctdk

using namespace ctdk;

extern "C" {

int ctdk_rmsnorm_fwd(const float* x, const float* w, float* y, float* rstd, int64_t rows,
                     int H, float eps, void* stream) {
  CTDK_REQUIRE(rows >= 0 && H > 0, "ctdk_rmsnorm_fwd: bad shape");
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(x && w && y, "ctdk_rmsnorm_fwd: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int grid = static_cast<int>(rows < cap ? rows : cap);
  const bool vec = (H % 4 == 0) && aligned16(x) && aligned16(w) && aligned16(y) && H <= 4096;
  void* tok = prof_begin(CTDK_PROF_NORM, 8.0 * static_cast<double>(rows) * H, s);
  if (vec) {
    const int H4 = H / 4;
    int threads = ((H4 + 31) / 32) * 32;
    if (threads > 256) threads = 256;
    const int nv = (H4 + threads - 1) / threads;
    switch (nv) {
      case 1: launch_rmsnorm_fwd<1>(x, w, y, rstd, rows, H, eps, threads, grid, s); break;
      case 2: launch_rmsnorm_fwd<2>(x, w, y, rstd, rows, H, eps, threads, grid, s); break;
      default: launch_rmsnorm_fwd<4>(x, w, y, rstd, rows, H, eps, threads, grid, s); break;
    }
  } else {
    rmsnorm_fwd_generic_kernel<<<grid, 256, 0, s>>>(x, w, y, rstd, rows, H, eps);
  }
  prof_end(tok, s);
  return check_launch("ctdk_rmsnorm_fwd");
}

int64_t ctdk_rmsnorm_bwd_scratch_floats(int H) {
  return static_cast<int64_t>(kNormPartialRows) * (H > 0 ? H : 0);
}

int ctdk_rmsnorm_bwd(const float* dy, const float* x, const float* w, float* dx, float* dw,
                     float* dw_scratch, int64_t rows, int H, float eps, int accumulate_dw,
                     int add_to_dx, void* stream) {
  CTDK_REQUIRE(rows >= 0 && H > 0, "ctdk_rmsnorm_bwd: bad shape");
  CTDK_REQUIRE(dw && dw_scratch, "ctdk_rmsnorm_bwd: null dw / scratch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    if (!accumulate_dw) cudaMemsetAsync(dw, 0, sizeof(float) * H, s);
    return CTDK_OK;
  }
  CTDK_REQUIRE(dy && x && w && dx, "ctdk_rmsnorm_bwd: null pointer");
  void* prof = prof_begin(CTDK_PROF_NORM_BWD, (add_to_dx ? 16.0 : 12.0) * static_cast<double>(rows) * H, s);
  int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (cap > kNormPartialRows) cap = kNormPartialRows;
  int grid = static_cast<int>(rows < cap ? rows : cap);
  const bool vec = (H % 4 == 0) && aligned16(dy) && aligned16(x) && aligned16(w) &&
                   aligned16(dx) && aligned16(dw_scratch) && H <= 4096;
  if (vec && H <= 1024 && rows >= 8 * static_cast<int64_t>(sm_count())) {
    // one warp per row
    const int H4 = H / 4;
    int64_t g = (rows + 7) / 8;
    const int64_t gcap = static_cast<int64_t>(sm_count()) * 2;
    if (g > gcap) g = gcap;
    grid = static_cast<int>(g);
    const size_t smem = static_cast<size_t>(8) * H4 * sizeof(float4);
    if (H4 <= 128)
      launch_pdl(rmsnorm_bwd_rows_kernel<4>, dim3(grid), dim3(256), smem, s, dy, x, w, dx, dw_scratch, rows, H4,
                 1.0f / static_cast<float>(H), eps, add_to_dx);
    else
      launch_pdl(rmsnorm_bwd_rows_kernel<8>, dim3(grid), dim3(256), smem, s, dy, x, w, dx, dw_scratch, rows, H4,
                 1.0f / static_cast<float>(H), eps, add_to_dx);
  } else if (vec) {
    const int H4 = H / 4;
    int threads = ((H4 + 31) / 32) * 32;
    if (threads > 256) threads = 256;
    const int nv = (H4 + threads - 1) / threads;
    switch (nv) {
      case 1:
        launch_rmsnorm_bwd<1>(dy, x, w, dx, dw_scratch, rows, H, eps, add_to_dx, threads, grid,
                              s);
        break;
      case 2:
        launch_rmsnorm_bwd<2>(dy, x, w, dx, dw_scratch, rows, H, eps, add_to_dx, threads, grid,
                              s);
        break;
      default:
        launch_rmsnorm_bwd<4>(dy, x, w, dx, dw_scratch, rows, H, eps, add_to_dx, threads, grid,
                              s);
        break;
    }
  } else {
    rmsnorm_bwd_generic_kernel<<<grid, 256, 0, s>>>(dy, x, w, dx, dw_scratch, rows, H, eps,
                                                    add_to_dx);
  }
  int rc = check_launch("ctdk_rmsnorm_bwd");
  if (rc != CTDK_OK) return rc;
  launch_pdl(dw_finalize_wide_kernel, dim3(ceil_div(H, 32)), dim3(1024), 0, s, static_cast<const float*>(dw_scratch), dw, dw, H, grid, H, accumulate_dw);
  prof_end(prof, s);
  return check_launch("ctdk_rmsnorm_bwd(finalize)");
}

// ---------------------------------------------------------------------------------------
// RMSNorm backward without any caller- or library-allocated scratch.
//
// Some hosts of this library cannot hand it scratch memory and cannot let it allocate
// either: a trainer that reserved the whole of HBM for its own arena at start-up (a
// cudaMalloc from inside a library call would simply fail, or would force the arena to
// shrink), and step loops that must not contain cudaMalloc/cudaFree because those calls
// synchronise the device and stall every stream (the very cost the reference pays per op).
// For them the per-CTA dw partial rows live in a fixed array inside the library image.
// It costs kStaticRows * kStaticMaxH * 4 bytes = 4 MiB of device memory on every GPU that
// loads the library, for the life of the process.
// ---------------------------------------------------------------------------------------
namespace ctdk {
namespace {
constexpr int kStaticRows = 256;   // per-CTA partial rows (upper bound of the grid)
constexpr int kStaticMaxH = 4096;  // widest row the static variant accepts
static __device__ __align__(256) float g_rmsnorm_static_scratch[kStaticRows * kStaticMaxH];

// Device address of the array, resolved once per device. In host code the array's name is
// only a handle for cudaGetSymbolAddress, never a pointer a kernel may be given.
float* g_static_scratch_ptr[64] = {nullptr};
std::mutex g_static_scratch_mu;   // callers on several host threads may make the first call together

int static_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64)
    return fail(CTDK_ELAUNCH, "ctdk_rmsnorm_bwd_static: no current device");
  std::lock_guard<std::mutex> lk(g_static_scratch_mu);
  if (g_static_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(CTDK_ELAUNCH, "ctdk_rmsnorm_bwd_static: cudaGetSymbolAddress failed: %s",
                  cudaGetErrorString(e));
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return CTDK_OK;
}
}  // namespace
}  // namespace ctdk

int ctdk_rmsnorm_bwd_static(const float* dy, const float* x, const float* w, float* dx,
                            float* dw, int64_t rows, int H, float eps, int accumulate_dw,
                            int add_to_dx, void* stream) {
  CTDK_REQUIRE(rows >= 0 && H > 0, "ctdk_rmsnorm_bwd_static: bad shape");
  CTDK_REQUIRE(H <= kStaticMaxH,
               "ctdk_rmsnorm_bwd_static: H = %d exceeds the built-in scratch (max %d); use "
               "ctdk_rmsnorm_bwd with caller-provided scratch",
               H, kStaticMaxH);
  CTDK_REQUIRE(dw != nullptr, "ctdk_rmsnorm_bwd_static: null dw");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    if (!accumulate_dw) cudaMemsetAsync(dw, 0, sizeof(float) * H, s);
    return CTDK_OK;
  }
  CTDK_REQUIRE(dy && x && w && dx, "ctdk_rmsnorm_bwd_static: null pointer");
  float* scratch = nullptr;
  int rc = static_scratch(&scratch);  // first call on a device resolves the symbol address
  if (rc != CTDK_OK) return rc;
  int64_t cap = static_cast<int64_t>(sm_count()) * 2;
  if (cap > kStaticRows) cap = kStaticRows;
  int grid = static_cast<int>(rows < cap ? rows : cap);
  // Nothing in the array has to start at zero: each of the `grid` CTAs overwrites its whole
  // partial row (the generic kernel zeroes its row itself) and the finalize pass reads only
  // those rows, so contents left by an earlier call are never observed.
  const bool vec =
      (H % 4 == 0) && aligned16(dy) && aligned16(x) && aligned16(w) && aligned16(dx);
  if (vec && H <= 1024 && rows >= 8 * static_cast<int64_t>(sm_count())) {
    // one warp per row, as ctdk_rmsnorm_bwd does for these shapes (dx is then bit-identical to it:
    // a row's result does not depend on the grid)
    const int H4 = H / 4;
    const int64_t g = (rows + 7) / 8;
    grid = static_cast<int>(g < cap ? g : cap);
    const size_t smem = static_cast<size_t>(8) * H4 * sizeof(float4);
    if (H4 <= 128)
      launch_pdl(rmsnorm_bwd_rows_kernel<4>, dim3(grid), dim3(256), smem, s, dy, x, w, dx, scratch, rows, H4,
                 1.0f / static_cast<float>(H), eps, add_to_dx);
    else
      launch_pdl(rmsnorm_bwd_rows_kernel<8>, dim3(grid), dim3(256), smem, s, dy, x, w, dx, scratch, rows, H4,
                 1.0f / static_cast<float>(H), eps, add_to_dx);
  } else if (vec) {
    const int H4 = H / 4;
    int threads = ((H4 + 31) / 32) * 32;
    if (threads > 256) threads = 256;
    const int nv = (H4 + threads - 1) / threads;
    if (nv == 1)
      launch_rmsnorm_bwd<1>(dy, x, w, dx, scratch, rows, H, eps, add_to_dx, threads, grid, s);
    else if (nv == 2)
      launch_rmsnorm_bwd<2>(dy, x, w, dx, scratch, rows, H, eps, add_to_dx, threads, grid, s);
    else
      launch_rmsnorm_bwd<4>(dy, x, w, dx, scratch, rows, H, eps, add_to_dx, threads, grid, s);
  } else {
    rmsnorm_bwd_generic_kernel<<<grid, 256, 0, s>>>(dy, x, w, dx, scratch, rows, H, eps,
                                                    add_to_dx);
  }
  rc = check_launch("ctdk_rmsnorm_bwd_static");
  if (rc != CTDK_OK) return rc;
  dw_finalize_kernel<<<ceil_div(H, 128), 128, 0, s>>>(scratch, dw, grid, H, accumulate_dw);
  return check_launch("ctdk_rmsnorm_bwd_static(finalize)");
}

int ctdk_rope_table(float* table, int64_t T, int D, int position_start,
                    const ctdk_rope_params* p, void* stream) {
  CTDK_REQUIRE(table && p, "ctdk_rope_table: null pointer");
  CTDK_REQUIRE(T >= 0 && D > 0 && D % 2 == 0, "ctdk_rope_table: D must be even");
  if (T == 0) return CTDK_OK;
  const int64_t n = T * (D / 2);
  rope_table_kernel<<<ceil_div(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<float2*>(table), T, D, position_start, *p);
  return check_launch("ctdk_rope_table");
}

int ctdk_rope(const float* x_in, float* x_out, int64_t B, int64_t T, int H, int D,
              int64_t row_stride, int position_start, const ctdk_rope_params* p,
              float sin_sign, void* stream) {
  CTDK_REQUIRE(p != nullptr, "ctdk_rope: null params");
  CTDK_REQUIRE(B >= 0 && T >= 0 && H > 0 && D > 0 && D % 2 == 0, "ctdk_rope: D must be even");
  const int64_t slots = B * T * H;
  if (slots == 0) return CTDK_OK;
  CTDK_REQUIRE(x_in && x_out, "ctdk_rope: null pointer");
  CTDK_REQUIRE(row_stride >= static_cast<int64_t>(H) * D, "ctdk_rope: row_stride < H*D");
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int64_t need = (slots + 7) / 8;
  rope_kernel<<<static_cast<int>(need < cap ? need : cap), 256, 0,
                static_cast<cudaStream_t>(stream)>>>(x_in, x_out, slots, T, H, D, row_stride,
                                                     position_start, *p, sin_sign);
  return check_launch("ctdk_rope");
}

int ctdk_qk_norm_rope_fwd(const float* qkv, float* qkv_out, const float* wq, const float* wk,
                          float* rstd_q, float* rstd_k, const float* rope_table, int64_t B,
                          int64_t T, int H, int Hk, int D, float eps, void* stream) {
  CTDK_REQUIRE(B >= 0 && T >= 0 && H > 0 && Hk > 0, "ctdk_qk_norm_rope_fwd: bad shape");
  CTDK_REQUIRE(D == 64 || D == 128, "ctdk_qk_norm_rope_fwd: head_dim must be 64 or 128");
  const int64_t rows = B * T;
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(qkv && qkv_out && rope_table, "ctdk_qk_norm_rope_fwd: null pointer");
  CTDK_REQUIRE(aligned16(qkv) && aligned16(qkv_out) && aligned16(rope_table) && aligned16(wq) &&
                   aligned16(wk),
               "ctdk_qk_norm_rope_fwd: pointers must be 16-byte aligned");
  CTDK_REQUIRE((wq == nullptr) == (wk == nullptr), "ctdk_qk_norm_rope_fwd: wq/wk mismatch");
  CTDK_REQUIRE(wq == nullptr || (rstd_q && rstd_k), "ctdk_qk_norm_rope_fwd: rstd required");
  CTDK_REQUIRE(wq == nullptr || qkv_out != qkv,
               "ctdk_qk_norm_rope_fwd: QK-Norm needs an out-of-place result");
  const int64_t items = rows * (H + Hk + (qkv_out != qkv ? Hk : 0));
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int per_cta = 256 / (D / 8);  // head slots per CTA and iteration
  const int64_t need = (items + per_cta - 1) / per_cta;
  const int grid = static_cast<int>(need < cap ? need : cap);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float2* tb = reinterpret_cast<const float2*>(rope_table);
  // q and k are read and written; v is copied only when the result goes to a second buffer
  void* prof = prof_begin(CTDK_PROF_QKROPE, 8.0 * static_cast<double>(rows) * D * (H + Hk + (qkv_out != qkv ? Hk : 0)), s);
  if (D == 64)
    launch_pdl(qk_norm_rope_fwd_kernel<1>, dim3(grid), dim3(256), 0, s, qkv, qkv_out, wq, wk, rstd_q, rstd_k, tb, rows, T, H,
               Hk, eps);
  else
    launch_pdl(qk_norm_rope_fwd_kernel<2>, dim3(grid), dim3(256), 0, s, qkv, qkv_out, wq, wk, rstd_q, rstd_k, tb, rows, T, H,
               Hk, eps);
  prof_end(prof, s);
  return check_launch("ctdk_qk_norm_rope_fwd");
}

int64_t ctdk_qk_norm_rope_bwd_scratch_floats(int D) {
  return static_cast<int64_t>(kMaxPartialRows) * 2 * (D > 0 ? D : 0);
}

int ctdk_qk_norm_rope_bwd(float* dqkv, const float* qkv_pre, const float* wq, const float* wk,
                          const float* rstd_q, const float* rstd_k, float* dwq, float* dwk,
                          float* scratch, const float* rope_table, int64_t B, int64_t T, int H,
                          int Hk, int D, int accumulate_dw, void* stream) {
  CTDK_REQUIRE(B >= 0 && T >= 0 && H > 0 && Hk > 0, "ctdk_qk_norm_rope_bwd: bad shape");
  CTDK_REQUIRE(D == 64 || D == 128, "ctdk_qk_norm_rope_bwd: head_dim must be 64 or 128");
  const int64_t rows = B * T;
  const bool has_norm = wq != nullptr;
  CTDK_REQUIRE((wq == nullptr) == (wk == nullptr), "ctdk_qk_norm_rope_bwd: wq/wk mismatch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    if (has_norm && !accumulate_dw) {
      cudaMemsetAsync(dwq, 0, sizeof(float) * D, s);
      cudaMemsetAsync(dwk, 0, sizeof(float) * D, s);
    }
    return CTDK_OK;
  }
  CTDK_REQUIRE(dqkv && rope_table, "ctdk_qk_norm_rope_bwd: null pointer");
  CTDK_REQUIRE(aligned16(dqkv) && aligned16(rope_table) && aligned16(qkv_pre) && aligned16(wq) &&
                   aligned16(wk),
               "ctdk_qk_norm_rope_bwd: pointers must be 16-byte aligned");
  CTDK_REQUIRE(!has_norm || (qkv_pre && rstd_q && rstd_k && dwq && dwk && scratch),
               "ctdk_qk_norm_rope_bwd: QK-Norm needs qkv_pre, rstd, dw and scratch");
  const int64_t items = rows * (H + Hk);
  // with QK-Norm every CTA leaves a dw partial row, so the grid is kept small; without it the grid only
  // has to fill the SMs
  int64_t cap = static_cast<int64_t>(sm_count()) * (has_norm ? 3 : 8);
  if (has_norm && cap > kMaxPartialRows) cap = kMaxPartialRows;
  const int per_cta = 256 / (D / 8);
  const int64_t need = (items + per_cta - 1) / per_cta;
  const int grid = static_cast<int>(need < cap ? need : cap);
  const float2* tb = reinterpret_cast<const float2*>(rope_table);
  // d(q), d(k) read and written in place; with QK-Norm the saved pre-norm q / k are read as well
  void* prof = prof_begin(CTDK_PROF_QKROPE, (has_norm ? 12.0 : 8.0) * static_cast<double>(rows) * D * (H + Hk), s);
  if (D == 64)
    launch_pdl(qk_norm_rope_bwd_kernel<1>, dim3(grid), dim3(256), 0, s, dqkv, qkv_pre, wq, wk, rstd_q, rstd_k, scratch, tb,
               rows, T, H, Hk);
  else
    launch_pdl(qk_norm_rope_bwd_kernel<2>, dim3(grid), dim3(256), 0, s, dqkv, qkv_pre, wq, wk, rstd_q, rstd_k, scratch, tb,
               rows, T, H, Hk);
  int rc = check_launch("ctdk_qk_norm_rope_bwd");
  if (rc != CTDK_OK || !has_norm) {
    prof_end(prof, s);
    return rc;
  }
  launch_pdl(dw_finalize_wide_kernel, dim3(ceil_div(2 * D, 32)), dim3(1024), 0, s, static_cast<const float*>(scratch), dwq, dwk, D, grid,
             2 * D, accumulate_dw);
  prof_end(prof, s);
  return check_launch("ctdk_qk_norm_rope_bwd(finalize)");
}

}  // extern "C"
