// KV-cache greedy decoding (batch 1): prefill with the training-path kernels, then one token per
// step with HBM-bound kernels, the whole step captured once in a CUDA graph and replayed.
//
// Replaces the inference path of the reference: Model::forward with a cache
// (emberlm include/ctd/nn/model.h:155-167), Attention::forward (include/ctd/nn/attention.h:43-97),
// write_kv_inplace / read_kv_expanded (src/ops/kv_cache.cu:14-47) and the greedy branch of the
// CPU sampler (src/core/sampling.cpp:13-20: first index of the maximum). Differences in execution:
// K/V are written to the cache by the same kernel that applies QK-Norm and RoPE; attention reads
// the cache in place (no expansion to [B,H,L,D] per token, no repeat of kv heads); the argmax runs
// on the GPU and the next token id never leaves the device; position and token counters live in
// device memory so that one captured graph serves every step.
// Cache layout: [layer][kv head][max_seq][D] for K and for V (as the reference's KVLayer,
// include/ctd/nn/kv_cache.h:23-37).
#include <cfloat>
#include <new>
#include <vector>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace ctdk {
namespace {

// y[n] = dot(W[n,:], f(x)) (+ residual[n]); one warp per output row, 128-bit loads, f(x) staged in
// shared memory once per CTA. f is the identity, RMSNorm (x * rsqrt(mean(x^2)+eps) * nw, the
// reference's norm kernel, emberlm src/ops/norm.cu:18-50) or SwiGLU of a packed gate|up vector
// (silu(g)*u, include/ctd/nn/mlp.h:16-21) so that no separate kernel has to run per token.
enum { kPreNone = 0, kPreRmsNorm = 1, kPreSwiglu = 2 };

// The kernels of a token step are launched with launch_pdl(): each one fetches what does not depend
// on its predecessor (weights) before pdl_wait().
template <int PRE>
__global__ void __launch_bounds__(256)
    gemv_kernel(const float* __restrict__ W, const float* __restrict__ x, float* __restrict__ y,
                const float* __restrict__ residual, const float* __restrict__ nw, float eps, int N, int K) {
  extern __shared__ float xs[];
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int warp0 = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int K4 = K >> 2;
  // The first weights of this warp's first row are requested before the input vector is staged
  // (and normalised), so the prologue runs under the first memory round trip instead of before it.
  constexpr int kPre = 8;
  float4 wpre[kPre];
  pdl_launch();
  {
    const float4* w4 = reinterpret_cast<const float4*>(W + static_cast<int64_t>(warp0 < N ? warp0 : 0) * K);
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      const int i = lane + 32 * j;
      wpre[j] = (warp0 < N && i < K4) ? __ldcs(w4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait();   // x (and the residual) come from the previous kernel
  if (PRE == kPreSwiglu) {
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
      const float g = x[i];
      xs[i] = g / (1.0f + __expf(-g)) * x[K + i];
    }
  } else {
    float ss = 0.0f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
      const float v = x[i];
      xs[i] = v;
      ss += v * v;
    }
    if (PRE == kPreRmsNorm) {
      ss = warp_sum(ss);
      if (lane == 0) red[wid] = ss;
      __syncthreads();
      float tot = 0.0f;
      for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
      const float sc = rsqrtf(tot / static_cast<float>(K) + eps);
      for (int i = threadIdx.x; i < K; i += blockDim.x) xs[i] = xs[i] * sc * nw[i];
    }
  }
  __syncthreads();
  const float4* x4 = reinterpret_cast<const float4*>(xs);
  for (int n = warp0; n < N; n += nwarps) {
    const float4* w4 = reinterpret_cast<const float4*>(W + static_cast<int64_t>(n) * K);
    float acc = 0.0f;
    int i0 = lane;
    if (n == warp0) {   // the prefetched part of the first row
#pragma unroll
      for (int j = 0; j < kPre; ++j) {
        const int i = lane + 32 * j;
        if (i < K4) {
          const float4 a = wpre[j], b = x4[i];
          acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
        }
      }
      i0 = lane + 32 * kPre;
    }
#pragma unroll 4
    for (int i = i0; i < K4; i += 32) {
      const float4 a = __ldcs(w4 + i), b = x4[i];
      acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    }
    acc = warp_sum(acc);
    if (lane == 0) y[n] = residual != nullptr ? acc + residual[n] : acc;
  }
}

// One warp per head slot of the single new row: per-head RMSNorm (optional) + RoPE at position
// *pos for q and k; q goes to q_out, k and v go into the cache at position *pos.
__global__ void __launch_bounds__(256)
    decode_qkv_post_kernel(const float* __restrict__ qkv, const float* __restrict__ wq,
                           const float* __restrict__ wk, const float2* __restrict__ table,
                           const int* __restrict__ pos_ptr, float* __restrict__ q_out,
                           float* __restrict__ kcache, float* __restrict__ vcache, int H, int Hk, int D,
                           int max_seq, float eps) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int slot = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (slot >= H + 2 * Hk) return;
  const int pos = *pos_ptr;
  const int Dh = D / 2;
  const float* xr = qkv + static_cast<int64_t>(slot) * D;
  if (slot >= H + Hk) {  // v head
    float* dst = vcache + (static_cast<int64_t>(slot - H - Hk) * max_seq + pos) * D;
    for (int i = lane; i < D; i += 32) dst[i] = xr[i];
    return;
  }
  const bool is_q = slot < H;
  const float* w = is_q ? wq : wk;
  float s = 1.0f;
  if (w != nullptr) {
    float ss = 0.0f;
    for (int i = lane; i < D; i += 32) ss += xr[i] * xr[i];
    ss = warp_sum(ss);
    s = rsqrtf(ss / static_cast<float>(D) + eps);
  }
  float* dst = is_q ? q_out + static_cast<int64_t>(slot) * D
                    : kcache + (static_cast<int64_t>(slot - H) * max_seq + pos) * D;
  for (int i = lane; i < Dh; i += 32) {
    float a = xr[i], b = xr[i + Dh];
    if (w != nullptr) {
      a = a * s * w[i];
      b = b * s * w[i + Dh];
    }
    const float2 cs = table[static_cast<int64_t>(pos) * Dh + i];
    dst[i] = a * cs.x - b * cs.y;
    dst[i + Dh] = a * cs.y + b * cs.x;
  }
}

// Copies post-RoPE k and v rows of a prefilled qkv[T, (H+2Hk)*D] into the cache at positions 0..T-1.
__global__ void __launch_bounds__(256)
    kv_write_rows_kernel(const float* __restrict__ qkv, float* __restrict__ kcache, float* __restrict__ vcache,
                         int T, int H, int Hk, int D, int max_seq) {
  const int64_t n = static_cast<int64_t>(T) * 2 * Hk * (D / 4);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int RS = (H + 2 * Hk) * D;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int c = static_cast<int>(i % (D / 4));
    const int hh = static_cast<int>((i / (D / 4)) % (2 * Hk));
    const int t = static_cast<int>(i / (static_cast<int64_t>(D / 4) * 2 * Hk));
    const float4 v = *reinterpret_cast<const float4*>(qkv + static_cast<int64_t>(t) * RS + (H + hh) * D + 4 * c);
    float* cache = hh < Hk ? kcache : vcache;
    const int hk = hh < Hk ? hh : hh - Hk;
    *reinterpret_cast<float4*>(cache + (static_cast<int64_t>(hk) * max_seq + t) * D + 4 * c) = v;
  }
}

constexpr int kAttnSplits = 8;   // key ranges per head in the decode attention

// Attention of the single new row over the cache, split over key ranges: CTA (h, sp) scores the
// keys [sp * n, (sp + 1) * n) of head h (n = ceil(L / kAttnSplits)), and leaves the range's maximum,
// exp-sum and exp-weighted V sum (relative to that maximum) in part[h][sp] = {m, l, o[D]};
// decode_attn_combine_kernel merges the ranges. One CTA per head kept 16 SMs busy and took longer
// than streaming the layer's weights.
__global__ void __launch_bounds__(256)
    decode_attn_kernel(const float* __restrict__ q, const float* __restrict__ kcache,
                       const float* __restrict__ vcache, float* __restrict__ part,
                       const int* __restrict__ pos_ptr, int H, int Hk, int D, int max_seq, float scale) {
  extern __shared__ float sm[];  // [keys per range] scores, [D] q, [256] reduction scratch
  pdl_launch();
  pdl_wait();
  const int h = blockIdx.x, sp = blockIdx.y, hk = h / (H / Hk);
  const int L = *pos_ptr + 1;
  const int per = (L + kAttnSplits - 1) / kAttnSplits;
  const int j0 = sp * per, j1 = min(L, j0 + per);
  const int cap = ((max_seq + kAttnSplits - 1) / kAttnSplits + 3) & ~3;   // keeps the q staging 16-byte aligned
  float* sc = sm;
  float* qs = sm + cap;
  float* red = qs + D;
  float* dst = part + (static_cast<int64_t>(h) * kAttnSplits + sp) * (D + 2);
  if (j0 >= j1) {   // empty range
    if (threadIdx.x == 0) {
      dst[0] = -FLT_MAX;
      dst[1] = 0.0f;
    }
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[2 + i] = 0.0f;
    return;
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int i = threadIdx.x; i < D; i += blockDim.x) qs[i] = q[static_cast<int64_t>(h) * D + i];
  __syncthreads();
  const float* kb = kcache + static_cast<int64_t>(hk) * max_seq * D;
  const float* vb = vcache + static_cast<int64_t>(hk) * max_seq * D;
  float mx = -FLT_MAX;
  for (int j = j0 + threadIdx.x; j < j1; j += blockDim.x) {
    const float4* kr = reinterpret_cast<const float4*>(kb + static_cast<int64_t>(j) * D);
    const float4* q4 = reinterpret_cast<const float4*>(qs);
    float acc = 0.0f;
    for (int i = 0; i < D / 4; ++i) {
      const float4 a = kr[i], b = q4[i];
      acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    }
    acc *= scale;
    sc[j - j0] = acc;
    mx = fmaxf(mx, acc);
  }
  mx = warp_max(mx);
  if (lane == 0) red[wid] = mx;
  __syncthreads();
  mx = -FLT_MAX;
  for (int i = 0; i < nw; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float sum = 0.0f;
  for (int j = j0 + threadIdx.x; j < j1; j += blockDim.x) {
    const float e = __expf(sc[j - j0] - mx);
    sc[j - j0] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if (lane == 0) red[wid] = sum;
  __syncthreads();
  sum = 0.0f;
  for (int i = 0; i < nw; ++i) sum += red[i];
  __syncthreads();
  const int d = threadIdx.x % D, pt = threadIdx.x / D, nparts = blockDim.x / D;
  float acc = 0.0f;
  for (int j = j0 + pt; j < j1; j += nparts) acc += sc[j - j0] * vb[static_cast<int64_t>(j) * D + d];
  red[pt * D + d] = acc;
  __syncthreads();
  if (threadIdx.x < D) {
    float t = 0.0f;
    for (int p = 0; p < nparts; ++p) t += red[p * D + threadIdx.x];
    dst[2 + threadIdx.x] = t;
  }
  if (threadIdx.x == 0) {
    dst[0] = mx;
    dst[1] = sum;
  }
}

// out[h][d] = sum_sp o_sp[d] e^(m_sp - M) / sum_sp l_sp e^(m_sp - M), M = max_sp m_sp.
__global__ void __launch_bounds__(128)
    decode_attn_combine_kernel(const float* __restrict__ part, float* __restrict__ out, int D) {
  pdl_launch();
  pdl_wait();
  const int h = blockIdx.x;
  const float* p = part + static_cast<int64_t>(h) * kAttnSplits * (D + 2);
  float M = -FLT_MAX;
#pragma unroll
  for (int s = 0; s < kAttnSplits; ++s) M = fmaxf(M, p[s * (D + 2)]);
  float l = 0.0f, w[kAttnSplits];
#pragma unroll
  for (int s = 0; s < kAttnSplits; ++s) {
    w[s] = __expf(p[s * (D + 2)] - M);
    l += p[s * (D + 2) + 1] * w[s];
  }
  const float inv = 1.0f / l;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.0f;
#pragma unroll
    for (int s = 0; s < kAttnSplits; ++s) o += p[s * (D + 2) + 2 + d] * w[s];
    out[static_cast<int64_t>(h) * D + d] = o * inv;
  }
}

// First index of the maximum (the reference's greedy sampler, src/core/sampling.cpp:13-20) over
// many CTAs: each reduces its share of the logits and folds (value, index) into one 64-bit word
// with atomicMax. The key orders floats as unsigned integers in the high half and prefers the
// smaller index in the low half; argmax_finish_kernel turns the word into the next input token.
__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
  unsigned u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return (static_cast<unsigned long long>(u) << 32) | (0xFFFFFFFFu - static_cast<unsigned>(idx));
}
__global__ void __launch_bounds__(256)
    argmax_kernel(const float* __restrict__ logits, int V, unsigned long long* __restrict__ word) {
  __shared__ unsigned long long best_s[8];
  pdl_launch();
  pdl_wait();
  unsigned long long best = 0ull;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) {
    const unsigned long long k = argmax_key(logits[i], i);
    best = k > best ? k : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) best_s[wid] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (blockDim.x >> 5); ++i) best = best_s[i] > best ? best_s[i] : best;
    atomicMax(word, best);
  }
}
// Stores the winning token as the next input, appends it to out_tokens[*count], clears the word and
// advances the counters (pos may point at a scratch int when the position must not move).
__global__ void argmax_finish_kernel(unsigned long long* word, int64_t* cur_token, int64_t* out_tokens, int* pos,
                                     int* count) {
  pdl_launch();
  pdl_wait();
  const int64_t idx = static_cast<int64_t>(0xFFFFFFFFu - static_cast<unsigned>(*word & 0xFFFFFFFFull));
  *cur_token = idx;
  if (out_tokens != nullptr) out_tokens[*count] = idx;
  *word = 0ull;
  *pos += 1;
  *count += 1;
}

__global__ void bump_kernel(int* pos, int* count) {
  pdl_launch();
  pdl_wait();
  *pos += 1;
  *count += 1;
}
__global__ void set_counters_kernel(int* pos, int* count, int p, int c) {
  *pos = p;
  *count = c;
  *reinterpret_cast<unsigned long long*>(pos + 4) = 0ull;   // the argmax word lives behind the counters
}


// ----------------------------------------------------------------------------------------
// Persistent token loop. The kernel-per-phase path above spends most of a token in the ~200
// launch-to-launch dependencies (each kernel streams 8-25 MB of weights in 2-4 us but waits ~8 us
// for its predecessor to drain). Here ONE cooperative kernel generates all the requested tokens:
// its CTAs stay resident, every phase of a layer is a grid-stride loop over weight rows, and the
// phases are separated by a grid barrier (an atomic counter in global memory, ~2 us) instead of a
// kernel boundary. While a CTA waits at a barrier, the weight rows of its next phase are already on
// their way into L2 (prefetch.global.L2), so the HBM stream of phase p+1 overlaps the barrier of
// phase p. Every wait is bounded: a barrier that does not complete within the budget sets the
// device status word, and every CTA leaves at its next barrier.
//   per layer: [RMSNorm + QKV rows] | [QK-Norm + RoPE + cache write + split attention + merge]
//              | [O rows + residual] | [RMSNorm + gate|up rows] | [SwiGLU + down rows + residual]
//   per token: ... | [RMSNorm + LM-head rows + arg-max]
// ----------------------------------------------------------------------------------------
constexpr int kSyncWords = 256;   // uint32: [0] barrier count, [2] abort flag, [8..8+H) head arrivals, [128..131] two 64-bit argmax words
constexpr int kMaxPersistLayers = 40;
constexpr int kPersistSplits = 16;  // key ranges per head in the persistent kernel (the partial buffer is sized for these)

struct PLayer {
  int64_t w_in, wq, wo, wqn, wkn, w_post, wg, wd;
};
struct PersistArgs {
  const float* P;
  PLayer lw[kMaxPersistLayers];
  int64_t embed, norm;
  int L, hid, I, D, H, Hk, V, QKVN, max_seq;
  int qk_norm;
  float eps, scale;
  const float2* table;
  float *kcache, *vcache, *x, *qkv, *attn, *hm, *gu, *logits, *attn_part;
  int64_t* cur_token;
  int* counters;
  unsigned int* sync;
  int64_t* out_tokens;
  int out_offset, n_tokens;
  int* status;
};

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// All CTAs of the grid meet here: one release reduction on a counter per CTA (no value comes back,
// so the arriving thread does not wait for it; the CTA's earlier writes are ordered before it by
// the bar.sync and the release), then one thread per CTA polls the counter. A flag per CTA watched
// by every other CTA measured twice as slow (all pollers hit the same few L2 lines). `epoch` counts
// the barriers this CTA has passed. Returns false once any CTA has given up (the abort flag is
// set): the caller unwinds.
__device__ __forceinline__ bool grid_barrier(const PersistArgs& a, unsigned int& epoch) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    ++epoch;
    const unsigned int target = epoch * gridDim.x;
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&a.sync[0]) : "memory");
    int ok = 1;
    if (ld_acquire_u32(&a.sync[0]) < target) {
      const uint64_t t0 = globaltimer_ns();
      unsigned int spins = 0;
      while (ld_acquire_u32(&a.sync[0]) < target) {
        if ((++spins & 0xffu) == 0u) {
          if (ld_acquire_u32(&a.sync[2]) != 0u) {   // someone else gave up
            ok = 0;
            break;
          }
          if (globaltimer_ns() - t0 > kWaitBudgetNs) {
            if (atomicCAS(a.status, 0, CTDK_ETIMEOUT) == 0) {
              a.status[1] = 90;
              a.status[2] = static_cast<int>(blockIdx.x);
              a.status[3] = static_cast<int>(epoch);
            }
            atomicExch(&a.sync[2], 1u);
            ok = 0;
            break;
          }
        }
      }
    }
    if (ok && ld_acquire_u32(&a.sync[2]) != 0u) ok = 0;
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}
// Rows n = first, first + step, ... of W[N, K] for this warp when WPR warps of a CTA share a row.
template <int WPR>
__device__ __forceinline__ void row_walk(int& first, int& step) {
  const int wid = threadIdx.x >> 5;
  first = blockIdx.x * (8 / WPR) + wid / WPR;
  step = gridDim.x * (8 / WPR);
}
// Requests this warp's share of W[N, K] into L2 (one 128-byte line per lane and iteration).
template <int WPR>
__device__ __forceinline__ void prefetch_rows(const float* __restrict__ W, int N, int K) {
  int first, step;
  row_walk<WPR>(first, step);
  const int lane = threadIdx.x & 31, part = (threadIdx.x >> 5) % WPR;
  const int Kp = K / WPR;
  for (int n = first; n < N; n += step) {
    const char* row = reinterpret_cast<const char*>(W + static_cast<int64_t>(n) * K + part * Kp);
    for (int off = lane * 128; off < Kp * 4; off += 32 * 128) prefetch_l2(row + off);
  }
}
// y[n] = dot(W[n, :], xs) (+ residual[n]); xs is the staged input in shared memory. With WPR > 1
// the warps of a group each take a K range and meet on a named barrier.
template <int WPR>
__device__ __forceinline__ void gemv_rows(const float* __restrict__ W, const float* xs, float* __restrict__ y,
                                          const float* __restrict__ residual, int N, int K, float* pair_red) {
  int first, step;
  row_walk<WPR>(first, step);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, part = wid % WPR;
  const int Kp4 = K / WPR / 4;
  const float4* x4 = reinterpret_cast<const float4*>(xs) + part * Kp4;
  for (int n = first; n < N; n += step) {
    const float4* w4 = reinterpret_cast<const float4*>(W + static_cast<int64_t>(n) * K) + part * Kp4;
    float acc = 0.0f;
#pragma unroll 8
    for (int i = lane; i < Kp4; i += 32) {
      const float4 w = __ldcs(w4 + i), v = x4[i];
      acc += w.x * v.x + w.y * v.y + w.z * v.z + w.w * v.w;
    }
    acc = warp_sum(acc);
    if (WPR == 1) {
      if (lane == 0) y[n] = residual != nullptr ? acc + __ldcg(residual + n) : acc;
    } else {
      if (lane == 0) pair_red[wid] = acc;
      asm volatile("bar.sync %0, %1;" ::"r"(1 + wid / WPR), "r"(32 * WPR) : "memory");
      if (part == 0 && lane == 0) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < WPR; ++k) t += pair_red[wid + k];
        y[n] = residual != nullptr ? t + __ldcg(residual + n) : t;
      }
      asm volatile("bar.sync %0, %1;" ::"r"(1 + wid / WPR), "r"(32 * WPR) : "memory");
    }
  }
}
// xs = x * rsqrt(mean(x^2) + eps) * nw (every CTA stages its own copy).
__device__ __forceinline__ void stage_rmsnorm(const float* __restrict__ x, const float* __restrict__ nw, float eps, int K,
                                              float* xs, float* red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < K; i += blockDim.x) {
    const float v = __ldcg(x + i);   // written by other CTAs one barrier ago: not through L1
    xs[i] = v;
    ss += v * v;
  }
  ss = warp_sum(ss);
  if (lane == 0) red[wid] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float sc = rsqrtf(tot / static_cast<float>(K) + eps);
  for (int i = threadIdx.x; i < K; i += blockDim.x) xs[i] = xs[i] * sc * nw[i];
  __syncthreads();
}

// Post-processes head `slot` of the new row (per-head RMSNorm when w != nullptr, then RoPE at pos)
// into dst[D]; one warp.
__device__ __forceinline__ void head_post(const float* __restrict__ xr, const float* __restrict__ w, const float2* __restrict__ table,
                                          int pos, int D, float eps, float* dst) {
  const int lane = threadIdx.x & 31, Dh = D / 2;
  float s = 1.0f;
  if (w != nullptr) {
    float ss = 0.0f;
    for (int i = lane; i < D; i += 32) {
      const float v = __ldcg(xr + i);
      ss += v * v;
    }
    ss = warp_sum(ss);
    s = rsqrtf(ss / static_cast<float>(D) + eps);
  }
  for (int i = lane; i < Dh; i += 32) {
    float p = __ldcg(xr + i), q = __ldcg(xr + i + Dh);
    if (w != nullptr) {
      p = p * s * w[i];
      q = q * s * w[i + Dh];
    }
    const float2 cs = table[static_cast<int64_t>(pos) * Dh + i];
    dst[i] = p * cs.x - q * cs.y;
    dst[i + Dh] = p * cs.y + q * cs.x;
  }
}

__global__ void __launch_bounds__(256, 2) decode_persistent_kernel(const __grid_constant__ PersistArgs a) {
  extern __shared__ float sm[];   // staged input vector (up to max(hid, H*D, I) floats), then attention scratch
  __shared__ float red[8];
  __shared__ float pair_red[8];
  __shared__ unsigned long long best_s[8];
  __shared__ int s_last;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int hid = a.hid, I = a.I, D = a.D, H = a.H, Hk = a.Hk, G = H / Hk;
  const int64_t cache_layer = static_cast<int64_t>(Hk) * a.max_seq * D;
  unsigned int epoch = 0;
  int pos = a.counters[0];
  int64_t tok = *a.cur_token;
  unsigned long long* words = reinterpret_cast<unsigned long long*>(a.sync + 128);
  bool alive = true;

  for (int t = 0; t < a.n_tokens && alive; ++t) {
    const float* xin = a.P + a.embed + tok * hid;   // layer 0 reads the embedding row in place
    for (int l = 0; l < a.L && alive; ++l) {
      const PLayer& w = a.lw[l];
      // ---- phase 1: qkv = Wqkv rmsnorm(x) ----
      stage_rmsnorm(xin, a.P + w.w_in, a.eps, hid, sm, red);
      gemv_rows<1>(a.P + w.wq, sm, a.qkv, nullptr, a.QKVN, hid, pair_red);
      prefetch_rows<2>(a.P + w.wo, hid, H * D);
      if (!(alive = grid_barrier(a, epoch))) break;

      // ---- phase 2: attention of the new row, split over key ranges; the last split of a head merges ----
      {
        float* kc = a.kcache + l * cache_layer;
        float* vc = a.vcache + l * cache_layer;
        const int Lk = pos + 1;
        const int per = (Lk + kPersistSplits - 1) / kPersistSplits;
        float* qs = sm;                 // [D] post-processed q of the head
        float* kn = sm + D;             // [D] post-processed new k of the kv head
        float* sc = sm + 2 * D;         // [per] scores
        float* scr = sc + (((a.max_seq + kPersistSplits - 1) / kPersistSplits + 4) & ~3);   // [8][D] per-warp partial sums
        for (int item = blockIdx.x; item < H * kPersistSplits; item += gridDim.x) {
          const int h = item / kPersistSplits, sp = item % kPersistSplits, hk = h / G;
          const int j0 = sp * per, j1 = min(Lk, j0 + per);
          float* dst = a.attn_part + (static_cast<int64_t>(h) * kPersistSplits + sp) * (D + 2);
          const bool has_new = pos >= j0 && pos < j1;   // this range ends with the new position
          if (wid == 0) head_post(a.qkv + static_cast<int64_t>(h) * D, a.qk_norm ? a.P + w.wqn : nullptr, a.table, pos, D, a.eps, qs);
          if (wid == 1 && has_new) {
            head_post(a.qkv + static_cast<int64_t>(H + hk) * D, a.qk_norm ? a.P + w.wkn : nullptr, a.table, pos, D, a.eps, kn);
            if (h % G == 0) {   // one head of the group puts the new K / V rows into the cache for later tokens
              __syncwarp();
              for (int i = lane; i < D; i += 32) {
                kc[(static_cast<int64_t>(hk) * a.max_seq + pos) * D + i] = kn[i];
                vc[(static_cast<int64_t>(hk) * a.max_seq + pos) * D + i] = __ldcg(a.qkv + static_cast<int64_t>(H + Hk + hk) * D + i);
              }
            }
          }
          __syncthreads();
          const float* kb = kc + static_cast<int64_t>(hk) * a.max_seq * D;
          const float* vb = vc + static_cast<int64_t>(hk) * a.max_seq * D;
          const float* vnew = a.qkv + static_cast<int64_t>(H + Hk + hk) * D;
          // scores: one warp per key (a key row is one coalesced read of the warp), four keys in flight
          float mx = -FLT_MAX;
          {
            const float4* q4 = reinterpret_cast<const float4*>(qs);
            const int D4 = D / 4;
            for (int jb = j0 + wid; jb < j1; jb += 32) {
              float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int j = jb + 8 * u;
                if (j < j1) {
                  const float4* kr = reinterpret_cast<const float4*>(j == pos ? kn : kb + static_cast<int64_t>(j) * D);
                  for (int i = lane; i < D4; i += 32) {
                    const float4 k4 = kr[i], b4 = q4[i];
                    part[u] += k4.x * b4.x + k4.y * b4.y + k4.z * b4.z + k4.w * b4.w;
                  }
                }
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int j = jb + 8 * u;
                const float v = warp_sum(part[u]) * a.scale;
                if (j < j1) {
                  if (lane == 0) sc[j - j0] = v;
                  mx = fmaxf(mx, v);
                }
              }
            }
          }
          mx = warp_max(mx);
          if (lane == 0) red[wid] = mx;
          __syncthreads();
          mx = -FLT_MAX;
#pragma unroll
          for (int i = 0; i < 8; ++i) mx = fmaxf(mx, red[i]);
          __syncthreads();
          float sum = 0.0f;
          for (int j = j0 + threadIdx.x; j < j1; j += blockDim.x) {
            const float e = __expf(sc[j - j0] - mx);
            sc[j - j0] = e;
            sum += e;
          }
          sum = warp_sum(sum);
          if (lane == 0) red[wid] = sum;
          __syncthreads();
          sum = 0.0f;
#pragma unroll
          for (int i = 0; i < 8; ++i) sum += red[i];
          // weighted sum of the value rows: one warp per key (a row is one coalesced read), four rows in
          // flight per warp; the eight warps' sums meet in shared memory
          {
            const int D4 = D / 4;
            float4 acc4[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};   // D <= 256: two float4 per lane
            for (int jb = j0 + wid; jb < j1; jb += 32) {
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int j = jb + 8 * u;
                if (j < j1) {
                  const float pj = sc[j - j0];
                  const float4* vr = reinterpret_cast<const float4*>(j == pos ? vnew : vb + static_cast<int64_t>(j) * D);
#pragma unroll
                  for (int c = 0; c < 2; ++c) {
                    const int i = lane + 32 * c;
                    if (i < D4) {
                      const float4 v4 = j == pos ? __ldcg(vr + i) : vr[i];
                      acc4[c].x += pj * v4.x;
                      acc4[c].y += pj * v4.y;
                      acc4[c].z += pj * v4.z;
                      acc4[c].w += pj * v4.w;
                    }
                  }
                }
              }
            }
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const int i = lane + 32 * c;
              if (i < D4) reinterpret_cast<float4*>(scr + wid * D)[i] = acc4[c];
            }
          }
          __syncthreads();
          if (threadIdx.x < D) {
            float tsum = 0.0f;
#pragma unroll
            for (int p2 = 0; p2 < 8; ++p2) tsum += scr[p2 * D + threadIdx.x];
            dst[2 + threadIdx.x] = j0 < j1 ? tsum : 0.0f;
          }
          if (threadIdx.x == 0) {
            dst[0] = j0 < j1 ? mx : -FLT_MAX;
            dst[1] = j0 < j1 ? sum : 0.0f;
          }
          // the split that arrives last at its head merges all of them
          __threadfence();
          __syncthreads();
          if (threadIdx.x == 0) {
            const unsigned int prev = atomicAdd(&a.sync[8 + h], 1u);
            s_last = prev == static_cast<unsigned int>(kPersistSplits - 1);
            if (s_last) a.sync[8 + h] = 0u;   // next use is a grid barrier away
          }
          __syncthreads();
          if (s_last) {
            __threadfence();
            const float* pp = a.attn_part + static_cast<int64_t>(h) * kPersistSplits * (D + 2);
            float M = -FLT_MAX;
#pragma unroll
            for (int s2 = 0; s2 < kPersistSplits; ++s2) M = fmaxf(M, __ldcg(pp + s2 * (D + 2)));
            float lsum = 0.0f, wv[kPersistSplits];
#pragma unroll
            for (int s2 = 0; s2 < kPersistSplits; ++s2) {
              wv[s2] = __expf(__ldcg(pp + s2 * (D + 2)) - M);
              lsum += __ldcg(pp + s2 * (D + 2) + 1) * wv[s2];
            }
            const float inv = 1.0f / lsum;
            for (int dd = threadIdx.x; dd < D; dd += blockDim.x) {
              float o = 0.0f;
#pragma unroll
              for (int s2 = 0; s2 < kPersistSplits; ++s2) o += __ldcg(pp + s2 * (D + 2) + 2 + dd) * wv[s2];
              a.attn[static_cast<int64_t>(h) * D + dd] = o * inv;
            }
          }
          __syncthreads();
        }
      }
      prefetch_rows<1>(a.P + w.wg, 2 * I, hid);
      if (!(alive = grid_barrier(a, epoch))) break;

      // ---- phase 3: hm = x + Wo attn ----
      for (int i = threadIdx.x; i < H * D; i += blockDim.x) sm[i] = __ldcg(a.attn + i);
      __syncthreads();
      gemv_rows<2>(a.P + w.wo, sm, a.hm, xin, hid, H * D, pair_red);
      prefetch_rows<2>(a.P + w.wd, hid, I);
      if (!(alive = grid_barrier(a, epoch))) break;

      // ---- phase 4: gu = Wgu rmsnorm(hm) ----
      stage_rmsnorm(a.hm, a.P + w.w_post, a.eps, hid, sm, red);
      gemv_rows<1>(a.P + w.wg, sm, a.gu, nullptr, 2 * I, hid, pair_red);
      if (l + 1 < a.L) prefetch_rows<1>(a.P + a.lw[l + 1].wq, a.QKVN, hid);
      if (!(alive = grid_barrier(a, epoch))) break;

      // ---- phase 5: x = hm + Wd (silu(gate) * up) ----
      for (int i = threadIdx.x; i < I; i += blockDim.x) {
        const float g = __ldcg(a.gu + i);
        sm[i] = g / (1.0f + __expf(-g)) * __ldcg(a.gu + I + i);
      }
      __syncthreads();
      gemv_rows<2>(a.P + w.wd, sm, a.x, a.hm, hid, I, pair_red);
      if (!(alive = grid_barrier(a, epoch))) break;
      xin = a.x;
    }
    if (!alive) break;

    // ---- LM head (tied embedding) + arg-max: first index of the maximum ----
    stage_rmsnorm(xin, a.P + a.norm, a.eps, hid, sm, red);
    {
      unsigned long long best = 0ull;
      int first, step;
      row_walk<1>(first, step);
      const int K4 = hid / 4;
      const float4* x4 = reinterpret_cast<const float4*>(sm);
      const float* E = a.P + a.embed;
      for (int n = first; n < a.V; n += step) {
        const float4* w4 = reinterpret_cast<const float4*>(E + static_cast<int64_t>(n) * hid);
        float acc = 0.0f;
#pragma unroll 8
        for (int i = lane; i < K4; i += 32) {
          const float4 wv4 = __ldcs(w4 + i), v = x4[i];
          acc += wv4.x * v.x + wv4.y * v.y + wv4.z * v.z + wv4.w * v.w;
        }
        acc = warp_sum(acc);
        if (lane == 0) {
          a.logits[n] = acc;
          const unsigned long long k = argmax_key(acc, n);
          best = k > best ? k : best;
        }
      }
      if (lane == 0) best_s[wid] = best;
      __syncthreads();
      if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 1; i < 8; ++i) best = best_s[i] > best ? best_s[i] : best;
        atomicMax(&words[t & 1], best);
      }
    }
    if (!(alive = grid_barrier(a, epoch))) break;
    {
      const unsigned long long wv = *reinterpret_cast<volatile unsigned long long*>(&words[t & 1]);
      tok = static_cast<int64_t>(0xFFFFFFFFu - static_cast<unsigned>(wv & 0xFFFFFFFFull));
      if (blockIdx.x == 0 && threadIdx.x == 0) {
        a.out_tokens[a.out_offset + t] = tok;
        words[(t + 1) & 1] = 0ull;   // last read one barrier ago
      }
      pos += 1;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    a.counters[0] = pos;
    a.counters[1] += a.n_tokens;
    *a.cur_token = tok;
  }
}

}  // namespace
}  // namespace ctdk

// ----------------------------------------------------------------------------------------
// Host side: the decode engine
// ----------------------------------------------------------------------------------------
namespace ctdk {
namespace {

struct LayerW {
  int64_t w_in, wq, wo, wqn, wkn, w_post, wg, wd;
};

struct Decoder {
  ctdk_model_config cfg;
  const float* params;
  int64_t embed, norm;
  std::vector<LayerW> lw;
  int max_seq, QKVN;
  // workspace
  float *rope_table, *kcache, *vcache;  // caches: [L][Hk][max_seq][D]
  float *x, *h1, *qkv, *q, *attn, *hm, *gu, *act, *logits;
  float* attn_part;   // [H][kAttnSplits][D + 2] partial results of the decode attention
  float *pa, *pb, *pqkv, *pattn, *plse, *pgu, *pact;  // prefill buffers ([max_seq, ...])
  int64_t* cur_token;
  int* counters;  // [0] = position of the next token, [1] = tokens generated
  unsigned int* sync = nullptr;
  int persistent_grid = -1;   // CTAs of the persistent token kernel; 0 = not usable here; -1 = not decided yet
  cudaGraphExec_t graph = nullptr;
  int64_t* graph_out = nullptr;
  cudaStream_t graph_stream = nullptr;
  int64_t prompt_len = 0, generated = 0;
  int64_t stepped = 0;   // tokens fed one by one through ctdk_decode_step since the prefill
};

struct Bump2 {
  char* base;
  int64_t used = 0;
  explicit Bump2(void* b) : base(static_cast<char*>(b)) {}
  float* floats(int64_t n) {
    const int64_t bytes = (n * 4 + 255) / 256 * 256;
    float* p = base ? reinterpret_cast<float*>(base + used) : nullptr;
    used += bytes;
    return p;
  }
};

void carve_decoder(Decoder& d, Bump2& b) {
  const ctdk_model_config& c = d.cfg;
  const int64_t hid = c.hidden_size, I = c.intermediate_size, D = c.head_dim, H = c.num_attention_heads,
                Hk = c.num_key_value_heads, L = c.num_hidden_layers, S = d.max_seq;
  d.rope_table = b.floats(S * D);
  d.kcache = b.floats(L * Hk * S * D);
  d.vcache = b.floats(L * Hk * S * D);
  d.x = b.floats(hid);
  d.h1 = b.floats(hid);
  d.qkv = b.floats(d.QKVN);
  d.q = b.floats(H * D);
  d.attn = b.floats(H * D);
  d.hm = b.floats(hid);
  d.gu = b.floats(2 * I);
  d.act = b.floats(I);
  d.logits = b.floats(c.vocab_size);
  d.pa = b.floats(S * hid);
  d.pb = b.floats(S * hid);
  d.pqkv = b.floats(S * d.QKVN);
  d.pattn = b.floats(S * H * D);
  d.plse = b.floats(H * S);
  d.pgu = b.floats(S * 2 * I);
  d.pact = b.floats(S * I);
  d.attn_part = b.floats(static_cast<int64_t>(H) * (kPersistSplits > kAttnSplits ? kPersistSplits : kAttnSplits) * (D + 2));
  d.cur_token = reinterpret_cast<int64_t*>(b.floats(2));
  d.counters = reinterpret_cast<int*>(b.floats(8));  // position, count, scratch, -, then the 64-bit argmax word
  d.sync = reinterpret_cast<unsigned int*>(b.floats(kSyncWords));   // persistent kernel: grid barrier, per-head arrivals, argmax words
}

int init_decoder(Decoder& d, const ctdk_model_config* cfg, int64_t max_seq) {
  CTDK_REQUIRE(cfg != nullptr && max_seq > 0 && max_seq < (1 << 20), "decoder: bad arguments");
  const int64_t n = ctdk_model_num_tensors(cfg);
  if (n < 0) return CTDK_EINVAL;
  d.cfg = *cfg;
  d.max_seq = static_cast<int>(max_seq);
  d.QKVN = (cfg->num_attention_heads + 2 * cfg->num_key_value_heads) * cfg->head_dim;
  std::vector<int64_t> off(n);
  int rc = ctdk_model_layout(cfg, off.data(), nullptr, nullptr, nullptr);
  if (rc != CTDK_OK) return rc;
  d.embed = off[0];
  d.norm = off[n - 1];
  const int per = cfg->qk_norm ? 11 : 9;
  d.lw.resize(cfg->num_hidden_layers);
  for (int l = 0; l < cfg->num_hidden_layers; ++l) {
    const int64_t* o = off.data() + 1 + static_cast<int64_t>(l) * per;
    LayerW& w = d.lw[l];
    w.w_in = o[0];
    w.wq = o[1];
    w.wo = o[4];
    int i = 5;
    if (cfg->qk_norm) {
      w.wqn = o[5];
      w.wkn = o[6];
      i = 7;
    } else {
      w.wqn = w.wkn = -1;
    }
    w.w_post = o[i];
    w.wg = o[i + 1];
    w.wd = o[i + 3];
  }
  return CTDK_OK;
}

#define DTRY(expr)                    \
  do {                                \
    int rc_ = (expr);                 \
    if (rc_ != CTDK_OK) return rc_;   \
  } while (0)

int gemv(const float* W, const float* x, float* y, const float* residual, int N, int K, cudaStream_t s,
         int pre = kPreNone, const float* nw = nullptr, float eps = 0.0f) {
  CTDK_REQUIRE(K % 4 == 0 && K <= 12288, "gemv: K must be a multiple of 4 and at most 12288");
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int64_t need = (N + 7) / 8;
  const int grid = static_cast<int>(need < cap ? need : cap);
  const size_t smem = K * sizeof(float);
  cudaError_t e;
  if (pre == kPreRmsNorm) e = launch_pdl(gemv_kernel<kPreRmsNorm>, grid, 256, smem, s, W, x, y, residual, nw, eps, N, K);
  else if (pre == kPreSwiglu) e = launch_pdl(gemv_kernel<kPreSwiglu>, grid, 256, smem, s, W, x, y, residual, nw, eps, N, K);
  else e = launch_pdl(gemv_kernel<kPreNone>, grid, 256, smem, s, W, x, y, residual, nw, eps, N, K);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "decode gemv: %s", cudaGetErrorString(e));
  return check_launch("decode gemv");
}

ctdk_rope_params decode_rope_params(const ctdk_model_config& c) {
  ctdk_rope_params p;
  p.theta = c.rope_theta;
  p.scaling_factor = c.rope_scaling_factor;
  p.low_freq_wavelen = static_cast<float>(c.rope_scaling_original_max_pos) / c.rope_scaling_low_freq_factor;
  p.high_freq_wavelen = static_cast<float>(c.rope_scaling_original_max_pos) / c.rope_scaling_high_freq_factor;
  return p;
}

// One token: embedding of *cur_token at position *pos -> logits -> argmax -> counters += 1.
int enqueue_token_forward(Decoder& d, cudaStream_t s) {
  const ctdk_model_config& c = d.cfg;
  const int hid = c.hidden_size, I = c.intermediate_size, D = c.head_dim, H = c.num_attention_heads,
            Hk = c.num_key_value_heads;
  const float* P = d.params;
  const int64_t cache_layer = static_cast<int64_t>(Hk) * d.max_seq * D;
  const float scale = 1.0f / sqrtf(static_cast<float>(D));
  DTRY(ctdk_embedding_fwd(d.cur_token, P + d.embed, d.x, 1, hid, c.vocab_size, s));
  for (int l = 0; l < c.num_hidden_layers; ++l) {
    const LayerW& w = d.lw[l];
    DTRY(gemv(P + w.wq, d.x, d.qkv, nullptr, d.QKVN, hid, s, kPreRmsNorm, P + w.w_in, c.rms_norm_eps));
    if (launch_pdl(decode_qkv_post_kernel, ceil_div((H + 2 * Hk) * 32, 256), 256, 0, s, d.qkv,
                   c.qk_norm ? P + w.wqn : nullptr, c.qk_norm ? P + w.wkn : nullptr,
                   reinterpret_cast<const float2*>(d.rope_table), d.counters, d.q, d.kcache + l * cache_layer,
                   d.vcache + l * cache_layer, H, Hk, D, d.max_seq, c.rms_norm_eps) != cudaSuccess)
      return fail(CTDK_ELAUNCH, "decode qkv post: launch failed");
    DTRY(check_launch("decode qkv post"));
    if (launch_pdl(decode_attn_kernel, dim3(H, kAttnSplits), 256,
                   ((d.max_seq + kAttnSplits - 1) / kAttnSplits + 4 + D + 256) * sizeof(float), s, d.q,
                   d.kcache + l * cache_layer, d.vcache + l * cache_layer, d.attn_part, d.counters, H, Hk, D, d.max_seq,
                   scale) != cudaSuccess)
      return fail(CTDK_ELAUNCH, "decode attention: launch failed");
    if (launch_pdl(decode_attn_combine_kernel, H, 128, 0, s, d.attn_part, d.attn, D) != cudaSuccess)
      return fail(CTDK_ELAUNCH, "decode attention combine: launch failed");
    DTRY(check_launch("decode attention"));
    DTRY(gemv(P + w.wo, d.attn, d.hm, d.x, hid, H * D, s));
    DTRY(gemv(P + w.wg, d.hm, d.gu, nullptr, 2 * I, hid, s, kPreRmsNorm, P + w.w_post, c.rms_norm_eps));
    DTRY(gemv(P + w.wd, d.gu, d.x, d.hm, hid, I, s, kPreSwiglu));
  }
  return gemv(P + d.embed, d.x, d.logits, nullptr, c.vocab_size, hid, s, kPreRmsNorm, P + d.norm, c.rms_norm_eps);
}

int enqueue_token_step(Decoder& d, int64_t* out_tokens, cudaStream_t s) {
  DTRY(enqueue_token_forward(d, s));
  unsigned long long* word = reinterpret_cast<unsigned long long*>(d.counters + 4);
  if (launch_pdl(argmax_kernel, 64, 256, 0, s, d.logits, d.cfg.vocab_size, word) != cudaSuccess)
    return fail(CTDK_ELAUNCH, "decode argmax: launch failed");
  DTRY(check_launch("decode argmax"));
  if (launch_pdl(argmax_finish_kernel, 1, 1, 0, s, word, d.cur_token, out_tokens, d.counters, d.counters + 1) != cudaSuccess)
    return fail(CTDK_ELAUNCH, "decode argmax finish: launch failed");
  return check_launch("decode argmax finish");
}

// Returns CTDK_OK when the persistent kernel was launched for `n` tokens, 1 when it does not apply
// (the caller takes the kernel-per-phase path), or a negative status.
int launch_persistent(Decoder& d, int64_t n, int64_t* out_tokens, cudaStream_t s) {
  const ctdk_model_config& c = d.cfg;
  const int hid = c.hidden_size, I = c.intermediate_size, D = c.head_dim, H = c.num_attention_heads;
  const size_t stage = static_cast<size_t>(std::max(std::max(hid, H * D), I));
  const size_t attn = static_cast<size_t>(2 * D + (d.max_seq + kPersistSplits - 1) / kPersistSplits + 8 + 8 * D);
  const size_t smem = std::max(stage, attn) * sizeof(float);
  if (d.persistent_grid < 0) {
    d.persistent_grid = 0;
    const char* env = std::getenv("CTDK_DECODE_PERSISTENT");
    const bool off = env != nullptr && env[0] == '0';
    int dev = 0, coop = 0, per_sm = 0;
    const bool shape_ok = c.num_hidden_layers <= kMaxPersistLayers && hid % 8 == 0 && (H * D) % 8 == 0 && I % 8 == 0 && D % 4 == 0 &&
                          256 % D == 0 && H <= 96 && smem <= 96 * 1024 && n < (1 << 20);
    if (!off && shape_ok && cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && coop != 0 &&
        cudaFuncSetAttribute(decode_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) == cudaSuccess &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_persistent_kernel, 256, smem) == cudaSuccess && per_sm >= 1)
      d.persistent_grid = sm_count() * (per_sm > 2 ? 2 : per_sm);
    cudaGetLastError();
  }
  if (d.persistent_grid <= 0) return 1;
  PersistArgs a{};
  a.P = d.params;
  for (int l = 0; l < c.num_hidden_layers; ++l) {
    const LayerW& w = d.lw[l];
    a.lw[l] = PLayer{w.w_in, w.wq, w.wo, w.wqn, w.wkn, w.w_post, w.wg, w.wd};
  }
  a.embed = d.embed;
  a.norm = d.norm;
  a.L = c.num_hidden_layers;
  a.hid = hid;
  a.I = I;
  a.D = D;
  a.H = H;
  a.Hk = c.num_key_value_heads;
  a.V = c.vocab_size;
  a.QKVN = d.QKVN;
  a.max_seq = d.max_seq;
  a.qk_norm = c.qk_norm;
  a.eps = c.rms_norm_eps;
  a.scale = 1.0f / sqrtf(static_cast<float>(D));
  a.table = reinterpret_cast<const float2*>(d.rope_table);
  a.kcache = d.kcache;
  a.vcache = d.vcache;
  a.x = d.x;
  a.qkv = d.qkv;
  a.attn = d.attn;
  a.hm = d.hm;
  a.gu = d.gu;
  a.logits = d.logits;
  a.attn_part = d.attn_part;
  a.cur_token = d.cur_token;
  a.counters = d.counters;
  a.sync = d.sync;
  a.out_tokens = out_tokens;
  a.out_offset = static_cast<int>(d.generated);
  a.n_tokens = static_cast<int>(n);
  a.status = device_status_word();
  if (a.status == nullptr) return fail(CTDK_ELAUNCH, "decode: no status word");
  if (cudaMemsetAsync(d.sync, 0, kSyncWords * sizeof(unsigned int), s) != cudaSuccess)
    return fail(CTDK_ELAUNCH, "decode: clearing the barrier words failed");
  void* params[] = {&a};
  const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(decode_persistent_kernel), dim3(d.persistent_grid),
                                                    dim3(256), params, smem, s);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "decode: cooperative launch failed: %s", cudaGetErrorString(e));
  return check_launch("decode persistent");
}

__global__ void set_token_kernel(int64_t* cur, int64_t value) { *cur = value; }
__global__ void bump_position_kernel(int* position) { *position += 1; }

}  // namespace
}  // namespace ctdk

using namespace ctdk;

extern "C" {

int64_t ctdk_decode_workspace_bytes(const ctdk_model_config* cfg, int64_t max_seq) {
  Decoder d;
  if (init_decoder(d, cfg, max_seq) != CTDK_OK) return -1;
  Bump2 b(nullptr);
  carve_decoder(d, b);
  return b.used;
}

int ctdk_decode_create(const ctdk_model_config* cfg, const float* params, void* workspace,
                       int64_t workspace_bytes, int64_t max_seq, void** decoder) {
  CTDK_REQUIRE(decoder && params && workspace, "ctdk_decode_create: null pointer");
  CTDK_REQUIRE((reinterpret_cast<uintptr_t>(params) & 255u) == 0 && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
               "ctdk_decode_create: arenas must be 256-byte aligned");
  Decoder* d = new (std::nothrow) Decoder();
  if (d == nullptr) return fail(CTDK_ENOMEM, "ctdk_decode_create: out of host memory");
  int rc = init_decoder(*d, cfg, max_seq);
  if (rc != CTDK_OK) {
    delete d;
    return rc;
  }
  const int64_t attn_smem = ((static_cast<int64_t>(max_seq) + kAttnSplits - 1) / kAttnSplits + 4 + cfg->head_dim + 256) * 4;
  CTDK_REQUIRE(attn_smem <= 200 * 1024, "ctdk_decode_create: max_seq too large for the decode attention kernel");
  CTDK_REQUIRE(cfg->head_dim <= 256 && 256 % cfg->head_dim == 0, "ctdk_decode_create: head_dim must divide 256");
  d->params = params;
  Bump2 b(workspace);
  carve_decoder(*d, b);
  if (b.used > workspace_bytes) {
    delete d;
    return fail(CTDK_EINVAL, "ctdk_decode_create: workspace too small");
  }
  cudaError_t e = cudaFuncSetAttribute(decode_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(attn_smem));
  if (e != cudaSuccess) {
    delete d;
    return fail(CTDK_ELAUNCH, "ctdk_decode_create: %s", cudaGetErrorString(e));
  }
  *decoder = d;
  return CTDK_OK;
}

int ctdk_decode_destroy(void* decoder) {
  Decoder* d = static_cast<Decoder*>(decoder);
  if (d != nullptr && d->graph != nullptr) cudaGraphExecDestroy(d->graph);
  delete d;
  return CTDK_OK;
}

int ctdk_decode_prefill(void* decoder, const int64_t* ids, int64_t T, void* stream) {
  CTDK_REQUIRE(decoder && ids, "ctdk_decode_prefill: null pointer");
  Decoder& d = *static_cast<Decoder*>(decoder);
  const ctdk_model_config& c = d.cfg;
  CTDK_REQUIRE(T > 0 && T < d.max_seq, "ctdk_decode_prefill: prompt length must be in [1, max_seq)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int hid = c.hidden_size, I = c.intermediate_size, D = c.head_dim, H = c.num_attention_heads,
            Hk = c.num_key_value_heads;
  const float* P = d.params;
  const int64_t cache_layer = static_cast<int64_t>(Hk) * d.max_seq * D;
  const ctdk_rope_params rp = decode_rope_params(c);
  DTRY(ctdk_rope_table(d.rope_table, d.max_seq, D, 0, &rp, s));
  DTRY(ctdk_embedding_fwd(ids, P + d.embed, d.pa, T, hid, c.vocab_size, s));
  const int prec = c.precision;
  for (int l = 0; l < c.num_hidden_layers; ++l) {
    const LayerW& w = d.lw[l];
    DTRY(ctdk_rmsnorm_fwd(d.pa, P + w.w_in, d.pb, nullptr, T, hid, c.rms_norm_eps, s));
    DTRY(ctdk_gemm(d.pb, P + w.wq, d.pqkv, T, d.QKVN, hid, hid, hid, d.QKVN, 0, 1, prec, CTDK_EPI_STORE, nullptr, s));
    if (c.qk_norm) {
      // out of place is required with norm weights: reuse the gate|up buffer as the destination
      CTDK_REQUIRE(2 * I >= d.QKVN, "ctdk_decode_prefill: intermediate size too small for the QK-Norm buffer");
      DTRY(ctdk_qk_norm_rope_fwd(d.pqkv, d.pgu, P + w.wqn, P + w.wkn, d.pattn, d.pattn + T * H, d.rope_table, 1, T, H,
                                 Hk, D, c.rms_norm_eps, s));
      DTRY(ctdk_scale(d.pgu, 1.0f, d.pqkv, T * static_cast<int64_t>(d.QKVN), s));
    } else {
      DTRY(ctdk_qk_norm_rope_fwd(d.pqkv, d.pqkv, nullptr, nullptr, nullptr, nullptr, d.rope_table, 1, T, H, Hk, D,
                                 c.rms_norm_eps, s));
    }
    kv_write_rows_kernel<<<sm_count() * 4, 256, 0, s>>>(d.pqkv, d.kcache + l * cache_layer, d.vcache + l * cache_layer,
                                                        static_cast<int>(T), H, Hk, D, d.max_seq);
    DTRY(check_launch("decode kv write"));
    DTRY(ctdk_attn_fwd_p(d.pqkv, d.pattn, d.plse, 1, T, H, Hk, D, prec, s));
    DTRY(ctdk_gemm(d.pattn, P + w.wo, d.pb, T, hid, H * D, H * D, H * D, hid, 0, 1, prec, CTDK_EPI_RESIDUAL, d.pa, s));
    DTRY(ctdk_rmsnorm_fwd(d.pb, P + w.w_post, d.pa, nullptr, T, hid, c.rms_norm_eps, s));
    DTRY(ctdk_gemm(d.pa, P + w.wg, d.pgu, T, 2 * I, hid, hid, hid, 2 * I, 0, 1, prec, CTDK_EPI_STORE, nullptr, s));
    DTRY(ctdk_swiglu_fwd(d.pgu, d.pact, T, I, s));
    DTRY(ctdk_gemm(d.pact, P + w.wd, d.pa, T, hid, I, I, I, hid, 0, 1, prec, CTDK_EPI_RESIDUAL, d.pb, s));
  }
  // logits of the last prompt position only, then the first generated token
  DTRY(ctdk_rmsnorm_fwd(d.pa + (T - 1) * hid, P + d.norm, d.h1, nullptr, 1, hid, c.rms_norm_eps, s));
  DTRY(gemv(P + d.embed, d.h1, d.logits, nullptr, c.vocab_size, hid, s));
  set_counters_kernel<<<1, 1, 0, s>>>(d.counters, d.counters + 1, static_cast<int>(T), 0);
  d.prompt_len = T;
  d.generated = 0;
  d.stepped = 0;
  return check_launch("decode counters");
}

int ctdk_decode_logits(void* decoder, const float** logits) {
  CTDK_REQUIRE(decoder && logits, "ctdk_decode_logits: null pointer");
  *logits = static_cast<Decoder*>(decoder)->logits;
  return CTDK_OK;
}

int ctdk_decode_step(void* decoder, int64_t token, void* stream) {
  CTDK_REQUIRE(decoder != nullptr, "ctdk_decode_step: null decoder");
  Decoder& d = *static_cast<Decoder*>(decoder);
  CTDK_REQUIRE(d.prompt_len > 0, "ctdk_decode_step: call ctdk_decode_prefill first");
  CTDK_REQUIRE(d.generated == 0, "ctdk_decode_step: cannot be mixed with ctdk_decode_greedy after one prefill");
  CTDK_REQUIRE(token >= 0 && token < d.cfg.vocab_size, "ctdk_decode_step: token id out of range");
  CTDK_REQUIRE(d.prompt_len + d.stepped < d.max_seq, "ctdk_decode_step: the cache is full (max_seq %d)", d.max_seq);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  set_token_kernel<<<1, 1, 0, s>>>(d.cur_token, token);
  DTRY(check_launch("decode set token"));
  DTRY(enqueue_token_forward(d, s));
  bump_position_kernel<<<1, 1, 0, s>>>(d.counters);
  DTRY(check_launch("decode bump"));
  ++d.stepped;
  return CTDK_OK;
}

int ctdk_decode_greedy(void* decoder, int64_t n_new, int64_t* out_tokens, void* stream) {
  CTDK_REQUIRE(decoder && out_tokens, "ctdk_decode_greedy: null pointer");
  CTDK_REQUIRE(n_new >= 0, "ctdk_decode_greedy: negative token count");
  Decoder& d = *static_cast<Decoder*>(decoder);
  CTDK_REQUIRE(d.prompt_len > 0, "ctdk_decode_greedy: call ctdk_decode_prefill first");
  CTDK_REQUIRE(d.stepped == 0, "ctdk_decode_greedy: cannot be mixed with ctdk_decode_step after one prefill");
  // n tokens after the prompt need n - 1 cache positions (the first comes from the prompt's logits, the
  // last is not fed back): the reference's loop emits max_seq - prompt + 1 tokens before it reports
  // max_seq_len (tools/ctd_generate/main.cpp:143-179)
  CTDK_REQUIRE(d.prompt_len + d.generated + n_new <= d.max_seq + 1,
               "ctdk_decode_greedy: %lld more tokens would exceed max_seq %d", static_cast<long long>(n_new),
               d.max_seq);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t todo = n_new;
  if (todo > 0 && d.generated == 0) {
    // the first new token comes from the prefill logits; its position is the prompt length
    unsigned long long* word = reinterpret_cast<unsigned long long*>(d.counters + 4);
    argmax_kernel<<<64, 256, 0, s>>>(d.logits, d.cfg.vocab_size, word);
    DTRY(check_launch("decode argmax"));
    // count += 1; the position is unchanged (a scratch int takes the increment)
    argmax_finish_kernel<<<1, 1, 0, s>>>(word, d.cur_token, out_tokens, d.counters + 2, d.counters + 1);
    DTRY(check_launch("decode argmax finish"));
    d.generated = 1;
    --todo;
  }
  if (todo == 0) return CTDK_OK;
  // All remaining tokens in one cooperative launch of the persistent kernel where it applies.
  {
    const int rc = launch_persistent(d, todo, out_tokens, s);
    if (rc <= 0) {
      if (rc == CTDK_OK) d.generated += todo;
      return rc;
    }
  }
  // One token step = ~9 kernels per layer; captured once and replayed, so a step costs one launch.
  const bool can_capture = s != nullptr;
  if (can_capture && (d.graph == nullptr || d.graph_out != out_tokens || d.graph_stream != s)) {
    if (d.graph != nullptr) {
      cudaGraphExecDestroy(d.graph);
      d.graph = nullptr;
    }
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "decode: begin capture: %s", cudaGetErrorString(e));
    const int rc = enqueue_token_step(d, out_tokens, s);
    e = cudaStreamEndCapture(s, &g);
    if (rc != CTDK_OK) {
      if (g != nullptr) cudaGraphDestroy(g);
      return rc;
    }
    if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "decode: end capture: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&d.graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "decode: graph instantiate: %s", cudaGetErrorString(e));
    d.graph_out = out_tokens;
    d.graph_stream = s;
  }
  for (int64_t i = 0; i < todo; ++i) {
    if (can_capture) {
      cudaError_t e = cudaGraphLaunch(d.graph, s);
      if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "decode: graph launch: %s", cudaGetErrorString(e));
    } else {
      DTRY(enqueue_token_step(d, out_tokens, s));
    }
  }
  d.generated += todo;
  return CTDK_OK;
}

}  // extern "C"
