// Token sampling on the device: greedy, temperature, top-k and top-p with the reference sampler's
// semantics (emberlm src/core/sampling.cpp:13-106), so that a seeded request draws the same tokens:
//   temperature <= 0      first index of the maximum logit
//   otherwise             x = logit / T; with 0 < top_k < V every x below the k-th largest becomes
//                         -inf (ties at the threshold survive); p = softmax(x) with the sum taken in
//                         double; with 0 < top_p < 1 the largest probabilities are kept, in
//                         descending order, until their running sum reaches top_p, the rest are
//                         zeroed and p is renormalised; the token is the first index i, in index
//                         order, whose running sum exceeds the uniform draw u.
// The reference copies the [V] logits to the host and sorts there for every token; here only the
// draw u (one uniform_real_distribution<double> value per row, drawn by the caller from its
// mt19937_64 in row order) goes to the device and one int64 per row comes back. One CTA per row;
// the k-th largest value and the top-p cut are found by a 4-pass radix descent over the float
// bits instead of a sort.
#include <cfloat>
#include <climits>

#include "common.cuh"

namespace ctdk {
namespace {

constexpr int kThreads = 1024;

// Monotonic map float -> uint32 (larger float = larger key).
__device__ __forceinline__ uint32_t key_of(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Shared {
  unsigned int count[256];
  double sum[256];
  double red[32];
  int redi[32];
  float redf[32];
  uint32_t prefix;       // key bits fixed so far
  unsigned int remaining;
  double cum;            // probability mass above the current prefix range
  int tie_keep;          // number of elements equal to the cut value that stay
  int result;
};

__device__ __forceinline__ double block_sum(double v, Shared& s) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) s.red[w] = v;
  __syncthreads();
  double t = lane < kThreads / 32 ? s.red[lane] : 0.0;
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}
__device__ __forceinline__ float block_max(float v, Shared& s) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) s.redf[w] = v;
  __syncthreads();
  float t = lane < kThreads / 32 ? s.redf[lane] : -FLT_MAX;
  return warp_max(t);
}

// Key of the k-th largest of x[0..V) (k >= 1).
__device__ uint32_t kth_largest_key(const float* __restrict__ x, int64_t V, float scale, unsigned int k, Shared& s) {
  if (threadIdx.x == 0) {
    s.prefix = 0;
    s.remaining = k;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    if (threadIdx.x < 256) s.count[threadIdx.x] = 0;
    __syncthreads();
    const uint32_t prefix = s.prefix;
    for (int64_t i = threadIdx.x; i < V; i += kThreads) {
      const uint32_t key = key_of(x[i] * scale);
      if ((key & mask) == prefix) atomicAdd(&s.count[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int need = s.remaining;
      int b = 255;
      for (; b > 0; --b) {
        if (s.count[b] >= need) break;
        need -= s.count[b];
      }
      s.prefix = prefix | (static_cast<uint32_t>(b) << shift);
      s.remaining = need;
    }
    __syncthreads();
  }
  return s.prefix;
}

__global__ void __launch_bounds__(kThreads) sample_kernel(const float* __restrict__ logits, int64_t V, float temperature, int top_k,
                                                          float top_p, const double* __restrict__ u, float* __restrict__ work,
                                                          int64_t* __restrict__ out) {
  __shared__ Shared s;
  const int64_t row = blockIdx.x;
  const float* x = logits + row * V;
  float* p = work + row * V;

  if (temperature <= 0.0f) {   // greedy: first index of the maximum
    float best = -FLT_MAX;
    int64_t bi = V;
    for (int64_t i = threadIdx.x; i < V; i += kThreads)
      if (x[i] > best) {
        best = x[i];
        bi = i;
      }
    const float m = block_max(best, s);
    int cand = (best == m && bi < V) ? static_cast<int>(bi) : INT_MAX;
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s.redi[threadIdx.x >> 5] = cand;
    __syncthreads();
    if (threadIdx.x == 0) {
      int r = INT_MAX;
      for (int w = 0; w < kThreads / 32; ++w) r = min(r, s.redi[w]);
      out[row] = r == INT_MAX ? 0 : r;
    }
    return;
  }

  const float inv_t = 1.0f / temperature;
  float thresh = -INFINITY;
  if (top_k > 0 && top_k < V) {
    const uint32_t key = kth_largest_key(x, V, inv_t, static_cast<unsigned int>(top_k), s);
    const uint32_t b = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
    thresh = __uint_as_float(b);
  }
  // softmax of the surviving logits, the sum in double
  float mx = -FLT_MAX;
  for (int64_t i = threadIdx.x; i < V; i += kThreads) {
    const float v = x[i] * inv_t;
    if (v >= thresh) mx = fmaxf(mx, v);
  }
  mx = block_max(mx, s);
  double part = 0.0;
  for (int64_t i = threadIdx.x; i < V; i += kThreads) {
    const float v = x[i] * inv_t;
    const float e = v >= thresh ? expf(v - mx) : 0.0f;
    p[i] = e;
    part += static_cast<double>(e);
  }
  const double total = block_sum(part, s);
  const float inv = static_cast<float>(1.0 / total);
  for (int64_t i = threadIdx.x; i < V; i += kThreads) p[i] *= inv;
  __syncthreads();

  if (top_p > 0.0f && top_p < 1.0f) {
    // Radix descent over the bits of p: after four passes `prefix` is the smallest probability
    // that is kept and `cum` the mass of everything larger.
    const double target = static_cast<double>(top_p);
    if (threadIdx.x == 0) {
      s.prefix = 0;
      s.cum = 0.0;
    }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      if (threadIdx.x < 256) {
        s.count[threadIdx.x] = 0;
        s.sum[threadIdx.x] = 0.0;
      }
      __syncthreads();
      const uint32_t prefix = s.prefix;
      for (int64_t i = threadIdx.x; i < V; i += kThreads) {
        const uint32_t key = __float_as_uint(p[i]);   // p >= 0: the bits order like the values
        if ((key & mask) == prefix) {
          const unsigned int b = (key >> shift) & 255u;
          atomicAdd(&s.count[b], 1u);
          atomicAdd(&s.sum[b], static_cast<double>(p[i]));
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        double cum = s.cum;
        int b = 255;
        for (; b > 0; --b) {
          if (s.count[b] != 0 && cum + s.sum[b] >= target) break;
          cum += s.sum[b];
        }
        s.prefix = prefix | (static_cast<uint32_t>(b) << shift);
        s.cum = cum;
        if (pass == 3) {
          // of the elements equal to the cut value, as many as it takes to reach the target
          const double v = static_cast<double>(__uint_as_float(s.prefix));
          int keep = 0;
          const int have = static_cast<int>(s.count[b]);
          while (keep < have) {
            cum += v;
            ++keep;
            if (cum >= target) break;
          }
          s.tie_keep = keep > 0 ? keep : 1;
          s.remaining = static_cast<unsigned int>(have);
        }
      }
      __syncthreads();
    }
    const float cut = __uint_as_float(s.prefix);
    // ties at the cut value: the first tie_keep in index order stay. Only when some of them must go
    // (rare: equal probabilities at the cut) does one thread walk the row.
    if (threadIdx.x == 0 && static_cast<unsigned int>(s.tie_keep) < s.remaining) {
      int left = s.tie_keep;
      for (int64_t i = 0; i < V; ++i)
        if (p[i] == cut) {
          if (left > 0) --left;
          else p[i] = 0.0f;
        }
    }
    __syncthreads();
    double kept = 0.0;
    for (int64_t i = threadIdx.x; i < V; i += kThreads) {
      if (p[i] < cut) p[i] = 0.0f;
      kept += static_cast<double>(p[i]);
    }
    const double ksum = block_sum(kept, s);
    if (ksum > 0.0) {
      const float inv2 = static_cast<float>(1.0 / ksum);
      for (int64_t i = threadIdx.x; i < V; i += kThreads) p[i] *= inv2;
    }
    __syncthreads();
  }

  // inverse CDF in index order: the first i with u < p[0] + ... + p[i]
  const int64_t chunk = (V + kThreads - 1) / kThreads;
  const int64_t lo = static_cast<int64_t>(threadIdx.x) * chunk, hi = lo + chunk < V ? lo + chunk : V;
  double mine = 0.0;
  for (int64_t i = lo; i < hi; ++i) mine += static_cast<double>(p[i]);
  // exclusive scan of the per-thread sums (warp scan, then the warp totals)
  double incl = mine;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (int o = 1; o < 32; o <<= 1) {
    const double t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (threadIdx.x == 0) s.result = INT_MAX;
  __syncthreads();
  if (lane == 31) s.red[w] = incl;
  __syncthreads();
  double base = 0.0;
  for (int k = 0; k < w; ++k) base += s.red[k];
  double c = base + incl - mine;
  const double r = u[row];
  for (int64_t i = lo; i < hi; ++i) {
    c += static_cast<double>(p[i]);
    if (r < c) {
      atomicMin(&s.result, static_cast<int>(i));
      break;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) out[row] = s.result == INT_MAX ? V - 1 : s.result;
}

}  // namespace
}  // namespace ctdk

using namespace ctdk;

extern "C" {

int64_t ctdk_sample_workspace_bytes(int64_t B, int64_t V) { return (B < 0 || V < 0) ? -1 : B * V * 4 + 256; }

int ctdk_sample(const float* logits, int64_t B, int64_t V, float temperature, int top_k, float top_p, const double* u,
                void* workspace, int64_t* out_tokens, void* stream) {
  CTDK_REQUIRE(B >= 0 && V > 0 && V < INT32_MAX, "ctdk_sample: bad shape");
  if (B == 0) return CTDK_OK;
  CTDK_REQUIRE(logits && out_tokens, "ctdk_sample: null pointer");
  CTDK_REQUIRE(temperature <= 0.0f || (u != nullptr && workspace != nullptr), "ctdk_sample: sampling needs the draws and the workspace");
  sample_kernel<<<static_cast<unsigned>(B), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, V, temperature, top_k, top_p, u, static_cast<float*>(workspace), out_tokens);
  return check_launch("ctdk_sample");
}

}  // extern "C"
