// The small stand-alone ops of the reference's per-op API that the fused training path absorbs
// but the public op surface (ctd::ops::softmax, permute, repeat_kv_heads, apply_causal_mask,
// mse_loss, the KV-cache copies) still offers: plain HBM-bound kernels with 64-bit indexing, so the
// reference's int32 / gridDim limits (rows * width < 2^31, B*T <= 65535) do not apply.
//   softmax            emberlm src/ops/softmax.cu:18-93
//   permute            src/ops/permute.cu:16-60
//   repeat_kv (+ sum)  src/ops/repeat_kv.cu:14-43
//   causal mask        src/ops/mask.cu:17-60
//   mse                src/ops/loss.cu:17-75
//   kv cache copies    src/ops/kv_cache.cu:14-47
#include <cfloat>

#include "common.cuh"

namespace ctdk {
namespace {

// One warp per row when the row fits a warp's registers comfortably, else one CTA per row.
template <int THREADS>
__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red) {
  v = is_max ? warp_max(v) : warp_sum(v);
  if constexpr (THREADS > 32) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = lane < THREADS / 32 ? red[lane] : (is_max ? -FLT_MAX : 0.0f);
    v = is_max ? warp_max(t) : warp_sum(t);
  }
  return v;
}

__global__ void __launch_bounds__(256) softmax_fwd_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                          int64_t rows, int64_t width) {
  __shared__ float red[8];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* xr = x + r * width;
    float* yr = y + r * width;
    float mx = -FLT_MAX;
    for (int64_t i = threadIdx.x; i < width; i += 256) mx = fmaxf(mx, xr[i]);
    mx = block_reduce<256>(mx, true, red);
    float sum = 0.0f;
    for (int64_t i = threadIdx.x; i < width; i += 256) {
      const float e = __expf(xr[i] - mx);
      yr[i] = e;
      sum += e;
    }
    sum = block_reduce<256>(sum, false, red);
    const float inv = 1.0f / sum;
    for (int64_t i = threadIdx.x; i < width; i += 256) yr[i] *= inv;
  }
}

// dx = y * (g - sum(g * y)) per row.
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const float* __restrict__ y, const float* __restrict__ g,
                                                          float* __restrict__ dx, int64_t rows, int64_t width) {
  __shared__ float red[8];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* yr = y + r * width;
    const float* gr = g + r * width;
    float dot = 0.0f;
    for (int64_t i = threadIdx.x; i < width; i += 256) dot += yr[i] * gr[i];
    dot = block_reduce<256>(dot, false, red);
    for (int64_t i = threadIdx.x; i < width; i += 256) dx[r * width + i] = yr[i] * (gr[i] - dot);
  }
}

struct PermuteArgs {
  int ndim;
  int64_t out_shape[6];
  int64_t in_stride_of_out_dim[6];   // stride in x of the axis that lands at output axis i
};

__global__ void __launch_bounds__(256) permute_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n,
                                                      PermuteArgs a) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t rem = i, src = 0;
#pragma unroll
    for (int d = 5; d >= 0; --d) {
      if (d < a.ndim) {
        const int64_t c = rem % a.out_shape[d];
        rem /= a.out_shape[d];
        src += c * a.in_stride_of_out_dim[d];
      }
    }
    y[i] = x[src];
  }
}

// y[r, hk * group + j, :] = x[r, hk, :]  (rows r = B*T)
__global__ void __launch_bounds__(256) repeat_kv_kernel(const float4* __restrict__ x, float4* __restrict__ y, int64_t rows,
                                                        int Hk, int D4, int group) {
  const int64_t n = rows * Hk * group * D4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t d = i % D4, h = (i / D4) % (static_cast<int64_t>(Hk) * group), r = i / (D4 * static_cast<int64_t>(Hk) * group);
    y[i] = x[(r * Hk + h / group) * D4 + d];
  }
}
__global__ void __launch_bounds__(256) repeat_kv_sum_kernel(const float4* __restrict__ y, float4* __restrict__ x,
                                                            int64_t rows, int Hk, int D4, int group) {
  const int64_t n = rows * Hk * D4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t d = i % D4, hk = (i / D4) % Hk, r = i / (static_cast<int64_t>(D4) * Hk);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < group; ++j) {
      const float4 v = y[((r * Hk + hk) * group + j) * D4 + d];
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    x[i] = acc;
  }
}

// out[m, i, j] = (j > q_pos_start + i) ? fill : in[m, i, j]
__global__ void __launch_bounds__(256) causal_mask_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t mats,
                                                          int64_t Tq, int64_t Tk, int q_pos_start, float fill) {
  const int64_t n = mats * Tq * Tk;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    const int64_t j = idx % Tk, i = (idx / Tk) % Tq;
    out[idx] = (j > q_pos_start + i) ? fill : in[idx];
  }
}

__global__ void __launch_bounds__(256) mse_fwd_kernel(const float* __restrict__ p, const float* __restrict__ t, int64_t n,
                                                      float inv_n, float* __restrict__ loss) {
  __shared__ float red[8];
  float acc = 0.0f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float d = p[i] - t[i];
    acc += d * d;
  }
  acc = block_reduce<256>(acc, false, red);
  if (threadIdx.x == 0) atomicAdd(loss, acc * inv_n);
}
__global__ void __launch_bounds__(256) mse_bwd_kernel(const float* __restrict__ p, const float* __restrict__ t,
                                                      const float* __restrict__ dy, float* __restrict__ dp, int64_t n,
                                                      float two_over_n) {
  const float s = two_over_n * dy[0];
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) dp[i] = s * (p[i] - t[i]);
}

// src [B, T, H, D] -> cache [B, H, max_seq, D] at positions pos .. pos+T-1
__global__ void __launch_bounds__(256) kv_write_kernel(const float* __restrict__ src, float* __restrict__ cache, int64_t B,
                                                       int64_t T, int H, int D, int64_t max_seq, int64_t pos) {
  const int64_t n = B * T * H * D;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t d = i % D, h = (i / D) % H, t = (i / (static_cast<int64_t>(D) * H)) % T, b = i / (static_cast<int64_t>(D) * H * T);
    cache[((b * H + h) * max_seq + pos + t) * D + d] = src[i];
  }
}
// cache [B, Hk, max_seq, D] -> out [B, Hk*group, valid, D]
__global__ void __launch_bounds__(256) kv_read_kernel(const float* __restrict__ cache, float* __restrict__ out, int64_t B, int Hk,
                                                      int group, int64_t valid, int D, int64_t max_seq) {
  const int64_t Ho = static_cast<int64_t>(Hk) * group, n = B * Ho * valid * D;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t d = i % D, t = (i / D) % valid, ho = (i / (D * valid)) % Ho, b = i / (D * valid * Ho);
    out[i] = cache[((b * Hk + ho / group) * max_seq + t) * D + d];
  }
}

// out[0] = sums[1] > 0 ? sums[0] / sums[1] : 0  (the masked-mean loss from the two CE sums)
__global__ void ratio_kernel(const float* __restrict__ sums, float* __restrict__ out) {
  out[0] = sums[1] > 0.0f ? sums[0] / sums[1] : 0.0f;
}
// w[i] = mask[i] * dy[0] / sums[1]: the per-row factor of the masked-CE backward, built on the device
__global__ void __launch_bounds__(256) ce_row_weight_kernel(const float* __restrict__ mask, const float* __restrict__ dy,
                                                            const float* __restrict__ mask_sum, float uniform, int64_t n,
                                                            float* __restrict__ w) {
  const float s = dy[0] / (mask != nullptr ? mask_sum[0] : uniform);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    w[i] = (mask != nullptr ? mask[i] : 1.0f) * s;
}

inline int grid_for(int64_t n) {
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8, need = (n + 255) / 256;
  return static_cast<int>(need < cap ? (need > 0 ? need : 1) : cap);
}

}  // namespace
}  // namespace ctdk

using namespace ctdk;

extern "C" {

int ctdk_softmax_fwd(const float* x, float* y, int64_t rows, int64_t width, void* stream) {
  CTDK_REQUIRE(rows >= 0 && width > 0, "ctdk_softmax_fwd: bad shape");
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(x && y, "ctdk_softmax_fwd: null pointer");
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  softmax_fwd_kernel<<<static_cast<int>(rows < cap ? rows : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, rows, width);
  return check_launch("ctdk_softmax_fwd");
}

int ctdk_softmax_bwd(const float* y, const float* g, float* dx, int64_t rows, int64_t width, void* stream) {
  CTDK_REQUIRE(rows >= 0 && width > 0, "ctdk_softmax_bwd: bad shape");
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(y && g && dx, "ctdk_softmax_bwd: null pointer");
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  softmax_bwd_kernel<<<static_cast<int>(rows < cap ? rows : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(y, g, dx, rows, width);
  return check_launch("ctdk_softmax_bwd");
}

int ctdk_permute(const float* x, float* y, int ndim, const int64_t* shape, const int* perm, void* stream) {
  CTDK_REQUIRE(ndim >= 1 && ndim <= 6 && shape && perm, "ctdk_permute: 1 to 6 dimensions");
  int64_t in_stride[6], n = 1;
  bool seen[6] = {false, false, false, false, false, false};
  for (int d = ndim - 1; d >= 0; --d) {
    CTDK_REQUIRE(shape[d] >= 0, "ctdk_permute: negative extent");
    in_stride[d] = n;
    n *= shape[d];
  }
  PermuteArgs a{};
  a.ndim = ndim;
  for (int i = 0; i < ndim; ++i) {
    CTDK_REQUIRE(perm[i] >= 0 && perm[i] < ndim && !seen[perm[i]], "ctdk_permute: perm is not a permutation");
    seen[perm[i]] = true;
    a.out_shape[i] = shape[perm[i]];
    a.in_stride_of_out_dim[i] = in_stride[perm[i]];
  }
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(x && y, "ctdk_permute: null pointer");
  permute_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, n, a);
  return check_launch("ctdk_permute");
}

int ctdk_repeat_kv(const float* x, float* y, int64_t rows, int Hk, int D, int group, void* stream) {
  CTDK_REQUIRE(rows >= 0 && Hk > 0 && D > 0 && group > 0 && D % 4 == 0, "ctdk_repeat_kv: bad shape (D must be a multiple of 4)");
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(x && y && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0,
               "ctdk_repeat_kv: null or unaligned pointer");
  repeat_kv_kernel<<<grid_for(rows * Hk * group * (D / 4)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), rows, Hk, D / 4, group);
  return check_launch("ctdk_repeat_kv");
}

int ctdk_repeat_kv_sum(const float* y, float* x, int64_t rows, int Hk, int D, int group, void* stream) {
  CTDK_REQUIRE(rows >= 0 && Hk > 0 && D > 0 && group > 0 && D % 4 == 0, "ctdk_repeat_kv_sum: bad shape (D must be a multiple of 4)");
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(x && y && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0,
               "ctdk_repeat_kv_sum: null or unaligned pointer");
  repeat_kv_sum_kernel<<<grid_for(rows * Hk * (D / 4)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(y), reinterpret_cast<float4*>(x), rows, Hk, D / 4, group);
  return check_launch("ctdk_repeat_kv_sum");
}

int ctdk_causal_mask(const float* in, float* out, int64_t mats, int64_t Tq, int64_t Tk, int q_pos_start, float fill,
                     void* stream) {
  CTDK_REQUIRE(mats >= 0 && Tq >= 0 && Tk >= 0, "ctdk_causal_mask: bad shape");
  if (mats * Tq * Tk == 0) return CTDK_OK;
  CTDK_REQUIRE(in && out, "ctdk_causal_mask: null pointer");
  causal_mask_kernel<<<grid_for(mats * Tq * Tk), 256, 0, static_cast<cudaStream_t>(stream)>>>(in, out, mats, Tq, Tk, q_pos_start, fill);
  return check_launch("ctdk_causal_mask");
}

int ctdk_mse_fwd(const float* pred, const float* target, int64_t n, float* loss, void* stream) {
  CTDK_REQUIRE(n > 0 && pred && target && loss, "ctdk_mse_fwd: bad argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(loss, 0, sizeof(float), s) != cudaSuccess) return fail(CTDK_ELAUNCH, "ctdk_mse_fwd: memset failed");
  mse_fwd_kernel<<<grid_for(n), 256, 0, s>>>(pred, target, n, 1.0f / static_cast<float>(n), loss);
  return check_launch("ctdk_mse_fwd");
}

int ctdk_mse_bwd(const float* pred, const float* target, const float* dy, float* dpred, int64_t n, void* stream) {
  CTDK_REQUIRE(n > 0 && pred && target && dy && dpred, "ctdk_mse_bwd: bad argument");
  mse_bwd_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(pred, target, dy, dpred, n, 2.0f / static_cast<float>(n));
  return check_launch("ctdk_mse_bwd");
}

int ctdk_kv_write(const float* src, float* cache, int64_t B, int64_t T, int H, int D, int64_t max_seq, int64_t pos,
                  void* stream) {
  CTDK_REQUIRE(B >= 0 && T >= 0 && H > 0 && D > 0, "ctdk_kv_write: bad shape");
  CTDK_REQUIRE(pos >= 0 && pos + T <= max_seq, "write_kv: write range out of cache bounds");
  if (B * T == 0) return CTDK_OK;
  CTDK_REQUIRE(src && cache, "ctdk_kv_write: null pointer");
  kv_write_kernel<<<grid_for(B * T * H * D), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, cache, B, T, H, D, max_seq, pos);
  return check_launch("ctdk_kv_write");
}

int ctdk_kv_read_expanded(const float* cache, float* out, int64_t B, int Hk, int group, int64_t valid_len, int D,
                          int64_t max_seq, void* stream) {
  CTDK_REQUIRE(B >= 0 && Hk > 0 && D > 0, "ctdk_kv_read_expanded: bad shape");
  CTDK_REQUIRE(valid_len >= 0 && valid_len <= max_seq, "read_kv_expanded: valid_len out of range");
  CTDK_REQUIRE(group > 0, "read_kv_expanded: group must be > 0");
  if (B * valid_len == 0) return CTDK_OK;
  CTDK_REQUIRE(cache && out, "ctdk_kv_read_expanded: null pointer");
  kv_read_kernel<<<grid_for(B * Hk * group * valid_len * D), 256, 0, static_cast<cudaStream_t>(stream)>>>(cache, out, B, Hk, group,
                                                                                                            valid_len, D, max_seq);
  return check_launch("ctdk_kv_read_expanded");
}

int ctdk_loss_ratio(const float* sums, float* out, void* stream) {
  CTDK_REQUIRE(sums && out, "ctdk_loss_ratio: null pointer");
  ratio_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(sums, out);
  return check_launch("ctdk_loss_ratio");
}

int ctdk_ce_row_weight(const float* loss_mask, const float* dy, const float* mask_sum, int64_t n, float* row_weight,
                       void* stream) {
  CTDK_REQUIRE(n > 0 && dy && row_weight, "ctdk_ce_row_weight: bad argument");
  CTDK_REQUIRE(loss_mask == nullptr || mask_sum != nullptr, "ctdk_ce_row_weight: a mask needs its sum");
  ce_row_weight_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(loss_mask, dy, mask_sum, static_cast<float>(n), n,
                                                                                  row_weight);
  return check_launch("ctdk_ce_row_weight");
}

}  // extern "C"
