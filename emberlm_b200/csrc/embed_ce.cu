// Embedding gather / scatter-add and the masked cross-entropy block kernel.
//
// Embedding follows the reference (emberlm src/ops/embedding.cu:15-39): row gather in the
// forward, dW[id] += dy[row] with float atomics in the backward — but straight into the
// caller's gradient buffer (the tied-embedding gradient arena) instead of a zeroed [V,H]
// temporary. Cross-entropy follows src/ops/loss.cu:254-329: per row
//   lse = max + logf(sum(__expf(z - max)));  loss += mask*(lse - z[target])
//   dlogits = row_weight * (softmax(z) - onehot(target))
// computed with an online max/sum so the row is read once, then rewritten in place.
#include <cfloat>

#include "common.cuh"

namespace ctdk {
namespace {

__global__ void __launch_bounds__(256)
    embedding_fwd_kernel(const int64_t* __restrict__ ids, const float* __restrict__ W,
                         float* __restrict__ out, int64_t rows, int H, int64_t V, int vec_ok,
                         int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t row = warp0; row < rows; row += nwarps) {
    const int64_t id = ids[row];
    float* o = out + row * H;
    if (id < 0 || id >= V) {
      if (lane == 0) atomicAdd(&status[2], 1);
      for (int i = lane; i < H; i += 32) o[i] = 0.0f;
      continue;
    }
    const float* w = W + id * H;
    if (vec_ok) {
      const float4* w4 = reinterpret_cast<const float4*>(w);
      float4* o4 = reinterpret_cast<float4*>(o);
      for (int i = lane; i < (H >> 2); i += 32) o4[i] = w4[i];
    } else {
      for (int i = lane; i < H; i += 32) o[i] = w[i];
    }
  }
}

__global__ void __launch_bounds__(256)
    embedding_bwd_kernel(const int64_t* __restrict__ ids, const float* __restrict__ dy,
                         float* __restrict__ dW, int64_t rows, int H, int64_t V,
                         int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t row = warp0; row < rows; row += nwarps) {
    const int64_t id = ids[row];
    if (id < 0 || id >= V) {
      if (lane == 0) atomicAdd(&status[2], 1);
      continue;
    }
    const float* g = dy + row * H;
    float* w = dW + id * H;
    for (int i = lane; i < H; i += 32) atomicAdd(&w[i], g[i]);
  }
}

// The same for rows that fit in the registers of one CTA (V <= 512 * 4 * NV, 16-byte aligned rows,
// in-place dlogits): every logit of the row is requested at once (NV float4 per thread in flight,
// i.e. the whole row), max and sum are formed from registers, and the rewrite needs no second read.
// Rows whose weight is 0 and whose loss is masked are zero-filled without being read.
template <int NV>
__global__ void __launch_bounds__(512, 1)
    ce_masked_rows_kernel(float* __restrict__ logits, const int64_t* __restrict__ targets,
                          const float* __restrict__ loss_mask, const float* __restrict__ row_weight,
                          float* __restrict__ loss_sum, float* __restrict__ lse_out, int64_t n, int64_t V) {
  __shared__ float s_red[16];
  __shared__ float s_out;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int V4 = static_cast<int>(V >> 2);
  auto block_reduce = [&](float v, bool is_max) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float u = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, u) : v + u;
    }
    if (lane == 0) s_red[wid] = v;
    __syncthreads();
    if (wid == 0) {
      float t = lane < 16 ? s_red[lane] : (is_max ? -FLT_MAX : 0.0f);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {
        const float u = __shfl_xor_sync(0xffffffffu, t, o);
        t = is_max ? fmaxf(t, u) : t + u;
      }
      if (lane == 0) s_out = t;
    }
    __syncthreads();
    const float r = s_out;
    __syncthreads();   // s_red / s_out are reused
    return r;
  };
  for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
    float4* z4 = reinterpret_cast<float4*>(logits + row * V);
    const float mk = loss_mask != nullptr ? loss_mask[row] : 1.0f;
    const float rw = row_weight[row];
    const bool need_fwd = (mk != 0.0f) || (lse_out != nullptr) || (rw != 0.0f);
    if (!need_fwd) {
      for (int i = threadIdx.x; i < V4; i += blockDim.x) z4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      continue;
    }
    float4 x[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = threadIdx.x + j * 512;
      x[j] = i < V4 ? z4[i] : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
    }
    float m = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < NV; ++j) m = fmaxf(m, fmaxf(fmaxf(x[j].x, x[j].y), fmaxf(x[j].z, x[j].w)));
    m = block_reduce(m, true);
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      // exp(x - m) is kept: it is the numerator of the probability written below
      x[j].x = __expf(x[j].x - m);
      x[j].y = __expf(x[j].y - m);
      x[j].z = __expf(x[j].z - m);
      x[j].w = __expf(x[j].w - m);
      sum += (x[j].x + x[j].y) + (x[j].z + x[j].w);   // padding: exp(-FLT_MAX - m) = 0
    }
    sum = block_reduce(sum, false);
    const int64_t tgt = targets[row];
    if (threadIdx.x == 0) {
      const float lse = m + logf(sum);
      if (lse_out != nullptr) lse_out[row] = lse;
      if (mk != 0.0f) {
        // the target's logit is still in memory: the row is rewritten only after this read (bar.sync below)
        const float zt = (tgt >= 0 && tgt < V) ? logits[row * V + tgt] : 0.0f;
        atomicAdd(&loss_sum[0], mk * (lse - zt));
        atomicAdd(&loss_sum[1], mk);
      }
    }
    __syncthreads();
    if (rw == 0.0f) {
      for (int i = threadIdx.x; i < V4; i += blockDim.x) z4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      const float sc = rw / sum;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int i = threadIdx.x + j * 512;
        if (i < V4) {
          float4 o = make_float4(x[j].x * sc, x[j].y * sc, x[j].z * sc, x[j].w * sc);
          const int64_t c = static_cast<int64_t>(i) << 2;
          if (tgt >= c && tgt < c + 4) {
            const int k = static_cast<int>(tgt - c);
            if (k == 0) o.x -= rw;
            else if (k == 1) o.y -= rw;
            else if (k == 2) o.z -= rw;
            else o.w -= rw;
          }
          z4[i] = o;
        }
      }
    }
  }
}

// One CTA per row. Pass 1: online (max, sum) over the row. Pass 2 (optional): rewrite the
// row as row_weight*(p - onehot). Rows whose weight is 0 are zero-filled without being read.
__global__ void __launch_bounds__(512, 2)
    ce_masked_kernel(float* __restrict__ logits, const int64_t* __restrict__ targets,
                     const float* __restrict__ loss_mask, const float* __restrict__ row_weight,
                     float* __restrict__ loss_sum, float* __restrict__ lse_out, int64_t n,
                     int64_t V, int dlogits_inplace, int vec_ok) {
  __shared__ float s_m[32], s_s[32];
  __shared__ float s_lse;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
    float* z = logits + row * V;
    const float mk = loss_mask != nullptr ? loss_mask[row] : 1.0f;
    const float rw = row_weight != nullptr ? row_weight[row] : 0.0f;
    const bool need_fwd = (mk != 0.0f) || (lse_out != nullptr) || (rw != 0.0f);
    if (need_fwd) {
      float m = -FLT_MAX, s = 0.0f;
      auto upd = [&](float x) {
        if (x > m) {
          s = s * __expf(m - x) + 1.0f;
          m = x;
        } else {
          s += __expf(x - m);
        }
      };
      if (vec_ok) {
        const float4* z4 = reinterpret_cast<const float4*>(z);
        const int64_t V4 = V >> 2, bd = blockDim.x;
        int64_t i = threadIdx.x;
        // four loads in flight per thread before the (serial) running max / sum takes them in
        for (; i + 3 * bd < V4; i += 4 * bd) {
          float4 x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) x[u] = z4[i + u * bd];
          float mx = m;
#pragma unroll
          for (int u = 0; u < 4; ++u) mx = fmaxf(mx, fmaxf(fmaxf(x[u].x, x[u].y), fmaxf(x[u].z, x[u].w)));
          if (mx > m) {
            s *= __expf(m - mx);
            m = mx;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) s += __expf(x[u].x - m) + __expf(x[u].y - m) + __expf(x[u].z - m) + __expf(x[u].w - m);
        }
        for (; i < V4; i += bd) {
          const float4 x = z4[i];
          const float mx = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
          if (mx > m) {
            s *= __expf(m - mx);
            m = mx;
          }
          s += __expf(x.x - m) + __expf(x.y - m) + __expf(x.z - m) + __expf(x.w - m);
        }
        for (int64_t i = ((V >> 2) << 2) + threadIdx.x; i < V; i += blockDim.x) upd(z[i]);
      } else {
        for (int64_t i = threadIdx.x; i < V; i += blockDim.x) upd(z[i]);
      }
      // combine (m, s) pairs across the warp, then across warps
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        const float mn = fmaxf(m, m2);
        s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
        m = mn;
      }
      if (lane == 0) {
        s_m[wid] = m;
        s_s[wid] = s;
      }
      __syncthreads();
      if (wid == 0) {
        m = (lane < nw) ? s_m[lane] : -FLT_MAX;
        s = (lane < nw) ? s_s[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
          const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
          const float mn = fmaxf(m, m2);
          s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
          m = mn;
        }
        if (lane == 0) {
          const float lse = m + logf(s);
          s_lse = lse;
          if (lse_out != nullptr) lse_out[row] = lse;
          if (mk != 0.0f) {
            const int64_t tgt = targets[row];
            const float zt = (tgt >= 0 && tgt < V) ? z[tgt] : 0.0f;
            atomicAdd(&loss_sum[0], mk * (lse - zt));
            atomicAdd(&loss_sum[1], mk);
          }
        }
      }
      __syncthreads();
    }
    if (dlogits_inplace) {
      if (rw == 0.0f) {
        if (vec_ok) {
          float4* z4 = reinterpret_cast<float4*>(z);
          for (int64_t i = threadIdx.x; i < (V >> 2); i += blockDim.x)
            z4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int64_t i = ((V >> 2) << 2) + threadIdx.x; i < V; i += blockDim.x) z[i] = 0.0f;
        } else {
          for (int64_t i = threadIdx.x; i < V; i += blockDim.x) z[i] = 0.0f;
        }
      } else {
        const float lse = s_lse;
        const int64_t tgt = targets[row];
        if (vec_ok) {
          float4* z4 = reinterpret_cast<float4*>(z);
#pragma unroll 4
          for (int64_t i = threadIdx.x; i < (V >> 2); i += blockDim.x) {
            float4 x = z4[i];
            x.x = __expf(x.x - lse);
            x.y = __expf(x.y - lse);
            x.z = __expf(x.z - lse);
            x.w = __expf(x.w - lse);
            const int64_t c = i << 2;
            if (tgt >= c && tgt < c + 4) {
              const int k = static_cast<int>(tgt - c);
              if (k == 0) x.x -= 1.0f;
              else if (k == 1) x.y -= 1.0f;
              else if (k == 2) x.z -= 1.0f;
              else x.w -= 1.0f;
            }
            x.x *= rw;
            x.y *= rw;
            x.z *= rw;
            x.w *= rw;
            z4[i] = x;
          }
          for (int64_t i = ((V >> 2) << 2) + threadIdx.x; i < V; i += blockDim.x) {
            float pz = __expf(z[i] - lse);
            if (i == tgt) pz -= 1.0f;
            z[i] = rw * pz;
          }
        } else {
          for (int64_t i = threadIdx.x; i < V; i += blockDim.x) {
            float pz = __expf(z[i] - lse);
            if (i == tgt) pz -= 1.0f;
            z[i] = rw * pz;
          }
        }
      }
    }
    __syncthreads();  // s_lse / s_m / s_s are reused by the next row
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// dst[i] = src[idx[i]] (gather) or dst[idx[i]] = src[i] (scatter), rows of H floats, one warp per row.
template <bool SCATTER>
__global__ void __launch_bounds__(256)
    move_rows_kernel(const float* __restrict__ src, const int32_t* __restrict__ idx, float* __restrict__ dst,
                     int64_t n, int H4) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t i = warp0; i < n; i += nwarps) {
    const int64_t r = idx[i];
    const float4* s4 = reinterpret_cast<const float4*>(src) + (SCATTER ? i : r) * H4;
    float4* d4 = reinterpret_cast<float4*>(dst) + (SCATTER ? r : i) * H4;
    for (int c = lane; c < H4; c += 32) d4[c] = s4[c];
  }
}

__global__ void __launch_bounds__(256)
    gather_ce_inputs_kernel(const int64_t* __restrict__ targets, const float* __restrict__ mask,
                            const float* __restrict__ weight, const int32_t* __restrict__ idx,
                            int64_t* __restrict__ t_out, float* __restrict__ m_out, float* __restrict__ w_out,
                            int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t r = idx[i];
  t_out[i] = targets[r];
  m_out[i] = mask != nullptr ? mask[r] : 1.0f;
  if (w_out != nullptr) w_out[i] = weight != nullptr ? weight[r] : 0.0f;
}

}  // namespace
}  // namespace ctdk

using namespace ctdk;

extern "C" {

int ctdk_embedding_fwd(const int64_t* ids, const float* W, float* out, int64_t rows, int H,
                       int64_t V, void* stream) {
  CTDK_REQUIRE(rows >= 0 && H > 0 && V > 0, "ctdk_embedding_fwd: bad shape");
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(ids && W && out, "ctdk_embedding_fwd: null pointer");
  int* st = device_status_word();
  CTDK_REQUIRE(st != nullptr, "ctdk_embedding_fwd: no status word");
  const int vec = (H % 4 == 0) && aligned16(W) && aligned16(out);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int64_t need = (rows + 7) / 8;
  void* prof = prof_begin(CTDK_PROF_EMBED, 8.0 * static_cast<double>(rows) * H, static_cast<cudaStream_t>(stream));
  embedding_fwd_kernel<<<static_cast<int>(need < cap ? need : cap), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(ids, W, out, rows, H, V, vec, st);
  prof_end(prof, static_cast<cudaStream_t>(stream));
  return check_launch("ctdk_embedding_fwd");
}

int ctdk_embedding_bwd(const int64_t* ids, const float* dy, float* dW, int64_t rows, int H,
                       int64_t V, void* stream) {
  CTDK_REQUIRE(rows >= 0 && H > 0 && V > 0, "ctdk_embedding_bwd: bad shape");
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(ids && dy && dW, "ctdk_embedding_bwd: null pointer");
  int* st = device_status_word();
  CTDK_REQUIRE(st != nullptr, "ctdk_embedding_bwd: no status word");
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int64_t need = (rows + 7) / 8;
  void* prof = prof_begin(CTDK_PROF_EMBED, 12.0 * static_cast<double>(rows) * H, static_cast<cudaStream_t>(stream));
  embedding_bwd_kernel<<<static_cast<int>(need < cap ? need : cap), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(ids, dy, dW, rows, H, V, st);
  prof_end(prof, static_cast<cudaStream_t>(stream));
  return check_launch("ctdk_embedding_bwd");
}

int ctdk_gather_rows(const float* src, const int32_t* idx, float* dst, int64_t n, int H, void* stream) {
  CTDK_REQUIRE(n >= 0 && H > 0 && H % 4 == 0, "ctdk_gather_rows: H must be a positive multiple of 4");
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(src && idx && dst && aligned16(src) && aligned16(dst), "ctdk_gather_rows: bad pointer");
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8, need = (n + 7) / 8;
  move_rows_kernel<false><<<static_cast<int>(need < cap ? need : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, idx, dst, n, H / 4);
  return check_launch("ctdk_gather_rows");
}

int ctdk_scatter_rows(const float* src, const int32_t* idx, float* dst, int64_t n, int H, void* stream) {
  CTDK_REQUIRE(n >= 0 && H > 0 && H % 4 == 0, "ctdk_scatter_rows: H must be a positive multiple of 4");
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(src && idx && dst && aligned16(src) && aligned16(dst), "ctdk_scatter_rows: bad pointer");
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8, need = (n + 7) / 8;
  move_rows_kernel<true><<<static_cast<int>(need < cap ? need : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, idx, dst, n, H / 4);
  return check_launch("ctdk_scatter_rows");
}

int ctdk_gather_ce_inputs(const int64_t* targets, const float* mask, const float* weight, const int32_t* idx,
                          int64_t* t_out, float* m_out, float* w_out, int64_t n, void* stream) {
  CTDK_REQUIRE(n >= 0, "ctdk_gather_ce_inputs: negative size");
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(targets && idx && t_out && m_out, "ctdk_gather_ce_inputs: null pointer");
  gather_ce_inputs_kernel<<<ceil_div(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(targets, mask, weight, idx,
                                                                                         t_out, m_out, w_out, n);
  return check_launch("ctdk_gather_ce_inputs");
}

int ctdk_ce_masked(float* logits, const int64_t* targets, const float* loss_mask,
                   const float* row_weight, float* loss_sum, float* lse_out, int64_t n,
                   int64_t V, int dlogits_inplace, void* stream) {
  CTDK_REQUIRE(n >= 0 && V > 0, "ctdk_ce_masked: bad shape");
  if (n == 0) return CTDK_OK;
  CTDK_REQUIRE(logits && targets && loss_sum, "ctdk_ce_masked: null pointer");
  CTDK_REQUIRE(!dlogits_inplace || row_weight, "ctdk_ce_masked: row_weight required");
  const int vec = (V % 4 == 0) && aligned16(logits);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 4;
  // one read of every logit, one rewrite when the block becomes dlogits (all rows counted: the
  // engine compacts the supervised rows before the head, so every row of a block is live)
  void* prof = prof_begin(CTDK_PROF_CE, (dlogits_inplace ? 8.0 : 4.0) * static_cast<double>(n) * V, static_cast<cudaStream_t>(stream));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t cap1 = static_cast<int64_t>(sm_count());
  const unsigned g1 = static_cast<unsigned>(n < cap1 ? n : cap1);
  if (vec && dlogits_inplace && V <= 512 * 4 * 8)
    ce_masked_rows_kernel<8><<<g1, 512, 0, st>>>(logits, targets, loss_mask, row_weight, loss_sum, lse_out, n, V);
  else if (vec && dlogits_inplace && V <= 512 * 4 * 16)
    ce_masked_rows_kernel<16><<<g1, 512, 0, st>>>(logits, targets, loss_mask, row_weight, loss_sum, lse_out, n, V);
  else if (vec && dlogits_inplace && V <= 512 * 4 * 24)
    ce_masked_rows_kernel<24><<<g1, 512, 0, st>>>(logits, targets, loss_mask, row_weight, loss_sum, lse_out, n, V);
  else
    ce_masked_kernel<<<static_cast<int>(n < cap ? n : cap), 512, 0, st>>>(
        logits, targets, loss_mask, row_weight, loss_sum, lse_out, n, V, dlogits_inplace, vec);
  prof_end(prof, static_cast<cudaStream_t>(stream));
  return check_launch("ctdk_ce_masked");
}

}  // extern "C"
