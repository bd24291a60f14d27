// Causal grouped-query attention, forward and backward, on the packed projection buffer.
//
// What the reference does with bmm -> 1/sqrt(D) -> causal mask -> softmax -> bmm plus four
// permutes and repeat_kv copies (emberlm include/ctd/nn/attention.h:123-141,
// src/ops/softmax.cu:18-54, src/ops/mask.cu:28-39) is computed here tile by tile with an
// online softmax, so the [B*H,T,T] score tensors never exist:
//   forward   : one CTA per (64-query tile, head, batch); S = Q K^T and O += P V on the
//               TF32 tensor-core path (mma.sync m16n8k8), running max/sum per row.
//   backward  : delta = rowsum(dO*O); a dQ kernel shaped like the forward; a dK/dV kernel
//               with one CTA per (64-key tile, kv head, batch) that loops over the query
//               heads of the group, so dK/dV need no atomics and no repeat_kv_sum pass.
// q/k/v are read in place from qkv[B*T, (H+2Hk)*D] (query head h uses kv head h/(H/Hk)).
#include <cfloat>

#include "common.cuh"

namespace ctdk {

// tcgen05 kernels (attention_tc.cu); return 1 when a shape is not eligible.
int attn_fwd_tcgen05(const float* qkv, float* out, float* lse, int64_t B, int64_t T, int H, int Hk,
                     int D, cudaStream_t stream);
int attn_bwd_dq_tcgen05(const float* qkv, const float* dout, const float* lse, const float* delta,
                        float* dqkv, int64_t B, int64_t T, int H, int Hk, int D, cudaStream_t stream);
int attn_bwd_dkv_tcgen05(const float* qkv, const float* dout, const float* lse, const float* delta,
                         float* dqkv, int64_t B, int64_t T, int H, int Hk, int D, cudaStream_t stream);
bool attn_use_legacy();

namespace {

constexpr int BQ = 64;   // query rows per CTA (4 warps x 16)
constexpr int BKV = 64;  // keys per tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t f2tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One m16n8k8 product in TF32, or (X3) the three-product split a = a_hi + a_lo, b = b_hi + b_lo,
// a*b ~ a_lo*b_hi + a_hi*b_lo + a_hi*b_hi, which recovers near-fp32 accuracy.
__device__ __forceinline__ void split_tf32(uint32_t x, uint32_t& hi, uint32_t& lo) {
  const float f = __uint_as_float(x);
  hi = f2tf32(f);
  lo = f2tf32(f - __uint_as_float(hi));
}
template <bool X3>
__device__ __forceinline__ void mma_x(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                      uint32_t b0, uint32_t b1) {
  if (!X3) {
    mma_tf32(c, a0, a1, a2, a3, b0, b1);
  } else {
    uint32_t ah[4], al[4], bh[2], bl[2];
    split_tf32(a0, ah[0], al[0]);
    split_tf32(a1, ah[1], al[1]);
    split_tf32(a2, ah[2], al[2]);
    split_tf32(a3, ah[3], al[3]);
    split_tf32(b0, bh[0], bl[0]);
    split_tf32(b1, bh[1], bl[1]);
    mma_tf32(c, al[0], al[1], al[2], al[3], bh[0], bh[1]);
    mma_tf32(c, ah[0], ah[1], ah[2], ah[3], bl[0], bl[1]);
    mma_tf32(c, ah[0], ah[1], ah[2], ah[3], bh[0], bh[1]);
  }
}

// Copies R rows of D floats (row r from g + (row0+r)*stride) into smem with pitch D+4;
// rows at or beyond `T` are zero-filled.
template <int D, int R, int NT>
__device__ __forceinline__ void load_tile(float* s, const float* __restrict__ g, int64_t stride,
                                          int row0, int T) {
  constexpr int P = D + 4, C4 = D / 4;
  for (int i = threadIdx.x; i < R * C4; i += NT) {
    const int r = i / C4, c = i - r * C4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + r < T) v = *reinterpret_cast<const float4*>(g + (row0 + r) * stride + c * 4);
    *reinterpret_cast<float4*>(s + r * P + c * 4) = v;
  }
}

// acc[nt] (16 x 8 each, NT8 tiles) += A[16 rows starting at a_row0 of sA][D] * B^T where
// B rows are the n index: B[n][k] = sB[(nt*8+n)*P + k]. Both tiles have k contiguous.
template <int D, int NT8, bool X3>
__device__ __forceinline__ void mma_ab_t(float (&acc)[NT8][4], const float* sA, int a_row0,
                                         const float* sB, int lane) {
  constexpr int P = D + 4;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int kk = 0; kk < D / 8; ++kk) {
    const uint32_t a0 = __float_as_uint(sA[(a_row0 + g) * P + kk * 8 + t]);
    const uint32_t a1 = __float_as_uint(sA[(a_row0 + g + 8) * P + kk * 8 + t]);
    const uint32_t a2 = __float_as_uint(sA[(a_row0 + g) * P + kk * 8 + t + 4]);
    const uint32_t a3 = __float_as_uint(sA[(a_row0 + g + 8) * P + kk * 8 + t + 4]);
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) {
      const uint32_t b0 = __float_as_uint(sB[(nt * 8 + g) * P + kk * 8 + t]);
      const uint32_t b1 = __float_as_uint(sB[(nt * 8 + g) * P + kk * 8 + t + 4]);
      mma_x<X3>(acc[nt], a0, a1, a2, a3, b0, b1);
    }
  }
}

// acc[nt] (16 x 8, D/8 tiles over the feature dim) += P[16 x KT*8] * B where P is held in
// accumulator layout p[kt][4] (row g: cols 2t,2t+1 -> p[kt][0..1]; row g+8 -> p[kt][2..3])
// and B[k][n] = sB[(kt*8+k)*P + n]. The k index inside each 8-wide slice is permuted
// (slot t <-> column 2t, slot t+4 <-> column 2t+1) on both operands, which leaves the
// contraction unchanged and needs no register shuffles.
template <int D, int KT, bool X3>
__device__ __forceinline__ void mma_p_b(float (&acc)[D / 8][4], const float (&p)[KT][4],
                                        const float* sB, int lane) {
  constexpr int P = D + 4;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int kt = 0; kt < KT; ++kt) {
    const uint32_t a0 = X3 ? __float_as_uint(p[kt][0]) : f2tf32(p[kt][0]);
    const uint32_t a1 = X3 ? __float_as_uint(p[kt][2]) : f2tf32(p[kt][2]);
    const uint32_t a2 = X3 ? __float_as_uint(p[kt][1]) : f2tf32(p[kt][1]);
    const uint32_t a3 = X3 ? __float_as_uint(p[kt][3]) : f2tf32(p[kt][3]);
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      const uint32_t b0 = __float_as_uint(sB[(kt * 8 + 2 * t) * P + nt * 8 + g]);
      const uint32_t b1 = __float_as_uint(sB[(kt * 8 + 2 * t + 1) * P + nt * 8 + g]);
      mma_x<X3>(acc[nt], a0, a1, a2, a3, b0, b1);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------
template <int D, bool X3>
__global__ void __launch_bounds__(128)
    attn_fwd_kernel(const float* __restrict__ qkv, float* __restrict__ out,
                    float* __restrict__ lse, int T, int H, int Hk, float scale_log2) {
  constexpr int P = D + 4;
  extern __shared__ float smem[];
  float* Qs = smem;
  float* Ks = Qs + BQ * P;
  float* Vs = Ks + BKV * P;
  const int qi = gridDim.x - 1 - blockIdx.x;  // heaviest tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (H / Hk);
  const int64_t RS = static_cast<int64_t>(H + 2 * Hk) * D;
  const float* qbase = qkv + static_cast<int64_t>(b) * T * RS + static_cast<int64_t>(h) * D;
  const float* kbase =
      qkv + static_cast<int64_t>(b) * T * RS + static_cast<int64_t>(H + hk) * D;
  const float* vbase =
      qkv + static_cast<int64_t>(b) * T * RS + static_cast<int64_t>(H + Hk + hk) * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int q0 = qi * BQ;

  load_tile<D, BQ, 128>(Qs, qbase, RS, q0, T);

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.0f, 0.0f};
  const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;

  for (int j = 0; j <= qi; ++j) {
    __syncthreads();  // previous tile fully consumed (and Qs visible on the first pass)
    load_tile<D, BKV, 128>(Ks, kbase, RS, j * BKV, T);
    load_tile<D, BKV, 128>(Vs, vbase, RS, j * BKV, T);
    __syncthreads();

    float s[BKV / 8][4];
#pragma unroll
    for (int i = 0; i < BKV / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
    mma_ab_t<D, BKV / 8, X3>(s, Qs, warp * 16, Ks, lane);

    float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
    for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = j * BKV + nt * 8 + 2 * t + (e & 1);
        const int row = (e < 2) ? row_a : row_b;
        float v = s[nt][e] * scale_log2;
        if (key > row) v = -FLT_MAX;
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], rs[2] = {0.0f, 0.0f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float mn = fmaxf(m_run[r], mx[r]);
      corr[r] = exp2f(m_run[r] - mn);
      m_run[r] = mn;
    }
#pragma unroll
    for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // masked entries hold -FLT_MAX: exp2f underflows to exactly 0 (the row max is
        // finite because key 0 is never masked)
        const float pv = exp2f(s[nt][e] - m_run[e >> 1]);
        s[nt][e] = pv;
        rs[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
      l_run[r] = l_run[r] * corr[r] + rs[r];
    }
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      o[nt][0] *= corr[0];
      o[nt][1] *= corr[0];
      o[nt][2] *= corr[1];
      o[nt][3] *= corr[1];
    }
    mma_p_b<D, BKV / 8, X3>(o, s, Vs, lane);
  }

  const float inv_a = 1.0f / l_run[0], inv_b = 1.0f / l_run[1];
  const int64_t OS = static_cast<int64_t>(H) * D;
  if (row_a < T) {
    float* op = out + (static_cast<int64_t>(b) * T + row_a) * OS + static_cast<int64_t>(h) * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt)
      *reinterpret_cast<float2*>(op + nt * 8 + 2 * t) =
          make_float2(o[nt][0] * inv_a, o[nt][1] * inv_a);
    if (t == 0)
      lse[(static_cast<int64_t>(b) * H + h) * T + row_a] = (m_run[0] + log2f(l_run[0])) * kLn2;
  }
  if (row_b < T) {
    float* op = out + (static_cast<int64_t>(b) * T + row_b) * OS + static_cast<int64_t>(h) * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt)
      *reinterpret_cast<float2*>(op + nt * 8 + 2 * t) =
          make_float2(o[nt][2] * inv_b, o[nt][3] * inv_b);
    if (t == 0)
      lse[(static_cast<int64_t>(b) * H + h) * T + row_b] = (m_run[1] + log2f(l_run[1])) * kLn2;
  }
}

// delta[b][h][t] = sum_d dO*O  (the rowsum of softmax backward, emberlm
// src/ops/softmax.cu:56-93). D/4 lanes per (row, head), one float4 of each operand per lane and
// four rows in flight per lane group, so the kernel runs at memory speed.
template <int D>
__global__ void __launch_bounds__(256)
    attn_delta_kernel(const float* __restrict__ out, const float* __restrict__ dout,
                      float* __restrict__ delta, int64_t B, int T, int H) {
  pdl_launch();
  pdl_wait();
  constexpr int LP = D / 4;          // lanes per item: 16 (D = 64) or 32 (D = 128)
  constexpr int UN = 4;              // items in flight per lane group
  const int sub = threadIdx.x % LP;
  const int64_t group0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / LP;
  const int64_t ngroups = (static_cast<int64_t>(gridDim.x) * blockDim.x) / LP;
  const int64_t items = B * T * H;
  for (int64_t base = group0 * UN; base < items; base += ngroups * UN) {
    float4 a[UN], c[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int64_t it = base + u;
      if (it < items) {
        a[u] = __ldcs(reinterpret_cast<const float4*>(out + it * D) + sub);
        c[u] = __ldg(reinterpret_cast<const float4*>(dout + it * D) + sub);   // read again by the dQ / dK,dV kernels
      } else {
        a[u] = c[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      float acc = a[u].x * c[u].x + a[u].y * c[u].y + a[u].z * c[u].z + a[u].w * c[u].w;
#pragma unroll
      for (int o = LP / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      const int64_t it = base + u;
      if (sub == 0 && it < items) {
        const int64_t bt = it / H;
        const int h = static_cast<int>(it - bt * H);
        const int64_t bb = bt / T;
        const int tt = static_cast<int>(bt - bb * T);
        delta[(bb * H + h) * T + tt] = acc;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Backward, dQ:  dS = P*(dP - delta)*scale, dQ = dS K
// ---------------------------------------------------------------------------------------
template <int D, bool X3>
__global__ void __launch_bounds__(128)
    attn_bwd_dq_kernel(const float* __restrict__ qkv, const float* __restrict__ dout,
                       const float* __restrict__ lse, const float* __restrict__ delta,
                       float* __restrict__ dqkv, int T, int H, int Hk, float scale) {
  constexpr int P = D + 4;
  extern __shared__ float smem[];
  float* Qs = smem;
  float* dOs = Qs + BQ * P;
  float* Ks = dOs + BQ * P;
  float* Vs = Ks + BKV * P;
  const int qi = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (H / Hk);
  const int64_t RS = static_cast<int64_t>(H + 2 * Hk) * D;
  const int64_t OS = static_cast<int64_t>(H) * D;
  const float* qbase = qkv + static_cast<int64_t>(b) * T * RS + static_cast<int64_t>(h) * D;
  const float* kbase =
      qkv + static_cast<int64_t>(b) * T * RS + static_cast<int64_t>(H + hk) * D;
  const float* vbase =
      qkv + static_cast<int64_t>(b) * T * RS + static_cast<int64_t>(H + Hk + hk) * D;
  const float* dobase = dout + static_cast<int64_t>(b) * T * OS + static_cast<int64_t>(h) * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int q0 = qi * BQ;
  const float scale_log2 = scale * kLog2e;

  load_tile<D, BQ, 128>(Qs, qbase, RS, q0, T);
  load_tile<D, BQ, 128>(dOs, dobase, OS, q0, T);

  const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
  const int64_t lbase = (static_cast<int64_t>(b) * H + h) * T;
  // rows past T: lse = +huge makes every probability 0
  const float lse_a = row_a < T ? lse[lbase + row_a] * kLog2e : FLT_MAX;
  const float lse_b = row_b < T ? lse[lbase + row_b] * kLog2e : FLT_MAX;
  const float del_a = row_a < T ? delta[lbase + row_a] : 0.0f;
  const float del_b = row_b < T ? delta[lbase + row_b] : 0.0f;

  float dq[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.0f;

  for (int j = 0; j <= qi; ++j) {
    __syncthreads();
    load_tile<D, BKV, 128>(Ks, kbase, RS, j * BKV, T);
    load_tile<D, BKV, 128>(Vs, vbase, RS, j * BKV, T);
    __syncthreads();

    float s[BKV / 8][4], dp[BKV / 8][4];
#pragma unroll
    for (int i = 0; i < BKV / 8; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.0f;
    }
    mma_ab_t<D, BKV / 8, X3>(s, Qs, warp * 16, Ks, lane);
    mma_ab_t<D, BKV / 8, X3>(dp, dOs, warp * 16, Vs, lane);
#pragma unroll
    for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = j * BKV + nt * 8 + 2 * t + (e & 1);
        const int row = (e < 2) ? row_a : row_b;
        const float l2 = (e < 2) ? lse_a : lse_b;
        const float dl = (e < 2) ? del_a : del_b;
        const float pv = (key > row) ? 0.0f : exp2f(s[nt][e] * scale_log2 - l2);
        s[nt][e] = pv * (dp[nt][e] - dl) * scale;
      }
    }
    mma_p_b<D, BKV / 8, X3>(dq, s, Ks, lane);
  }

  if (row_a < T) {
    float* p = dqkv + (static_cast<int64_t>(b) * T + row_a) * RS + static_cast<int64_t>(h) * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt)
      *reinterpret_cast<float2*>(p + nt * 8 + 2 * t) = make_float2(dq[nt][0], dq[nt][1]);
  }
  if (row_b < T) {
    float* p = dqkv + (static_cast<int64_t>(b) * T + row_b) * RS + static_cast<int64_t>(h) * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt)
      *reinterpret_cast<float2*>(p + nt * 8 + 2 * t) = make_float2(dq[nt][2], dq[nt][3]);
  }
}

// ---------------------------------------------------------------------------------------
// Backward, dK/dV: keys are the M dimension. For a tile of 64 keys, loop over the query
// heads of the group and over query tiles at or after the key tile:
//   S^T = K Q^T, P^T = exp(S^T*scale - lse[q]), dP^T = V dO^T,
//   dS^T = P^T*(dP^T - delta[q])*scale, dV += P^T dO, dK += dS^T Q.
// QT = queries per inner tile (64 for D=64, 32 for D=128 to bound registers).
// ---------------------------------------------------------------------------------------
template <int D, int QT, bool X3>
__global__ void __launch_bounds__(128)
    attn_bwd_dkv_kernel(const float* __restrict__ qkv, const float* __restrict__ dout,
                        const float* __restrict__ lse, const float* __restrict__ delta,
                        float* __restrict__ dqkv, int T, int H, int Hk, float scale) {
  constexpr int P = D + 4;
  extern __shared__ float smem[];
  float* Ks = smem;
  float* Vs = Ks + BKV * P;
  float* Qs = Vs + BKV * P;
  float* dOs = Qs + QT * P;
  float* s_lse = dOs + QT * P;  // [QT]
  float* s_del = s_lse + QT;    // [QT]
  const int kj = blockIdx.x;    // key tile; low tiles have the most query tiles
  const int hk = blockIdx.y, b = blockIdx.z;
  const int G = H / Hk;
  const int64_t RS = static_cast<int64_t>(H + 2 * Hk) * D;
  const int64_t OS = static_cast<int64_t>(H) * D;
  const float* kbase =
      qkv + static_cast<int64_t>(b) * T * RS + static_cast<int64_t>(H + hk) * D;
  const float* vbase =
      qkv + static_cast<int64_t>(b) * T * RS + static_cast<int64_t>(H + Hk + hk) * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int k0 = kj * BKV;
  const float scale_log2 = scale * kLog2e;

  load_tile<D, BKV, 128>(Ks, kbase, RS, k0, T);
  load_tile<D, BKV, 128>(Vs, vbase, RS, k0, T);

  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.0f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.0f;
  }
  const int key_a = k0 + warp * 16 + g, key_b = key_a + 8;
  const int n_qt = (T + QT - 1) / QT;
  const int first_qt = k0 / QT;

  for (int hh = 0; hh < G; ++hh) {
    const int h = hk * G + hh;
    const float* qbase = qkv + static_cast<int64_t>(b) * T * RS + static_cast<int64_t>(h) * D;
    const float* dobase = dout + static_cast<int64_t>(b) * T * OS + static_cast<int64_t>(h) * D;
    const int64_t lbase = (static_cast<int64_t>(b) * H + h) * T;
    for (int qt = first_qt; qt < n_qt; ++qt) {
      const int q0 = qt * QT;
      __syncthreads();  // previous Q/dO tile consumed (and K/V visible on the first pass)
      load_tile<D, QT, 128>(Qs, qbase, RS, q0, T);
      load_tile<D, QT, 128>(dOs, dobase, OS, q0, T);
      if (threadIdx.x < QT) {
        const int q = q0 + threadIdx.x;
        s_lse[threadIdx.x] = q < T ? lse[lbase + q] * kLog2e : FLT_MAX;
        s_del[threadIdx.x] = q < T ? delta[lbase + q] : 0.0f;
      }
      __syncthreads();

      float st[QT / 8][4], dpt[QT / 8][4];
#pragma unroll
      for (int i = 0; i < QT / 8; ++i) {
        st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.0f;
        dpt[i][0] = dpt[i][1] = dpt[i][2] = dpt[i][3] = 0.0f;
      }
      mma_ab_t<D, QT / 8, X3>(st, Ks, warp * 16, Qs, lane);
      mma_ab_t<D, QT / 8, X3>(dpt, Vs, warp * 16, dOs, lane);
      float pt[QT / 8][4];
#pragma unroll
      for (int nt = 0; nt < QT / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int ql = nt * 8 + 2 * t + (e & 1);
          const int q = q0 + ql;
          const int key = (e < 2) ? key_a : key_b;
          const float pv = (key > q) ? 0.0f : exp2f(st[nt][e] * scale_log2 - s_lse[ql]);
          pt[nt][e] = pv;
          st[nt][e] = pv * (dpt[nt][e] - s_del[ql]) * scale;
        }
      }
      mma_p_b<D, QT / 8, X3>(dv, pt, dOs, lane);
      mma_p_b<D, QT / 8, X3>(dk, st, Qs, lane);
    }
  }

  if (key_a < T) {
    float* pk = dqkv + (static_cast<int64_t>(b) * T + key_a) * RS +
                static_cast<int64_t>(H + hk) * D;
    float* pv = dqkv + (static_cast<int64_t>(b) * T + key_a) * RS +
                static_cast<int64_t>(H + Hk + hk) * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      *reinterpret_cast<float2*>(pk + nt * 8 + 2 * t) = make_float2(dk[nt][0], dk[nt][1]);
      *reinterpret_cast<float2*>(pv + nt * 8 + 2 * t) = make_float2(dv[nt][0], dv[nt][1]);
    }
  }
  if (key_b < T) {
    float* pk = dqkv + (static_cast<int64_t>(b) * T + key_b) * RS +
                static_cast<int64_t>(H + hk) * D;
    float* pv = dqkv + (static_cast<int64_t>(b) * T + key_b) * RS +
                static_cast<int64_t>(H + Hk + hk) * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      *reinterpret_cast<float2*>(pk + nt * 8 + 2 * t) = make_float2(dk[nt][2], dk[nt][3]);
      *reinterpret_cast<float2*>(pv + nt * 8 + 2 * t) = make_float2(dv[nt][2], dv[nt][3]);
    }
  }
}

template <typename K>
int set_smem(K kern, int bytes, const char* what) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess)
    return fail(CTDK_ELAUNCH, "%s: cannot opt in to %d bytes of shared memory: %s", what, bytes,
                cudaGetErrorString(e));
  return CTDK_OK;
}

int check_attn_args(const char* name, int64_t B, int64_t T, int H, int Hk, int D) {
  CTDK_REQUIRE(B >= 0 && T >= 0, "%s: negative size", name);
  CTDK_REQUIRE(H > 0 && Hk > 0 && H % Hk == 0, "%s: H must be a positive multiple of Hk", name);
  CTDK_REQUIRE(D == 64 || D == 128, "%s: head_dim must be 64 or 128", name);
  CTDK_REQUIRE(T < (1 << 24) && B <= 65535 && H <= 65535, "%s: shape too large", name);
  return CTDK_OK;
}

template <int D, bool X3>
int run_fwd_legacy(const float* qkv, float* out, float* lse, int64_t B, int64_t T, int H, int Hk, cudaStream_t s) {
  const float scale_log2 = (1.0f / sqrtf(static_cast<float>(D))) * kLog2e;
  dim3 grid(static_cast<unsigned>((T + BQ - 1) / BQ), static_cast<unsigned>(H), static_cast<unsigned>(B));
  const int smem = (BQ + 2 * BKV) * (D + 4) * static_cast<int>(sizeof(float));
  int rc = set_smem(attn_fwd_kernel<D, X3>, smem, "ctdk_attn_fwd");
  if (rc != CTDK_OK) return rc;
  attn_fwd_kernel<D, X3><<<grid, 128, smem, s>>>(qkv, out, lse, static_cast<int>(T), H, Hk, scale_log2);
  return check_launch("ctdk_attn_fwd");
}

template <int D, int QT, bool X3>
int run_bwd_legacy(const float* qkv, const float* dout, const float* lse, const float* delta, float* dqkv,
                   int64_t B, int64_t T, int H, int Hk, bool do_dq, bool do_dkv, cudaStream_t s) {
  const float scale = 1.0f / sqrtf(static_cast<float>(D));
  const int Ti = static_cast<int>(T);
  dim3 gq(static_cast<unsigned>((T + BQ - 1) / BQ), static_cast<unsigned>(H), static_cast<unsigned>(B));
  dim3 gk(static_cast<unsigned>((T + BKV - 1) / BKV), static_cast<unsigned>(Hk), static_cast<unsigned>(B));
  const int smem_q = (2 * BQ + 2 * BKV) * (D + 4) * static_cast<int>(sizeof(float));
  const int smem_k = ((2 * BKV + 2 * QT) * (D + 4) + 2 * QT) * static_cast<int>(sizeof(float));
  int rc = CTDK_OK;
  if (do_dq) {
    rc = set_smem(attn_bwd_dq_kernel<D, X3>, smem_q, "ctdk_attn_bwd");
    if (rc != CTDK_OK) return rc;
    attn_bwd_dq_kernel<D, X3><<<gq, 128, smem_q, s>>>(qkv, dout, lse, delta, dqkv, Ti, H, Hk, scale);
    rc = check_launch("ctdk_attn_bwd(dq)");
    if (rc != CTDK_OK) return rc;
  }
  if (do_dkv) {
    rc = set_smem(attn_bwd_dkv_kernel<D, QT, X3>, smem_k, "ctdk_attn_bwd");
    if (rc != CTDK_OK) return rc;
    attn_bwd_dkv_kernel<D, QT, X3><<<gk, 128, smem_k, s>>>(qkv, dout, lse, delta, dqkv, Ti, H, Hk, scale);
    rc = check_launch("ctdk_attn_bwd(dkv)");
  }
  return rc;
}

}  // namespace
}  // namespace ctdk

using namespace ctdk;

namespace ctdk {
// delta[b, h, t] = sum_d dout * out (the row term of the softmax backward).
int attn_delta_launch(const float* out, const float* dout, float* delta, int64_t B, int64_t T, int H, int D, cudaStream_t s) {
  const int64_t items = B * T * H;
  const int lp = D / 4;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  const int64_t need = (items + (256 / lp) * 4 - 1) / ((256 / lp) * 4);
  const int grid = static_cast<int>(need < cap ? need : cap);
  if (D == 64)
    launch_pdl(attn_delta_kernel<64>, dim3(grid), dim3(256), 0, s, out, dout, delta, B, static_cast<int>(T), H);
  else
    launch_pdl(attn_delta_kernel<128>, dim3(grid), dim3(256), 0, s, out, dout, delta, B, static_cast<int>(T), H);
  return check_launch("ctdk_attn_bwd(delta)");
}
}  // namespace ctdk

extern "C" {

int ctdk_attn_fwd_p(const float* qkv, float* out, float* lse, int64_t B, int64_t T, int H, int Hk, int D,
                    int precision, void* stream) {
  int rc = check_attn_args("ctdk_attn_fwd", B, T, H, Hk, D);
  if (rc != CTDK_OK) return rc;
  CTDK_REQUIRE(precision == CTDK_GEMM_TF32 || precision == CTDK_GEMM_3XTF32, "ctdk_attn_fwd: unknown precision");
  if (B == 0 || T == 0) return CTDK_OK;
  CTDK_REQUIRE(qkv && out && lse, "ctdk_attn_fwd: null pointer");
  CTDK_REQUIRE((reinterpret_cast<uintptr_t>(qkv) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 7u) == 0,
               "ctdk_attn_fwd: qkv must be 16-byte aligned, out 8-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool x3 = precision == CTDK_GEMM_3XTF32;
  // causal half of 2 GEMMs: 2 * (2*T*T*D)/2 per (batch, head)
  void* tok = prof_begin(CTDK_PROF_ATTN, 2.0 * B * H * static_cast<double>(T) * T * D, s);
  if (!x3 && !attn_use_legacy()) {
    rc = attn_fwd_tcgen05(qkv, out, lse, B, T, H, Hk, D, s);
    if (rc <= 0) {
      prof_end(tok, s);
      return rc;
    }
  }
  if (D == 64) rc = x3 ? run_fwd_legacy<64, true>(qkv, out, lse, B, T, H, Hk, s) : run_fwd_legacy<64, false>(qkv, out, lse, B, T, H, Hk, s);
  else rc = x3 ? run_fwd_legacy<128, true>(qkv, out, lse, B, T, H, Hk, s) : run_fwd_legacy<128, false>(qkv, out, lse, B, T, H, Hk, s);
  prof_end(tok, s);
  return rc;
}

int ctdk_attn_fwd(const float* qkv, float* out, float* lse, int64_t B, int64_t T, int H, int Hk, int D,
                  void* stream) {
  return ctdk_attn_fwd_p(qkv, out, lse, B, T, H, Hk, D, CTDK_GEMM_TF32, stream);
}

int ctdk_attn_bwd_p(const float* qkv, const float* out, const float* dout, const float* lse, float* delta,
                    float* dqkv, int64_t B, int64_t T, int H, int Hk, int D, int precision, void* stream) {
  int rc = check_attn_args("ctdk_attn_bwd", B, T, H, Hk, D);
  if (rc != CTDK_OK) return rc;
  CTDK_REQUIRE(precision == CTDK_GEMM_TF32 || precision == CTDK_GEMM_3XTF32, "ctdk_attn_bwd: unknown precision");
  if (B == 0 || T == 0) return CTDK_OK;
  CTDK_REQUIRE(qkv && dout && lse && delta && dqkv, "ctdk_attn_bwd: null pointer");
  CTDK_REQUIRE((reinterpret_cast<uintptr_t>(qkv) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(dout) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dqkv) & 7u) == 0,
               "ctdk_attn_bwd: qkv/out/dout must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool x3 = precision == CTDK_GEMM_3XTF32;
  // backward = 2x the forward's algorithmic FLOPs (recomputation is not counted)
  void* tok = prof_begin(CTDK_PROF_ATTN, 4.0 * B * H * static_cast<double>(T) * T * D, s);
  if (out != nullptr) {   // otherwise delta already holds rowsum(dout * out) (ctdk_gemm_dattn_delta)
    rc = attn_delta_launch(out, dout, delta, B, T, H, D, s);
    if (rc != CTDK_OK) return rc;
  }
  // tcgen05 kernels first; each returns 1 when it does not take the shape.
  int dq_done = 1, dkv_done = 1;
  if (!x3 && !attn_use_legacy()) {
    dq_done = attn_bwd_dq_tcgen05(qkv, dout, lse, delta, dqkv, B, T, H, Hk, D, s);
    if (dq_done < 0) return dq_done;
    dkv_done = attn_bwd_dkv_tcgen05(qkv, dout, lse, delta, dqkv, B, T, H, Hk, D, s);
    if (dkv_done < 0) return dkv_done;
  }
  const bool dq = dq_done == 1, dkv = dkv_done == 1;
  if (dq || dkv) {
    if (D == 64)
      rc = x3 ? run_bwd_legacy<64, 64, true>(qkv, dout, lse, delta, dqkv, B, T, H, Hk, dq, dkv, s)
              : run_bwd_legacy<64, 64, false>(qkv, dout, lse, delta, dqkv, B, T, H, Hk, dq, dkv, s);
    else
      rc = x3 ? run_bwd_legacy<128, 32, true>(qkv, dout, lse, delta, dqkv, B, T, H, Hk, dq, dkv, s)
              : run_bwd_legacy<128, 32, false>(qkv, dout, lse, delta, dqkv, B, T, H, Hk, dq, dkv, s);
  }
  prof_end(tok, s);
  return rc;
}

int ctdk_attn_bwd(const float* qkv, const float* out, const float* dout, const float* lse, float* delta,
                  float* dqkv, int64_t B, int64_t T, int H, int Hk, int D, void* stream) {
  return ctdk_attn_bwd_p(qkv, out, dout, lse, delta, dqkv, B, T, H, Hk, D, CTDK_GEMM_TF32, stream);
}

}  // extern "C"
