// ctdk_gemm / ctdk_bmm entry points and the exact-fp32 SIMT kernel used for shapes the
// tensor-core path cannot take (leading dimensions that are not multiples of 4 floats,
// unaligned pointers, N < 8) or when CTDK_GEMM_FP32_SIMT is requested.
#include "common.cuh"

namespace ctdk {

int gemm_tcgen05(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                 int64_t lda, int64_t ldb, int64_t ldc, int transa, int transb, int epilogue,
                 const float* aux, cudaStream_t stream);
void gemm_set_kblock_limit(int k_blocks);
int gemm_dattn_delta_tcgen05(const float* dy, const float* Wo, const float* out, float* dattn, float* delta, int64_t M,
                             int64_t T, int H, int D, int64_t K, cudaStream_t stream);
int attn_delta_launch(const float* out, const float* dout, float* delta, int64_t B, int64_t T, int H, int D, cudaStream_t s);
int gemm_3xtf32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                int64_t lda, int64_t ldb, int64_t ldc, int transa, int transb, int epilogue,
                const float* aux, cudaStream_t stream);

namespace {

constexpr int TS = 64;  // C tile
constexpr int TK = 16;

// 256 threads, each owns a 4x4 block of the 64x64 tile. fp32 FMA, k ascending.
__global__ void __launch_bounds__(256)
    gemm_simt_kernel(const float* __restrict__ A, const float* __restrict__ B,
                     float* __restrict__ C, const float* __restrict__ aux, int64_t M, int64_t N,
                     int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int transa, int transb,
                     int epilogue) {
  __shared__ float As[TK][TS + 1];
  __shared__ float Bs[TK][TS + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * TS, n0 = static_cast<int64_t>(blockIdx.x) * TS;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TS * TK; i += 256) {
      const int kk = i % TK, mm = i / TK;
      const int64_t gm = m0 + mm, gk = k0 + kk;
      float va = 0.0f;
      if (gm < M && gk < K) va = transa ? A[gk * lda + gm] : A[gm * lda + gk];
      As[kk][mm] = va;
      const int64_t gn = n0 + mm;
      float vb = 0.0f;
      if (gn < N && gk < K) vb = transb ? B[gn * ldb + gk] : B[gk * ldb + gn];
      Bs[kk][mm] = vb;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = As[kk][ty * 4 + i];
        b[i] = Bs[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float r = acc[i][j];
      if (epilogue == CTDK_EPI_ACCUMULATE) r += C[gm * ldc + gn];
      else if (epilogue == CTDK_EPI_RESIDUAL) r += aux[gm * ldc + gn];
      C[gm * ldc + gn] = r;
    }
  }
}

// hi = x rounded to TF32 (10-bit mantissa, round to nearest), lo = x - hi (exact in fp32).
__global__ void __launch_bounds__(256) split_tf32_kernel(const float* __restrict__ x, float* __restrict__ hi,
                                                         float* __restrict__ lo, int64_t n4) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  auto sp = [](float v, float& h, float& l) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    h = __uint_as_float(r);
    l = v - h;
  };
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    float4 h, l;
    sp(v.x, h.x, l.x);
    sp(v.y, h.y, l.y);
    sp(v.z, h.z, l.z);
    sp(v.w, h.w, l.w);
    reinterpret_cast<float4*>(hi)[i] = h;
    reinterpret_cast<float4*>(lo)[i] = l;
  }
}

__global__ void fill_rows_kernel(float* C, const float* aux, int64_t M, int64_t N, int64_t ldc,
                                 int epilogue) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  const int64_t r = i / N, c = i - r * N;
  if (epilogue == CTDK_EPI_STORE) C[r * ldc + c] = 0.0f;
  else if (epilogue == CTDK_EPI_RESIDUAL) C[r * ldc + c] = aux[r * ldc + c];
}

}  // namespace
}  // namespace ctdk

namespace ctdk {
int gemm_swiglu_tcgen05(const float* A, const float* W, float* gu, float* act, int64_t M, int64_t I, int64_t K,
                        cudaStream_t stream);
int gemm_swiglu_bwd_tcgen05(const float* dy, const float* Wd, const float* gu, float* dgu, int64_t M, int64_t I, int64_t K,
                            cudaStream_t stream);
}  // namespace ctdk

using namespace ctdk;

extern "C" {

int ctdk_gemm_swiglu_bwd(const float* dy, const float* Wd, const float* gu, float* dgu, float* dact_scratch, int64_t M,
                         int64_t I, int64_t K, int precision, void* stream) {
  CTDK_REQUIRE(M >= 0 && I > 0 && K > 0, "ctdk_gemm_swiglu_bwd: bad shape");
  if (M == 0) return CTDK_OK;
  CTDK_REQUIRE(dy && Wd && gu && dgu, "ctdk_gemm_swiglu_bwd: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (precision == CTDK_GEMM_TF32) {
    void* tok = prof_begin(CTDK_PROF_GEMM, 2.0 * static_cast<double>(M) * I * K, s);
    const int rc = gemm_swiglu_bwd_tcgen05(dy, Wd, gu, dgu, M, I, K, s);
    prof_end(tok, s);
    if (rc <= 0) return rc;
  }
  CTDK_REQUIRE(dact_scratch != nullptr, "ctdk_gemm_swiglu_bwd: this shape needs the [M, I] scratch buffer");
  int rc = ctdk_gemm(dy, Wd, dact_scratch, M, I, K, K, I, I, 0, 0, precision, CTDK_EPI_STORE, nullptr, stream);
  if (rc != CTDK_OK) return rc;
  return ctdk_swiglu_bwd(gu, dact_scratch, dgu, M, static_cast<int>(I), stream);
}

int ctdk_gemm_dattn_delta(const float* dy, const float* Wo, const float* attn_out, float* dattn, float* delta, int64_t B,
                          int64_t T, int H, int D, int64_t hid, int precision, void* stream) {
  CTDK_REQUIRE(B >= 0 && T >= 0 && H > 0 && hid > 0 && (D == 64 || D == 128), "ctdk_gemm_dattn_delta: bad shape");
  if (B == 0 || T == 0) return CTDK_OK;
  CTDK_REQUIRE(dy && Wo && attn_out && dattn && delta, "ctdk_gemm_dattn_delta: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t M = B * T, N = static_cast<int64_t>(H) * D;
  if (precision == CTDK_GEMM_TF32) {
    void* tok = prof_begin(CTDK_PROF_GEMM, 2.0 * static_cast<double>(M) * N * hid, s);
    const int rc = gemm_dattn_delta_tcgen05(dy, Wo, attn_out, dattn, delta, M, T, H, D, hid, s);
    prof_end(tok, s);
    if (rc <= 0) return rc;
  }
  int rc = ctdk_gemm(dy, Wo, dattn, M, N, hid, hid, N, N, 0, 0, precision, CTDK_EPI_STORE, nullptr, stream);
  if (rc != CTDK_OK) return rc;
  return attn_delta_launch(attn_out, dattn, delta, B, T, H, D, s);
}

int ctdk_gemm_swiglu(const float* A, const float* W, float* gu, float* act, int64_t M, int64_t I, int64_t K,
                     int precision, void* stream) {
  CTDK_REQUIRE(M >= 0 && I > 0 && K > 0, "ctdk_gemm_swiglu: bad shape");
  if (M == 0) return CTDK_OK;
  CTDK_REQUIRE(A && W && gu && act, "ctdk_gemm_swiglu: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (precision == CTDK_GEMM_TF32) {
    void* tok = prof_begin(CTDK_PROF_GEMM, 4.0 * static_cast<double>(M) * I * K, s);
    const int rc = gemm_swiglu_tcgen05(A, W, gu, act, M, I, K, s);
    if (rc <= 0) {
      prof_end(tok, s);
      return rc;
    }
    prof_end(tok, s);   // not eligible: nothing was enqueued; the two-kernel path below reports itself
  }
  int rc = ctdk_gemm(A, W, gu, M, 2 * I, K, K, K, 2 * I, 0, 1, precision, CTDK_EPI_STORE, nullptr, stream);
  if (rc != CTDK_OK) return rc;
  return ctdk_swiglu_fwd(gu, act, M, static_cast<int>(I), stream);
}

int ctdk_gemm(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
              int64_t lda, int64_t ldb, int64_t ldc, int transa, int transb, int precision,
              int epilogue, const float* aux, void* stream) {
  CTDK_REQUIRE(M >= 0 && N >= 0 && K >= 0, "ctdk_gemm: negative dimension");
  CTDK_REQUIRE(epilogue == CTDK_EPI_STORE || epilogue == CTDK_EPI_ACCUMULATE ||
                   epilogue == CTDK_EPI_RESIDUAL,
               "ctdk_gemm: unknown epilogue %d", epilogue);
  CTDK_REQUIRE(precision == CTDK_GEMM_TF32 || precision == CTDK_GEMM_3XTF32 ||
                   precision == CTDK_GEMM_FP32_SIMT,
               "ctdk_gemm: unknown precision %d", precision);
  if (M == 0 || N == 0) return CTDK_OK;
  CTDK_REQUIRE(C != nullptr, "ctdk_gemm: null C");
  CTDK_REQUIRE(epilogue != CTDK_EPI_RESIDUAL || aux != nullptr, "ctdk_gemm: residual needs aux");
  CTDK_REQUIRE(ldc >= N, "ctdk_gemm: ldc < N");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (K == 0) {
    if (epilogue != CTDK_EPI_ACCUMULATE) {
      fill_rows_kernel<<<ceil_div(M * N, 256), 256, 0, s>>>(C, aux, M, N, ldc, epilogue);
      return check_launch("ctdk_gemm(K=0)");
    }
    return CTDK_OK;
  }
  CTDK_REQUIRE(A && B, "ctdk_gemm: null operand");
  CTDK_REQUIRE(lda >= (transa ? M : K), "ctdk_gemm: lda too small");
  CTDK_REQUIRE(ldb >= (transb ? K : N), "ctdk_gemm: ldb too small");
  void* tok = prof_begin(CTDK_PROF_GEMM, 2.0 * static_cast<double>(M) * N * K, s);
  if (precision != CTDK_GEMM_FP32_SIMT) {
    int rc = (precision == CTDK_GEMM_3XTF32)
                 ? gemm_3xtf32(A, B, C, M, N, K, lda, ldb, ldc, transa, transb, epilogue, aux, s)
                 : gemm_tcgen05(A, B, C, M, N, K, lda, ldb, ldc, transa, transb, epilogue, aux,
                                s);
    if (rc <= 0) {  // enqueued, or a real error
      prof_end(tok, s);
      return rc;
    }
  }
  dim3 grid(static_cast<unsigned>((N + TS - 1) / TS), static_cast<unsigned>((M + TS - 1) / TS));
  CTDK_REQUIRE(grid.y <= 65535u, "ctdk_gemm: M too large for the SIMT path");
  gemm_simt_kernel<<<grid, 256, 0, s>>>(A, B, C, aux, M, N, K, lda, ldb, ldc, transa, transb,
                                        epilogue);
  prof_end(tok, s);
  return check_launch("ctdk_gemm(simt)");
}

int64_t ctdk_gemm_3xtf32_workspace_floats(int64_t M, int64_t N, int64_t K) {
  if (M < 0 || N < 0 || K < 0) return -1;
  return 2 * (M * K + K * N) + 64;
}

int ctdk_gemm_ws(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                 int64_t lda, int64_t ldb, int64_t ldc, int transa, int transb, int precision,
                 int epilogue, const float* aux, float* workspace, int64_t workspace_floats,
                 void* stream) {
  const bool dense = lda == (transa ? M : K) && ldb == (transb ? K : N);
  const bool aligned = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
                         reinterpret_cast<uintptr_t>(workspace)) & 15u) == 0 &&
                       ((M * K) % 4 == 0) && ((K * N) % 4 == 0) && (lda % 4 == 0) && (ldb % 4 == 0);
  if (precision != CTDK_GEMM_3XTF32 || workspace == nullptr || !dense || !aligned || M == 0 || N == 0 ||
      K == 0 || N < 8)
    return ctdk_gemm(A, B, C, M, N, K, lda, ldb, ldc, transa, transb, precision, epilogue, aux, stream);
  CTDK_REQUIRE(workspace_floats >= ctdk_gemm_3xtf32_workspace_floats(M, N, K),
               "ctdk_gemm_ws: workspace too small for the 3xTF32 split");
  // a = a_hi + a_lo, b = b_hi + b_lo with hi exactly representable in TF32:
  // a*b = a_hi*b_hi + a_hi*b_lo + a_lo*b_hi (+ a_lo*b_lo, below fp32 resolution and dropped).
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t na = M * K, nb = K * N;
  auto up = [](int64_t v) { return (v + 15) / 16 * 16; };
  float* a_hi = workspace;
  float* a_lo = a_hi + up(na);
  float* b_hi = a_lo + up(na);
  float* b_lo = b_hi + up(nb);
  const int cap = sm_count() * 8;
  auto blocks = [&](int64_t n4) { return static_cast<int>(n4 / 256 + 1 < cap ? n4 / 256 + 1 : cap); };
  split_tf32_kernel<<<blocks(na / 4), 256, 0, s>>>(A, a_hi, a_lo, na / 4);
  int rc = check_launch("ctdk_gemm_ws(split A)");
  if (rc != CTDK_OK) return rc;
  split_tf32_kernel<<<blocks(nb / 4), 256, 0, s>>>(B, b_hi, b_lo, nb / 4);
  rc = check_launch("ctdk_gemm_ws(split B)");
  if (rc != CTDK_OK) return rc;
  // the leading product in accumulation runs of at most 16 k-blocks (512 deep); the two correction
  // products are 2^-11 of it and keep the usual schedule
  gemm_set_kblock_limit(16);
  rc = ctdk_gemm(a_hi, b_hi, C, M, N, K, lda, ldb, ldc, transa, transb, CTDK_GEMM_TF32, epilogue, aux, stream);
  gemm_set_kblock_limit(0);
  if (rc != CTDK_OK) return rc;
  rc = ctdk_gemm(a_hi, b_lo, C, M, N, K, lda, ldb, ldc, transa, transb, CTDK_GEMM_TF32, CTDK_EPI_ACCUMULATE,
                 nullptr, stream);
  if (rc != CTDK_OK) return rc;
  return ctdk_gemm(a_lo, b_hi, C, M, N, K, lda, ldb, ldc, transa, transb, CTDK_GEMM_TF32, CTDK_EPI_ACCUMULATE,
                   nullptr, stream);
}

int ctdk_bmm(const float* A, const float* B, float* C, int64_t batch, int64_t M, int64_t N,
             int64_t K, int transa, int transb, int precision, void* stream) {
  CTDK_REQUIRE(batch >= 0 && M >= 0 && N >= 0 && K >= 0, "ctdk_bmm: negative dimension");
  const int64_t lda = transa ? M : K, ldb = transb ? K : N;
  for (int64_t b = 0; b < batch; ++b) {
    int rc = ctdk_gemm(A + b * M * K, B + b * K * N, C + b * M * N, M, N, K, lda, ldb, N,
                       transa, transb, precision, CTDK_EPI_STORE, nullptr, stream);
    if (rc != CTDK_OK) return rc;
  }
  return CTDK_OK;
}

}  // extern "C"
