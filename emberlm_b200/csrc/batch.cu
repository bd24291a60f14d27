// Data feed of the training step: widens token / mask rows of the reference's bin format on the
// device (emberlm tools/ctd_train/main.cpp:145-174 builds int64 / fp32 host vectors instead).
#include "common.cuh"

namespace ctdk {
namespace {

// One CTA per micro-batch: sum of the loss mask over its rows, positions 1 .. S-1. The values are
// 0/1, so the fp32 sum is an exact integer whatever the order.
__global__ void __launch_bounds__(256) micro_mask_sum_kernel(const int8_t* __restrict__ msk, int64_t rows, int S,
                                                             int micro_rows, float* __restrict__ sums) {
  __shared__ float red[8];
  const int64_t r0 = static_cast<int64_t>(blockIdx.x) * micro_rows;
  const int64_t r1 = r0 + micro_rows < rows ? r0 + micro_rows : rows;
  const int T = S - 1;
  float acc = 0.0f;
  for (int64_t i = threadIdx.x; i < (r1 - r0) * T; i += blockDim.x) {
    const int64_t r = r0 + i / T;
    const int t = static_cast<int>(i % T);
    acc += static_cast<float>(msk[r * S + t + 1] != 0);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < 8 ? red[threadIdx.x] : 0.0f;
    v = warp_sum(v);
    if (threadIdx.x == 0) sums[blockIdx.x] = v;
  }
}

__global__ void __launch_bounds__(256) batch_widen_kernel(const int32_t* __restrict__ tok, const int8_t* __restrict__ msk,
                                                          int64_t rows, int S, int micro_rows, float accum,
                                                          const float* __restrict__ sums, int64_t* __restrict__ ids,
                                                          int64_t* __restrict__ targets, float* __restrict__ mask,
                                                          float* __restrict__ weight) {
  const int T = S - 1;
  const int64_t n = rows * T;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t r = i / T;
    const int t = static_cast<int>(i - r * T);
    const int32_t a = tok[r * S + t], b = tok[r * S + t + 1];
    const float mk = static_cast<float>(msk[r * S + t + 1] != 0);
    const float sm = sums[r / micro_rows];
    ids[i] = a;
    targets[i] = b;
    mask[i] = mk;
    weight[i] = sm > 0.0f ? mk / (sm * accum) : 0.0f;
  }
}

}  // namespace
}  // namespace ctdk

using namespace ctdk;

extern "C" int ctdk_batch_widen(const int32_t* tok, const int8_t* msk, int64_t rows, int S, int micro_rows,
                                int accum_total, int64_t* ids, int64_t* targets, float* mask, float* weight,
                                float* micro_sums, void* stream) {
  CTDK_REQUIRE(rows >= 0 && S >= 2 && micro_rows >= 1 && accum_total >= 1, "ctdk_batch_widen: bad shape");
  if (rows == 0) return CTDK_OK;
  CTDK_REQUIRE(tok && msk && ids && targets && mask && weight && micro_sums, "ctdk_batch_widen: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int n_micro = static_cast<int>((rows + micro_rows - 1) / micro_rows);
  micro_mask_sum_kernel<<<n_micro, 256, 0, s>>>(msk, rows, S, micro_rows, micro_sums);
  int rc = check_launch("ctdk_batch_widen (mask sums)");
  if (rc != CTDK_OK) return rc;
  const int64_t n = rows * (S - 1);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8, need = (n + 255) / 256;
  batch_widen_kernel<<<static_cast<int>(need < cap ? need : cap), 256, 0, s>>>(
      tok, msk, rows, S, micro_rows, static_cast<float>(accum_total), micro_sums, ids, targets, mask, weight);
  return check_launch("ctdk_batch_widen");
}
