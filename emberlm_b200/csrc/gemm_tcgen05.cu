// TF32 GEMM on the 5th-generation tensor cores: C[M,N] = op(A)·op(B) with fp32 operands in
// HBM, fp32 accumulators in tensor memory.
//
// One persistent CTA per SM, 6 warps:
//   warp 0   TMA producer: fills a ring of shared-memory stages (128-byte swizzled tiles),
//            one elected lane, plain (non-multicast) cp.async.bulk.tensor loads.
//   warp 1   MMA issuer: one elected lane issues tcgen05.mma.kind::tf32 (M=128, N=BN, K=8)
//            four times per 32-float stage and releases the stage with tcgen05.commit.
//   warps 2-5 epilogue: read the accumulator with tcgen05.ld (each warp owns one 32-lane
//            quarter of tensor memory) and write C. Two accumulator buffers let the epilogue
//            of tile i overlap the main loop of tile i+1.
// Operands that are contiguous along K are loaded as one box {32 floats, rows}; operands
// contiguous along M or N (the transposed cases of the reference's matmul, emberlm
// src/ops/matmul.cpp:25-47,99-118) are loaded as {32 floats of M/N, 32 rows of K} boxes with
// the 32-byte-atom variant of the 128-byte swizzle and described to the tensor core as
// MN-major. M, N and K tails are zero-filled by TMA bounds
// checking; the epilogue predicates stores. Every mbarrier wait is bounded.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace ctdk {
namespace {

constexpr int BM = 128;
constexpr int BK = 32;                    // floats per stage along K = one 128-byte swizzle row
constexpr int kATileBytes = BM * BK * 4;  // 16 KB
constexpr int kChunkBytes = 32 * BK * 4;  // 4 KB: one {32 x 32} box of an MN-major operand
constexpr int kThreads = 192;
constexpr int kGroupM = 16;               // m-blocks per scheduling group (L2 reuse of B tiles)

template <int BN>
struct Cfg {
  static constexpr int kBTileBytes = BN * BK * 4;
  static constexpr int kStageBytes = kATileBytes + kBTileBytes;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * BN;  // two accumulator buffers
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

struct GemmArgs {
  float* C;
  const float* aux;
  int64_t ldc;
  int M, N, K;
  int epilogue;
  int vec_ok;  // C (and aux) rows are 16-byte aligned and N%4==0
  int splits;  // K is cut into `splits` ranges; >1: partial tiles are added to C with atomics
  int* status;
};

// Instruction descriptor for kind::tf32: D=F32 (bit 4), A,B=TF32 (value 2 at bits 7 and 10),
// major-ness bits 15/16 (0 = K-major, 1 = MN-major), N>>3 at bit 17, M>>4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(bool a_mn, bool b_mn, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(a_mn) << 15) |
         (static_cast<uint32_t>(b_mn) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(BM >> 4) << 24);
}

__device__ __forceinline__ void tile_coords(int tile, int m_blocks, int n_blocks, int& mb,
                                            int& nb) {
  const int per_group = kGroupM * n_blocks;
  const int g = tile / per_group;
  const int first_m = g * kGroupM;
  const int gm = min(kGroupM, m_blocks - first_m);
  const int local = tile - g * per_group;
  mb = first_m + local % gm;
  nb = local / gm;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_tf32_kernel(const __grid_constant__ CUtensorMap tmA,
                     const __grid_constant__ CUtensorMap tmB, const GemmArgs args) {
  using C = Cfg<BN>;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* full = bars;                      // [kStages]
  uint64_t* empty = bars + C::kStages;        // [kStages]
  uint64_t* tfull = bars + 2 * C::kStages;    // [2]
  uint64_t* tempty = tfull + 2;               // [2]
  uint64_t* final_bar = tempty + 2;           // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(final_bar + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = (args.M + BM - 1) / BM;
  const int n_blocks = (args.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int k_blocks = (args.K + BK - 1) / BK;
  const int num_units = num_tiles * args.splits;  // unit u: tile u % num_tiles, k-range u / num_tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    mbar_init(final_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        int mb, nb;
        tile_coords(unit % num_tiles, m_blocks, n_blocks, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        const int split = unit / num_tiles;
        const int kb0 = static_cast<int>(static_cast<int64_t>(split) * k_blocks / args.splits);
        const int kb1 = static_cast<int>(static_cast<int64_t>(split + 1) * k_blocks / args.splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&empty[s], ph ^ 1u, args.status, 1)) {
            ok = false;
            break;
          }
          unsigned char* a_dst = smem + s * C::kStageBytes;
          unsigned char* b_dst = a_dst + kATileBytes;
          mbar_expect_tx(&full[s], C::kStageBytes);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 32; ++c)
              tma_load_2d(a_dst + c * kChunkBytes, &tmA, &full[s], m0 + 32 * c, k0);
          } else {
            tma_load_2d(a_dst, &tmA, &full[s], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 32; ++c)
              tma_load_2d(b_dst + c * kChunkBytes, &tmB, &full[s], n0 + 32 * c, k0);
          } else {
            tma_load_2d(b_dst, &tmB, &full[s], k0, n0);
          }
          if (++s == C::kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(A_MN, B_MN, BN);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++it) {
        const int split = unit / num_tiles;
        const int kb0 = static_cast<int>(static_cast<int64_t>(split) * k_blocks / args.splits);
        const int kb1 = static_cast<int>(static_cast<int64_t>(split + 1) * k_blocks / args.splits);
        const int acc = it & 1;
        const uint32_t acc_ph = (static_cast<uint32_t>(it) >> 1) & 1u;
        if (!mbar_wait_bounded(&tempty[acc], acc_ph ^ 1u, args.status, 2)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&full[s], ph, args.status, 3)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * C::kStageBytes);
          const uint32_t b_addr = a_addr + kATileBytes;
#pragma unroll
          for (int ks = 0; ks < BK / 8; ++ks) {
            // K-major (SWIZZLE_128B): the 8-float k-slice starts 32 bytes further inside the
            // swizzled row; rows are 128 bytes apart, 8-row groups 1024 bytes apart (SBO).
            // MN-major (SWIZZLE_128B_BASE32B): a k-slice is 8 rows of 128 bytes = two 4-row
            // swizzle groups 512 bytes apart (SBO); the 32-float chunks along M/N are
            // kChunkBytes apart (LBO).
            const uint64_t adesc =
                A_MN ? make_smem_desc(a_addr + ks * 1024, kChunkBytes, 512, kLayoutSw128Base32)
                     : make_smem_desc(a_addr + ks * 32, 16, 1024, kLayoutSw128);
            const uint64_t bdesc =
                B_MN ? make_smem_desc(b_addr + ks * 1024, kChunkBytes, 512, kLayoutSw128Base32)
                     : make_smem_desc(b_addr + ks * 32, 16, 1024, kLayoutSw128);
            umma_tf32(d_tmem, adesc, bdesc, idesc, (kb != kb0 || ks != 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // stage is free once these MMAs have read it
          if (++s == C::kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) umma_commit(&tfull[acc]);  // accumulator complete
      }
      // All MMAs retired before tensor memory is released.
      umma_commit(final_bar);
      mbar_wait_bounded(final_bar, 0, args.status, 4);
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue -------------------------------
    const int q = warp & 3;  // tensor-memory lane quarter this warp may access
    const int row_in_tile = q * 32 + lane;
    int it = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++it) {
      int mb, nb;
      tile_coords(unit % num_tiles, m_blocks, n_blocks, mb, nb);
      const bool first_split = unit < num_tiles;
      const bool atomic = args.splits > 1;
      const int acc = it & 1;
      const uint32_t acc_ph = (static_cast<uint32_t>(it) >> 1) & 1u;
      if (!mbar_wait_bounded(&tfull[acc], acc_ph, args.status, 5)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int64_t grow = static_cast<int64_t>(mb) * BM + row_in_tile;
      const bool row_ok = grow < args.M;
      float* crow = args.C + grow * args.ldc;
      const float* xrow = args.aux != nullptr ? args.aux + grow * args.ldc : nullptr;
      const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * BN) +
                             (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        const int col0 = nb * BN + ch * 32;
        if (col0 >= args.N) break;  // warp-uniform
        float v[32];
        tmem_ld_32x32(t_row + static_cast<uint32_t>(ch * 32), v);
        if (!row_ok) {
          // rows past M hold zero-filled garbage: nothing to store
        } else if (atomic) {
          // split-K: C was zeroed (STORE / RESIDUAL) or holds the running sum (ACCUMULATE);
          // every k-range adds its partial tile, the first one also adds the residual.
          const bool add_aux = first_split && args.epilogue == CTDK_EPI_RESIDUAL;
          if (args.vec_ok && col0 + 32 <= args.N) {
            float4* c4 = reinterpret_cast<float4*>(crow + col0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 r = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              if (add_aux) {
                const float4 x = reinterpret_cast<const float4*>(xrow + col0)[j];
                r.x += x.x;
                r.y += x.y;
                r.z += x.z;
                r.w += x.w;
              }
              atomicAdd(&c4[j], r);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = col0 + j;
              if (col < args.N) atomicAdd(&crow[col], v[j] + (add_aux ? xrow[col] : 0.0f));
            }
          }
        } else if (args.vec_ok && col0 + 32 <= args.N) {
          float4* c4 = reinterpret_cast<float4*>(crow + col0);
          if (args.epilogue == CTDK_EPI_STORE) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              c4[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
            const float4* x4 = args.epilogue == CTDK_EPI_ACCUMULATE
                                   ? reinterpret_cast<const float4*>(crow + col0)
                                   : reinterpret_cast<const float4*>(xrow + col0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 x = x4[j];
              c4[j] = make_float4(v[4 * j] + x.x, v[4 * j + 1] + x.y, v[4 * j + 2] + x.z,
                                  v[4 * j + 3] + x.w);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = col0 + j;
            if (col < args.N) {
              float r = v[j];
              if (args.epilogue == CTDK_EPI_ACCUMULATE) r += crow[col];
              else if (args.epilogue == CTDK_EPI_RESIDUAL) r += xrow[col];
              crow[col] = r;
            }
          }
        }
        __syncwarp();  // tcgen05.ld is warp-collective: reconverge before the next chunk
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ----------------------------------------------------------------------------------------
// Host side
// ----------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::once_flag g_encode_once;

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  });
  return g_encode;
}

bool tma_rounds_to_tf32() {
  // CTDK_TMA_F32=1 loads raw fp32 bits (the tensor core then ignores the low mantissa bits);
  // the default asks the copy engine for the TF32 data type.
  static const bool raw = [] {
    const char* e = std::getenv("CTDK_TMA_F32");
    return e != nullptr && e[0] == '1';
  }();
  return !raw;
}

// 2-D map over a row-major fp32 matrix: dim0 = contiguous extent `inner`, dim1 = `outer`
// rows `ld` floats apart; box = {32, box_rows}; 128-byte rows swizzled in 16-byte chunks
// (K-major tiles) or 32-byte chunks (MN-major tiles); out-of-range reads give 0.
int make_map(CUtensorMap* map, const float* base, int64_t inner, int64_t outer, int64_t ld,
             int box_rows, bool mn_major, bool exact_fp32) {
  auto enc = encode_fn();
  if (enc == nullptr) return fail(CTDK_ELAUNCH, "cuTensorMapEncodeTiled unavailable");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * sizeof(float)};
  cuuint32_t box[2] = {32u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  const CUtensorMapDataType dt = (!exact_fp32 && tma_rounds_to_tf32())
                                     ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32
                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(map, dt, 2, const_cast<float*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(CTDK_ELAUNCH, "cuTensorMapEncodeTiled failed (%d): inner=%lld outer=%lld ld=%lld",
                static_cast<int>(r), static_cast<long long>(inner),
                static_cast<long long>(outer), static_cast<long long>(ld));
  return CTDK_OK;
}

}  // namespace

int encode_tensor_map(CUtensorMap* map, const float* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, bool atom32) {
  auto enc = encode_fn();
  if (enc == nullptr) return fail(CTDK_ELAUNCH, "cuTensorMapEncodeTiled unavailable");
  cuuint64_t d[5], st[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) st[i] = strides_bytes[i];
  }
  const CUtensorMapDataType dt =
      tma_rounds_to_tf32() ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(map, dt, rank, const_cast<float*>(base), d, st, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(CTDK_ELAUNCH, "cuTensorMapEncodeTiled failed (%d), rank %d", static_cast<int>(r), rank);
  return CTDK_OK;
}

namespace {

template <int BN, bool A_MN, bool B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args,
           cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto* kern = gemm_tf32_kernel<BN, A_MN, B_MN>;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess)
      return fail(CTDK_ELAUNCH, "gemm: cannot opt in to %d bytes of shared memory: %s",
                  C::kSmemBytes, cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  const int m_blocks = (args.M + BM - 1) / BM, n_blocks = (args.N + BN - 1) / BN;
  const int tiles = m_blocks * n_blocks * args.splits;
  const int sms = sm_count();
  const int grid = tiles < sms ? tiles : sms;
  kern<<<grid, kThreads, C::kSmemBytes, stream>>>(ta, tb, args);
  return check_launch("ctdk_gemm(tcgen05)");
}

template <int BN>
int dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb,
                   const GemmArgs& args, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch<BN, false, false>(ta, tb, args, stream);
  if (!a_mn && b_mn) return launch<BN, false, true>(ta, tb, args, stream);
  if (a_mn && !b_mn) return launch<BN, true, false>(ta, tb, args, stream);
  return launch<BN, true, true>(ta, tb, args, stream);
}

}  // namespace

int gemm_tcgen05_2cta(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, bool a_mn, bool b_mn,
                      bool a3d, bool b3d, int tma_out, float* C, const float* aux, int64_t ldc, int M, int N, int K,
                      int epilogue, int vec_ok, int splits, int* status, cudaStream_t stream);

int gemm_tcgen05_2cta_swiglu(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tgu, const CUtensorMap& tact,
                             int M, int N, int K, int* status, cudaStream_t stream);

// gu[M, 2I] = A[M, K] W[2I, K]^T and act[M, I] = silu(gu[:, :I]) * gu[:, I:] in one paired-CTA launch.
// Returns CTDK_OK after enqueueing, a negative status, or 1 when the shape is not eligible.
int gemm_swiglu_tcgen05(const float* A, const float* W, float* gu, float* act, int64_t M, int64_t I, int64_t K,
                        cudaStream_t stream) {
  auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!a16(A) || !a16(W) || !a16(gu) || !a16(act) || (K & 3) || (I % 128) != 0) return 1;
  if (M < 256 || M > INT32_MAX || 2 * I > INT32_MAX || K > INT32_MAX || K < 1) return 1;
  CUtensorMap ta, tb, tgu, tact;
  int rc = make_map(&ta, A, K, M, K, BM, false, false);
  if (rc == CTDK_OK) rc = make_map(&tb, W, K, 2 * I, K, 128, false, false);
  if (rc == CTDK_OK) rc = make_map(&tgu, gu, 2 * I, M, 2 * I, 32, false, true);
  if (rc == CTDK_OK) rc = make_map(&tact, act, I, M, I, 32, false, true);
  if (rc != CTDK_OK) return rc;
  int* st = device_status_word();
  if (st == nullptr) return fail(CTDK_ELAUNCH, "gemm: no status word");
  return gemm_tcgen05_2cta_swiglu(ta, tb, tgu, tact, static_cast<int>(M), static_cast<int>(I), static_cast<int>(K), st, stream);
}

int gemm_tcgen05_2cta_swiglu_bwd(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tgu, const CUtensorMap& tdgu,
                                 bool b3d, int M, int N, int K, int* status, cudaStream_t stream);

// dgu[M, 2I] = SwiGLU backward of (dy[M, K] * Wd[K, I]) against gu[M, 2I], in one paired-CTA launch.
// Returns CTDK_OK after enqueueing, a negative status, or 1 when the shape is not eligible.
int gemm_swiglu_bwd_tcgen05(const float* dy, const float* Wd, const float* gu, float* dgu, int64_t M, int64_t I, int64_t K,
                            cudaStream_t stream) {
  auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!a16(dy) || !a16(Wd) || !a16(gu) || !a16(dgu) || (K & 3) || (I % 32) != 0) return 1;
  if (M < 256 || I < 256 || M > INT32_MAX || 2 * I > INT32_MAX || K > INT32_MAX || K < 1) return 1;
  CUtensorMap ta, tb, tgu, tdgu;
  int rc = make_map(&ta, dy, K, M, K, BM, false, false);
  if (rc == CTDK_OK) {
    const uint64_t dims[3] = {32u, static_cast<uint64_t>(K), static_cast<uint64_t>(I / 32)};
    const uint64_t strides[2] = {static_cast<uint64_t>(I) * sizeof(float), 128u};
    const uint32_t box[3] = {32u, 32u, 4u};
    rc = encode_tensor_map(&tb, Wd, 3, dims, strides, box, true);
  }
  if (rc == CTDK_OK) rc = make_map(&tgu, gu, 2 * I, M, 2 * I, 32, false, true);
  if (rc == CTDK_OK) rc = make_map(&tdgu, dgu, 2 * I, M, 2 * I, 32, false, true);
  if (rc != CTDK_OK) return rc;
  int* st = device_status_word();
  if (st == nullptr) return fail(CTDK_ELAUNCH, "gemm: no status word");
  return gemm_tcgen05_2cta_swiglu_bwd(ta, tb, tgu, tdgu, true, static_cast<int>(M), static_cast<int>(I), static_cast<int>(K), st,
                                      stream);
}

int gemm_tcgen05_2cta_dattn_delta(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& to,
                                  bool b3d, float* delta, int M, int N, int K, int T, int H, int D, int* status,
                                  cudaStream_t stream);

// dattn[M, H*D] = dy[M, K] * Wo[K, H*D] and delta[b, h, t] = sum_d dattn * out over each head, in one paired-CTA
// launch (M = B * T rows). Returns CTDK_OK after enqueueing, a negative status, or 1 when not eligible.
int gemm_dattn_delta_tcgen05(const float* dy, const float* Wo, const float* out, float* dattn, float* delta, int64_t M,
                             int64_t T, int H, int D, int64_t K, cudaStream_t stream) {
  auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const int64_t N = static_cast<int64_t>(H) * D;
  if (!a16(dy) || !a16(Wo) || !a16(out) || !a16(dattn) || (K & 3) || (D != 64 && D != 128)) return 1;
  if (M < 256 || N < 256 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || K < 1 || T < 1 || M % T != 0) return 1;
  CUtensorMap ta, tb, tc, to;
  int rc = make_map(&ta, dy, K, M, K, BM, false, false);
  if (rc == CTDK_OK) {
    const uint64_t dims[3] = {32u, static_cast<uint64_t>(K), static_cast<uint64_t>(N / 32)};
    const uint64_t strides[2] = {static_cast<uint64_t>(N) * sizeof(float), 128u};
    const uint32_t box[3] = {32u, 32u, 4u};
    rc = encode_tensor_map(&tb, Wo, 3, dims, strides, box, true);
  }
  if (rc == CTDK_OK) rc = make_map(&tc, dattn, N, M, N, 32, false, true);
  if (rc == CTDK_OK) rc = make_map(&to, out, N, M, N, 32, false, true);
  if (rc != CTDK_OK) return rc;
  int* st = device_status_word();
  if (st == nullptr) return fail(CTDK_ELAUNCH, "gemm: no status word");
  return gemm_tcgen05_2cta_dattn_delta(ta, tb, tc, to, true, delta, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
                                       static_cast<int>(T), H, D, st, stream);
}

// Upper bound on the k-blocks one unit accumulates in tensor memory (0 = none), per host thread.
// The tensor core's fp32 accumulation loses low bits with every addition, so the error of a product
// grows with the length of the accumulation (measured: 2.1e-5 of the largest element at K = 8192 in
// one run against 1.3e-6 when the same K is added up from 512-deep pieces in fp32). The 3xTF32 mode
// sets it for its leading (hi x hi) product: K is then cut into ranges of at most that many
// k-blocks whose partial tiles are added at L2 in fp32.
static thread_local int t_kblock_limit = 0;
void gemm_set_kblock_limit(int k_blocks) { t_kblock_limit = k_blocks; }

// Returns CTDK_OK after enqueueing, or 1 when the shape/alignment is not eligible for the
// tensor-core path (the caller then uses the SIMT kernel).
int gemm_tcgen05(const float* A, const float* B, float* Cp, int64_t M, int64_t N, int64_t K,
                 int64_t lda, int64_t ldb, int64_t ldc, int transa, int transb, int epilogue,
                 const float* aux, cudaStream_t stream) {
  auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!a16(A) || !a16(B) || (lda & 3) || (ldb & 3)) return 1;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return 1;
  if (M < 1 || N < 8 || K < 1) return 1;

  const bool a_mn = transa != 0;  // A stored [K,M]: contiguous along M
  const bool b_mn = transb == 0;  // B stored [K,N]: contiguous along N
  // Tile width and K split: estimated time = rounds of the persistent grid x k-blocks per
  // unit x relative cost of a k-block (a 128-wide tile does half the work of a 256-wide one
  // but moves 2/3 of the operand bytes, hence the 0.6). Splitting K only pays when the output
  // tiles alone cannot fill the SMs (weight gradients: few tiles, K = all tokens).
  const int sms = sm_budget();
  const int64_t m_blocks = (M + BM - 1) / BM;
  const int64_t k_blocks = (K + BK - 1) / BK;
  int bn = 64, splits = 1;
  if (N > 64) {
    double best = 1e300;
    const int widths[2] = {256, 128};
    for (int wi = 0; wi < 2; ++wi) {
      const int w = widths[wi];
      if (w == 256 && N <= 128) continue;
      const int64_t tiles = m_blocks * ((N + w - 1) / w);
      const int max_splits = static_cast<int>(k_blocks / 16 < 1 ? 1 : (k_blocks / 16 > 32 ? 32 : k_blocks / 16));
      for (int sp = 1; sp <= max_splits; ++sp) {
        if (sp > 1 && tiles >= 2 * sms) break;
        const int64_t units = tiles * sp;
        const double rounds = static_cast<double>((units + sms - 1) / sms);
        const double kb = static_cast<double>((k_blocks + sp - 1) / sp);
        // + a fixed per-unit cost (epilogue / atomics) in k-block equivalents
        const double t = rounds * (kb + (sp > 1 ? 12.0 : 6.0)) * (w == 256 ? 1.0 : 0.6);
        if (t < best * 0.97) {
          best = t;
          bn = w;
          splits = sp;
        }
      }
    }
  }

  // Paired-CTA kernel (256 x 256 tile per CTA pair, half of B per CTA): same cost model, a pair
  // round does the work of two 256-wide rounds in about 1.7x the time of one.
  static const bool pair_off = [] {
    const char* e = std::getenv("CTDK_GEMM_1CTA");
    return e != nullptr && e[0] == '1';
  }();
  bool use_pair = false;
  if (!pair_off && M >= 256 && N >= 256) {
    double best1 = 1e300;
    {
      const int64_t tiles = m_blocks * ((N + bn - 1) / bn);
      const double rounds = static_cast<double>((tiles * splits + sms - 1) / sms);
      best1 = rounds * (static_cast<double>((k_blocks + splits - 1) / splits) + (splits > 1 ? 12.0 : 6.0)) *
              (bn == 256 ? 1.0 : (bn == 128 ? 0.6 : 0.4));
    }
    const int pairs = sms / 2;
    const int64_t tiles2 = ((M + 255) / 256) * ((N + 255) / 256);
    const int max_splits = static_cast<int>(k_blocks / 16 < 1 ? 1 : (k_blocks / 16 > 32 ? 32 : k_blocks / 16));
    double bestp = 1e300;
    int sp_best = 1;
    for (int sp = 1; sp <= max_splits; ++sp) {
      if (sp > 1 && tiles2 >= 2 * pairs) break;
      const double rounds = static_cast<double>((tiles2 * sp + pairs - 1) / pairs);
      const double t = rounds * (static_cast<double>((k_blocks + sp - 1) / sp) + (sp > 1 ? 12.0 : 6.0)) * 1.7;
      if (t < bestp * 0.97) {
        bestp = t;
        sp_best = sp;
      }
    }
    // compare per-SM-round costs: a one-CTA round covers `sms` tiles, a pair round `pairs` tiles
    if (bestp < best1 * 2.0 * 0.98) {
      use_pair = true;
      splits = sp_best;
      bn = 256;
    }
  }

  if (t_kblock_limit > 0) {
    int64_t need = (k_blocks + t_kblock_limit - 1) / t_kblock_limit;
    if (need > 64) need = 64;
    if (need > splits) splits = static_cast<int>(need);
  }

  CUtensorMap ta, tb;
  int rc;
  // The pair kernel takes an MN-major operand whose contiguous extent is a multiple of 32 through
  // a 3-D map {32 columns, K rows, extent / 32 column groups}: one {32, 32, 4} box per k-block
  // instead of four {32, 32} boxes (issuing a TMA copy costs the producer thread ~140 cycles).
  auto make_map3 = [&](CUtensorMap* m, const float* base, int64_t extent, int64_t ld) {
    const uint64_t dims[3] = {32u, static_cast<uint64_t>(K), static_cast<uint64_t>(extent / 32)};
    const uint64_t strides[2] = {static_cast<uint64_t>(ld) * sizeof(float), 128u};
    const uint32_t box[3] = {32u, 32u, 4u};
    return encode_tensor_map(m, base, 3, dims, strides, box, true);
  };
  const bool a3d = use_pair && a_mn && (M % 32 == 0);
  const bool b3d = use_pair && b_mn && (N % 32 == 0);
  if (a3d) rc = make_map3(&ta, A, M, lda);
  else if (a_mn) rc = make_map(&ta, A, M, K, lda, BK, true, false);
  else rc = make_map(&ta, A, K, M, lda, BM, false, false);
  if (rc != CTDK_OK) return rc;
  if (b3d) rc = make_map3(&tb, B, N, ldb);
  else if (b_mn) rc = make_map(&tb, B, N, K, ldb, BK, true, false);
  else rc = make_map(&tb, B, K, N, ldb, use_pair ? 128 : bn, false, false);
  if (rc != CTDK_OK) return rc;

  if (use_pair) {
    int* st = device_status_word();
    if (st == nullptr) return fail(CTDK_ELAUNCH, "gemm: no status word");
    const int vec = (a16(Cp) && (ldc & 3) == 0 && (aux == nullptr || a16(aux))) ? 1 : 0;
    if (splits > 1 && epilogue != CTDK_EPI_ACCUMULATE) {
      cudaError_t e = cudaMemset2DAsync(Cp, static_cast<size_t>(ldc) * sizeof(float), 0,
                                        static_cast<size_t>(N) * sizeof(float), static_cast<size_t>(M), stream);
      if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "gemm: memset failed: %s", cudaGetErrorString(e));
    }
    // Output through TMA (coalesced, off the load/store pipe): plain store, or an fp32 add at L2
    // for accumulation and for split-K partial tiles. The residual epilogue reads a second
    // matrix and keeps the direct path.
    int tma_out = 0;
    CUtensorMap tc = ta;
    if (vec && epilogue != CTDK_EPI_RESIDUAL) {
      tma_out = (epilogue == CTDK_EPI_ACCUMULATE || splits > 1) ? 2 : 1;
      rc = make_map(&tc, Cp, N, M, ldc, 32, false, true);
      if (rc != CTDK_OK) return rc;
    }
    return gemm_tcgen05_2cta(ta, tb, tc, a_mn, b_mn, a3d, b3d, tma_out, Cp, aux, ldc, static_cast<int>(M),
                             static_cast<int>(N), static_cast<int>(K), epilogue, vec, splits, st, stream);
  }

  GemmArgs args;
  args.C = Cp;
  args.aux = aux;
  args.ldc = ldc;
  args.M = static_cast<int>(M);
  args.N = static_cast<int>(N);
  args.K = static_cast<int>(K);
  args.epilogue = epilogue;
  args.vec_ok = (a16(Cp) && (ldc & 3) == 0 && (aux == nullptr || a16(aux))) ? 1 : 0;
  args.splits = splits;
  args.status = device_status_word();
  if (args.status == nullptr) return fail(CTDK_ELAUNCH, "gemm: no status word");
  if (splits > 1 && epilogue != CTDK_EPI_ACCUMULATE) {
    cudaError_t e = cudaMemset2DAsync(Cp, static_cast<size_t>(ldc) * sizeof(float), 0,
                                      static_cast<size_t>(N) * sizeof(float),
                                      static_cast<size_t>(M), stream);
    if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "gemm: memset failed: %s", cudaGetErrorString(e));
  }

  switch (bn) {
    case 64: return dispatch_major<64>(a_mn, b_mn, ta, tb, args, stream);
    case 128: return dispatch_major<128>(a_mn, b_mn, ta, tb, args, stream);
    default: return dispatch_major<256>(a_mn, b_mn, ta, tb, args, stream);
  }
}

// Near-fp32 GEMM (3xTF32 split). Returns 1 (not eligible) until the split kernel is built,
// so the caller computes the exact fp32 result with the SIMT kernel.
int gemm_3xtf32(const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t, int64_t,
                int64_t, int, int, int, const float*, cudaStream_t) {
  return 1;
}

}  // namespace ctdk
