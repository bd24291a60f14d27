// Causal grouped-query attention on the tcgen05 tensor cores (forward).
//
// One CTA per (128-query tile, head, batch), 6 warps:
//   warp 0    TMA producer: Q once, then K/V tiles of 128 keys through a small ring, read in
//             place from the packed qkv[B, T, (H+2Hk)*D] buffer through 3-D tensor maps (rows past
//             the end of a sequence are zero-filled by TMA bounds checking).
//   warp 1    MMA issuer: S = Q K^T (A, B from shared memory, TF32) into one of two tensor-memory
//             score buffers; O_j = P V with P read from tensor memory (written there by the
//             softmax warps) and V as an MN-major shared-memory operand.
//   warps 2-5 softmax: one query row per thread (no shuffles): running max / sum in the log2
//             domain, P written back over S with tcgen05.st, per-tile P V results folded into
//             register accumulators with the usual rescaling, final normalisation and stores.
// S for tile j+1 is issued before the softmax of tile j has finished, so tensor core and
// softmax overlap. Every mbarrier wait is bounded.
//
// Replaces, like attention.cu, the bmm -> scale -> causal mask -> softmax -> bmm chain of the
// reference's Attention::forward_train (emberlm include/ctd/nn/attention.h:123-141).
#include <cfloat>
#include <cstdlib>

#include "common.cuh"

namespace ctdk {
namespace {

constexpr int TQ = 128;   // query rows per CTA = tensor-memory lanes
constexpr int TK = 128;   // keys per tile
constexpr int kChunk = TQ * 128;  // bytes of one {32 floats x 128 rows} box
constexpr float kLn2f = 0.6931471805599453f;

// NB = number of score / PV buffers in tensor memory and of K/V stages in shared memory.
// NB == 1 keeps a CTA small enough (<= 113 KB, 256 tensor-memory columns) for two CTAs per
// SM at D = 64, so one CTA's softmax overlaps the other's MMAs; NB == 2 overlaps inside one CTA.
template <int D, int NB>
struct FwdCfg {
  static constexpr int kTileBytes = TK * D * 4;  // one K or V tile (= one Q tile)
  static constexpr int kSmem = kTileBytes * (1 + 2 * NB) + 1024 + 256;
  static constexpr uint32_t kTmemCols = (NB == 1) ? 256 : 512;  // NB x (128 score + D PV columns)
  static constexpr int kCtasPerSm = (NB == 1 && D == 64) ? 2 : 1;
};

__device__ __forceinline__ uint32_t idesc_tf32(bool b_mn, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(TQ >> 4) << 24);
}

__device__ __forceinline__ uint32_t f2tf32_bits(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct FwdArgs {
  float* out;
  float* lse;
  int T, H, Hk;
  float scale_log2;
  int* status;
};

template <int D, int NB>
__global__ void __launch_bounds__(192, FwdCfg<D, NB>::kCtasPerSm)
    attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_k,   // 16-byte-chunk swizzle (Q, K)
                       const __grid_constant__ CUtensorMap tm_v,   // 32-byte-chunk swizzle (V)
                       const FwdArgs args) {
  using C = FwdCfg<D, NB>;
  constexpr int NC = D / 32;  // 32-float chunks per row
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + C::kTileBytes;            // [NB] tiles
  unsigned char* v_s = k_s + NB * C::kTileBytes;       // [NB] tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + NB * C::kTileBytes);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2]
  uint64_t* p_ready = bars + 11;      // [2]
  uint64_t* pv_full = bars + 13;      // [2]
  uint64_t* pv_empty = bars + 15;     // [2]
  uint64_t* final_bar = bars + 17;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi = gridDim.x - 1 - blockIdx.x;  // heaviest tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (args.H / args.Hk);
  const int n_tiles = qi + 1;
  const int q0 = qi * TQ;
  const int col_q = h * D, col_k = (args.H + hk) * D, col_v = (args.H + args.Hk + hk) * D;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 128);
      mbar_init(&pv_full[i], 1);
      mbar_init(&pv_empty[i], 128);
    }
    mbar_init(final_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tm_s = [&](int i) { return tmem_base + static_cast<uint32_t>(i * 128); };
  auto tm_pv = [&](int i) { return tmem_base + static_cast<uint32_t>(NB * 128 + i * D); };

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, C::kTileBytes);
#pragma unroll
      for (int c = 0; c < NC; ++c) tma_load_3d(q_s + c * kChunk, &tm_k, q_full, col_q + 32 * c, q0, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % NB;
        const uint32_t ph = static_cast<uint32_t>(j / NB) & 1u;
        if (!mbar_wait_bounded(&k_empty[s], ph ^ 1u, args.status, 11)) break;
        mbar_expect_tx(&k_full[s], C::kTileBytes);
#pragma unroll
        for (int c = 0; c < NC; ++c)
          tma_load_3d(k_s + s * C::kTileBytes + c * kChunk, &tm_k, &k_full[s], col_k + 32 * c, j * TK, b);
        if (!mbar_wait_bounded(&v_empty[s], ph ^ 1u, args.status, 12)) break;
        mbar_expect_tx(&v_full[s], C::kTileBytes);
#pragma unroll
        for (int c = 0; c < NC; ++c)
          tma_load_3d(v_s + s * C::kTileBytes + c * kChunk, &tm_v, &v_full[s], col_v + 32 * c, j * TK, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      const uint32_t idesc_s = idesc_tf32(false, TK);
      const uint32_t idesc_pv = idesc_tf32(true, D);
      bool ok = mbar_wait_bounded(q_full, 0, args.status, 21);
      tc_fence_after();
      const uint32_t q_addr = smem_u32(q_s);
      auto issue_s = [&](int j) {
        const int s = j % NB;
        const uint32_t ph = static_cast<uint32_t>(j / NB) & 1u;
        if (!mbar_wait_bounded(&k_full[s], ph, args.status, 22)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(k_s + s * C::kTileBytes);
#pragma unroll
        for (int ks = 0; ks < D / 8; ++ks) {
          const uint32_t off = static_cast<uint32_t>((ks >> 2) * kChunk + (ks & 3) * 32);
          umma_tf32(tm_s(s), make_smem_desc(q_addr + off, 16, 1024, kLayoutSw128),
                    make_smem_desc(k_addr + off, 16, 1024, kLayoutSw128), idesc_s, ks != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[s]);
        return true;
      };
      auto issue_pv = [&](int jj) {
        const int s = jj % NB;
        const uint32_t ph = static_cast<uint32_t>(jj / NB) & 1u;
        if (!mbar_wait_bounded(&p_ready[s], ph, args.status, 23)) return false;
        if (!mbar_wait_bounded(&v_full[s], ph, args.status, 24)) return false;
        if (!mbar_wait_bounded(&pv_empty[s], ph ^ 1u, args.status, 25)) return false;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(v_s + s * C::kTileBytes);
#pragma unroll
        for (int ks = 0; ks < TK / 8; ++ks) {
          // A: 8 probability columns of tensor memory; B: 8 key rows (two 4-row swizzle
          // groups, SBO 512) of every 32-float chunk of V (chunks kChunk apart, LBO).
          umma_tf32_ta(tm_pv(s), tm_s(s) + static_cast<uint32_t>(ks * 8),
                       make_smem_desc(v_addr + ks * 1024, kChunk, 512, kLayoutSw128Base32), idesc_pv,
                       ks != 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[s]);
        umma_commit(&pv_full[s]);
        return true;
      };
      // With two buffers S(j) is issued before P(j-1) is awaited, so it overlaps the softmax of
      // tile j-1; with one buffer P(j-1) lives where S(j) goes, so P V comes first.
      for (int j = 0; j <= n_tiles && ok; ++j) {
        if (NB == 2 && j < n_tiles) ok = issue_s(j);
        if (ok && j >= 1) ok = issue_pv(j - 1);
        if (NB == 1 && ok && j < n_tiles) ok = issue_s(j);
      }
      umma_commit(final_bar);
      mbar_wait_bounded(final_bar, 0, args.status, 26);
    }
    __syncwarp();
  } else {
    // ------------------------------- softmax / output -------------------------------
    const int qd = warp & 3;                 // tensor-memory lane quarter of this warp
    const int row = q0 + qd * 32 + lane;     // query position inside the sequence
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sc = args.scale_log2;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.0f;
    float m_run = -FLT_MAX, l_run = 0.0f, c_prev = 0.0f;
    bool ok = true;
    auto fold_pv = [&](int jj) {
      const int s = jj % NB;
      if (!mbar_wait_bounded(&pv_full[s], static_cast<uint32_t>(jj / NB) & 1u, args.status, 32)) return false;
      tc_fence_after();
#pragma unroll
      for (int hf = 0; hf < D / 64; ++hf) {
        float v[64];
        tmem_ld_32x64_nowait(tm_pv(s) + lane_off + hf * 64, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 64; ++i) o[hf * 64 + i] = o[hf * 64 + i] * c_prev + v[i];
      }
      tc_fence_before();
      mbar_arrive(&pv_empty[s]);
      return true;
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % NB;
      if (!mbar_wait_bounded(&s_full[s], static_cast<uint32_t>(j / NB) & 1u, args.status, 31)) { ok = false; break; }
      tc_fence_after();
      const uint32_t ts = tm_s(s) + lane_off;
      // keys of this tile this row may attend to (causal): all 128 except on the diagonal tile
      const int n_valid = (j == qi) ? (row - j * TK + 1) : TK;
      float a[64];
      // pass 1: row maximum; the second half stays in registers for pass 2
      tmem_ld_32x64_nowait(ts, a);
      tmem_wait_ld();
      float mx = -FLT_MAX;
#pragma unroll
      for (int i = 0; i < 64; ++i) mx = fmaxf(mx, (i < n_valid) ? a[i] : -FLT_MAX);
      tmem_ld_32x64_nowait(ts + 64, a);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 64; ++i) mx = fmaxf(mx, (64 + i < n_valid) ? a[i] : -FLT_MAX);
      const float m_new = fmaxf(m_run, mx * sc);
      // pass 2: probabilities (rounded to TF32) back into tensor memory
      float sum = 0.0f;
      {
        uint32_t* pb = reinterpret_cast<uint32_t*>(a);
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float p = (64 + i < n_valid) ? fast_exp2(a[i] * sc - m_new) : 0.0f;
          sum += p;
          pb[i] = f2tf32_bits(p);
        }
        tmem_st_32x64(ts + 64, *reinterpret_cast<uint32_t(*)[64]>(pb));
      }
      tmem_wait_st();  // the registers are reused by the next load
      tmem_ld_32x64_nowait(ts, a);
      tmem_wait_ld();
      {
        uint32_t* pb = reinterpret_cast<uint32_t*>(a);
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float p = (i < n_valid) ? fast_exp2(a[i] * sc - m_new) : 0.0f;
          sum += p;
          pb[i] = f2tf32_bits(p);
        }
        tmem_st_32x64(ts, *reinterpret_cast<uint32_t(*)[64]>(pb));
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_ready[s]);
      const float c_j = fast_exp2(m_run - m_new);
      l_run = l_run * c_j + sum;
      m_run = m_new;
      if (j >= 1) ok = fold_pv(j - 1);
      c_prev = c_j;
    }
    if (ok && fold_pv(n_tiles - 1) && row < args.T) {
      const float inv = 1.0f / l_run;
      float* op = args.out + (static_cast<int64_t>(b) * args.T + row) * (static_cast<int64_t>(args.H) * D) +
                  static_cast<int64_t>(h) * D;
#pragma unroll
      for (int i = 0; i < D / 4; ++i)
        reinterpret_cast<float4*>(op)[i] =
            make_float4(o[4 * i] * inv, o[4 * i + 1] * inv, o[4 * i + 2] * inv, o[4 * i + 3] * inv);
      args.lse[(static_cast<int64_t>(b) * args.H + h) * args.T + row] = (m_run + log2f(l_run)) * kLn2f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

int make_qkv_maps(const float* qkv, int64_t B, int64_t T, int RS, CUtensorMap* tm_k, CUtensorMap* tm_v) {
  const uint64_t dims[3] = {static_cast<uint64_t>(RS), static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
  const uint64_t strides[2] = {static_cast<uint64_t>(RS) * 4, static_cast<uint64_t>(T) * RS * 4};
  const uint32_t box[3] = {32u, 128u, 1u};
  int rc = encode_tensor_map(tm_k, qkv, 3, dims, strides, box, false);
  if (rc != CTDK_OK) return rc;
  return encode_tensor_map(tm_v, qkv, 3, dims, strides, box, true);
}

template <int D, int NB>
int launch_fwd(const CUtensorMap& tk, const CUtensorMap& tv, const FwdArgs& a, dim3 grid, cudaStream_t s) {
  using C = FwdCfg<D, NB>;
  cudaError_t e =
      cudaFuncSetAttribute(attn_fwd_tc_kernel<D, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "attn_fwd(tcgen05): shared memory opt-in failed: %s", cudaGetErrorString(e));
  attn_fwd_tc_kernel<D, NB><<<grid, 192, C::kSmem, s>>>(tk, tv, a);
  return check_launch("ctdk_attn_fwd(tcgen05)");
}

}  // namespace

// CTDK_ATTN_LEGACY=1 selects the mma.sync kernels of attention.cu (kept for comparison).
bool attn_use_legacy() {
  static const bool legacy = [] {
    const char* e = getenv("CTDK_ATTN_LEGACY");
    return e != nullptr && e[0] == '1';
  }();
  return legacy;
}

// Returns CTDK_OK after enqueueing, a negative status on error, or 1 when the shape is not
// eligible (the caller then uses the mma.sync kernel).
int attn_fwd_tcgen05(const float* qkv, float* out, float* lse, int64_t B, int64_t T, int H, int Hk, int D,
                     cudaStream_t stream) {
  const int RS = (H + 2 * Hk) * D;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) return 1;
  CUtensorMap tk, tv;
  int rc = make_qkv_maps(qkv, B, T, RS, &tk, &tv);
  if (rc != CTDK_OK) return rc;
  FwdArgs a;
  a.out = out;
  a.lse = lse;
  a.T = static_cast<int>(T);
  a.H = H;
  a.Hk = Hk;
  a.scale_log2 = (1.0f / sqrtf(static_cast<float>(D))) * 1.4426950408889634f;
  a.status = device_status_word();
  if (a.status == nullptr) return fail(CTDK_ELAUNCH, "attn_fwd(tcgen05): no status word");
  dim3 grid(static_cast<unsigned>((T + TQ - 1) / TQ), static_cast<unsigned>(H), static_cast<unsigned>(B));
  return D == 64 ? launch_fwd<64, 1>(tk, tv, a, grid, stream) : launch_fwd<128, 1>(tk, tv, a, grid, stream);
}

}  // namespace ctdk
