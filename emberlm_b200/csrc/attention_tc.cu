// Causal grouped-query attention on the tcgen05 tensor cores (forward).
//
// Persistent CTAs (two per SM at D = 64), each walking a list of (128-query tile, head, batch) items
// so that loads, score MMAs and the epilogue of consecutive items overlap. 6 warps:
//   warp 0    TMA producer: Q once, then K/V steps of 64 keys through two-stage rings, read in
//             place from the packed qkv[B, T, (H+2Hk)*D] buffer through 3-D tensor maps (rows past
//             the end of a sequence are zero-filled by TMA bounds checking).
//   warp 1    MMA issuer: S(j) = Q K(j)^T (A, B from shared memory, TF32) into one of two 64-column
//             score buffers in tensor memory; O += P(j) V(j) with P read from tensor memory
//             (written there by the softmax warps) and V as an MN-major shared-memory operand.
//             S(j+2) is queued right behind P V(j), so scores are always one step ahead.
//   warps 2-5 softmax: one query row per thread (no shuffles): maximum, exp2 and sum in the log2
//             domain with packed two-wide fp32 arithmetic, P written back over S with tcgen05.st.
//             O stays in tensor memory and is rescaled lazily (only when a row's maximum grew by
//             more than 2^8 since the last rescale), then normalised and stored at the end.
// Every mbarrier wait is bounded.
//
// Replaces, like attention.cu, the bmm -> scale -> causal mask -> softmax -> bmm chain of the
// reference's Attention::forward_train (emberlm include/ctd/nn/attention.h:123-141).
#include <cfloat>
#include <climits>
#include <cstdlib>

#include "common.cuh"

namespace ctdk {
namespace {

constexpr int TQ = 128;   // query rows per CTA = tensor-memory lanes
constexpr int TK = 64;    // keys per step
constexpr int kQChunk = TQ * 128;  // bytes of one {32 floats x 128 rows} box (Q)
constexpr int kKChunk = TK * 128;  // bytes of one {32 floats x 64 rows} box (K, V)
constexpr float kLn2f = 0.6931471805599453f;

// Per CTA: Q tile, two K and two V stages of 64 keys in shared memory; two 64-column score
// buffers and D output columns in tensor memory. At D = 64 that is 97 KB and 256 columns, so two
// CTAs share an SM.
template <int D>
struct FwdCfg {
  static constexpr int kQBytes = TQ * D * 4;
  static constexpr int kKBytes = TK * D * 4;     // one K or V stage
  static constexpr int kStageBytes = 4 * 2048;   // per softmax warp: 32 rows x 16 floats of output in transit
  static constexpr int kSmem = kQBytes + 4 * kKBytes + kStageBytes + 1024 + 256;
  static constexpr uint32_t kTmemCols = 256;     // 2 x 64 score + D output columns
  static constexpr int kCtasPerSm = (D == 64) ? 2 : 1;
};

__device__ __forceinline__ uint32_t idesc_tf32(bool b_mn, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(TQ >> 4) << 24);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Round-to-nearest (ties away) to TF32 as an integer add: the tensor core ignores the 13 low
// mantissa bits, so adding half a TF32 ulp to the bit pattern is cvt.rna.tf32.f32 without the
// conversion pipe.
__device__ __forceinline__ uint32_t tf32_rna_bits(float x) { return __float_as_uint(x) + 0x1000u; }


struct FwdArgs {
  float* out;
  float* lse;
  int T, H, Hk, B;
  int n_qtiles;   // ceil(T / 128)
  int n_items;    // n_qtiles * H * B
  float scale_log2;
  int* status;
};

// How far (log2 units) a row's running maximum may grow before the output accumulator in tensor
// memory is rescaled: probabilities stay below 2^8 relative to the reference point, far inside
// fp32 range, and most steps need no rescaling pass at all.
constexpr float kRescaleSlack = 8.0f;

// One work item = one (128-query tile, head, batch). Items are numbered batch-major so that the
// CTAs running at any moment work on two or three sequences whose Q/K/V (a few MB each) stay in
// L2 and are read from DRAM once; inside a sequence the heaviest query tile comes first and heads
// run fastest (the query heads of one key/value group sit side by side). CTA c takes items
// c, c + gridDim.x, ...
struct FwdItem {
  int qi, h, b, q0, n_steps;
};
__device__ __forceinline__ FwdItem fwd_item(const FwdArgs& a, int it) {
  FwdItem w;
  const int per_b = a.n_qtiles * a.H;
  w.b = it / per_b;
  const int r = it % per_b;
  w.qi = a.n_qtiles - 1 - r / a.H;
  w.h = r % a.H;
  w.q0 = w.qi * TQ;
  // key steps up to and including the diagonal, never past the end of the sequence
  w.n_steps = min((w.q0 + TQ) / TK, (a.T + TK - 1) / TK);
  return w;
}

template <int D>
__global__ void __launch_bounds__(192, FwdCfg<D>::kCtasPerSm)
    attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q,   // {32 x 128} boxes, 16-byte-chunk swizzle
                       const __grid_constant__ CUtensorMap tm_k,   // {32 x 64} boxes, 16-byte-chunk swizzle
                       const __grid_constant__ CUtensorMap tm_v,   // {32 x 64} boxes, 32-byte-chunk swizzle
                       const FwdArgs args) {
  using C = FwdCfg<D>;
  constexpr int NC = D / 32;  // 32-float chunks per row
  extern __shared__ unsigned char smem_raw[];
  pdl_launch();
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + C::kQBytes;          // [2] stages
  unsigned char* v_s = k_s + 2 * C::kKBytes;      // [2] stages
  unsigned char* o_stage = v_s + 2 * C::kKBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(o_stage + C::kStageBytes);
  uint64_t* q_full = bars;          // 1    one phase per item
  uint64_t* q_empty = bars + 1;     // 1    every score MMA of the item has read Q
  uint64_t* k_full = bars + 2;      // [2]  stage / phase by the running step count
  uint64_t* k_empty = bars + 4;     // [2]
  uint64_t* v_full = bars + 6;      // [2]
  uint64_t* v_empty = bars + 8;     // [2]
  uint64_t* s_full = bars + 10;     // [2]  S(g) is in tensor memory
  uint64_t* p_ready = bars + 12;    // [2]  P(g) has replaced S(g) (128 arrivals)
  uint64_t* pv_full = bars + 14;    // 1    O += P(g) V(g) has finished (one phase per step)
  uint64_t* o_full = bars + 15;     // 1    the item's last P V has finished (one phase per item)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 128);
    }
    mbar_init(pv_full, 1);
    mbar_init(o_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
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
  pdl_wait();   // inputs come from earlier kernels in the stream
  const uint32_t tm_o = tmem_base + 128u;
  auto tm_s = [&](uint32_t g) { return tmem_base + (g & 1u) * static_cast<uint32_t>(TK); };
  // g = running count of key steps over all items of this CTA: stage g & 1, phase (g >> 1) & 1.

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      uint32_t g0 = 0, n_it = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < args.n_items && ok; it += gridDim.x, ++n_it) {
        const FwdItem w = fwd_item(args, it);
        const int hk = w.h / (args.H / args.Hk);
        const int col_q = w.h * D, col_k = (args.H + hk) * D, col_v = (args.H + args.Hk + hk) * D;
        if (!mbar_wait_bounded(q_empty, (n_it & 1u) ^ 1u, args.status, 10)) break;
        mbar_expect_tx(q_full, C::kQBytes);
#pragma unroll
        for (int c = 0; c < NC; ++c) tma_load_3d(q_s + c * kQChunk, &tm_q, q_full, col_q + 32 * c, w.q0, w.b);
        auto load_k = [&](int j) {
          const uint32_t g = g0 + static_cast<uint32_t>(j), s = g & 1u;
          if (!mbar_wait_bounded(&k_empty[s], ((g >> 1) & 1u) ^ 1u, args.status, 11)) return false;
          mbar_expect_tx(&k_full[s], C::kKBytes);
#pragma unroll
          for (int c = 0; c < NC; ++c)
            tma_load_3d(k_s + s * C::kKBytes + c * kKChunk, &tm_k, &k_full[s], col_k + 32 * c, j * TK, w.b);
          return true;
        };
        auto load_v = [&](int j) {
          const uint32_t g = g0 + static_cast<uint32_t>(j), s = g & 1u;
          if (!mbar_wait_bounded(&v_empty[s], ((g >> 1) & 1u) ^ 1u, args.status, 12)) return false;
          mbar_expect_tx(&v_full[s], C::kKBytes);
#pragma unroll
          for (int c = 0; c < NC; ++c)
            tma_load_3d(v_s + s * C::kKBytes + c * kKChunk, &tm_v, &v_full[s], col_v + 32 * c, j * TK, w.b);
          return true;
        };
        // K runs one step ahead of V: the score MMA of step j+2 is queued right behind P V(j).
        ok = load_k(0);
        for (int j = 0; j < w.n_steps && ok; ++j) {
          if (j + 1 < w.n_steps) ok = load_k(j + 1);
          if (ok) ok = load_v(j);
        }
        g0 += static_cast<uint32_t>(w.n_steps);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    // The whole warp runs this role converged; one elected lane issues each MMA / commit.
    {
      const uint32_t idesc_s = idesc_tf32(false, TK);
      const uint32_t idesc_pv = idesc_tf32(true, D);
      const uint32_t k_base = smem_u32(k_s), v_base = smem_u32(v_s);
      const uint64_t qd_ = make_smem_desc(smem_u32(q_s), 16, 1024, kLayoutSw128);
      uint32_t g0 = 0, n_it = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < args.n_items && ok; it += gridDim.x, ++n_it) {
        const FwdItem w = fwd_item(args, it);
        auto issue_s = [&](int j) {
          const uint32_t g = g0 + static_cast<uint32_t>(j), s = g & 1u;
          {
            if (!mbar_wait_bounded_w(&k_full[s], (g >> 1) & 1u, args.status, 22)) return false;
          }
          tc_fence_after();
          const uint64_t kd = make_smem_desc(k_base + s * C::kKBytes, 16, 1024, kLayoutSw128);
          const uint32_t ts = tm_s(g);
#pragma unroll
          for (int ks = 0; ks < D / 8; ++ks)   // descriptor address field counts 16-byte units
            umma_tf32_w(ts, qd_ + (((ks >> 2) * kQChunk + (ks & 3) * 32) >> 4),
                        kd + (((ks >> 2) * kKChunk + (ks & 3) * 32) >> 4), idesc_s, ks != 0 ? 1u : 0u);
          umma_commit_w(&k_empty[s]);
          umma_commit_w(&s_full[s]);
          if (j == w.n_steps - 1) umma_commit_w(q_empty);   // the item's last use of Q
          return true;
        };
        {
          if (!mbar_wait_bounded_w(q_full, n_it & 1u, args.status, 21)) break;
        }
        tc_fence_after();
        // Tensor-pipe order: S(0) S(1) | PV(0) S(2) | PV(1) S(3) | ... S(j+2) reuses the columns
        // P(j) lives in; it is queued behind P V(j) on the in-order pipe.
        ok = issue_s(0);
        if (ok && w.n_steps > 1) ok = issue_s(1);
        for (int j = 0; j < w.n_steps && ok; ++j) {
          const uint32_t g = g0 + static_cast<uint32_t>(j), s = g & 1u, ph = (g >> 1) & 1u;
          {
            if (!mbar_wait_bounded_w(&p_ready[s], ph, args.status, 23)) { ok = false; break; }
          }
          {
            if (!mbar_wait_bounded_w(&v_full[s], ph, args.status, 24)) { ok = false; break; }
          }
          tc_fence_after();
          // A: 8 probability columns of tensor memory; B: 8 key rows (two 4-row swizzle
          // groups, SBO 512) of every 32-float chunk of V (chunks kKChunk apart, LBO).
          const uint64_t vd = make_smem_desc(v_base + s * C::kKBytes, kKChunk, 512, kLayoutSw128Base32);
          const uint32_t ts = tm_s(g);
          const uint32_t acc0 = j != 0 ? 1u : 0u;
#pragma unroll
          for (int ks = 0; ks < TK / 8; ++ks)
            umma_tf32_ta_w(tm_o, ts + static_cast<uint32_t>(ks * 8), vd + ((ks * 1024) >> 4), idesc_pv, ks != 0 ? 1u : acc0);
          umma_commit_w(&v_empty[s]);
          umma_commit_w(pv_full);
          if (j == w.n_steps - 1) umma_commit_w(o_full);
          if (j + 2 < w.n_steps) ok = issue_s(j + 2);
        }
        g0 += static_cast<uint32_t>(w.n_steps);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- softmax / output -------------------------------
    // One query row per thread, the 64 scores of a step in registers. The output accumulator
    // stays in tensor memory; it is rescaled (by this row's own thread) only when the running
    // maximum has grown by more than kRescaleSlack since the last rescale.
    const int qd = warp & 3;                 // tensor-memory lane quarter of this warp
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sc = args.scale_log2;
    const uint32_t to = tm_o + lane_off;
    uint32_t g0 = 0, n_done = 0;
    bool ok = true;
    for (int it = blockIdx.x; it < args.n_items && ok; it += gridDim.x, ++n_done) {
      const FwdItem w = fwd_item(args, it);
      const int row = w.q0 + qd * 32 + lane;   // query position inside the sequence
      float m_ref = 0.0f, l_run = 0.0f;
      for (int j = 0; j < w.n_steps && ok; ++j) {
        const uint32_t g = g0 + static_cast<uint32_t>(j), s = g & 1u;
        {
          if (!mbar_wait_bounded(&s_full[s], (g >> 1) & 1u, args.status, 31)) { ok = false; break; }
        }
        tc_fence_after();
        const uint32_t ts = tm_s(g) + lane_off;
        float a[64];
        tmem_ld_32x64_nowait(ts, a);
        tmem_wait_ld();
        if ((j + 1) * TK > w.q0 + 1) {  // a step that reaches past the first row's own position
          const int n_valid = row - j * TK + 1;   // may be <= 0: the whole step is in this row's future
#pragma unroll
          for (int i = 0; i < 64; ++i) a[i] = (i < n_valid) ? a[i] : -FLT_MAX;
        }
        float mx0 = fmax3(a[0], a[1], a[2]), mx1 = fmax3(a[3], a[4], a[5]);
#pragma unroll
        for (int i = 6; i < 62; i += 4) {
          mx0 = fmax3(mx0, a[i], a[i + 1]);
          mx1 = fmax3(mx1, a[i + 2], a[i + 3]);
        }
        const float mxs = fmax3(mx0, mx1, fmaxf(a[62], a[63])) * sc;
        float c = 1.0f;
        bool grow = false;
        if (j == 0) {
          m_ref = mxs;   // step 0 always holds key 0, which every row sees
        } else if (mxs > m_ref + kRescaleSlack) {
          c = fast_exp2(m_ref - mxs);
          m_ref = mxs;
          grow = true;
        }
        if (__any_sync(0xffffffffu, grow)) {
          // P V(g-1) must have landed before the accumulator is touched; P V(g) cannot start
          // before every row has arrived at p_ready below.
          if (!mbar_wait_bounded(pv_full, (g - 1u) & 1u, args.status, 32)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int hf = 0; hf < D / 64; ++hf) {
            float o[64];
            tmem_ld_32x64_nowait(to + hf * 64, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 64; i += 2) fmul2(o[i], o[i + 1], o[i], o[i + 1], c, c);
            tmem_st_32x64(to + hf * 64, *reinterpret_cast<uint32_t(*)[64]>(o));
            tmem_wait_st();
          }
          l_run *= c;
        }
        const float neg_m = -m_ref;
        float s0 = 0.0f, s1 = 0.0f;
        uint32_t* pb = reinterpret_cast<uint32_t*>(a);
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          float x0, x1;
          ffma2(x0, x1, a[i], a[i + 1], sc, sc, neg_m, neg_m);
          x0 = fast_exp2(x0);
          x1 = fast_exp2(x1);
          fadd2(s0, s1, s0, s1, x0, x1);
          pb[i] = tf32_rna_bits(x0);
          pb[i + 1] = tf32_rna_bits(x1);
        }
        tmem_st_32x64(ts, *reinterpret_cast<uint32_t(*)[64]>(pb));
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_ready[s]);
        l_run += s0 + s1;
      }
      g0 += static_cast<uint32_t>(w.n_steps);
      // The item's last P V, on a barrier of its own with one phase per item: pv_full cannot be
      // used here, because up to two of its phases may still be outstanding at this point and a
      // parity wait cannot tell them apart. The next item's first P V cannot start before these
      // threads have read O and arrived at its p_ready.
      {
        if (!ok || !mbar_wait_bounded(o_full, n_done & 1u, args.status, 33)) { ok = false; break; }
      }
      tc_fence_after();
      // Normalised output rows go through a small per-warp staging area (16 rows x 32 floats,
      // 128-byte rows with the 16-byte chunks XORed by the row number) so that each store
      // instruction writes 4 rows x 128 contiguous bytes instead of 32 rows x 16 bytes.
      const float inv = 1.0f / l_run;
      float* stg = reinterpret_cast<float*>(o_stage + qd * 2048);
      float* obase = args.out + (static_cast<int64_t>(w.b) * args.T + w.q0 + qd * 32) * (static_cast<int64_t>(args.H) * D) +
                     static_cast<int64_t>(w.h) * D;
      const int rows_left = args.T - (w.q0 + qd * 32);   // rows of this warp that exist
#pragma unroll
      for (int hf = 0; hf < D / 64; ++hf) {
        float o[64];
        tmem_ld_32x64_nowait(to + hf * 64, o);   // warp-collective: rows past T take part too
        tmem_wait_ld();
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const int ch2 = pass >> 1, rh = pass & 1;   // column half, row half
          if ((lane >> 4) == rh) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const int i = ch2 * 32 + c * 4;
              *reinterpret_cast<float4*>(stg + (lane & 15) * 32 + ((c ^ (lane & 7)) << 2)) =
                  make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
            }
          }
          __syncwarp();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int r = (lane >> 3) + 4 * k, ch = lane & 7;
            const float4 v = *reinterpret_cast<const float4*>(stg + r * 32 + ((ch ^ (r & 7)) << 2));
            if (rh * 16 + r < rows_left)
              *reinterpret_cast<float4*>(obase + static_cast<int64_t>(rh * 16 + r) * (args.H * D) + hf * 64 + ch2 * 32 +
                                         ch * 4) = v;
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      if (row < args.T)
        args.lse[(static_cast<int64_t>(w.b) * args.H + w.h) * args.T + row] = (m_ref + log2f(l_run)) * kLn2f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

int make_qkv_maps(const float* qkv, int64_t B, int64_t T, int RS, CUtensorMap* tm_q, CUtensorMap* tm_k,
                  CUtensorMap* tm_v) {
  const uint64_t dims[3] = {static_cast<uint64_t>(RS), static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
  const uint64_t strides[2] = {static_cast<uint64_t>(RS) * 4, static_cast<uint64_t>(T) * RS * 4};
  const uint32_t box_q[3] = {32u, static_cast<uint32_t>(TQ), 1u};
  const uint32_t box_k[3] = {32u, static_cast<uint32_t>(TK), 1u};
  int rc = encode_tensor_map(tm_q, qkv, 3, dims, strides, box_q, false);
  if (rc != CTDK_OK) return rc;
  rc = encode_tensor_map(tm_k, qkv, 3, dims, strides, box_k, false);
  if (rc != CTDK_OK) return rc;
  return encode_tensor_map(tm_v, qkv, 3, dims, strides, box_k, true);
}

template <int D>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdArgs& a, dim3 grid,
               cudaStream_t s) {
  using C = FwdCfg<D>;
  cudaError_t e =
      cudaFuncSetAttribute(attn_fwd_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "attn_fwd(tcgen05): shared memory opt-in failed: %s", cudaGetErrorString(e));
  launch_pdl(attn_fwd_tc_kernel<D>, dim3(grid), dim3(192), C::kSmem, s, tq, tk, tv, a);
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
  CUtensorMap tq, tk, tv;
  int rc = make_qkv_maps(qkv, B, T, RS, &tq, &tk, &tv);
  if (rc != CTDK_OK) return rc;
  FwdArgs a;
  a.out = out;
  a.lse = lse;
  a.T = static_cast<int>(T);
  a.H = H;
  a.Hk = Hk;
  a.B = static_cast<int>(B);
  a.n_qtiles = static_cast<int>((T + TQ - 1) / TQ);
  const int64_t items = static_cast<int64_t>(a.n_qtiles) * H * B;
  if (items > INT32_MAX) return 1;
  a.n_items = static_cast<int>(items);
  a.scale_log2 = (1.0f / sqrtf(static_cast<float>(D))) * 1.4426950408889634f;
  a.status = device_status_word();
  if (a.status == nullptr) return fail(CTDK_ELAUNCH, "attn_fwd(tcgen05): no status word");
  // persistent CTAs: as many as fit on the device at once
  const int64_t slots = static_cast<int64_t>(sm_budget()) * (D == 64 ? 2 : 1);
  dim3 grid(static_cast<unsigned>(items < slots ? items : slots));
  return D == 64 ? launch_fwd<64>(tq, tk, tv, a, grid, stream) : launch_fwd<128>(tq, tk, tv, a, grid, stream);
}

}  // namespace ctdk
