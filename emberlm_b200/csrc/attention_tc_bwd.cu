// Causal grouped-query attention backward on the tcgen05 tensor cores.
//
// Two kernels, as in the mma.sync version (attention.cu), after delta = rowsum(dO*O):
//   dQ kernel   one CTA per (128-query tile, head, batch), loop over key tiles:
//               S = Q K^T and dP = dO V^T into tensor memory, the compute warps turn them into
//               dS = P*(dP - delta)*scale in place (P = exp(S*scale - lse)), then
//               dQ += dS K with dS read from tensor memory and K as an MN-major operand;
//               dQ accumulates in tensor memory over all key tiles and is read once.
//   dK/dV kernel one CTA per (128-key tile, kv head, batch), loop over the query heads of the
//               group and the query tiles at or after the key tile (keys are the M dimension):
//               S^T = K Q^T, dP^T = V dO^T, P^T and dS^T in place, dV += P^T dO, dK += dS^T Q;
//               dK and dV accumulate in tensor memory, so the group sum (the reference's
//               repeat_kv_sum, emberlm src/ops/repeat_kv.cu:29-43) needs no atomics.
// Operands that are needed both K-major and MN-major (K in the dQ kernel; Q and dO in the dK/dV
// kernel) are loaded twice by TMA, once per swizzle layout. Every mbarrier wait is bounded.
#include <cfloat>
#include <cstdlib>

#include "common.cuh"

namespace ctdk {
namespace {

constexpr int TM = 128;  // rows of the CTA tile = tensor-memory lanes
constexpr float kLog2ef = 1.4426950408889634f;

__device__ __forceinline__ uint32_t idesc_b(bool b_mn, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(TM >> 4) << 24);
}
__device__ __forceinline__ uint32_t tf32_bits(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct BwdArgs {
  const float* lse;
  const float* delta;
  float* dqkv;
  int T, H, Hk;
  int B, n_qtiles;   // batch rows; ceil(T / 128)
  float scale;
  int* status;
};

// ----------------------------------------------------------------------------------------
// dQ kernel. TKB keys per tile, NB score buffers in tensor memory, STG K/V stages in shared memory
// (STG >= NB). QT: Q and dO live in tensor memory (copied there once by the compute warps through
// the K/V stage area, where they land), so S = Q K^T and dP = dO V^T read their left-hand operand
// at the math rate and the 128 KB they would occupy in shared memory hold a second K/V stage: the
// loads of tile j+1 run under the products of tile j instead of after them.
// ----------------------------------------------------------------------------------------
template <int D, int TKB, int NB, int STG, bool QT>
struct DqCfg {
  static constexpr int kRowTile = TM * D * 4;    // Q or dO
  static constexpr int kKeyTile = TKB * D * 4;   // K (either layout) or V
  static constexpr int kSmem = (QT ? 0 : 2 * kRowTile) + STG * 3 * kKeyTile + 1024 + 256;
  static constexpr int kCols = NB * 2 * TKB + D + (QT ? 2 * D : 0);
  static constexpr uint32_t kTmemCols = kCols <= 256 ? 256 : 512;
  static_assert(STG >= NB && STG <= 2 && NB <= 2, "barrier arrays hold two entries");
  static_assert(!QT || STG * 2 * kKeyTile >= 2 * kRowTile, "the K-major and MN-major K stages are the landing area of Q and dO");
  static_assert(kCols <= 512, "tensor memory");
};

template <int D, int TKB, int NB, int STG, bool QT>
__global__ void __launch_bounds__(320, 1)
    attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tm_q,    // qkv, box 128 rows, K-major
                          const __grid_constant__ CUtensorMap tm_do,   // dout, box 128 rows, K-major
                          const __grid_constant__ CUtensorMap tm_kk,   // qkv, box TKB rows, K-major
                          const __grid_constant__ CUtensorMap tm_km,   // qkv, box TKB rows, MN-major
                          const BwdArgs args) {
  using C = DqCfg<D, TKB, NB, STG, QT>;
  constexpr int NC = D / 32;
  constexpr int kRowChunk = TM * 128, kKeyChunk = TKB * 128;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* kk_s = smem + (QT ? 0 : 2 * C::kRowTile);   // [STG]
  unsigned char* km_s = kk_s + STG * C::kKeyTile;            // [STG]
  unsigned char* v_s = km_s + STG * C::kKeyTile;             // [STG]
  unsigned char* q_s = QT ? kk_s : smem;                     // QT: Q and dO only land here on their way to tensor memory
  unsigned char* do_s = q_s + C::kRowTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + STG * C::kKeyTile);
  uint64_t* q_full = bars;          // 1 (Q and dO)
  uint64_t* kv_full = bars + 1;     // [2] K (K-major) and V
  uint64_t* kv_empty = bars + 3;    // [2]
  uint64_t* km_full = bars + 5;     // [2] K (MN-major)
  uint64_t* km_empty = bars + 7;    // [2]
  uint64_t* sdp_full = bars + 9;    // [2]
  uint64_t* ds_ready = bars + 11;   // [2] 256 arrivals
  uint64_t* dq_full = bars + 13;    // 1
  uint64_t* qdo_ready = bars + 14;  // 1    QT: Q and dO have been copied to tensor memory (256 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // One-dimensional grid, longest items first: CTAs start in index order, so all tiles with the most
  // key steps (the last query tile of every head and sequence) run before any shorter one.
  const int hb = args.H * args.B;
  const int qi = args.n_qtiles - 1 - static_cast<int>(blockIdx.x) / hb;
  const int h = (static_cast<int>(blockIdx.x) % hb) % args.H, b = (static_cast<int>(blockIdx.x) % hb) / args.H;
  const int hk = h / (args.H / args.Hk);
  const int q0 = qi * TM;
  const int last_key = min(q0 + TM, args.T) - 1;
  const int n_tiles = last_key / TKB + 1;
  const int col_q = h * D, col_k = (args.H + hk) * D, col_v = (args.H + args.Hk + hk) * D;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&km_full[i], 1);
      mbar_init(&km_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
      mbar_init(&ds_ready[i], 256);
    }
    mbar_init(dq_full, 1);
    mbar_init(qdo_ready, 256);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_kk);
    tma_prefetch_desc(&tm_km);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tm_s = [&](int i) { return tmem_base + static_cast<uint32_t>(i * 2 * TKB); };          // S, later dS
  auto tm_dp = [&](int i) { return tmem_base + static_cast<uint32_t>(i * 2 * TKB + TKB); };   // dP
  const uint32_t tm_dq = tmem_base + static_cast<uint32_t>(NB * 2 * TKB);
  const uint32_t tm_qa = tm_dq + static_cast<uint32_t>(D), tm_doa = tm_qa + static_cast<uint32_t>(D);   // QT only

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * C::kRowTile);
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        tma_load_3d(q_s + c * kRowChunk, &tm_q, q_full, col_q + 32 * c, q0, b);
        tma_load_3d(do_s + c * kRowChunk, &tm_do, q_full, col_q + 32 * c, q0, b);
      }
      // QT: the K/V stages are where Q and dO landed, so those have to be in tensor memory first
      const bool moved = !QT || mbar_wait_bounded(qdo_ready, 0, args.status, 40);
      for (int j = 0; j < n_tiles && moved; ++j) {
        const int s = j % STG;
        const uint32_t ph = static_cast<uint32_t>(j / STG) & 1u;
        if (!mbar_wait_bounded(&kv_empty[s], ph ^ 1u, args.status, 41)) break;
        mbar_expect_tx(&kv_full[s], 2 * C::kKeyTile);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          tma_load_3d(kk_s + s * C::kKeyTile + c * kKeyChunk, &tm_kk, &kv_full[s], col_k + 32 * c, j * TKB, b);
          tma_load_3d(v_s + s * C::kKeyTile + c * kKeyChunk, &tm_kk, &kv_full[s], col_v + 32 * c, j * TKB, b);
        }
        if (!mbar_wait_bounded(&km_empty[s], ph ^ 1u, args.status, 42)) break;
        mbar_expect_tx(&km_full[s], C::kKeyTile);
#pragma unroll
        for (int c = 0; c < NC; ++c)
          tma_load_3d(km_s + s * C::kKeyTile + c * kKeyChunk, &tm_km, &km_full[s], col_k + 32 * c, j * TKB, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // The whole warp runs this role converged; one elected lane issues each MMA / commit (issued
    // from inside a one-lane branch an MMA costs the thread ~80 cycles, more than its pipe time).
    const uint32_t idesc_s = idesc_b(false, TKB);
    const uint32_t idesc_dq = idesc_b(true, D);
    bool ok = mbar_wait_bounded_w(QT ? qdo_ready : q_full, 0, args.status, 43);
    tc_fence_after();
    const uint64_t qd = make_smem_desc(smem_u32(q_s), 16, 1024, kLayoutSw128);     // unused with QT
    const uint64_t dod = make_smem_desc(smem_u32(do_s), 16, 1024, kLayoutSw128);
    auto issue_sdp = [&](int j) {
      const int s = j % STG, sb = j % NB;   // shared-memory stage, score buffer
      if (!mbar_wait_bounded_w(&kv_full[s], static_cast<uint32_t>(j / STG) & 1u, args.status, 44)) return false;
      tc_fence_after();
      const uint64_t kd = make_smem_desc(smem_u32(kk_s + s * C::kKeyTile), 16, 1024, kLayoutSw128);
      const uint64_t vd = make_smem_desc(smem_u32(v_s + s * C::kKeyTile), 16, 1024, kLayoutSw128);
      const uint32_t ts = tm_s(sb), tp = tm_dp(sb);
#pragma unroll
      for (int ks = 0; ks < D / 8; ++ks) {
        const uint64_t bd = kd + static_cast<uint64_t>(((ks >> 2) * kKeyChunk + (ks & 3) * 32) >> 4);
        if (QT) umma_tf32_ta_w(ts, tm_qa + static_cast<uint32_t>(ks * 8), bd, idesc_s, ks != 0 ? 1u : 0u);
        else umma_tf32_w(ts, qd + static_cast<uint64_t>(((ks >> 2) * kRowChunk + (ks & 3) * 32) >> 4), bd, idesc_s, ks != 0 ? 1u : 0u);
      }
#pragma unroll
      for (int ks = 0; ks < D / 8; ++ks) {
        const uint64_t bd = vd + static_cast<uint64_t>(((ks >> 2) * kKeyChunk + (ks & 3) * 32) >> 4);
        if (QT) umma_tf32_ta_w(tp, tm_doa + static_cast<uint32_t>(ks * 8), bd, idesc_s, ks != 0 ? 1u : 0u);
        else umma_tf32_w(tp, dod + static_cast<uint64_t>(((ks >> 2) * kRowChunk + (ks & 3) * 32) >> 4), bd, idesc_s, ks != 0 ? 1u : 0u);
      }
      umma_commit_w(&kv_empty[s]);
      umma_commit_w(&sdp_full[sb]);
      return true;
    };
    auto issue_dq = [&](int jj) {
      const int s = jj % STG, sb = jj % NB;
      if (!mbar_wait_bounded_w(&ds_ready[sb], static_cast<uint32_t>(jj / NB) & 1u, args.status, 45)) return false;
      if (!mbar_wait_bounded_w(&km_full[s], static_cast<uint32_t>(jj / STG) & 1u, args.status, 46)) return false;
      tc_fence_after();
      const uint64_t kmd = make_smem_desc(smem_u32(km_s + s * C::kKeyTile), kKeyChunk, 512, kLayoutSw128Base32);
      const uint32_t ts = tm_s(sb);
#pragma unroll
      for (int ks = 0; ks < TKB / 8; ++ks)
        umma_tf32_ta_w(tm_dq, ts + static_cast<uint32_t>(ks * 8), kmd + static_cast<uint64_t>((ks * 1024) >> 4), idesc_dq,
                       (jj != 0 || ks != 0) ? 1u : 0u);
      umma_commit_w(&km_empty[s]);
      return true;
    };
    for (int j = 0; j <= n_tiles && ok; ++j) {
      if (NB == 2 && j < n_tiles) ok = issue_sdp(j);
      if (ok && j >= 1) ok = issue_dq(j - 1);
      if (NB == 1 && ok && j < n_tiles) ok = issue_sdp(j);
    }
    umma_commit_w(dq_full);
    __syncwarp();
  } else {
    // 8 compute warps: warp pair (w, w+4) shares a lane quarter, each takes half of the keys.
    const int cw = warp - 2;
    const int qd = warp & 3, half = cw >> 2;
    const int row = q0 + qd * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const int64_t lbase = (static_cast<int64_t>(b) * args.H + h) * args.T;
    const bool row_ok = row < args.T;
    const float lse2 = row_ok ? args.lse[lbase + row] * kLog2ef : FLT_MAX;
    const float dl = row_ok ? args.delta[lbase + row] : 0.0f;
    const float sc2 = args.scale * kLog2ef;
    constexpr int HC = TKB / 2;  // columns per thread and tile
    bool ok = true;
    if (QT) {
      // the first warp of a lane quarter moves its rows of Q, the second its rows of dO: shared memory
      // (16-byte pieces XORed with the row number inside each 128-byte chunk row) -> tensor memory
      ok = mbar_wait_bounded(q_full, 0, args.status, 49);
      if (ok) {
        const int r = qd * 32 + lane;
        const unsigned char* src = half == 0 ? q_s : do_s;
        const uint32_t dst = (half == 0 ? tm_qa : tm_doa) + lane_off;
#pragma unroll
        for (int chunk = 0; chunk < NC; ++chunk) {
          uint32_t vb[32];
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const uint4 x = *reinterpret_cast<const uint4*>(src + chunk * kRowChunk + r * 128 + ((jj ^ (r & 7)) << 4));
            vb[4 * jj] = x.x;
            vb[4 * jj + 1] = x.y;
            vb[4 * jj + 2] = x.z;
            vb[4 * jj + 3] = x.w;
          }
          tmem_st_32x32(dst + static_cast<uint32_t>(chunk * 32), vb);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(qdo_ready);
      }
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % NB;
      if (!mbar_wait_bounded(&sdp_full[s], static_cast<uint32_t>(j / NB) & 1u, args.status, 47)) { ok = false; break; }
      tc_fence_after();
      const int key0 = j * TKB + half * HC;
#pragma unroll
      for (int c = 0; c < HC / 32; ++c) {
        float sv[32], dv[32];
        uint32_t ob[32];
        tmem_ld_32x32(tm_s(s) + lane_off + half * HC + c * 32, sv);
        tmem_ld_32x32(tm_dp(s) + lane_off + half * HC + c * 32, dv);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float p = (key0 + c * 32 + i > row) ? 0.0f : ex2(sv[i] * sc2 - lse2);
          ob[i] = tf32_bits(p * (dv[i] - dl) * args.scale);
        }
        tmem_st_32x32(tm_s(s) + lane_off + half * HC + c * 32, ob);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&ds_ready[s]);
    }
    if (ok && mbar_wait_bounded(dq_full, 0, args.status, 48)) {
      tc_fence_after();
      const int64_t RS = static_cast<int64_t>(args.H + 2 * args.Hk) * D;
      float* dst = args.dqkv + (static_cast<int64_t>(b) * args.T + row) * RS + static_cast<int64_t>(h) * D;
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        float v[32];
        const int col = half * (D / 2) + c * 32;
        tmem_ld_32x32(tm_dq + lane_off + col, v);
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            reinterpret_cast<float4*>(dst + col)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
        __syncwarp();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

int map3(CUtensorMap* m, const float* base, int64_t inner, int64_t T, int64_t B, int rows, bool atom32) {
  const uint64_t dims[3] = {static_cast<uint64_t>(inner), static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
  const uint64_t strides[2] = {static_cast<uint64_t>(inner) * 4, static_cast<uint64_t>(T) * inner * 4};
  const uint32_t box[3] = {32u, static_cast<uint32_t>(rows), 1u};
  return encode_tensor_map(m, base, 3, dims, strides, box, atom32);
}

template <int D, int TKB, int NB, int STG, bool QT>
int launch_dq(const float* qkv, const float* dout, const BwdArgs& a, int64_t B, cudaStream_t s) {
  using C = DqCfg<D, TKB, NB, STG, QT>;
  const int RS = (a.H + 2 * a.Hk) * D;
  CUtensorMap tq, tdo, tkk, tkm;
  int rc = map3(&tq, qkv, RS, a.T, B, TM, false);
  if (rc == CTDK_OK) rc = map3(&tdo, dout, static_cast<int64_t>(a.H) * D, a.T, B, TM, false);
  if (rc == CTDK_OK) rc = map3(&tkk, qkv, RS, a.T, B, TKB, false);
  if (rc == CTDK_OK) rc = map3(&tkm, qkv, RS, a.T, B, TKB, true);
  if (rc != CTDK_OK) return rc;
  auto* kern = attn_bwd_dq_tc_kernel<D, TKB, NB, STG, QT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "attn_bwd dq(tcgen05): shared memory opt-in failed: %s", cudaGetErrorString(e));
  dim3 grid(static_cast<unsigned>(static_cast<int64_t>(a.n_qtiles) * a.H * B));
  kern<<<grid, 320, C::kSmem, s>>>(tq, tdo, tkk, tkm, a);
  return check_launch("ctdk_attn_bwd(dq, tcgen05)");
}

}  // namespace

// Head size 64: persistent kernels with the left-hand operands in tensor memory (attention_tc_bwd64.cu).
int attn_bwd_dq_tc64(const float* qkv, const float* dout, const float* lse, const float* delta, float* dqkv,
                     int64_t B, int64_t T, int H, int Hk, cudaStream_t stream);
int attn_bwd_dkv_tc64(const float* qkv, const float* dout, const float* lse, const float* delta, float* dqkv,
                      int64_t B, int64_t T, int H, int Hk, cudaStream_t stream);
static bool bwd64_off() {
  static const bool off = [] {
    const char* e = getenv("CTDK_ATTN_BWD_GENERIC");
    return e != nullptr && e[0] == '1';
  }();
  return off;
}

// dQ part of the backward. Returns CTDK_OK, a negative status, or 1 when not eligible.
int attn_bwd_dq_tcgen05(const float* qkv, const float* dout, const float* lse, const float* delta, float* dqkv,
                        int64_t B, int64_t T, int H, int Hk, int D, cudaStream_t stream) {
  if ((reinterpret_cast<uintptr_t>(qkv) & 15u) || (reinterpret_cast<uintptr_t>(dout) & 15u) ||
      (reinterpret_cast<uintptr_t>(dqkv) & 15u))
    return 1;
  if (D == 64 && !bwd64_off()) return attn_bwd_dq_tc64(qkv, dout, lse, delta, dqkv, B, T, H, Hk, stream);
  BwdArgs a;
  a.lse = lse;
  a.delta = delta;
  a.dqkv = dqkv;
  a.T = static_cast<int>(T);
  a.H = H;
  a.Hk = Hk;
  a.B = static_cast<int>(B);
  a.n_qtiles = static_cast<int>((T + TM - 1) / TM);
  a.scale = 1.0f / sqrtf(static_cast<float>(D));
  a.status = device_status_word();
  if (a.status == nullptr) return fail(CTDK_ELAUNCH, "attn_bwd(tcgen05): no status word");
  return D == 64 ? launch_dq<64, 64, 2, 2, false>(qkv, dout, a, B, stream) : launch_dq<128, 64, 1, 2, true>(qkv, dout, a, B, stream);
}

// ----------------------------------------------------------------------------------------
// dK/dV kernel. Keys are the M dimension (tensor-memory lanes). TQB queries per step, NB stages.
// ----------------------------------------------------------------------------------------
namespace {

// VT: V lives in tensor memory (copied there once by the compute warps through the Q / dO landing
// area), so dP^T = V dO^T reads its left-hand operand at the math rate and the 64 KB it would
// occupy in shared memory go to a 64-query step instead of a 32-query one.
template <int D, int TQB, int NB, bool VT>
struct DkvCfg {
  static constexpr int kKeyTile = TM * D * 4;    // K or V, resident
  static constexpr int kQTile = TQB * D * 4;     // Q or dO in one layout
  static constexpr int kKeyTiles = VT ? 1 : 2;
  static constexpr int kSmem = kKeyTiles * kKeyTile + NB * 4 * kQTile + 1024 /*align*/ + 1024 /*lse, delta*/ + 256;
  static constexpr int kCols = NB * 2 * TQB + 2 * D + (VT ? D : 0);
  static_assert(!VT || NB * 2 * kQTile >= kKeyTile, "the K-major Q and dO buffers are V's landing area");
  static_assert(kCols <= 512, "tensor memory");
  static constexpr uint32_t kTmemCols = kCols <= 256 ? 256 : 512;
  static constexpr int kComputeWarps = 4 * (TQB / 32);
  static constexpr int kThreads = 64 + 32 * kComputeWarps;
};

template <int D, int TQB, int NB, bool VT>
__global__ void __launch_bounds__(DkvCfg<D, TQB, NB, VT>::kThreads, 1)
    attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tm_kv,   // qkv, box 128 rows, K-major
                           const __grid_constant__ CUtensorMap tm_qk,   // qkv, box TQB rows, K-major
                           const __grid_constant__ CUtensorMap tm_dok,  // dout, box TQB rows, K-major
                           const __grid_constant__ CUtensorMap tm_qm,   // qkv, box TQB rows, MN-major
                           const __grid_constant__ CUtensorMap tm_dom,  // dout, box TQB rows, MN-major
                           const BwdArgs args) {
  using C = DkvCfg<D, TQB, NB, VT>;
  constexpr int NC = D / 32;
  constexpr int kKeyChunk = TM * 128, kQChunk = TQB * 128;
  constexpr int NCW = C::kComputeWarps * 32;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* k_s = smem;
  unsigned char* qk_s = k_s + C::kKeyTiles * C::kKeyTile;   // [NB] Q  K-major
  unsigned char* v_s = VT ? qk_s : k_s + C::kKeyTile;  // VT: V only lands here (in the Q / dO buffers) on its way to tensor memory
  unsigned char* dok_s = qk_s + NB * C::kQTile;       // [NB] dO K-major
  unsigned char* qm_s = dok_s + NB * C::kQTile;       // [NB] Q  MN-major
  unsigned char* dom_s = qm_s + NB * C::kQTile;       // [NB] dO MN-major
  float* s_lse = reinterpret_cast<float*>(dom_s + NB * C::kQTile);   // [2][TQB]
  float* s_del = s_lse + 2 * TQB;                                    // [2][TQB]  (NB <= 2)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kKeyTiles * C::kKeyTile + NB * 4 * C::kQTile + 1024);
  uint64_t* kv_full = bars;         // 1
  uint64_t* qk_full = bars + 1;     // [2]
  uint64_t* qk_empty = bars + 3;    // [2]
  uint64_t* qm_full = bars + 5;     // [2]
  uint64_t* qm_empty = bars + 7;    // [2]
  uint64_t* sdp_full = bars + 9;    // [2]
  uint64_t* pds_ready = bars + 11;  // [2] NCW arrivals
  uint64_t* done_bar = bars + 13;   // 1
  uint64_t* v_land = bars + 14;     // 1    VT: V has arrived in shared memory
  uint64_t* v_ready = bars + 15;    // 1    VT: ... and has been copied to tensor memory (NCW arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // One-dimensional grid, longest items first (the first key tile of every kv head and sequence
  // meets the most query tiles).
  const int hb = args.Hk * args.B;
  const int kj = static_cast<int>(blockIdx.x) / hb;
  const int hk = (static_cast<int>(blockIdx.x) % hb) % args.Hk, b = (static_cast<int>(blockIdx.x) % hb) / args.Hk;
  const int G = args.H / args.Hk;
  const int k0 = kj * TM;
  const int n_qt = (args.T + TQB - 1) / TQB;
  const int first_qt = k0 / TQB;
  const int per_head = n_qt - first_qt;
  const int n_units = G * per_head;
  const int col_k = (args.H + hk) * D, col_v = (args.H + args.Hk + hk) * D;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qk_full[i], 1);
      mbar_init(&qk_empty[i], 1);
      mbar_init(&qm_full[i], 1);
      mbar_init(&qm_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
      mbar_init(&pds_ready[i], NCW);
    }
    mbar_init(done_bar, 1);
    mbar_init(v_land, 1);
    mbar_init(v_ready, NCW);
    mbar_fence_init();
    tma_prefetch_desc(&tm_kv);
    tma_prefetch_desc(&tm_qk);
    tma_prefetch_desc(&tm_dok);
    tma_prefetch_desc(&tm_qm);
    tma_prefetch_desc(&tm_dom);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tm_s = [&](int i) { return tmem_base + static_cast<uint32_t>(i * 2 * TQB); };         // S^T, then P^T
  auto tm_dp = [&](int i) { return tmem_base + static_cast<uint32_t>(i * 2 * TQB + TQB); };  // dP^T, then dS^T
  const uint32_t tm_dv = tmem_base + static_cast<uint32_t>(NB * 2 * TQB);
  const uint32_t tm_dk = tm_dv + static_cast<uint32_t>(D);
  const uint32_t tm_v = tm_dk + static_cast<uint32_t>(D);   // VT only

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, C::kKeyTiles * C::kKeyTile);
      if (VT) mbar_expect_tx(v_land, C::kKeyTile);
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        tma_load_3d(k_s + c * kKeyChunk, &tm_kv, kv_full, col_k + 32 * c, k0, b);
        tma_load_3d(v_s + c * kKeyChunk, &tm_kv, VT ? v_land : kv_full, col_v + 32 * c, k0, b);
      }
      // VT: the first Q / dO tiles go where V landed, so V has to be in tensor memory first
      bool v_out = !VT || mbar_wait_bounded(v_ready, 0, args.status, 59);
      for (int u = 0; u < n_units && v_out; ++u) {
        const int s = u % NB;
        const uint32_t ph = static_cast<uint32_t>(u / NB) & 1u;
        const int g = u / per_head;
        const int qrow = (first_qt + (u - g * per_head)) * TQB;
        const int col_q = (hk * G + g) * D;
        if (!mbar_wait_bounded(&qk_empty[s], ph ^ 1u, args.status, 51)) break;
        mbar_expect_tx(&qk_full[s], 2 * C::kQTile);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          tma_load_3d(qk_s + s * C::kQTile + c * kQChunk, &tm_qk, &qk_full[s], col_q + 32 * c, qrow, b);
          tma_load_3d(dok_s + s * C::kQTile + c * kQChunk, &tm_dok, &qk_full[s], col_q + 32 * c, qrow, b);
        }
        if (!mbar_wait_bounded(&qm_empty[s], ph ^ 1u, args.status, 52)) break;
        mbar_expect_tx(&qm_full[s], 2 * C::kQTile);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          tma_load_3d(qm_s + s * C::kQTile + c * kQChunk, &tm_qm, &qm_full[s], col_q + 32 * c, qrow, b);
          tma_load_3d(dom_s + s * C::kQTile + c * kQChunk, &tm_dom, &qm_full[s], col_q + 32 * c, qrow, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // converged-warp issue, as in the dQ kernel
    const uint32_t idesc_s = idesc_b(false, TQB);
    const uint32_t idesc_d = idesc_b(true, D);
    bool ok = mbar_wait_bounded_w(kv_full, 0, args.status, 53);
    if (VT && ok) ok = mbar_wait_bounded_w(v_ready, 0, args.status, 53);
    tc_fence_after();
    const uint64_t kd = make_smem_desc(smem_u32(k_s), 16, 1024, kLayoutSw128);
    const uint64_t vd = make_smem_desc(smem_u32(v_s), 16, 1024, kLayoutSw128);   // unused with VT
    auto issue_sdp = [&](int u) {
      const int s = u % NB;
      if (!mbar_wait_bounded_w(&qk_full[s], static_cast<uint32_t>(u / NB) & 1u, args.status, 54)) return false;
      tc_fence_after();
      const uint64_t qd_ = make_smem_desc(smem_u32(qk_s + s * C::kQTile), 16, 1024, kLayoutSw128);
      const uint64_t dod = make_smem_desc(smem_u32(dok_s + s * C::kQTile), 16, 1024, kLayoutSw128);
      const uint32_t ts = tm_s(s), tp = tm_dp(s);
#pragma unroll
      for (int ks = 0; ks < D / 8; ++ks)
        umma_tf32_w(ts, kd + static_cast<uint64_t>(((ks >> 2) * kKeyChunk + (ks & 3) * 32) >> 4),
                    qd_ + static_cast<uint64_t>(((ks >> 2) * kQChunk + (ks & 3) * 32) >> 4), idesc_s, ks != 0 ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < D / 8; ++ks) {
        const uint64_t bd = dod + static_cast<uint64_t>(((ks >> 2) * kQChunk + (ks & 3) * 32) >> 4);
        if (VT) umma_tf32_ta_w(tp, tm_v + static_cast<uint32_t>(ks * 8), bd, idesc_s, ks != 0 ? 1u : 0u);
        else umma_tf32_w(tp, vd + static_cast<uint64_t>(((ks >> 2) * kKeyChunk + (ks & 3) * 32) >> 4), bd, idesc_s, ks != 0 ? 1u : 0u);
      }
      umma_commit_w(&qk_empty[s]);
      umma_commit_w(&sdp_full[s]);
      return true;
    };
    auto issue_dvdk = [&](int u) {
      const int s = u % NB;
      const uint32_t ph = static_cast<uint32_t>(u / NB) & 1u;
      if (!mbar_wait_bounded_w(&pds_ready[s], ph, args.status, 55)) return false;
      if (!mbar_wait_bounded_w(&qm_full[s], ph, args.status, 56)) return false;
      tc_fence_after();
      const uint64_t qmd = make_smem_desc(smem_u32(qm_s + s * C::kQTile), kQChunk, 512, kLayoutSw128Base32);
      const uint64_t domd = make_smem_desc(smem_u32(dom_s + s * C::kQTile), kQChunk, 512, kLayoutSw128Base32);
      const uint32_t ts = tm_s(s), tp = tm_dp(s);
#pragma unroll
      for (int ks = 0; ks < TQB / 8; ++ks)
        umma_tf32_ta_w(tm_dv, ts + static_cast<uint32_t>(ks * 8), domd + static_cast<uint64_t>((ks * 1024) >> 4), idesc_d,
                       (u != 0 || ks != 0) ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < TQB / 8; ++ks)
        umma_tf32_ta_w(tm_dk, tp + static_cast<uint32_t>(ks * 8), qmd + static_cast<uint64_t>((ks * 1024) >> 4), idesc_d,
                       (u != 0 || ks != 0) ? 1u : 0u);
      umma_commit_w(&qm_empty[s]);
      return true;
    };
    for (int u = 0; u <= n_units && ok; ++u) {
      if (NB == 2 && u < n_units) ok = issue_sdp(u);
      if (ok && u >= 1) ok = issue_dvdk(u - 1);
      if (NB == 1 && ok && u < n_units) ok = issue_sdp(u);
    }
    umma_commit_w(done_bar);
    __syncwarp();
  } else {
    const int cw = warp - 2;
    const int qd = warp & 3, half = cw >> 2;
    const int ctid = cw * 32 + lane;  // 0 .. NCW-1
    const int key = k0 + qd * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sc2 = args.scale * kLog2ef;
    bool ok = true;
    if (VT) {
      // this thread's key row, half of its D columns: shared memory (16-byte pieces XORed with the
      // row number inside each 128-byte chunk row) -> tensor memory
      ok = mbar_wait_bounded(v_land, 0, args.status, 50);
      if (ok) {
        const int r = qd * 32 + lane;
        constexpr int kPerHalf = D / (C::kComputeWarps / 4);   // columns per warp of a lane quarter
#pragma unroll
        for (int cc = 0; cc < kPerHalf / 32; ++cc) {
          const int chunk = half * (kPerHalf / 32) + cc;
          uint32_t vb[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 x = *reinterpret_cast<const uint4*>(v_s + chunk * kKeyChunk + r * 128 + ((j ^ (r & 7)) << 4));
            vb[4 * j] = x.x;
            vb[4 * j + 1] = x.y;
            vb[4 * j + 2] = x.z;
            vb[4 * j + 3] = x.w;
          }
          tmem_st_32x32(tm_v + lane_off + static_cast<uint32_t>(chunk * 32), vb);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(v_ready);
      }
    }
    for (int u = 0; u < n_units && ok; ++u) {
      const int s = u % NB;
      const int g = u / per_head;
      const int q0 = (first_qt + (u - g * per_head)) * TQB;
      const int64_t lbase = (static_cast<int64_t>(b) * args.H + hk * G + g) * args.T;
      float* bl = s_lse + (u & 1) * TQB;
      float* bd = s_del + (u & 1) * TQB;
      for (int t = ctid; t < 2 * TQB; t += NCW) {
        const int q = q0 + (t < TQB ? t : t - TQB);
        if (t < TQB) bl[t] = q < args.T ? args.lse[lbase + q] * kLog2ef : FLT_MAX;
        else bd[t - TQB] = q < args.T ? args.delta[lbase + q] : 0.0f;
      }
      asm volatile("bar.sync 1, %0;" ::"r"(NCW) : "memory");
      if (!mbar_wait_bounded(&sdp_full[s], static_cast<uint32_t>(u / NB) & 1u, args.status, 57)) { ok = false; break; }
      tc_fence_after();
      float sv[32], dv[32];
      uint32_t pb[32], db[32];
      tmem_ld_32x32(tm_s(s) + lane_off + half * 32, sv);
      tmem_ld_32x32(tm_dp(s) + lane_off + half * 32, dv);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int ql = half * 32 + i;
        const float p = (key > q0 + ql) ? 0.0f : ex2(sv[i] * sc2 - bl[ql]);
        pb[i] = tf32_bits(p);
        db[i] = tf32_bits(p * (dv[i] - bd[ql]) * args.scale);
      }
      tmem_st_32x32(tm_s(s) + lane_off + half * 32, pb);
      tmem_st_32x32(tm_dp(s) + lane_off + half * 32, db);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&pds_ready[s]);
    }
    if (ok && mbar_wait_bounded(done_bar, 0, args.status, 58)) {
      tc_fence_after();
      const int64_t RS = static_cast<int64_t>(args.H + 2 * args.Hk) * D;
      float* row = args.dqkv + (static_cast<int64_t>(b) * args.T + key) * RS;
      constexpr int kChunks = 2 * D / 32;               // dV chunks then dK chunks
      constexpr int kPerWarpSet = kChunks / (C::kComputeWarps / 4);
      for (int c = half * kPerWarpSet; c < (half + 1) * kPerWarpSet; ++c) {
        float v[32];
        tmem_ld_32x32(tm_dv + lane_off + c * 32, v);   // dK follows dV in tensor memory
        const bool is_dv = c < D / 32;
        float* dst = row + (is_dv ? col_v + c * 32 : col_k + (c - D / 32) * 32);
        if (key < args.T) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
        __syncwarp();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int D, int TQB, int NB, bool VT>
int launch_dkv(const float* qkv, const float* dout, const BwdArgs& a, int64_t B, cudaStream_t s) {
  using C = DkvCfg<D, TQB, NB, VT>;
  const int RS = (a.H + 2 * a.Hk) * D;
  const int64_t HD = static_cast<int64_t>(a.H) * D;
  CUtensorMap tkv, tqk, tdok, tqm, tdom;
  int rc = map3(&tkv, qkv, RS, a.T, B, TM, false);
  if (rc == CTDK_OK) rc = map3(&tqk, qkv, RS, a.T, B, TQB, false);
  if (rc == CTDK_OK) rc = map3(&tdok, dout, HD, a.T, B, TQB, false);
  if (rc == CTDK_OK) rc = map3(&tqm, qkv, RS, a.T, B, TQB, true);
  if (rc == CTDK_OK) rc = map3(&tdom, dout, HD, a.T, B, TQB, true);
  if (rc != CTDK_OK) return rc;
  auto* kern = attn_bwd_dkv_tc_kernel<D, TQB, NB, VT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "attn_bwd dkv(tcgen05): shared memory opt-in failed: %s", cudaGetErrorString(e));
  dim3 grid(static_cast<unsigned>(static_cast<int64_t>(a.n_qtiles) * a.Hk * B));
  kern<<<grid, C::kThreads, C::kSmem, s>>>(tkv, tqk, tdok, tqm, tdom, a);
  return check_launch("ctdk_attn_bwd(dkv, tcgen05)");
}

}  // namespace

// dK/dV part of the backward. Returns CTDK_OK, a negative status, or 1 when not eligible.
int attn_bwd_dkv_tcgen05(const float* qkv, const float* dout, const float* lse, const float* delta, float* dqkv,
                         int64_t B, int64_t T, int H, int Hk, int D, cudaStream_t stream) {
  if ((reinterpret_cast<uintptr_t>(qkv) & 15u) || (reinterpret_cast<uintptr_t>(dout) & 15u) ||
      (reinterpret_cast<uintptr_t>(dqkv) & 15u))
    return 1;
  if (D == 64 && !bwd64_off()) return attn_bwd_dkv_tc64(qkv, dout, lse, delta, dqkv, B, T, H, Hk, stream);
  BwdArgs a;
  a.lse = lse;
  a.delta = delta;
  a.dqkv = dqkv;
  a.T = static_cast<int>(T);
  a.H = H;
  a.Hk = Hk;
  a.B = static_cast<int>(B);
  a.n_qtiles = static_cast<int>((T + TM - 1) / TM);
  a.scale = 1.0f / sqrtf(static_cast<float>(D));
  a.status = device_status_word();
  if (a.status == nullptr) return fail(CTDK_ELAUNCH, "attn_bwd(tcgen05): no status word");
  return D == 64 ? launch_dkv<64, 64, 2, false>(qkv, dout, a, B, stream) : launch_dkv<128, 64, 1, true>(qkv, dout, a, B, stream);
}

}  // namespace ctdk
