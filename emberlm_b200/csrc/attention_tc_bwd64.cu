// Causal grouped-query attention backward for head size 64 on the tcgen05 tensor cores:
// persistent kernels with every left-hand MMA operand in tensor memory.
//
// With 4-byte operands an MMA whose A operand comes from shared memory is bound by shared-memory
// bandwidth unless its N is 256 (a 128 x 8 slice of A plus an N x 8 slice of B per instruction),
// and the N of these products is only 64. Reading A from tensor memory removes that bound, so
//   dQ kernel     keeps Q and dO of its 128-query tile in tensor memory (copied there once per
//                 work item by the compute warps) next to the dQ accumulator and two S / dP
//                 buffers:  S = Q K^T,  dP = dO V^T,  dS = P (dP - delta) scale,  dQ += dS K;
//   dK/dV kernel  keeps K and V of its 128-key tile in tensor memory next to the dK and dV
//                 accumulators and two S^T / dP^T buffers:  S^T = K Q^T,  dP^T = V dO^T,
//                 dV += P^T dO,  dK += dS^T Q, summed over the query heads of the group (the
//                 reference's repeat_kv_sum, emberlm src/ops/repeat_kv.cu:29-43) without atomics.
// Both kernels walk a batch-major list of work items per CTA so that loads, MMAs and the epilogue
// of consecutive items overlap and the operands of the sequences in flight stay in L2. All
// right-hand operands arrive by TMA, one multi-dimensional box per tile (issuing a TMA copy
// occupies the producer thread for ~140 cycles whatever its size). P and dS are written with
// packed two-wide fp32 arithmetic. Every mbarrier wait is bounded.
//
// Replaces, with attention_tc.cu, the backward of the bmm -> scale -> mask -> softmax -> bmm chain
// of the reference's Attention::forward_train (emberlm include/ctd/nn/attention.h:123-141,
// softmax backward src/ops/softmax.cu:56-93).
#include <atomic>
#include <cfloat>
#include <climits>

#include "common.cuh"

namespace ctdk {
namespace {

constexpr int D = 64;          // head size
constexpr int TM = 128;        // rows of the CTA tile = tensor-memory lanes
constexpr int TN = 64;         // columns of one S / dP step
constexpr float kLog2ef = 1.4426950408889634f;
constexpr int kRowTileBytes = TM * D * 4;   // 32 KB: a 128-row operand tile
constexpr int kColTileBytes = TN * D * 4;   // 16 KB: a 64-row operand tile
constexpr int kRowChunk = TM * 128;         // bytes of one {32 floats x 128 rows} sub-box
constexpr int kColChunk = TN * 128;         // bytes of one {32 floats x 64 rows} sub-box

__device__ __forceinline__ uint32_t idesc64(bool b_mn) {   // M = 128, N = 64, TF32, fp32 accumulate
  return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(64 >> 3) << 17) | (static_cast<uint32_t>(TM >> 4) << 24);
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Round-to-nearest to TF32 as an integer add (the tensor core ignores the 13 low mantissa bits).
__device__ __forceinline__ uint32_t rna_bits(float x) { return __float_as_uint(x) + 0x1000u; }


struct Bwd64Args {
  const float* lse;
  const float* delta;
  float* dqkv;
  int T, H, Hk, B;
  int n_tiles;    // ceil(T / 128)
  int n_items;
  float scale;
  int* status;
  int* work_counter;   // dK/dV kernel: next unclaimed item (zeroed before the launch)
};

// Copies this thread's row (64 floats, 256 bytes) of a {2 x [128 rows x 128 bytes]} tile with the
// 16-byte-chunk swizzle out of shared memory.
__device__ __forceinline__ void load_row_sw128(const unsigned char* tile, int r, float (&v)[64]) {
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    const float4 x = *reinterpret_cast<const float4*>(tile + (c >> 3) * kRowChunk + r * 128 + (((c & 7) ^ (r & 7)) << 4));
    v[4 * c] = x.x;
    v[4 * c + 1] = x.y;
    v[4 * c + 2] = x.z;
    v[4 * c + 3] = x.w;
  }
}

// Writes 32 rows x 32 columns held one row per lane (v) to global memory through a 2 KB per-warp
// staging area, 16 rows at a time, so that each store instruction covers 4 rows x 128 bytes.
// dst points at row 0, column 0 of the 32 x 32 block; rows_left = number of rows that exist.
__device__ __forceinline__ void store_block_32x32(float* stg, const float (&v)[32], float* dst, int64_t ld,
                                                  int rows_left, int lane) {
#pragma unroll
  for (int rh = 0; rh < 2; ++rh) {
    if ((lane >> 4) == rh) {
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<float4*>(stg + (lane & 15) * 32 + ((c ^ (lane & 7)) << 2)) =
            make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int r = (lane >> 3) + 4 * k, ch = lane & 7;
      const float4 x = *reinterpret_cast<const float4*>(stg + r * 32 + ((ch ^ (r & 7)) << 2));
      if (rh * 16 + r < rows_left) *reinterpret_cast<float4*>(dst + static_cast<int64_t>(rh * 16 + r) * ld + ch * 4) = x;
    }
    __syncwarp();
  }
}

// ----------------------------------------------------------------------------------------
// dQ kernel
// ----------------------------------------------------------------------------------------
constexpr int kDqStages = 3;
constexpr int kDqStageBytes = 3 * kColTileBytes;   // K and V (16-byte swizzle) + K (32-byte swizzle)
constexpr int kDqSmem = 2 * kRowTileBytes + kDqStages * kDqStageBytes + 8 * 2048 + 1024 + 256;

struct DqItem {
  int qi, h, b, q0, n_steps;
};
// Batch-major item order (see attention_tc.cu): heaviest query tile of a sequence first, heads fastest.
__device__ __forceinline__ DqItem dq_item(const Bwd64Args& a, int it) {
  DqItem w;
  const int per_b = a.n_tiles * a.H;
  w.b = it / per_b;
  const int r = it % per_b;
  w.qi = a.n_tiles - 1 - r / a.H;
  w.h = r % a.H;
  w.q0 = w.qi * TM;
  w.n_steps = min((w.q0 + TM) / TN, (a.T + TN - 1) / TN);
  return w;
}

__global__ void __launch_bounds__(320, 1)
    attn_bwd_dq64_kernel(const __grid_constant__ CUtensorMap tm_q,    // qkv  {32, 128, 2, 1}      16-byte swizzle
                         const __grid_constant__ CUtensorMap tm_do,   // dout {32, 128, 2, 1}      16-byte swizzle
                         const __grid_constant__ CUtensorMap tm_kv,   // qkv  {32, 64, 2, 2, 1}    16-byte swizzle: K then V
                         const __grid_constant__ CUtensorMap tm_km,   // qkv  {32, 64, 2, 1}       32-byte swizzle: K
                         const Bwd64Args args) {
  extern __shared__ unsigned char smem_raw[];
  pdl_launch();
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* q_land = smem;                        // Q tile as it arrives
  unsigned char* do_land = q_land + kRowTileBytes;     // dO tile
  unsigned char* stages = do_land + kRowTileBytes;     // [3] x {K, V (K-major), K (MN-major)}
  unsigned char* o_stage = stages + kDqStages * kDqStageBytes;   // 8 x 2 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(o_stage + 8 * 2048);
  uint64_t* land_full = bars;        // 1    Q and dO of the item have arrived (one phase per item)
  uint64_t* qdo_ready = bars + 1;    // 1    ... and have been copied to tensor memory (256 arrivals)
  uint64_t* kv_full = bars + 2;      // [3]
  uint64_t* kv_empty = bars + 5;     // [3]
  uint64_t* km_full = bars + 8;      // [3]
  uint64_t* km_empty = bars + 11;    // [3]
  uint64_t* sdp_full = bars + 14;    // [2]  S(g) and dP(g) are in tensor memory
  uint64_t* ds_ready = bars + 16;    // [2]  dS(g) has replaced S(g) (256 arrivals)
  uint64_t* dq_done = bars + 18;     // 1    the item's last dQ MMA has finished (one phase per item)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(land_full, 1);
    mbar_init(qdo_ready, 256);
    for (int i = 0; i < kDqStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&km_full[i], 1);
      mbar_init(&km_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sdp_full[i], 1);
      mbar_init(&ds_ready[i], 256);
    }
    mbar_init(dq_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_kv);
    tma_prefetch_desc(&tm_km);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // inputs come from earlier kernels in the stream
  const uint32_t tm_qa = tmem_base, tm_doa = tmem_base + 64u;
  // two dQ accumulators (items alternate), so that an item's result is read and stored while the
  // next item's first MMAs are already running
  auto tm_dq = [&](uint32_t n) { return tmem_base + ((n & 1u) ? 448u : 128u); };
  auto tm_s = [&](uint32_t g) { return tmem_base + 192u + (g & 1u) * 128u; };    // S, later dS
  auto tm_dp = [&](uint32_t g) { return tmem_base + 256u + (g & 1u) * 128u; };   // dP
  // g = running count of key steps over all items of this CTA: stage g % 3, score buffer g & 1.

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      uint32_t g0 = 0, n_it = 0;
      bool ok = true;
      auto load_qdo = [&](const DqItem& w) {
        mbar_expect_tx(land_full, 2 * kRowTileBytes);
        tma_load_4d(q_land, &tm_q, land_full, 0, w.q0, (w.h * D) >> 5, w.b);
        tma_load_4d(do_land, &tm_do, land_full, 0, w.q0, (w.h * D) >> 5, w.b);
      };
      if (static_cast<int>(blockIdx.x) < args.n_items) load_qdo(dq_item(args, blockIdx.x));
      for (int it = blockIdx.x; it < args.n_items && ok; it += gridDim.x, ++n_it) {
        const DqItem w = dq_item(args, it);
        const int hk = w.h / (args.H / args.Hk);
        const int chunk_k = ((args.H + hk) * D) >> 5;
        for (int j = 0; j < w.n_steps && ok; ++j) {
          const uint32_t g = g0 + static_cast<uint32_t>(j), st = g % kDqStages, ph = (g / kDqStages) & 1u;
          unsigned char* sb = stages + st * kDqStageBytes;
          if (!mbar_wait_bounded(&kv_empty[st], ph ^ 1u, args.status, 41)) { ok = false; break; }
          mbar_expect_tx(&kv_full[st], 2 * kColTileBytes);
          tma_load_5d(sb, &tm_kv, &kv_full[st], 0, j * TN, chunk_k, 0, w.b);
          if (!mbar_wait_bounded(&km_empty[st], ph ^ 1u, args.status, 42)) { ok = false; break; }
          mbar_expect_tx(&km_full[st], kColTileBytes);
          tma_load_4d(sb + 2 * kColTileBytes, &tm_km, &km_full[st], 0, j * TN, chunk_k, w.b);
          if (j == min(1, w.n_steps - 1) && it + static_cast<int>(gridDim.x) < args.n_items) {
            // the landing buffers are free once this item's Q / dO sit in tensor memory
            if (!mbar_wait_bounded(qdo_ready, n_it & 1u, args.status, 40)) { ok = false; break; }
            load_qdo(dq_item(args, it + gridDim.x));
          }
        }
        g0 += static_cast<uint32_t>(w.n_steps);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    // The whole warp runs this role converged; one elected lane issues each MMA / commit.
    {
      const uint32_t id_k = idesc64(false), id_mn = idesc64(true);
      const uint32_t stages_addr = smem_u32(stages);
      uint32_t g0 = 0, n_it = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < args.n_items && ok; it += gridDim.x, ++n_it) {
        const DqItem w = dq_item(args, it);
        auto issue_sdp = [&](int j) {
          const uint32_t g = g0 + static_cast<uint32_t>(j), st = g % kDqStages;
          {
            if (!mbar_wait_bounded_w(&kv_full[st], (g / kDqStages) & 1u, args.status, 44)) return false;
          }
          tc_fence_after();
          const uint64_t kd = make_smem_desc(stages_addr + st * kDqStageBytes, 16, 1024, kLayoutSw128);
          const uint64_t vd = make_smem_desc(stages_addr + st * kDqStageBytes + kColTileBytes, 16, 1024, kLayoutSw128);
          const uint32_t ts = tm_s(g), tp = tm_dp(g);
#pragma unroll
          for (int ks = 0; ks < D / 8; ++ks)   // descriptor address field counts 16-byte units
            umma_tf32_ta_w(ts, tm_qa + static_cast<uint32_t>(ks * 8), kd + (((ks >> 2) * kColChunk + (ks & 3) * 32) >> 4),
                           id_k, ks != 0 ? 1u : 0u);
#pragma unroll
          for (int ks = 0; ks < D / 8; ++ks)
            umma_tf32_ta_w(tp, tm_doa + static_cast<uint32_t>(ks * 8), vd + (((ks >> 2) * kColChunk + (ks & 3) * 32) >> 4),
                           id_k, ks != 0 ? 1u : 0u);
          umma_commit_w(&kv_empty[st]);
          umma_commit_w(&sdp_full[g & 1u]);
          return true;
        };
        {
          if (!mbar_wait_bounded_w(qdo_ready, n_it & 1u, args.status, 43)) break;
        }
        tc_fence_after();
        // Tensor-pipe order: SdP(0) SdP(1) | dQ(0) SdP(2) | dQ(1) SdP(3) | ...
        ok = issue_sdp(0);
        if (ok && w.n_steps > 1) ok = issue_sdp(1);
        for (int j = 0; j < w.n_steps && ok; ++j) {
          const uint32_t g = g0 + static_cast<uint32_t>(j), st = g % kDqStages;
          {
            if (!mbar_wait_bounded_w(&ds_ready[g & 1u], (g >> 1) & 1u, args.status, 45)) { ok = false; break; }
          }
          {
            if (!mbar_wait_bounded_w(&km_full[st], (g / kDqStages) & 1u, args.status, 46)) { ok = false; break; }
          }
          tc_fence_after();
          const uint64_t kmd =
              make_smem_desc(stages_addr + st * kDqStageBytes + 2 * kColTileBytes, kColChunk, 512, kLayoutSw128Base32);
          const uint32_t ts = tm_s(g), tdq = tm_dq(n_it);
          const uint32_t acc0 = j != 0 ? 1u : 0u;
#pragma unroll
          for (int ks = 0; ks < TN / 8; ++ks)
            umma_tf32_ta_w(tdq, ts + static_cast<uint32_t>(ks * 8), kmd + ((ks * 1024) >> 4), id_mn, ks != 0 ? 1u : acc0);
          umma_commit_w(&km_empty[st]);
          if (j == w.n_steps - 1) umma_commit_w(dq_done);
          if (j + 2 < w.n_steps) ok = issue_sdp(j + 2);
        }
        g0 += static_cast<uint32_t>(w.n_steps);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- compute warps -------------------------------
    // Warp pair (w, w+4) shares a tensor-memory lane quarter; each thread owns one query row and
    // 32 of the 64 keys of a step.
    const int cw = warp - 2;
    const int qd = warp & 3, half = cw >> 2;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sc2 = args.scale * kLog2ef;
    float* stg = reinterpret_cast<float*>(o_stage + cw * 2048);
    uint32_t g0 = 0, n_it = 0;
    bool ok = true;
    const int64_t RS = static_cast<int64_t>(args.H + 2 * args.Hk) * D;
    // Reads item n's finished dQ out of its accumulator and stores it. Runs after the NEXT item's
    // Q / dO have been handed to the MMA warp, i.e. while that item's first S / dP MMAs execute.
    auto epilogue = [&](const DqItem& w, uint32_t n) {
      {
        if (!mbar_wait_bounded(dq_done, n & 1u, args.status, 49)) return false;
      }
      tc_fence_after();
      float v[32];
      tmem_ld_32x32(tm_dq(n) + lane_off + static_cast<uint32_t>(half * 32), v);
      float* dst = args.dqkv + (static_cast<int64_t>(w.b) * args.T + w.q0 + qd * 32) * RS + w.h * D + half * 32;
      store_block_32x32(stg, v, dst, RS, args.T - (w.q0 + qd * 32), lane);
      tc_fence_before();
      return true;
    };
    DqItem prev{};
    bool have_prev = false;
    for (int it = blockIdx.x; it < args.n_items && ok; it += gridDim.x, ++n_it) {
      const DqItem w = dq_item(args, it);
      const int row = w.q0 + qd * 32 + lane;
      const bool row_ok = row < args.T;
      const int64_t lbase = (static_cast<int64_t>(w.b) * args.H + w.h) * args.T;
      const float neg_lse2 = row_ok ? -args.lse[lbase + row] * kLog2ef : -FLT_MAX;
      const float neg_dls = row_ok ? -args.delta[lbase + row] * args.scale : 0.0f;
      // Q (first warp of the pair) or dO (second) row of this thread: shared -> tensor memory
      {
        if (!mbar_wait_bounded(land_full, n_it & 1u, args.status, 47)) { ok = false; break; }
      }
      {
        float v[64];
        load_row_sw128(half == 0 ? q_land : do_land, qd * 32 + lane, v);
        tmem_st_32x64((half == 0 ? tm_qa : tm_doa) + lane_off, *reinterpret_cast<uint32_t(*)[64]>(v));
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive(qdo_ready);
      if (have_prev && !epilogue(prev, n_it - 1u)) { ok = false; break; }
      for (int j = 0; j < w.n_steps && ok; ++j) {
        const uint32_t g = g0 + static_cast<uint32_t>(j);
        {
          if (!mbar_wait_bounded(&sdp_full[g & 1u], (g >> 1) & 1u, args.status, 48)) { ok = false; break; }
        }
        tc_fence_after();
        const uint32_t ts = tm_s(g) + lane_off + static_cast<uint32_t>(half * 32);
        const uint32_t tp = tm_dp(g) + lane_off + static_cast<uint32_t>(half * 32);
        float sv[32], dv[32];
        tmem_ld_32x32_nowait(ts, sv);
        tmem_ld_32x32_nowait(tp, dv);
        tmem_wait_ld();
        uint32_t* ob = reinterpret_cast<uint32_t*>(sv);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float t0, t1, u0, u1;
          ffma2(t0, t1, sv[i], sv[i + 1], sc2, sc2, neg_lse2, neg_lse2);
          ffma2(u0, u1, dv[i], dv[i + 1], args.scale, args.scale, neg_dls, neg_dls);
          t0 = ex2f(t0);
          t1 = ex2f(t1);
          fmul2(t0, t1, t0, t1, u0, u1);
          ob[i] = rna_bits(t0);
          ob[i + 1] = rna_bits(t1);
        }
        if ((j + 1) * TN > w.q0 + 1) {   // a step that reaches past the tile's first row: causal mask
          const int key0 = j * TN + half * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i) ob[i] = (key0 + i > row) ? 0u : ob[i];
        }
        tmem_st_32x32(ts, *reinterpret_cast<uint32_t(*)[32]>(ob));
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&ds_ready[g & 1u]);
      }
      g0 += static_cast<uint32_t>(w.n_steps);
      prev = w;
      have_prev = true;
    }
    if (ok && have_prev) epilogue(prev, n_it - 1u);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ----------------------------------------------------------------------------------------
// dK/dV kernel. Keys are the M dimension (tensor-memory lanes); a unit is 64 queries of one of
// the group's query heads.
// ----------------------------------------------------------------------------------------
constexpr int kKvStages = 3;
constexpr int kKvStageBytes = 4 * kColTileBytes;   // Q, dO (16-byte swizzle) + Q, dO (32-byte swizzle)
constexpr int kKvSmem = kKvStages * kKvStageBytes + 8 * 2048 + 2048 /*lse, delta*/ + 1024 + 256;

struct KvItem {
  int kj, hk, b, k0, first_qt, per_head, n_units;
};
// Batch-major item order; inside a sequence the key tile with the most query blocks comes first.
__device__ __forceinline__ KvItem kv_item(const Bwd64Args& a, int it) {
  KvItem w;
  const int per_b = a.n_tiles * a.Hk;
  w.b = it / per_b;
  const int r = it % per_b;
  w.kj = r / a.Hk;
  w.hk = r % a.Hk;
  w.k0 = w.kj * TM;
  w.first_qt = w.k0 / TN;
  w.per_head = (a.T + TN - 1) / TN - w.first_qt;
  w.n_units = (a.H / a.Hk) * w.per_head;
  return w;
}

__global__ void __launch_bounds__(320, 1)
    attn_bwd_dkv64_kernel(const __grid_constant__ CUtensorMap tm_qk,    // qkv  {32, 64, 2, 1} 16-byte swizzle
                          const __grid_constant__ CUtensorMap tm_dok,   // dout {32, 64, 2, 1} 16-byte swizzle
                          const __grid_constant__ CUtensorMap tm_qm,    // qkv  {32, 64, 2, 1} 32-byte swizzle
                          const __grid_constant__ CUtensorMap tm_dom,   // dout {32, 64, 2, 1} 32-byte swizzle
                          const __grid_constant__ CUtensorMap tm_kvt,   // qkv  {32, 128, 2, 1} 16-byte swizzle (K, V tiles)
                          const Bwd64Args args) {
  extern __shared__ unsigned char smem_raw[];
  pdl_launch();
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  unsigned char* stages = smem;                                   // [3] x {Q, dO K-major, Q, dO MN-major}
  unsigned char* o_stage = stages + kKvStages * kKvStageBytes;    // 8 x 2 KB
  float* s_nl = reinterpret_cast<float*>(o_stage + 8 * 2048);     // [3][64]  -lse * log2(e) per query
  float* s_nd = s_nl + 3 * TN;                                    // [3][64]  -delta * scale per query
  uint64_t* bars = reinterpret_cast<uint64_t*>(o_stage + 8 * 2048 + 2048);
  uint64_t* kvt_ready = bars;        // 1    K and V of the item sit in tensor memory (256 arrivals)
  uint64_t* qk_full = bars + 1;      // [3]
  uint64_t* qk_empty = bars + 4;     // [3]
  uint64_t* qm_full = bars + 7;      // [3]
  uint64_t* qm_empty = bars + 10;    // [3]
  uint64_t* sdp_full = bars + 13;    // [2]
  uint64_t* pds_ready = bars + 15;   // [2]  P^T and dS^T are in place (256 arrivals)
  uint64_t* done_bar = bars + 17;    // 1    the item's last dV / dK MMA has finished
  uint64_t* const_full = bars + 18;  // [3]  the unit's per-query constants are in shared memory (128 arrivals)
  uint64_t* iq_full = bars + 21;     // [2]  work queue: item number published by the producer
  uint64_t* iq_empty = bars + 23;    // [2]  ... and read by the MMA warp (1) and every compute thread (256)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 25);
  volatile int* item_q = reinterpret_cast<volatile int*>(tmem_slot + 1);   // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = args.H / args.Hk;
  const int64_t RS = static_cast<int64_t>(args.H + 2 * args.Hk) * D;

  if (threadIdx.x == 0) {
    mbar_init(kvt_ready, 256);
    for (int i = 0; i < kKvStages; ++i) {
      mbar_init(&qk_full[i], 1);
      mbar_init(&qk_empty[i], 1);
      mbar_init(&qm_full[i], 1);
      mbar_init(&qm_empty[i], 1);
      mbar_init(&const_full[i], 2 * TN);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sdp_full[i], 1);
      mbar_init(&pds_ready[i], 256);
      mbar_init(&iq_full[i], 1);
      mbar_init(&iq_empty[i], 257);
    }
    mbar_init(done_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_qk);
    tma_prefetch_desc(&tm_dok);
    tma_prefetch_desc(&tm_qm);
    tma_prefetch_desc(&tm_dom);
    tma_prefetch_desc(&tm_kvt);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // inputs come from earlier kernels in the stream
  const uint32_t tm_ka = tmem_base, tm_va = tmem_base + 64u, tm_dv = tmem_base + 128u, tm_dk = tmem_base + 192u;
  auto tm_s = [&](uint32_t g) { return tmem_base + 256u + (g & 1u) * 128u; };    // S^T, later P^T
  auto tm_dp = [&](uint32_t g) { return tmem_base + 320u + (g & 1u) * 128u; };   // dP^T, later dS^T
  // Two running counts over all items of this CTA: r numbers the entries of the 3-stage operand
  // ring (the item's K / V tiles take one entry, then one per unit); g numbers the units (score
  // buffer g & 1, constant buffer g % 3).

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      // Items differ in length by up to 8x (a key tile meets between 2 and 16 query blocks per
      // head), so they are claimed one at a time from a global counter, in batch-major order with
      // the longest items of a sequence first, and published to the other warps through a
      // two-entry queue in shared memory.
      uint32_t r0 = 0;
      bool ok = true;
      for (uint32_t n = 0; ok; ++n) {
        const uint32_t slot = n & 1u;
        if (!mbar_wait_bounded(&iq_empty[slot], ((n >> 1) & 1u) ^ 1u, args.status, 50)) break;
        int it = atomicAdd(args.work_counter, 1);
        if (it >= args.n_items) it = -1;
        item_q[slot] = it;
        mbar_arrive(&iq_full[slot]);
        if (it < 0) break;
        const KvItem w = kv_item(args, it);
        {
          // the item's K and V tiles land in one ring entry (K in the first half, V in the
          // second) and are moved to tensor memory by the compute warps
          const uint32_t st = r0 % kKvStages, ph = (r0 / kKvStages) & 1u;
          unsigned char* sb = stages + st * kKvStageBytes;
          if (!mbar_wait_bounded(&qk_empty[st], ph ^ 1u, args.status, 51)) break;
          mbar_expect_tx(&qk_full[st], kRowTileBytes);
          tma_load_4d(sb, &tm_kvt, &qk_full[st], 0, w.k0, ((args.H + w.hk) * D) >> 5, w.b);
          if (!mbar_wait_bounded(&qm_empty[st], ph ^ 1u, args.status, 52)) break;
          mbar_expect_tx(&qm_full[st], kRowTileBytes);
          tma_load_4d(sb + kRowTileBytes, &tm_kvt, &qm_full[st], 0, w.k0, ((args.H + args.Hk + w.hk) * D) >> 5, w.b);
        }
        for (int u = 0; u < w.n_units && ok; ++u) {
          const uint32_t g = r0 + 1u + static_cast<uint32_t>(u), st = g % kKvStages, ph = (g / kKvStages) & 1u;
          const int gi = u / w.per_head;
          const int q0 = (w.first_qt + (u - gi * w.per_head)) * TN;
          const int chunk_q = ((w.hk * G + gi) * D) >> 5;
          unsigned char* sb = stages + st * kKvStageBytes;
          if (!mbar_wait_bounded(&qk_empty[st], ph ^ 1u, args.status, 51)) { ok = false; break; }
          mbar_expect_tx(&qk_full[st], 2 * kColTileBytes);
          tma_load_4d(sb, &tm_qk, &qk_full[st], 0, q0, chunk_q, w.b);
          tma_load_4d(sb + kColTileBytes, &tm_dok, &qk_full[st], 0, q0, chunk_q, w.b);
          if (!mbar_wait_bounded(&qm_empty[st], ph ^ 1u, args.status, 52)) { ok = false; break; }
          mbar_expect_tx(&qm_full[st], 2 * kColTileBytes);
          tma_load_4d(sb + 2 * kColTileBytes, &tm_qm, &qm_full[st], 0, q0, chunk_q, w.b);
          tma_load_4d(sb + 3 * kColTileBytes, &tm_dom, &qm_full[st], 0, q0, chunk_q, w.b);
        }
        r0 += static_cast<uint32_t>(w.n_units) + 1u;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    // The whole warp runs this role converged; one elected lane issues each MMA / commit.
    {
      const uint32_t id_k = idesc64(false), id_mn = idesc64(true);
      const uint32_t stages_addr = smem_u32(stages);
      uint32_t g0 = 0, r0 = 0, n_it = 0;
      bool ok = true;
      for (;; ++n_it) {
        if (!mbar_wait_bounded_w(&iq_full[n_it & 1u], (n_it >> 1) & 1u, args.status, 60)) break;
        const int it = item_q[n_it & 1u];
        __syncwarp();
        if (lane == 0) mbar_arrive(&iq_empty[n_it & 1u]);
        if (it < 0 || !ok) break;
        const KvItem w = kv_item(args, it);
        auto issue_sdp = [&](int u) {
          const uint32_t g = g0 + static_cast<uint32_t>(u), r = r0 + 1u + static_cast<uint32_t>(u), st = r % kKvStages;
          {
            if (!mbar_wait_bounded_w(&qk_full[st], (r / kKvStages) & 1u, args.status, 54)) return false;
          }
          tc_fence_after();
          const uint64_t qd_ = make_smem_desc(stages_addr + st * kKvStageBytes, 16, 1024, kLayoutSw128);
          const uint64_t dod = make_smem_desc(stages_addr + st * kKvStageBytes + kColTileBytes, 16, 1024, kLayoutSw128);
          const uint32_t ts = tm_s(g), tp = tm_dp(g);
#pragma unroll
          for (int ks = 0; ks < D / 8; ++ks)   // descriptor address field counts 16-byte units
            umma_tf32_ta_w(ts, tm_ka + static_cast<uint32_t>(ks * 8), qd_ + (((ks >> 2) * kColChunk + (ks & 3) * 32) >> 4),
                           id_k, ks != 0 ? 1u : 0u);
#pragma unroll
          for (int ks = 0; ks < D / 8; ++ks)
            umma_tf32_ta_w(tp, tm_va + static_cast<uint32_t>(ks * 8), dod + (((ks >> 2) * kColChunk + (ks & 3) * 32) >> 4),
                           id_k, ks != 0 ? 1u : 0u);
          umma_commit_w(&qk_empty[st]);
          umma_commit_w(&sdp_full[g & 1u]);
          return true;
        };
        {
          if (!mbar_wait_bounded_w(kvt_ready, n_it & 1u, args.status, 53)) break;
        }
        tc_fence_after();
        if (lane == 0) {   // K and V sit in tensor memory: their ring entry is free again
          mbar_arrive(&qk_empty[r0 % kKvStages]);
          mbar_arrive(&qm_empty[r0 % kKvStages]);
        }
        __syncwarp();
        ok = issue_sdp(0);
        if (ok && w.n_units > 1) ok = issue_sdp(1);
        for (int u = 0; u < w.n_units && ok; ++u) {
          const uint32_t g = g0 + static_cast<uint32_t>(u), r = r0 + 1u + static_cast<uint32_t>(u), st = r % kKvStages;
          {
            if (!mbar_wait_bounded_w(&pds_ready[g & 1u], (g >> 1) & 1u, args.status, 55)) { ok = false; break; }
          }
          {
            if (!mbar_wait_bounded_w(&qm_full[st], (r / kKvStages) & 1u, args.status, 56)) { ok = false; break; }
          }
          tc_fence_after();
          const uint64_t qmd =
              make_smem_desc(stages_addr + st * kKvStageBytes + 2 * kColTileBytes, kColChunk, 512, kLayoutSw128Base32);
          const uint64_t domd =
              make_smem_desc(stages_addr + st * kKvStageBytes + 3 * kColTileBytes, kColChunk, 512, kLayoutSw128Base32);
          const uint32_t ts = tm_s(g), tp = tm_dp(g);
          const uint32_t acc0 = u != 0 ? 1u : 0u;
#pragma unroll
          for (int ks = 0; ks < TN / 8; ++ks)
            umma_tf32_ta_w(tm_dv, ts + static_cast<uint32_t>(ks * 8), domd + ((ks * 1024) >> 4), id_mn, ks != 0 ? 1u : acc0);
#pragma unroll
          for (int ks = 0; ks < TN / 8; ++ks)
            umma_tf32_ta_w(tm_dk, tp + static_cast<uint32_t>(ks * 8), qmd + ((ks * 1024) >> 4), id_mn, ks != 0 ? 1u : acc0);
          umma_commit_w(&qm_empty[st]);
          if (u == w.n_units - 1) umma_commit_w(done_bar);
          if (u + 2 < w.n_units) ok = issue_sdp(u + 2);
        }
        g0 += static_cast<uint32_t>(w.n_units);
        r0 += static_cast<uint32_t>(w.n_units) + 1u;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- compute warps -------------------------------
    // Warp pair (w, w+4) shares a lane quarter; each thread owns one key row and 32 of the 64
    // queries of a unit.
    const int cw = warp - 2;
    const int qd = warp & 3, half = cw >> 2;
    const int ctid = cw * 32 + lane;   // 0..255
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sc2 = args.scale * kLog2ef;
    float* stg = reinterpret_cast<float*>(o_stage + cw * 2048);
    uint32_t g0 = 0, r0 = 0, n_it = 0;
    bool ok = true;
    for (;; ++n_it) {
      if (!mbar_wait_bounded(&iq_full[n_it & 1u], (n_it >> 1) & 1u, args.status, 61)) break;
      const int it = item_q[n_it & 1u];
      mbar_arrive(&iq_empty[n_it & 1u]);
      if (it < 0 || !ok) break;
      const KvItem w = kv_item(args, it);
      const int key = w.k0 + qd * 32 + lane;
      const int col_k = (args.H + w.hk) * D, col_v = (args.H + args.Hk + w.hk) * D;
      // per-query constants of unit u: threads 0..63 fetch -lse*log2e, threads 64..127 -delta*scale
      auto fetch_const = [&](int u) {
        float r = 0.0f;
        if (ctid < 2 * TN && u < w.n_units) {
          const int gi = u / w.per_head;
          const int q = (w.first_qt + (u - gi * w.per_head)) * TN + (ctid & (TN - 1));
          const int64_t lbase = (static_cast<int64_t>(w.b) * args.H + w.hk * G + gi) * args.T;
          if (ctid < TN) r = q < args.T ? -args.lse[lbase + q] * kLog2ef : -FLT_MAX;
          else r = q < args.T ? -args.delta[lbase + q] * args.scale : 0.0f;
        }
        return r;
      };
      float next_const = fetch_const(0);
      // K (first warp of the pair) or V (second) row of this thread: shared -> tensor memory.
      // The tensor-memory copies of the previous item are free: its last MMA was awaited below.
      {
        const uint32_t st = r0 % kKvStages, ph = (r0 / kKvStages) & 1u;
        if (!mbar_wait_bounded(half == 0 ? &qk_full[st] : &qm_full[st], ph, args.status, 62)) { ok = false; break; }
        float v[64];
        load_row_sw128(stages + st * kKvStageBytes + half * kRowTileBytes, qd * 32 + lane, v);
        tmem_st_32x64((half == 0 ? tm_ka : tm_va) + lane_off, *reinterpret_cast<uint32_t(*)[64]>(v));
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive(kvt_ready);
      for (int u = 0; u < w.n_units && ok; ++u) {
        const uint32_t g = g0 + static_cast<uint32_t>(u);
        const int gi = u / w.per_head;
        const int q0 = (w.first_qt + (u - gi * w.per_head)) * TN;
        // Three constant buffers: a thread can run at most two units ahead of the slowest one
        // (S^T(u) is only issued once every thread has delivered P^T(u-2)), so the buffer
        // written here is no longer being read.
        const uint32_t cb = g % 3u;
        float* nl = s_nl + cb * TN;
        float* nd = s_nd + cb * TN;
        if (ctid < 2 * TN) {
          if (ctid < TN) nl[ctid] = next_const;
          else nd[ctid - TN] = next_const;
          mbar_arrive(&const_full[cb]);
        }
        next_const = fetch_const(u + 1);
        {
          if (!mbar_wait_bounded(&const_full[cb], (g / 3u) & 1u, args.status, 59)) { ok = false; break; }
        }
        {
          if (!mbar_wait_bounded(&sdp_full[g & 1u], (g >> 1) & 1u, args.status, 57)) { ok = false; break; }
        }
        tc_fence_after();
        const uint32_t ts = tm_s(g) + lane_off + static_cast<uint32_t>(half * 32);
        const uint32_t tp = tm_dp(g) + lane_off + static_cast<uint32_t>(half * 32);
        float sv[32], dv[32];
        tmem_ld_32x32_nowait(ts, sv);
        tmem_ld_32x32_nowait(tp, dv);
        tmem_wait_ld();
        uint32_t* pb = reinterpret_cast<uint32_t*>(sv);
        uint32_t* db = reinterpret_cast<uint32_t*>(dv);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(nl + half * 32 + i);
          const float4 d4 = *reinterpret_cast<const float4*>(nd + half * 32 + i);
          float t0, t1, t2, t3, u0, u1, u2, u3;
          ffma2(t0, t1, sv[i], sv[i + 1], sc2, sc2, l4.x, l4.y);
          ffma2(t2, t3, sv[i + 2], sv[i + 3], sc2, sc2, l4.z, l4.w);
          ffma2(u0, u1, dv[i], dv[i + 1], args.scale, args.scale, d4.x, d4.y);
          ffma2(u2, u3, dv[i + 2], dv[i + 3], args.scale, args.scale, d4.z, d4.w);
          t0 = ex2f(t0);
          t1 = ex2f(t1);
          t2 = ex2f(t2);
          t3 = ex2f(t3);
          fmul2(u0, u1, t0, t1, u0, u1);
          fmul2(u2, u3, t2, t3, u2, u3);
          pb[i] = rna_bits(t0);
          pb[i + 1] = rna_bits(t1);
          pb[i + 2] = rna_bits(t2);
          pb[i + 3] = rna_bits(t3);
          db[i] = rna_bits(u0);
          db[i + 1] = rna_bits(u1);
          db[i + 2] = rna_bits(u2);
          db[i + 3] = rna_bits(u3);
        }
        if (q0 < w.k0 + TM) {   // queries that may lie before this tile's last key: causal mask
          const int qq = q0 + half * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const bool dead = key > qq + i;
            pb[i] = dead ? 0u : pb[i];
            db[i] = dead ? 0u : db[i];
          }
        }
        tmem_st_32x32(ts, *reinterpret_cast<uint32_t(*)[32]>(pb));
        tmem_st_32x32(tp, *reinterpret_cast<uint32_t(*)[32]>(db));
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&pds_ready[g & 1u]);
      }
      g0 += static_cast<uint32_t>(w.n_units);
      r0 += static_cast<uint32_t>(w.n_units) + 1u;
      {
        if (!ok || !mbar_wait_bounded(done_bar, n_it & 1u, args.status, 58)) { ok = false; break; }
      }
      tc_fence_after();
      {
        float* rowp = args.dqkv + (static_cast<int64_t>(w.b) * args.T + w.k0 + qd * 32) * RS;
        const int rows_left = args.T - (w.k0 + qd * 32);
        float v[32];
        tmem_ld_32x32(tm_dv + lane_off + static_cast<uint32_t>(half * 32), v);
        store_block_32x32(stg, v, rowp + col_v + half * 32, RS, rows_left, lane);
        tmem_ld_32x32(tm_dk + lane_off + static_cast<uint32_t>(half * 32), v);
        store_block_32x32(stg, v, rowp + col_k + half * 32, RS, rows_left, lane);
      }
      tc_fence_before();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// 4-D view {32 floats, T rows, width / 32 column groups, B} of a [B, T, width] buffer; a box takes
// `rows` rows of `groups` consecutive column groups and lands as [group][row][32 floats].
int map4(CUtensorMap* m, const float* base, int64_t width, int64_t T, int64_t B, int rows, int groups, bool atom32) {
  const uint64_t dims[4] = {32u, static_cast<uint64_t>(T), static_cast<uint64_t>(width / 32), static_cast<uint64_t>(B)};
  const uint64_t strides[3] = {static_cast<uint64_t>(width) * 4, 128u, static_cast<uint64_t>(T) * width * 4};
  const uint32_t box[4] = {32u, static_cast<uint32_t>(rows), static_cast<uint32_t>(groups), 1u};
  return encode_tensor_map(m, base, 4, dims, strides, box, atom32);
}

}  // namespace

// dQ part of the backward for D = 64. Returns CTDK_OK or a negative status.
int attn_bwd_dq_tc64(const float* qkv, const float* dout, const float* lse, const float* delta, float* dqkv,
                     int64_t B, int64_t T, int H, int Hk, cudaStream_t stream) {
  const int64_t RS = static_cast<int64_t>(H + 2 * Hk) * D, HD = static_cast<int64_t>(H) * D;
  Bwd64Args a;
  a.lse = lse;
  a.delta = delta;
  a.dqkv = dqkv;
  a.T = static_cast<int>(T);
  a.H = H;
  a.Hk = Hk;
  a.B = static_cast<int>(B);
  a.n_tiles = static_cast<int>((T + TM - 1) / TM);
  const int64_t items = static_cast<int64_t>(a.n_tiles) * H * B;
  if (items > INT32_MAX) return 1;
  a.n_items = static_cast<int>(items);
  a.scale = 1.0f / sqrtf(static_cast<float>(D));
  a.status = device_status_word();
  a.work_counter = nullptr;
  if (a.status == nullptr) return fail(CTDK_ELAUNCH, "attn_bwd(tcgen05): no status word");
  CUtensorMap tq, tdo, tkv, tkm;
  int rc = map4(&tq, qkv, RS, T, B, TM, D / 32, false);
  if (rc == CTDK_OK) rc = map4(&tdo, dout, HD, T, B, TM, D / 32, false);
  if (rc == CTDK_OK) rc = map4(&tkm, qkv, RS, T, B, TN, D / 32, true);
  if (rc == CTDK_OK) {
    // K and V tiles of one key/value head in one box: a fifth dimension steps from the K columns
    // to the V columns (Hk * D floats further on).
    const uint64_t dims[5] = {32u, static_cast<uint64_t>(T), static_cast<uint64_t>(RS / 32), 2u, static_cast<uint64_t>(B)};
    const uint64_t strides[4] = {static_cast<uint64_t>(RS) * 4, 128u, static_cast<uint64_t>(Hk) * D * 4,
                                 static_cast<uint64_t>(T) * RS * 4};
    const uint32_t box[5] = {32u, static_cast<uint32_t>(TN), static_cast<uint32_t>(D / 32), 2u, 1u};
    rc = encode_tensor_map(&tkv, qkv, 5, dims, strides, box, false);
  }
  if (rc != CTDK_OK) return rc;
  cudaError_t e = cudaFuncSetAttribute(attn_bwd_dq64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqSmem);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "attn_bwd dq(tcgen05): shared memory opt-in failed: %s", cudaGetErrorString(e));
  const int sms = sm_budget();
  launch_pdl(attn_bwd_dq64_kernel, dim3(a.n_items < sms ? a.n_items : sms), dim3(320), kDqSmem, stream, tq, tdo, tkv, tkm, a);
  return check_launch("ctdk_attn_bwd(dq, tcgen05)");
}

namespace {
// Work counters of the dK/dV kernel: every call takes the next one of a ring and zeroes it in its
// own stream, so calls on different streams of a device do not draw from each other's sequence.
// A counter is reused after kKvCounters further calls, long after its kernel has finished.
constexpr int kKvCounters = 64;
__device__ int g_kv_work_counter[kKvCounters];
std::atomic<unsigned> g_kv_counter_next{0};
}  // namespace

// dK/dV part of the backward for D = 64. Returns CTDK_OK or a negative status.
int attn_bwd_dkv_tc64(const float* qkv, const float* dout, const float* lse, const float* delta, float* dqkv,
                      int64_t B, int64_t T, int H, int Hk, cudaStream_t stream) {
  const int64_t RS = static_cast<int64_t>(H + 2 * Hk) * D, HD = static_cast<int64_t>(H) * D;
  Bwd64Args a;
  a.lse = lse;
  a.delta = delta;
  a.dqkv = dqkv;
  a.T = static_cast<int>(T);
  a.H = H;
  a.Hk = Hk;
  a.B = static_cast<int>(B);
  a.n_tiles = static_cast<int>((T + TM - 1) / TM);
  const int64_t items = static_cast<int64_t>(a.n_tiles) * Hk * B;
  if (items > INT32_MAX) return 1;
  a.n_items = static_cast<int>(items);
  a.scale = 1.0f / sqrtf(static_cast<float>(D));
  a.status = device_status_word();
  if (a.status == nullptr) return fail(CTDK_ELAUNCH, "attn_bwd(tcgen05): no status word");
  {
    void* cptr = nullptr;
    if (cudaGetSymbolAddress(&cptr, g_kv_work_counter) != cudaSuccess || cptr == nullptr)
      return fail(CTDK_ELAUNCH, "attn_bwd dkv(tcgen05): no work counter");
    a.work_counter = static_cast<int*>(cptr) + g_kv_counter_next.fetch_add(1, std::memory_order_relaxed) % kKvCounters;
    if (cudaMemsetAsync(a.work_counter, 0, sizeof(int), stream) != cudaSuccess)
      return fail(CTDK_ELAUNCH, "attn_bwd dkv(tcgen05): counter reset failed");
  }
  CUtensorMap tqk, tdok, tqm, tdom, tkvt;
  int rc = map4(&tqk, qkv, RS, T, B, TN, D / 32, false);
  if (rc == CTDK_OK) rc = map4(&tkvt, qkv, RS, T, B, TM, D / 32, false);
  if (rc == CTDK_OK) rc = map4(&tdok, dout, HD, T, B, TN, D / 32, false);
  if (rc == CTDK_OK) rc = map4(&tqm, qkv, RS, T, B, TN, D / 32, true);
  if (rc == CTDK_OK) rc = map4(&tdom, dout, HD, T, B, TN, D / 32, true);
  if (rc != CTDK_OK) return rc;
  cudaError_t e = cudaFuncSetAttribute(attn_bwd_dkv64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kKvSmem);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "attn_bwd dkv(tcgen05): shared memory opt-in failed: %s", cudaGetErrorString(e));
  const int sms = sm_budget();
  launch_pdl(attn_bwd_dkv64_kernel, dim3(a.n_items < sms ? a.n_items : sms), dim3(320), kKvSmem, stream, tqk, tdok, tqm, tdom, tkvt, a);
  return check_launch("ctdk_attn_bwd(dkv, tcgen05)");
}

}  // namespace ctdk
