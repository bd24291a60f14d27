// TF32 GEMM with paired CTAs (tcgen05 cta_group::2): a cluster of two CTAs on one TPC computes a
// 256 x 256 output tile. Each CTA loads its own 128 rows of A and only HALF of the B tile
// (128 of the 256 columns) per k-block; the tensor cores of both SMs read both halves. Per FLOP
// this moves one third fewer operand bytes through L2 and shared memory than the one-CTA
// 128 x 256 tile of gemm_tcgen05.cu, which is what bounds that kernel with 4-byte operands.
//
// Roles per CTA (10 warps): TMA producer, MMA warp, 8 epilogue warps. Only the even CTA of the
// pair (the leader) issues MMAs; both CTAs' TMA loads report their bytes to the leader's
// "full" barrier; the leader releases stages and publishes finished accumulators to both CTAs
// with a multicast tcgen05.commit; both CTAs' epilogue warps report to the leader's
// "accumulator free" barrier. Loads are plain per-CTA TMA loads. All waits are bounded.
#include <cuda.h>

#include "common.cuh"

namespace ctdk {
namespace {

constexpr int BM2 = 128;                 // rows of A per CTA (pair: 256)
constexpr int BN2 = 256;                 // tile width (each CTA loads 128 columns of B)
constexpr int BK2 = 32;
constexpr int kATile = BM2 * BK2 * 4;    // 16 KB
constexpr int kBHalf = (BN2 / 2) * BK2 * 4;  // 16 KB
constexpr int kStage2 = kATile + kBHalf;
constexpr int kStages2 = 6;
constexpr int kChunk2 = 32 * BK2 * 4;    // one {32 x 32} box of an MN-major operand
constexpr int kEpiBuf = 32 * 128;         // one {32 x 32} fp32 output box in transit
constexpr int kEpiWarps = 8;              // two per tensor-memory lane quarter, each takes half of the tile's columns
constexpr int kThreads2 = 32 * (2 + kEpiWarps);
constexpr int kEpiStage = kEpiWarps * kEpiBuf;  // one staging box per epilogue warp (two for the SwiGLU backward, which runs 5 stages)
constexpr int kTiles2 = kStages2 * kStage2 + kEpiStage;   // operand ring + output staging: 224 KB, split per mode
constexpr int kSmem2 = kTiles2 + 1024 + 256;
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address
constexpr int kGroupM2 = 8;

struct Gemm2Args {
  float* C;
  const float* aux;
  int64_t ldc;
  int M, N, K;
  int epilogue;
  int vec_ok;
  int splits;  // K ranges per tile; >1: partial tiles are added to C with atomics
  int a3d, b3d;   // MN-major operand described by a 3-D map: one {32 x 32 x 4} box per k-block
  int tma_out;    // 1: C is written (2: added to) through TMA from shared-memory staging
  int swiglu;     // 1: B = [gate rows; up rows] of an MLP ([2N, K]); C = packed gate|up [M, 2N] and a second
                  //    output act = silu(gate) * up [M, N]: each tile holds 128 gate and the matching 128 up columns
                  // 2: the product is d(act) [M, N]; the epilogue reads gate|up [M, 2N] through map C and
                  //    writes d(gate)|d(up) [M, 2N] through map D (SwiGLU backward), d(act) is never stored
  int narrow;     // 1: the plain epilogue (store / add of the bare accumulator) is run by the first warp of each lane
                  //    quarter through both staging boxes of its pair, which measured ~1 % faster than eight warps with
                  //    one box each; the epilogues that compute (SwiGLU, +residual) use all eight warps
  float* delta;   // != nullptr: C = d(attention output) [M, N = H * dl_D]; map D covers the attention output itself and the
                  // epilogue also writes delta[(b * dl_H + h) * dl_T + t] = sum over the head's columns of C * O, the row
                  // term of the softmax backward (row = b * dl_T + t); needs swiglu == 0, splits == 1, a plain store
  int dl_T, dl_H, dl_D;
  int stages;     // operand ring depth: 6, or 5 when the epilogue needs 64 KB of staging (swiglu == 2)
  int* status;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Load into this CTA's shared memory; the bytes are counted on the LEADER CTA's barrier.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & kPeerMask), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                                 int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & kPeerMask), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Shared-memory box -> global tile (out-of-range rows / columns are clipped by the map).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
// Same, but added to the tile in global memory (fp32 add performed at L2).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, const void* smem_src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this offset in BOTH CTAs of the pair once prior MMAs retire.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "{\n"
      ".reg .b16 m;\n"
      "mov.b16 m, 3;\n"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n"
      "}\n" ::"r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kPeerMask)
               : "memory");
}

__device__ __forceinline__ void tile_coords2(int tile, int m_blocks, int n_blocks, int& mb, int& nb) {
  const int per_group = kGroupM2 * n_blocks;
  const int g = tile / per_group;
  const int first_m = g * kGroupM2;
  const int gm = min(kGroupM2, m_blocks - first_m);
  const int local = tile - g * per_group;
  mb = first_m + local % gm;
  nb = local / gm;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
    gemm_tf32_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmD,
                          const Gemm2Args args) {
  extern __shared__ unsigned char smem_raw[];
  pdl_launch();   // the next kernel in the stream may set itself up while this one runs
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  const int n_stages = args.stages;
  unsigned char* epi_stage = smem + n_stages * kStage2;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kTiles2);
  uint64_t* full = bars;                   // [kStages2]  used in the leader only
  uint64_t* empty = bars + kStages2;       // [kStages2]  one per CTA, signalled by multicast commit
  uint64_t* tfull = bars + 2 * kStages2;   // [2]         one per CTA, multicast commit
  uint64_t* tempty = tfull + 2;            // [2]         leader only, 16 arrivals (8 warps x 2 CTAs)
  uint64_t* ld_bar = tempty + 2;           // [8 warps]   gate / up boxes of the SwiGLU-backward epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ld_bar + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int m_blocks = (args.M + 2 * BM2 - 1) / (2 * BM2);
  const int n_blocks = args.swiglu == 1 ? args.N / (BN2 / 2) : (args.N + BN2 - 1) / BN2;
  const int num_tiles = m_blocks * n_blocks;
  const int k_blocks = (args.K + BK2 - 1) / BK2;
  const int num_units = num_tiles * args.splits;  // unit u: tile u % num_tiles, k-range u / num_tiles
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 2 * kEpiWarps);
    }
    for (int a = 0; a < 8; ++a) mbar_init(&ld_bar[a], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (args.tma_out) tma_prefetch_desc(&tmC);
    if (args.swiglu || args.delta != nullptr) tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote signal
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();     // operands (and C, when it is accumulated into) come from earlier kernels

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int unit = pair; unit < num_units && ok; unit += n_pairs) {
        int mb, nb;
        tile_coords2(unit % num_tiles, m_blocks, n_blocks, mb, nb);
        const int m0 = mb * 2 * BM2 + static_cast<int>(rank) * BM2;
        // B rows of this CTA: its half of the 256 columns, or (fused SwiGLU) 128 gate rows in the
        // even CTA and the matching 128 up rows, N rows further on, in the odd one
        const int n0 = args.swiglu == 1 ? nb * (BN2 / 2) + static_cast<int>(rank) * args.N
                                   : nb * BN2 + static_cast<int>(rank) * (BN2 / 2);
        const int split = unit / num_tiles;
        const int kb0 = static_cast<int>(static_cast<int64_t>(split) * k_blocks / args.splits);
        const int kb1 = static_cast<int>(static_cast<int64_t>(split + 1) * k_blocks / args.splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          {
            if (!mbar_wait_bounded(&empty[s], ph ^ 1u, args.status, 61)) {
              ok = false;
              break;
            }
          }
          unsigned char* a_dst = smem + s * kStage2;
          unsigned char* b_dst = a_dst + kATile;
          if (leader) mbar_expect_tx(&full[s], 2 * kStage2);  // bytes of both CTAs
          const int k0 = kb * BK2;
          if (A_MN) {
            if (args.a3d) {
              tma_load_3d_pair(a_dst, &tmA, &full[s], 0, k0, m0 >> 5);
            } else {
#pragma unroll
              for (int c = 0; c < BM2 / 32; ++c)
                tma_load_2d_pair(a_dst + c * kChunk2, &tmA, &full[s], m0 + 32 * c, k0);
            }
          } else {
            tma_load_2d_pair(a_dst, &tmA, &full[s], k0, m0);
          }
          if (B_MN) {
            if (args.b3d) {
              tma_load_3d_pair(b_dst, &tmB, &full[s], 0, k0, n0 >> 5);
            } else {
#pragma unroll
              for (int c = 0; c < BN2 / 64; ++c)
                tma_load_2d_pair(b_dst + c * kChunk2, &tmB, &full[s], n0 + 32 * c, k0);
            }
          } else {
            tma_load_2d_pair(b_dst, &tmB, &full[s], k0, n0);
          }
          if (++s == n_stages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      // M = 256 (both CTAs), N = 256
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(A_MN) << 15) |
                             (static_cast<uint32_t>(B_MN) << 16) | (static_cast<uint32_t>(BN2 >> 3) << 17) |
                             (static_cast<uint32_t>(256 >> 4) << 24);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      for (int unit = pair; unit < num_units && ok; unit += n_pairs, ++it) {
        const int split = unit / num_tiles;
        const int kb0 = static_cast<int>(static_cast<int64_t>(split) * k_blocks / args.splits);
        const int kb1 = static_cast<int>(static_cast<int64_t>(split + 1) * k_blocks / args.splits);
        const int acc = it & 1;
        const uint32_t acc_ph = (static_cast<uint32_t>(it) >> 1) & 1u;
        {
          if (!mbar_wait_bounded(&tempty[acc], acc_ph ^ 1u, args.status, 62)) {
            ok = false;
            break;
          }
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN2);
        for (int kb = kb0; kb < kb1; ++kb) {
          {
            if (!mbar_wait_bounded(&full[s], ph, args.status, 63)) {
              ok = false;
              break;
            }
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * kStage2);
          const uint32_t b_addr = a_addr + kATile;
#pragma unroll
          for (int ks = 0; ks < BK2 / 8; ++ks) {
            const uint64_t adesc = A_MN ? make_smem_desc(a_addr + ks * 1024, kChunk2, 512, kLayoutSw128Base32)
                                        : make_smem_desc(a_addr + ks * 32, 16, 1024, kLayoutSw128);
            const uint64_t bdesc = B_MN ? make_smem_desc(b_addr + ks * 1024, kChunk2, 512, kLayoutSw128Base32)
                                        : make_smem_desc(b_addr + ks * 32, 16, 1024, kLayoutSw128);
            umma_tf32_pair(d_tmem, adesc, bdesc, idesc, (kb != kb0 || ks != 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty[s]);
          if (++s == n_stages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) umma_commit_pair(&tfull[acc]);
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (both CTAs, own 128 rows, all 256 columns) ----------------
    // A warp may read the tensor-memory lanes of quarter (warp id % 4); the two warps of a quarter
    // take the first and the second half of the tile's 32-column chunks.
    const int q = warp & 3;
    const int ew = warp - 2, half = ew >> 2;
    const int row_in_tile = static_cast<int>(rank) * BM2 + q * 32 + lane;
    int it = 0;
    bool ok = true;
    uint32_t chunk_cnt = 0;   // chunks this warp has fetched gate / up boxes for (SwiGLU backward): the parity of its barrier
    for (int unit = pair; unit < num_units && ok; unit += n_pairs, ++it) {
      int mb, nb;
      tile_coords2(unit % num_tiles, m_blocks, n_blocks, mb, nb);
      const bool first_split = unit < num_tiles;
      const bool atomic = args.splits > 1;
      const int acc = it & 1;
      const uint32_t acc_ph = (static_cast<uint32_t>(it) >> 1) & 1u;
      {
        if (!mbar_wait_bounded(&tfull[acc], acc_ph, args.status, 64)) {
          ok = false;
          break;
        }
      }
      tc_fence_after();
      const int64_t grow = static_cast<int64_t>(mb) * 2 * BM2 + row_in_tile;
      const bool row_ok = grow < args.M;
      float* crow = args.C + grow * args.ldc;
      const float* xrow = args.aux != nullptr ? args.aux + grow * args.ldc : nullptr;
      const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * BN2) + (static_cast<uint32_t>(q * 32) << 16);
      if (args.swiglu == 2) {
        // SwiGLU backward on the accumulator: d(act) stays in registers; the gate and up boxes of a
        // chunk are fetched by TMA into the warp's box pair, turned into d(gate) and d(up) in place
        // and stored from there (the eight warps of the CTA hide one another's fetch latency).
        const int r0 = mb * 2 * BM2 + static_cast<int>(rank) * BM2 + q * 32;
        int n_ch = (args.N - nb * BN2 + 31) / 32;
        if (n_ch > BN2 / 32) n_ch = BN2 / 32;
        unsigned char* boxes = epi_stage + ew * (2 * kEpiBuf);   // [gate, up]
        const int ch_end = n_ch < half * 4 + 4 ? n_ch : half * 4 + 4;
#pragma unroll 1
        for (int ch = half * 4; ch < ch_end && ok; ++ch) {
          if (lane == 0) {
            bulk_wait_read<0>();   // the boxes were last read by the stores of the chunk before
            const int col = nb * BN2 + ch * 32;
            mbar_expect_tx(&ld_bar[ew], 2 * kEpiBuf);
            tma_load_2d(boxes, &tmC, &ld_bar[ew], col, r0);
            tma_load_2d(boxes + kEpiBuf, &tmC, &ld_bar[ew], args.N + col, r0);
          }
          float v[32];
          tmem_ld_32x32(t_row + static_cast<uint32_t>(ch * 32), v);
          if (!mbar_wait_bounded(&ld_bar[ew], chunk_cnt & 1u, args.status, 65)) {
            ok = false;
            break;
          }
          ++chunk_cnt;
          unsigned char* bg = boxes + lane * 128;
          unsigned char* bu = bg + kEpiBuf;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const int off = (c ^ (lane & 7)) << 4;
            const float4 g = *reinterpret_cast<const float4*>(bg + off);
            const float4 u = *reinterpret_cast<const float4*>(bu + off);
            float4 dg, du;
            swiglu_bwd_elem(v[4 * c], g.x, u.x, dg.x, du.x);
            swiglu_bwd_elem(v[4 * c + 1], g.y, u.y, dg.y, du.y);
            swiglu_bwd_elem(v[4 * c + 2], g.z, u.z, dg.z, du.z);
            swiglu_bwd_elem(v[4 * c + 3], g.w, u.w, dg.w, du.w);
            *reinterpret_cast<float4*>(bg + off) = dg;
            *reinterpret_cast<float4*>(bu + off) = du;
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int col = nb * BN2 + ch * 32;
            if (r0 < args.M) {
              tma_store_2d(&tmD, boxes, col, r0);
              tma_store_2d(&tmD, boxes + kEpiBuf, args.N + col, r0);
            }
            bulk_commit();
          }
          __syncwarp();
        }
      } else if (args.delta != nullptr) {
        // d(attention output) tile: stored as it is, and dotted with the same tile of the attention
        // output O on the way: a lane holds one row, a warp's four chunks are whole heads (two of 64
        // columns or one of 128). O's box is fetched by TMA while the accumulator chunk is staged
        // and sent.
        const int r0 = mb * 2 * BM2 + static_cast<int>(rank) * BM2 + q * 32;
        int n_ch = (args.N - nb * BN2 + 31) / 32;
        if (n_ch > BN2 / 32) n_ch = BN2 / 32;
        unsigned char* box_o = epi_stage + ew * (2 * kEpiBuf);
        unsigned char* box_c = box_o + kEpiBuf;
        const int ch_end = n_ch < half * 4 + 4 ? n_ch : half * 4 + 4;
        const int cph = args.dl_D >> 5;   // chunks per head
        const int64_t bsq = grow / args.dl_T;
        float* drow = args.delta + bsq * args.dl_H * args.dl_T + (grow - bsq * args.dl_T);
        float hsum = 0.0f;
#pragma unroll 1
        for (int ch = half * 4; ch < ch_end && ok; ++ch) {
          const int col = nb * BN2 + ch * 32;
          if (lane == 0) {
            bulk_wait_read<0>();   // the staging box's last store has left
            mbar_expect_tx(&ld_bar[ew], kEpiBuf);
            tma_load_2d(box_o, &tmD, &ld_bar[ew], col, r0);
          }
          float v[32];
          tmem_ld_32x32(t_row + static_cast<uint32_t>(ch * 32), v);
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<float4*>(box_c + lane * 128 + ((c ^ (lane & 7)) << 4)) =
                make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (r0 < args.M) tma_store_2d(&tmC, box_c, col, r0);
            bulk_commit();
          }
          if (!mbar_wait_bounded(&ld_bar[ew], chunk_cnt & 1u, args.status, 66)) {
            ok = false;
            break;
          }
          ++chunk_cnt;
          const unsigned char* bo = box_o + lane * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 o = *reinterpret_cast<const float4*>(bo + ((c ^ (lane & 7)) << 4));
            hsum += v[4 * c] * o.x + v[4 * c + 1] * o.y + v[4 * c + 2] * o.z + v[4 * c + 3] * o.w;
          }
          if ((ch + 1) % cph == 0) {
            if (row_ok) drow[static_cast<int64_t>(col / args.dl_D) * args.dl_T] = hsum;
            hsum = 0.0f;
          }
          fence_async_smem();   // the reads of O's box come before the next fetch into it
          __syncwarp();
        }
      } else if (args.swiglu) {
        // columns 0..127 of the accumulator are gate, 128..255 the matching up columns: three boxes
        // per 32-column chunk (gate and up into the packed buffer, silu(gate)*up into the second
        // output) through the warp's staging box
        const int r0 = mb * 2 * BM2 + static_cast<int>(rank) * BM2 + q * 32;
        auto send = [&](const float (&v)[32], const CUtensorMap* map, int col) {
          unsigned char* buf = epi_stage + ew * kEpiBuf;
          if (lane == 0) bulk_wait_read<0>();   // the box sent before has left
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<float4*>(buf + lane * 128 + ((c ^ (lane & 7)) << 4)) =
                make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (r0 < args.M) tma_store_2d(map, buf, col, r0);
            bulk_commit();
          }
        };
#pragma unroll 1
        for (int ch = half * 2; ch < half * 2 + 2; ++ch) {
          const int col = nb * (BN2 / 2) + ch * 32;
          float g[32], u[32];
          tmem_ld_32x32(t_row + static_cast<uint32_t>(ch * 32), g);
          tmem_ld_32x32(t_row + static_cast<uint32_t>(BN2 / 2 + ch * 32), u);
          send(g, &tmC, col);
          send(u, &tmC, args.N + col);
#pragma unroll
          for (int i = 0; i < 32; ++i) g[i] = g[i] / (1.0f + __expf(-g[i])) * u[i];
          send(g, &tmD, col);
        }
      } else if (args.epilogue == CTDK_EPI_RESIDUAL && !atomic && args.vec_ok && (args.N & 3) == 0) {
        // C = acc + aux. Lane i holds row i of a chunk after tcgen05.ld; read and written like
        // that, every 16-byte access would touch its own 128-byte line. So the chunk goes through
        // a 4 KB shared-memory tile (128-byte rows, 16-byte pieces XORed with the row number) and
        // comes back with 8 lanes covering one 128-byte row: coalesced loads of aux (fetched one
        // chunk ahead) and coalesced stores of C.
        const int r0 = mb * 2 * BM2 + static_cast<int>(rank) * BM2 + q * 32;
        const int lr = lane >> 3, lc = lane & 7;   // after the transpose: rows j*4+lr, columns lc*4..+3
        float* buf = reinterpret_cast<float*>(epi_stage + ew * kEpiBuf);
        float4 X[8], Xn[8];
        auto fetch = [&](int ch, float4 (&x)[8]) {
          const int col = nb * BN2 + ch * 32 + lc * 4;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int64_t row = r0 + j * 4 + lr;
            x[j] = (row < args.M && col < args.N) ? __ldg(reinterpret_cast<const float4*>(args.aux + row * args.ldc + col))
                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        };
        fetch(half * 4, X);
#pragma unroll 1
        for (int ch = half * 4; ch < half * 4 + 4; ++ch) {
          const int col0 = nb * BN2 + ch * 32;
          if (col0 >= args.N) break;
          if (ch + 1 < half * 4 + 4) fetch(ch + 1, Xn);
          float v[32];
          tmem_ld_32x32(t_row + static_cast<uint32_t>(ch * 32), v);
          __syncwarp();   // the reads of the chunk before are done
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<float4*>(buf + lane * 32 + ((c ^ (lane & 7)) << 2)) =
                make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
          __syncwarp();
          const int col = col0 + lc * 4;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int rl = j * 4 + lr;
            const int64_t row = r0 + rl;
            float4 o = *reinterpret_cast<const float4*>(buf + rl * 32 + ((lc ^ (rl & 7)) << 2));
            o.x += X[j].x;
            o.y += X[j].y;
            o.z += X[j].z;
            o.w += X[j].w;
            if (row < args.M && col < args.N) *reinterpret_cast<float4*>(args.C + row * args.ldc + col) = o;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) X[j] = Xn[j];
        }
      } else
#pragma unroll 1
      for (int ch = args.narrow ? half * 8 : half * 4; ch < (args.narrow ? 8 : half * 4 + 4); ++ch) {
        const int col0 = nb * BN2 + ch * 32;
        if (col0 >= args.N) break;
        float v[32];
        tmem_ld_32x32(t_row + static_cast<uint32_t>(ch * 32), v);
        if (args.tma_out) {
          // 32 rows x 32 columns through a 4 KB staging box (128-byte rows, 16-byte chunks XORed
          // with the row number as the map's swizzle expects), then one TMA store / reduce-add.
          unsigned char* buf = epi_stage + (args.narrow ? ew + 4 * (ch & 1) : ew) * kEpiBuf;
          if (lane == 0) {
            if (!args.narrow) bulk_wait_read<0>();   // the box sent before has left
            else if (ch >= 2) bulk_wait_read<1>();
          }
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<float4*>(buf + lane * 128 + ((c ^ (lane & 7)) << 4)) =
                make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int r0 = mb * 2 * BM2 + static_cast<int>(rank) * BM2 + q * 32;
            if (r0 < args.M) {
              if (args.tma_out == 2) tma_reduce_add_2d(&tmC, buf, col0, r0);
              else tma_store_2d(&tmC, buf, col0, r0);
            }
            bulk_commit();
          }
        } else if (!row_ok) {
        } else if (atomic) {
          // split-K: C was zeroed (STORE / RESIDUAL) or holds the running sum (ACCUMULATE)
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
            for (int j = 0; j < 8; ++j) c4[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
            const float4* x4 = args.epilogue == CTDK_EPI_ACCUMULATE ? reinterpret_cast<const float4*>(crow + col0)
                                                                    : reinterpret_cast<const float4*>(xrow + col0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 x = x4[j];
              c4[j] = make_float4(v[4 * j] + x.x, v[4 * j + 1] + x.y, v[4 * j + 2] + x.z, v[4 * j + 3] + x.w);
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
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_leader(&tempty[acc]);
        if (args.tma_out) bulk_wait_read<0>();   // the staging box is free for the next tile (and before the CTA ends)
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer has drained its accumulators and sent its last signals
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

template <bool A_MN, bool B_MN>
int launch2(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& td,
            const Gemm2Args& args, cudaStream_t stream) {
  auto* kern = gemm_tf32_2cta_kernel<A_MN, B_MN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "gemm(2cta): shared memory opt-in failed: %s", cudaGetErrorString(e));
  const int tiles = ((args.M + 255) / 256) * (args.swiglu == 1 ? args.N / (BN2 / 2) : (args.N + BN2 - 1) / BN2) * args.splits;
  int pairs = sm_budget() / 2;
  if (tiles < pairs) pairs = tiles;
  e = launch_pdl(kern, dim3(2 * pairs), dim3(kThreads2), kSmem2, stream, ta, tb, tc, td, args);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "gemm(2cta): launch failed: %s", cudaGetErrorString(e));
  return check_launch("ctdk_gemm(tcgen05, cta pair)");
}

}  // namespace

// Enqueues the paired-CTA kernel. K-major operands: 2-D maps with {32, 128} boxes. MN-major operands:
// 2-D maps with {32, 32} boxes, or (a3d / b3d) 3-D maps {32 columns, K rows, columns / 32} with
// {32, 32, 4} boxes. tc: 2-D map of C with {32, 32} boxes, used when tma_out != 0.
int gemm_tcgen05_2cta(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, bool a_mn, bool b_mn,
                      bool a3d, bool b3d, int tma_out, float* C, const float* aux, int64_t ldc, int M, int N, int K,
                      int epilogue, int vec_ok, int splits, int* status, cudaStream_t stream) {
  Gemm2Args args{C, aux, ldc, M, N, K, epilogue, vec_ok, splits, a3d ? 1 : 0, b3d ? 1 : 0, tma_out, 0, 1, nullptr, 0, 0, 0, kStages2, status};
  if (!a_mn && !b_mn) return launch2<false, false>(ta, tb, tc, tc, args, stream);
  if (!a_mn && b_mn) return launch2<false, true>(ta, tb, tc, tc, args, stream);
  if (a_mn && !b_mn) return launch2<true, false>(ta, tb, tc, tc, args, stream);
  return launch2<true, true>(ta, tb, tc, tc, args, stream);
}

// Fused MLP input projection: gu[M, 2N] = A[M, K] * W[2N, K]^T (gate rows then up rows) and
// act[M, N] = silu(gate) * up. ta: A, {32, 128} boxes; tb: W, {32, 128} boxes; tgu / tact: the two
// outputs, {32, 32} boxes. N must be a multiple of 128.
int gemm_tcgen05_2cta_swiglu(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tgu, const CUtensorMap& tact,
                             int M, int N, int K, int* status, cudaStream_t stream) {
  Gemm2Args args{nullptr, nullptr, 0, M, N, K, CTDK_EPI_STORE, 1, 1, 0, 0, 1, 1, 0, nullptr, 0, 0, 0, kStages2, status};
  return launch2<false, false>(ta, tb, tgu, tact, args, stream);
}

// Fused SwiGLU backward: d(act)[M, N] = A[M, K] * B[K, N] (B MN-major, 3-D map when b3d) stays in the
// accumulator; tgu: gate|up [M, 2N] for loading, tdgu: d(gate)|d(up) [M, 2N] for storing, {32, 32} boxes.
int gemm_tcgen05_2cta_swiglu_bwd(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tgu, const CUtensorMap& tdgu,
                                 bool b3d, int M, int N, int K, int* status, cudaStream_t stream) {
  Gemm2Args args{nullptr, nullptr, 0, M, N, K, CTDK_EPI_STORE, 1, 1, 0, b3d ? 1 : 0, 1, 2, 0, nullptr, 0, 0, 0, kStages2 - 1, status};
  return launch2<false, true>(ta, tb, tgu, tdgu, args, stream);
}

// d(attention output)[M, N] = A[M, K] * B[K, N] (B MN-major, 3-D map when b3d), stored through map tc, and
// delta[b, h, t] = sum over head h's D columns of that product times the attention output (map to, {32, 32} boxes).
int gemm_tcgen05_2cta_dattn_delta(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& to,
                                  bool b3d, float* delta, int M, int N, int K, int T, int H, int D, int* status,
                                  cudaStream_t stream) {
  Gemm2Args args{nullptr, nullptr, 0, M, N, K, CTDK_EPI_STORE, 1, 1, 0, b3d ? 1 : 0, 1, 0, 0, delta, T, H, D, kStages2 - 1, status};
  return launch2<false, true>(ta, tb, tc, to, args, stream);
}

}  // namespace ctdk
