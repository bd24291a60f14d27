/* ctdk — C-ABI of the sm_100a kernels behind emberlm's decoder training step.
 *
 * Every entry point takes raw device pointers and sizes, enqueues work on `stream`
 * (a cudaStream_t passed as void*; NULL = the legacy default stream, which is what the
 * reference runs on) and returns 0 or a negative CTDK_E* status. Unless stated, entry
 * points never allocate, never synchronise and never throw; ctdk_last_error() returns
 * the message of the calling thread's last failure. Tensors are fp32, row-major and
 * contiguous unless a leading dimension is given, exactly as the reference's ops demand
 * (e.g. src/ops/elementwise.cu:71-81 in the reference).
 *
 * Each declaration cites the reference interface (file:line inside KyleCr4ne/emberlm)
 * whose arithmetic it replaces.
 */
#ifndef CTDK_H_
#define CTDK_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CTDK_OK 0
#define CTDK_EINVAL (-1)   /* bad argument (shape, alignment, null pointer) */
#define CTDK_ELAUNCH (-2)  /* CUDA reported an error at launch / encode time */
#define CTDK_ETIMEOUT (-3) /* a bounded device-side wait ran out (status word set) */
#define CTDK_ENOMEM (-4)   /* an allocating entry point could not allocate */

const char* ctdk_last_error(void);
/* Reads (and clears) the device status word written by bounded waits; synchronises
 * `stream`. Returns 0 or CTDK_ETIMEOUT; where[0..3] (optional) receives the raw words. */
int ctdk_device_status(void* stream, int* where);
int ctdk_sm_count(void);
/* Leaves n SMs (rounded down to whole pairs) out of the grids of the persistent tensor-core kernels
 * (GEMM, attention), for kernels that run beside them on other streams: a collective that takes a few
 * SMs while a one-wave persistent GEMM wants all of them makes that GEMM run in two waves. 0 restores
 * the default. Process-wide; set it before the step loop, not between launches in flight. */
int ctdk_reserve_sms(int n);
/* Number of kernel launches this library has enqueued in this process. */
long long ctdk_launch_count(void);
/* Optional live timing: while enabled, every launch of a profiled class is bracketed by CUDA
 * events on its own stream. ctdk_prof_collect synchronises the device and returns (and clears)
 * the summed duration in ms, the summed algorithmic work (FLOPs for CTDK_PROF_GEMM, bytes for
 * the others) and the number of launches of class `cls`. */
#define CTDK_PROF_GEMM 0
#define CTDK_PROF_ATTN 1
#define CTDK_PROF_ADAMW 2
#define CTDK_PROF_NORM 3      /* RMSNorm forward: 8 B per element */
#define CTDK_PROF_NORM_BWD 4  /* RMSNorm backward incl. the dw column sums: 12 B per element (+ 4 when it adds into dx) */
#define CTDK_PROF_QKROPE 5    /* fused QK-Norm + RoPE, forward and backward: 8 B per q / k element (+ v copy when out of place) */
#define CTDK_PROF_CE 6        /* masked cross-entropy on a logits block: 8 B per logit of a supervised row */
#define CTDK_PROF_EMBED 7     /* embedding gather / scatter-add: 8 B / 12 B per element */
int ctdk_prof_enable(int on);
int ctdk_prof_collect(int cls, double* total_ms, double* total_work, long long* launches);

/* ------------------------------------------------------------------------------------
 * GEMM  —  C[M,N] = op(A)·op(B) (+ epilogue), TF32 tensor cores (tcgen05, TMEM fp32
 * accumulators, TMA-fed), optional 3xTF32 split for near-fp32 results.
 * Replaces cublasSgemm in ops::matmul_impl (src/ops/matmul.cpp:13-49) and the two
 * backward GEMMs of MatmulBackward (src/ops/matmul.cpp:99-118).
 *   transa==0: A is [M,K] with leading dimension lda;  transa!=0: A is [K,M].
 *   transb==0: B is [K,N] with leading dimension ldb;  transb!=0: B is [N,K].
 * Shapes whose leading dimensions are not multiples of 4 floats, or pointers not
 * 16-byte aligned, take a plain fp32 SIMT kernel (exact fp32, any shape).
 * ------------------------------------------------------------------------------------ */
#define CTDK_GEMM_TF32 0
#define CTDK_GEMM_3XTF32 1
#define CTDK_GEMM_FP32_SIMT 2 /* force the SIMT kernel (exact fp32) */

#define CTDK_EPI_STORE 0      /* C = acc */
#define CTDK_EPI_ACCUMULATE 1 /* C += acc (gradient accumulation over micro-batches) */
#define CTDK_EPI_RESIDUAL 2   /* C = acc + aux, aux is [M,N] with leading dimension ldc */

int ctdk_gemm(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
              int64_t lda, int64_t ldb, int64_t ldc, int transa, int transb, int precision,
              int epilogue, const float* aux, void* stream);

/* Same as ctdk_gemm with a caller-provided workspace, which CTDK_GEMM_3XTF32 needs to run on the
 * tensor cores: both operands are split into a TF32-exact high part and an fp32 remainder and
 * C = A_hi B_hi + A_hi B_lo + A_lo B_hi is accumulated in three tensor-core passes (relative
 * error ~1e-6, i.e. near the reference's fp32 cublasSgemm). Needs dense operands (leading
 * dimensions equal to the row lengths); otherwise, or without a workspace, behaves as ctdk_gemm
 * (where CTDK_GEMM_3XTF32 selects the exact-fp32 SIMT kernel). */
int64_t ctdk_gemm_3xtf32_workspace_floats(int64_t M, int64_t N, int64_t K);
int ctdk_gemm_ws(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                 int64_t lda, int64_t ldb, int64_t ldc, int transa, int transb, int precision,
                 int epilogue, const float* aux, float* workspace, int64_t workspace_floats,
                 void* stream);

/* Fused MLP input projection (nn::MLP::forward, include/ctd/nn/mlp.h:16-21: gate_proj and up_proj
 * matmuls followed by silu(gate) * up): W is the [2I, K] stack of the gate_proj rows and the up_proj
 * rows (adjacent in the parameter arena); gu[M, 2I] receives gate | up (kept for the backward pass)
 * and act[M, I] = silu(gate) * up, both from the accumulator of one paired-CTA GEMM, so the
 * activation never re-reads gate and up from memory. Shapes the fused kernel does not take
 * (I not a multiple of 128, M < 256, unaligned pointers, 3xTF32) run as ctdk_gemm + ctdk_swiglu_fwd. */
int ctdk_gemm_swiglu(const float* A, const float* W, float* gu, float* act, int64_t M, int64_t I,
                     int64_t K, int precision, void* stream);
/* The matching backward step: d(act)[M, I] = dy[M, K] * Wd[K, I] (the dX product of down_proj,
 * MatmulBackward, src/ops/matmul.cpp:120-168) followed by MulBackward and SiluBackward
 * (src/ops/elementwise.cu:89-238): dgu[M, 2I] = d(gate) | d(up) with d(gate) = d(act) * up *
 * silu'(gate), d(up) = d(act) * silu(gate), gate | up read from gu[M, 2I]. In the fused kernel
 * d(act) never leaves the accumulator: the epilogue fetches the gate / up boxes by TMA, rewrites
 * them in place and stores them. Shapes it does not take run as ctdk_gemm into dact_scratch[M, I]
 * + ctdk_swiglu_bwd (dact_scratch may be NULL only when the fused kernel is known to apply). */
int ctdk_gemm_swiglu_bwd(const float* dy, const float* Wd, const float* gu, float* dgu,
                         float* dact_scratch, int64_t M, int64_t I, int64_t K, int precision,
                         void* stream);

/* The dX product of o_proj in the backward pass (MatmulBackward, src/ops/matmul.cpp:120-168) fused with
 * the row term of the softmax backward (softmax_backward_kernel, src/ops/softmax.cu:56-93, after the
 * P V product's backward): dattn[B*T, H*D] = dy[B*T, hid] * Wo[hid, H*D] and delta[b, h, t] = sum over
 * head h's D columns of dattn * attn_out, formed in the GEMM's epilogue while the tile is still in
 * registers (attn_out's tile is fetched by TMA), so the attention output and its gradient are not
 * read again for it. ctdk_attn_bwd(_p) called afterwards with out == NULL takes delta as given. Shapes
 * the fused kernel does not take (3xTF32, B*T < 256, unaligned pointers) run as ctdk_gemm + the
 * separate delta pass. D is 64 or 128. */
int ctdk_gemm_dattn_delta(const float* dy, const float* Wo, const float* attn_out, float* dattn,
                          float* delta, int64_t B, int64_t T, int H, int D, int64_t hid,
                          int precision, void* stream);

/* Batched variant with full-matrix strides, as cublasSgemmStridedBatched in
 * ops::bmm_impl (src/ops/matmul.cpp:51-93). */
int ctdk_bmm(const float* A, const float* B, float* C, int64_t batch, int64_t M, int64_t N,
             int64_t K, int transa, int transb, int precision, void* stream);

/* ------------------------------------------------------------------------------------
 * RMSNorm — y = x * rsqrt(mean(x^2)+eps) * w per row of length H.
 * Replaces rms_norm_kernel_f32 / rms_norm_backward_kernel_f32 (src/ops/norm.cu:18-106).
 * rstd (optional, [rows]) receives the per-row scale. The backward writes dx and
 * dw (+)= sum_rows dy*x*rstd; `dw_scratch` must hold ctdk_rmsnorm_bwd_scratch_floats(H)
 * floats; accumulate_dw != 0 adds into dw instead of overwriting it. If add_to_dx != 0,
 * dx += result (the residual-stream gradient is kept in one buffer).
 * ------------------------------------------------------------------------------------ */
int ctdk_rmsnorm_fwd(const float* x, const float* w, float* y, float* rstd, int64_t rows,
                     int H, float eps, void* stream);
int64_t ctdk_rmsnorm_bwd_scratch_floats(int H);
int ctdk_rmsnorm_bwd(const float* dy, const float* x, const float* w, float* dx, float* dw,
                     float* dw_scratch, int64_t rows, int H, float eps, int accumulate_dw,
                     int add_to_dx, void* stream);

/* Same result as ctdk_rmsnorm_bwd, for callers that can neither pass scratch nor let the
 * library allocate: hosts that gave all of HBM to their own arena at start-up, and step
 * loops that must stay free of cudaMalloc/cudaFree because those stall every stream.
 * (No counterpart in the reference, whose ops allocate on every call.)
 * The dw partial rows live in a 4 MiB array built into the library (256 rows x 4096 floats),
 * resident on every GPU that loads it until the process exits. H above 4096 is rejected
 * with CTDK_EINVAL. The entry point calls no cudaMalloc, cudaFree or allocating library
 * routine. The first call on each device looks up the array's device address (with that
 * device current); make that first call outside any stream capture. All calls share the one
 * array: two calls whose kernels can overlap on the GPU (different streams, no ordering
 * between them) race on it — keep them on one stream or order them with events. */
int ctdk_rmsnorm_bwd_static(const float* dy, const float* x, const float* w, float* dx,
                            float* dw, int64_t rows, int H, float eps, int accumulate_dw,
                            int add_to_dx, void* stream);

/* ------------------------------------------------------------------------------------
 * RoPE — non-interleaved rotation of pairs (i, i+D/2) of x[B,T,H,D] by
 * (position_start+t)*freq_i, freq_i = theta^(-2i/D) with the llama3 wavelength scaling.
 * Replaces rope_kernel_f32 (src/ops/rope.cu:17-56); RopeScaling fields as in
 * include/ctd/ops/rope.h:9-22 (scaling_factor <= 1 disables scaling). sin_sign = +1
 * forward, -1 for the transpose (backward). x_out may alias x_in. `row_stride` is the
 * distance in floats between consecutive (b,t) rows (H*D when contiguous).
 * ------------------------------------------------------------------------------------ */
typedef struct {
  float theta;
  float scaling_factor;
  float low_freq_wavelen;
  float high_freq_wavelen;
} ctdk_rope_params;

int ctdk_rope(const float* x_in, float* x_out, int64_t B, int64_t T, int H, int D,
              int64_t row_stride, int position_start, const ctdk_rope_params* p,
              float sin_sign, void* stream);

/* (cos, sin) table for positions position_start .. position_start+T-1:
 * table[t][i] = {cosf(a), sinf(a)}, a = float(position_start+t) * freq_i, i < D/2
 * (T*D floats). The fused kernels below read it instead of recomputing powf/sin/cos per
 * element as rope_kernel_f32 does (src/ops/rope.cu:32-50). */
int ctdk_rope_table(float* table, int64_t T, int D, int position_start,
                    const ctdk_rope_params* p, void* stream);

/* Fused per-head RMSNorm (optional, Qwen3 QK-Norm: include/ctd/nn/attention.h:115-118)
 * followed by RoPE (attention.h:120-121) on the q and k slices of a packed
 * qkv[B*T, (H+2*Hk)*D] buffer, written to qkv_out (v is copied; qkv_out may alias qkv when
 * no norm weights are given). When wq/wk are NULL only RoPE is applied. rstd_q [B*T*H] and
 * rstd_k [B*T*Hk] are saved for the backward. D must be 64 or 128.
 * The backward takes d(qkv_out) in dqkv and overwrites its q and k slices with d(qkv)
 * (v is left as is); dwq, dwk (+)= the norm-weight gradients. `scratch` must hold
 * ctdk_qk_norm_rope_bwd_scratch_floats(D) floats when norm weights are given. */
int ctdk_qk_norm_rope_fwd(const float* qkv, float* qkv_out, const float* wq, const float* wk,
                          float* rstd_q, float* rstd_k, const float* rope_table, int64_t B,
                          int64_t T, int H, int Hk, int D, float eps, void* stream);
int64_t ctdk_qk_norm_rope_bwd_scratch_floats(int D);
int ctdk_qk_norm_rope_bwd(float* dqkv, const float* qkv_pre, const float* wq, const float* wk,
                          const float* rstd_q, const float* rstd_k, float* dwq, float* dwk,
                          float* scratch, const float* rope_table, int64_t B, int64_t T, int H,
                          int Hk, int D, int accumulate_dw, void* stream);

/* ------------------------------------------------------------------------------------
 * Elementwise. Replace add/sub/mul/scale/silu/silu_backward kernels
 * (src/ops/elementwise.cu:15-69) and mul_scalar (src/ops/repeat_kv.cu:45).
 * ------------------------------------------------------------------------------------ */
int ctdk_add(const float* a, const float* b, float* out, int64_t n, void* stream);
int ctdk_sub(const float* a, const float* b, float* out, int64_t n, void* stream);
int ctdk_mul(const float* a, const float* b, float* out, int64_t n, void* stream);
int ctdk_scale(const float* x, float alpha, float* out, int64_t n, void* stream);
int ctdk_silu(const float* x, float* out, int64_t n, void* stream);
int ctdk_silu_bwd(const float* x, const float* g, float* out, int64_t n, void* stream);
/* SwiGLU of nn::MLP::forward (include/ctd/nn/mlp.h:16-21): act = silu(g)*u on a packed
 * gu[rows, 2*I] buffer (gate columns first) -> act[rows, I]; backward writes dgu in the
 * same packed layout from d(act). */
int ctdk_swiglu_fwd(const float* gu, float* act, int64_t rows, int I, void* stream);
int ctdk_swiglu_bwd(const float* gu, const float* dact, float* dgu, int64_t rows, int I,
                    void* stream);

/* ------------------------------------------------------------------------------------
 * Embedding. Replaces embedding_kernel_f32 / embedding_backward_kernel_f32
 * (src/ops/embedding.cu:15-39). ids are int64 as at the reference's ops:: API
 * (embedding.cu:44). The backward adds dy rows into dW (the caller owns zeroing, so the
 * tied-embedding gradient can be accumulated in place). Out-of-range ids are skipped and
 * counted in the device status word.
 * ------------------------------------------------------------------------------------ */
int ctdk_embedding_fwd(const int64_t* ids, const float* W, float* out, int64_t rows, int H,
                       int64_t V, void* stream);
int ctdk_embedding_bwd(const int64_t* ids, const float* dy, float* dW, int64_t rows, int H,
                       int64_t V, void* stream);

/* ------------------------------------------------------------------------------------
 * Masked cross-entropy on a block of logits[n,V] (leading dimension V).
 * Replaces ce_masked_fwd_kernel_f32 / ce_masked_bwd_kernel_f32 (src/ops/loss.cu:254-329).
 * row_weight[i] = mask_i * dy / sum(mask) (the factor the reference applies in
 * CrossEntropyMaskedBackward, loss.cu:388-411). In one pass per row it computes
 * lse_i, adds mask_i*(lse_i - z_target) to loss_sum[0] and mask_i to loss_sum[1]
 * (loss_mask[i] is 0/1), and overwrites the logits with
 * dlogits = row_weight_i * (softmax(z) - onehot(target)); rows of weight 0 are zero-filled
 * exactly. lse_out (optional) receives lse per row. If dlogits_inplace == 0 the logits are
 * left untouched (forward only).
 * ------------------------------------------------------------------------------------ */
int ctdk_ce_masked(float* logits, const int64_t* targets, const float* loss_mask,
                   const float* row_weight, float* loss_sum, float* lse_out, int64_t n,
                   int64_t V, int dlogits_inplace, void* stream);

/* Row gather / scatter used to run the LM head and the loss only on supervised positions: rows
 * whose loss mask is 0 contribute exactly 0 to the loss and to every gradient
 * (ce_masked_bwd_kernel_f32 scales them by mk = 0, src/ops/loss.cu:318-327), so they need no
 * logits at all. idx holds the kept row numbers (int32, ascending). */
int ctdk_gather_rows(const float* src, const int32_t* idx, float* dst, int64_t n, int H, void* stream);
int ctdk_scatter_rows(const float* src, const int32_t* idx, float* dst, int64_t n, int H, void* stream);
int ctdk_gather_ce_inputs(const int64_t* targets, const float* mask, const float* weight, const int32_t* idx,
                          int64_t* t_out, float* m_out, float* w_out, int64_t n, void* stream);

/* ------------------------------------------------------------------------------------
 * Causal softmax attention with grouped-query heads on packed projections.
 * Replaces the bmm -> mul_scalar -> causal mask -> softmax -> bmm chain of
 * nn::Attention::forward_train (include/ctd/nn/attention.h:123-141) including
 * repeat_kv_heads and the permutes. q is read at qkv[(b*T+t)*row_stride + h*D], k at
 * column offset H*D + hk*D, v at (H+Hk)*D + hk*D; query head h uses kv head h/(H/Hk).
 * out is [B*T, H*D]; lse [B,H,T] holds the log-sum-exp of the scaled scores.
 * The backward takes dout [B*T,H*D] and writes dqkv in the packed layout; delta [B,H,T] is
 * scratch for rowsum(dout * out), computed from out here, or taken as given when out is NULL
 * (ctdk_gemm_dattn_delta has produced it).
 * ------------------------------------------------------------------------------------ */
int ctdk_attn_fwd(const float* qkv, float* out, float* lse, int64_t B, int64_t T, int H,
                  int Hk, int D, void* stream);
int ctdk_attn_bwd(const float* qkv, const float* out, const float* dout, const float* lse,
                  float* delta, float* dqkv, int64_t B, int64_t T, int H, int Hk, int D,
                  void* stream);
/* Same with a precision: CTDK_GEMM_TF32 (what the plain entry points use) or CTDK_GEMM_3XTF32,
 * which splits every operand of every contraction into TF32 high and low parts (three tensor-core
 * products per product) for results close to the reference's fp32 bmm. */
int ctdk_attn_fwd_p(const float* qkv, float* out, float* lse, int64_t B, int64_t T, int H,
                    int Hk, int D, int precision, void* stream);
int ctdk_attn_bwd_p(const float* qkv, const float* out, const float* dout, const float* lse,
                    float* delta, float* dqkv, int64_t B, int64_t T, int H, int Hk, int D,
                    int precision, void* stream);

/* ------------------------------------------------------------------------------------
 * Stand-alone ops of the reference's per-op API that the fused training path absorbs (kept for the
 * public op surface; 64-bit indexing throughout):
 *   softmax over the last axis and its backward dx = y * (g - sum(g*y))   (src/ops/softmax.cu:18-93)
 *   permute of up to 6 axes into a new contiguous tensor: out axis i = in axis perm[i]
 *                                                                         (src/ops/permute.cu:16-60)
 *   repeat_kv: [rows, Hk, D] -> [rows, Hk*group, D], and the group sum that is its backward
 *                                                                         (src/ops/repeat_kv.cu:14-43)
 *   causal mask on [mats, Tq, Tk]: out = (j > q_pos_start + i) ? fill : in; fill = -FLT_MAX forward,
 *   0 for the backward; in == out is allowed                               (src/ops/mask.cu:17-60)
 *   mse: loss[0] = mean((pred - target)^2); dpred = 2 (pred - target) / n * dy[0] with dy on the device
 *                                                                         (src/ops/loss.cu:17-75)
 *   KV cache: write src [B, T, H, D] into cache [B, H, max_seq, D] at position pos; read the first
 *   valid_len positions with every KV head repeated `group` times -> [B, H*group, valid_len, D]
 *                                                                         (src/ops/kv_cache.cu:14-109)
 *   loss_ratio: out[0] = sums[1] > 0 ? sums[0] / sums[1] : 0 (the masked mean from ctdk_ce_masked's sums)
 *   ce_row_weight: row_weight[i] = mask[i] * dy[0] / mask_sum[0] (mask NULL: dy[0] / n), the factor of
 *   CrossEntropy(Masked)Backward built without a host round trip           (src/ops/loss.cu:388-411)
 * ------------------------------------------------------------------------------------ */
int ctdk_softmax_fwd(const float* x, float* y, int64_t rows, int64_t width, void* stream);
int ctdk_softmax_bwd(const float* y, const float* g, float* dx, int64_t rows, int64_t width, void* stream);
int ctdk_permute(const float* x, float* y, int ndim, const int64_t* shape, const int* perm, void* stream);
int ctdk_repeat_kv(const float* x, float* y, int64_t rows, int Hk, int D, int group, void* stream);
int ctdk_repeat_kv_sum(const float* y, float* x, int64_t rows, int Hk, int D, int group, void* stream);
int ctdk_causal_mask(const float* in, float* out, int64_t mats, int64_t Tq, int64_t Tk, int q_pos_start,
                     float fill, void* stream);
int ctdk_mse_fwd(const float* pred, const float* target, int64_t n, float* loss, void* stream);
int ctdk_mse_bwd(const float* pred, const float* target, const float* dy, float* dpred, int64_t n,
                 void* stream);
int ctdk_kv_write(const float* src, float* cache, int64_t B, int64_t T, int H, int D, int64_t max_seq,
                  int64_t pos, void* stream);
int ctdk_kv_read_expanded(const float* cache, float* out, int64_t B, int Hk, int group, int64_t valid_len,
                          int D, int64_t max_seq, void* stream);
int ctdk_loss_ratio(const float* sums, float* out, void* stream);
int ctdk_ce_row_weight(const float* loss_mask, const float* dy, const float* mask_sum, int64_t n,
                       float* row_weight, void* stream);

/* ------------------------------------------------------------------------------------
 * Optimizer. ctdk_sumsq adds sum(g^2) into out[0] (sum_sq_kernel_f32,
 * src/core/optim.cu:221-239). ctdk_adamw is one launch over a flat range of parameters:
 *   g' = g * grad_scale            (clip_grad_norm_'s scale, optim.cu:276-290; read from
 *                                   device memory so no host sync is needed; NULL = 1)
 *   m = b1 m + (1-b1) g';  v = b2 v + (1-b2) g'^2
 *   p = p - lr * ((m/bc1) / (sqrtf(v/bc2) + eps) + wd * p)   (adamw_step_kernel_f32,
 *                                                              optim.cu:54-73)
 * Weight decay applies per segment: seg_end[i] is the exclusive end offset (in floats,
 * relative to p, multiple of 4) of segment i and seg_wd[i] its decay (the reference's two
 * ParamGroups, tools/ctd_train/main.cpp:304-311). nseg == 0 applies `wd` everywhere.
 * ------------------------------------------------------------------------------------ */
typedef struct {
  float lr, beta1, beta2, eps, wd, bc1, bc2;
} ctdk_adamw_params;

int ctdk_sumsq(const float* g, int64_t n, float* out, void* stream);
/* scale_out[0] = norm > max_norm ? max_norm/(norm+eps) : 1, norm_out[0] = norm with
 * norm = sqrt(sumsq[0]) (clip_grad_norm_, optim.cu:274-279). */
int ctdk_clip_scale(const float* sumsq, float max_norm, float eps, float* scale_out,
                    float* norm_out, void* stream);
int ctdk_adamw(float* p, const float* g, float* m, float* v, int64_t n,
               const ctdk_adamw_params* hp, const float* grad_scale, const int64_t* seg_end,
               const float* seg_wd, int nseg, void* stream);

/* ------------------------------------------------------------------------------------
 * Training-step engine: the fused per-layer forward/backward schedule that replaces the
 * autograd tape walk of Model::forward_train_masked + Tensor::backward
 * (include/ctd/nn/model.h:170-206, src/core/autograd.cu:158-237) for the decoder.
 * The caller owns all device memory: a flat fp32 parameter arena, a gradient arena of the
 * same layout and a workspace. The arena holds the tensors in Model::collect_parameters
 * order (src/nn/model.cpp:78-98), each padded to a multiple of 64 floats, so q/k/v and
 * gate/up weights are adjacent and run as one GEMM each.
 * ------------------------------------------------------------------------------------ */
typedef struct {
  int vocab_size, hidden_size, intermediate_size, num_hidden_layers;
  int num_attention_heads, num_key_value_heads, head_dim;
  float rms_norm_eps, rope_theta;
  int qk_norm; /* Qwen3 per-head RMSNorm on q and k before RoPE */
  float rope_scaling_factor, rope_scaling_low_freq_factor, rope_scaling_high_freq_factor;
  int rope_scaling_original_max_pos;
  int gradient_checkpointing; /* keep only layer inputs; recompute inside the backward */
  int precision;              /* CTDK_GEMM_TF32 or CTDK_GEMM_3XTF32 */
} ctdk_model_config;          /* fields as LlamaConfig, include/ctd/nn/model.h:19-37 */

/* Number of parameter tensors, and their arena layout: offsets[i], numels[i] (floats),
 * decay[i] (1 = weight-decay group) in collect_parameters order; *total = arena floats. */
int64_t ctdk_model_num_tensors(const ctdk_model_config* cfg);
int ctdk_model_layout(const ctdk_model_config* cfg, int64_t* offsets, int64_t* numels,
                      int* decay, int64_t* total);
int64_t ctdk_engine_workspace_bytes(const ctdk_model_config* cfg, int64_t B, int64_t T);
/* Host-side object only (no device allocation). B, T are the largest batch and sequence
 * (positions per row, i.e. seq_len-1) the workspace was sized for. */
int ctdk_engine_create(const ctdk_model_config* cfg, float* params, float* grads,
                       void* workspace, int64_t workspace_bytes, int64_t B, int64_t T,
                       void** engine);
int ctdk_engine_destroy(void* engine);
/* One micro-batch (or several concatenated along B): forward, masked CE and backward.
 * ids/targets int64 [B,T], loss_mask fp32 [B,T] (0/1), row_weight fp32 [B,T] =
 * mask * dy / sum(mask of the row's micro-batch). accumulate == 0 overwrites the gradient
 * arena, != 0 adds to it. loss_sums (device float[2]) += {sum mask*row_loss, sum mask}. */
int ctdk_engine_forward_backward(void* engine, const int64_t* ids, const int64_t* targets,
                                 const float* loss_mask, const float* row_weight, int64_t B,
                                 int64_t T, int accumulate, float* loss_sums, void* stream);
/* Optional, before the next forward_backward / forward_loss call only: the rows (positions of the
 * flattened [B*T] batch) whose loss mask is non-zero, as an ascending int32 device array. The final
 * norm output is then compacted to these rows before the LM head, so the head GEMMs and the loss
 * skip the unsupervised half of a typical SFT batch. n == 0 or never calling it keeps all rows. */
int ctdk_engine_set_active_rows(void* engine, const int32_t* rows, int64_t n);
/* Forward and loss only (the no-grad validation pass, tools/ctd_train/main.cpp:191-206). */
int ctdk_engine_forward_loss(void* engine, const int64_t* ids, const int64_t* targets,
                             const float* loss_mask, int64_t B, int64_t T, float* loss_sums,
                             void* stream);
/* Optional host callback invoked once everything that writes the gradients of layer `layer` is
 * ordered before the caller's stream at this point of the enqueue (layer == num_hidden_layers:
 * final norm + LM head; -1: embedding, i.e. all done), so the caller can start reducing that
 * layer's gradients while earlier layers still run. Layers come in descending order. The engine
 * runs the weight-gradient GEMMs of the TF32 path on a stream of its own (they feed nothing before
 * the optimizer and fill SMs the dependency chain leaves idle) and joins them one layer later, so
 * the callback of layer l is made after layer l-1 has been enqueued; when the pass returns, all
 * of its work is ordered before the caller's stream again. CTDK_ENGINE_SIDE_STREAM=0 in the
 * environment keeps everything on the caller's stream. */
typedef void (*ctdk_layer_callback)(int layer, void* user);
int ctdk_engine_set_layer_callback(void* engine, ctdk_layer_callback cb, void* user);
/* Optional host callback invoked right BEFORE the forward kernels that first read a part of the
 * parameter arena are enqueued (layer == -1: embedding; 0..L-1: decoder layer; L: final norm + LM
 * head), so a data-parallel caller can let the all-gather of the updated parameters of later
 * layers run underneath the forward pass of earlier ones and only make the stream wait here. */
int ctdk_engine_set_forward_callback(void* engine, ctdk_layer_callback cb, void* user);

/* ------------------------------------------------------------------------------------
 * Data feed: widens one pass's rows from the reference's bin format (int32 token rows and int8
 * 0/1 loss masks of length S, tools/ctd_train/main.cpp:121-136) to what the engine takes, on the
 * device, so that only 5 bytes per token cross PCIe instead of the 24 bytes of the int64 / fp32
 * host vectors make_batch builds (main.cpp:145-174):
 *   ids[r,t] = tok[r,t], targets[r,t] = tok[r,t+1], mask[r,t] = msk[r,t+1]   (t < S-1)
 *   weight[r,t] = mask[r,t] / (accum_total * sum(mask of the row's micro-batch))
 * where consecutive groups of micro_rows rows form a micro-batch and accum_total counts the
 * micro-batches of the whole step over all ranks (mul_scalar(loss, 1/A) and the masked-CE backward,
 * main.cpp:346-361, src/ops/loss.cu:388-411). A micro-batch with an empty mask gets weight 0
 * (main.cpp:357). micro_sums is scratch of ceil(rows / micro_rows) floats.
 * ------------------------------------------------------------------------------------ */
int ctdk_batch_widen(const int32_t* tok, const int8_t* msk, int64_t rows, int S, int micro_rows,
                     int accum_total, int64_t* ids, int64_t* targets, float* mask, float* weight,
                     float* micro_sums, void* stream);

/* ------------------------------------------------------------------------------------
 * Data-parallel trainer: the part of the step loop after the backward pass (clip_grad_norm_,
 * AdamW::step, zero_grad; tools/ctd_train/main.cpp:362-373) for one process per GPU, with ZeRO-1
 * sharding of AdamW's m / v over buckets of the arena in place of the reference's host offload
 * (src/core/optim.cu:94-130): ncclReduceScatter per gradient bucket started from the engine's
 * layer callback underneath the backward pass, one scalar ncclAllReduce, fused AdamW on the rank's
 * slices, ncclAllGather of the parameters left in flight under the next forward pass.
 *
 * Plan (host only, no GPU needed): the arena is padded to a multiple of 64*world floats
 * (ctdk_dp_arena_floats) and cut into contiguous buckets — the embedding, then groups of
 * layers_per_bucket decoder layers, cuts rounded down to 64*world floats; 0 = one bucket. For
 * bucket i, [lo, hi) is its arena range, [own_lo, own_hi) the slice rank `rank` owns,
 * state_offset where that slice starts in the rank's m / v arrays (the slices back to back) and
 * ready the lowest completion index of the tensors it overlaps (-1 embedding, l decoder layer,
 * L final norm): its gradients are final once the layer callback has fired for `ready`, and the
 * forward pass first reads it at the forward callback of `ready`. ctdk_dp_segments returns the
 * number of weight-decay segments of an arena range (decay group = embedding + linear weights,
 * norm weights and padding 0; main.cpp:304-311) and fills up to `capacity` of them.
 * ------------------------------------------------------------------------------------ */
int64_t ctdk_dp_arena_floats(const ctdk_model_config* cfg, int world);
int ctdk_dp_num_buckets(const ctdk_model_config* cfg, int world, int layers_per_bucket);
int ctdk_dp_buckets(const ctdk_model_config* cfg, int world, int rank, int layers_per_bucket,
                    int64_t* lo, int64_t* hi, int64_t* own_lo, int64_t* own_hi,
                    int64_t* state_offset, int* ready);
int ctdk_dp_segments(const ctdk_model_config* cfg, float weight_decay, int64_t lo, int64_t hi,
                     int64_t* seg_end, float* seg_wd, int capacity);

typedef struct {
  float lr, beta1, beta2, eps, weight_decay, clip; /* AdamW + clip_grad_norm_ (main.cpp:304-313) */
  int layers_per_bucket;                           /* < 0: default (4); 0: one bucket */
} ctdk_trainer_hparams;

/* Rank 0 makes the 128-byte NCCL unique id and hands it to the other ranks (file, socket, ...). */
int ctdk_trainer_unique_id(void* id128);
/* params / grads: arenas of ctdk_dp_arena_floats(cfg, world) floats; m / v: that / world floats
 * (zeroed by the caller, or loaded); workspace as for ctdk_engine_create, which it calls. With
 * world > 1 every rank must call it (communicator set-up is collective) with the same id. Allocates
 * a few KB of device memory for scalars and segment tables; nothing is allocated afterwards. */
int ctdk_trainer_create(const ctdk_model_config* cfg, float* params, float* grads, float* m, float* v,
                        void* workspace, int64_t workspace_bytes, int64_t B, int64_t T, int rank,
                        int world, const void* nccl_id, const ctdk_trainer_hparams* hp, void** trainer);
int ctdk_trainer_destroy(void* trainer);
void* ctdk_trainer_engine(void* trainer); /* the ctdk_engine_* handle inside (set_active_rows) */
/* Called in front of the trainer's own layer callback (same contract as the engine's). */
int ctdk_trainer_set_layer_callback(void* trainer, ctdk_layer_callback cb, void* user);
/* One optimizer step on this rank's rows: zero the loss sums, forward + backward with the bucket
 * reduce-scatters, then ctdk_trainer_optimizer_step. active_rows as ctdk_engine_set_active_rows. */
int ctdk_trainer_step(void* trainer, const int64_t* ids, const int64_t* targets, const float* loss_mask,
                      const float* row_weight, int64_t B, int64_t T, const int32_t* active_rows,
                      int64_t n_active, float lr, void* stream);
/* The pieces, for steps of several passes (gradient accumulation): `last` != 0 marks the final
 * backward pass of the step, whose buckets are reduce-scattered as they complete. */
int ctdk_trainer_zero_loss(void* trainer, void* stream);
int ctdk_trainer_forward_backward(void* trainer, const int64_t* ids, const int64_t* targets,
                                  const float* loss_mask, const float* row_weight, int64_t B, int64_t T,
                                  int accumulate, int last, void* stream);
int ctdk_trainer_forward_loss(void* trainer, const int64_t* ids, const int64_t* targets,
                              const float* loss_mask, int64_t B, int64_t T, void* stream);
int ctdk_trainer_optimizer_step(void* trainer, float lr, void* stream);
/* Sums the two loss sums over the ranks (validation split over ranks; the optimizer step does this
 * itself for training passes). Collective: every rank calls it the same number of times. */
int ctdk_trainer_allreduce_loss(void* trainer, void* stream);
/* Makes `stream` wait for the parameter all-gathers the last optimizer step left in flight; call it
 * before anything but the trainer's own forward pass reads the parameter arena. */
int ctdk_trainer_wait_parameters(void* trainer, void* stream);
/* Synchronises `stream` and returns {sum mask*loss, sum mask, sum g^2, clip scale, gradient norm}
 * of the last step (summed over ranks), then checks the device status word: CTDK_ETIMEOUT if a
 * bounded device-side wait gave up since the last check. */
int ctdk_trainer_read_metrics(void* trainer, float* out5, void* stream);
const float* ctdk_trainer_loss_sums(void* trainer); /* device float[2] the passes add to */
int64_t ctdk_trainer_step_count(void* trainer);
int ctdk_trainer_set_step_count(void* trainer, int64_t n);
/* Checkpoints (tools/ctd_train/main.cpp:208-271 keep m / v per parameter): gather assembles the
 * ranks' slices of m or v into arena order in `full` (arena floats, device; every rank calls it);
 * scatter copies this rank's slices out of an arena-order array at load. */
int ctdk_trainer_gather_state(void* trainer, const float* shard_state, float* full, void* stream);
int ctdk_trainer_scatter_state(void* trainer, const float* full, float* shard_state, void* stream);

/* ------------------------------------------------------------------------------------
 * Token sampling on the device with the semantics of the reference's host sampler
 * (src/core/sampling.cpp:13-106; include/ctd/sampling.h:11-21): logits fp32 [B, V] on the device;
 * temperature <= 0 is greedy (first index of the maximum); otherwise logits / temperature, optional
 * top-k (0 < top_k < V: everything below the k-th largest is dropped, ties at the threshold stay),
 * softmax, optional top-p (0 < top_p < 1: the largest probabilities in descending order until their
 * sum reaches top_p, renormalised) and inverse-CDF selection in index order with the draw u[b]: one
 * std::uniform_real_distribution<double>(0, 1) value per row from the caller's mt19937_64, in row
 * order, which is the reference's draw order, so a seeded request picks the same tokens. u and
 * out_tokens are device pointers (u may be NULL for greedy); workspace holds
 * ctdk_sample_workspace_bytes(B, V) bytes (unused for greedy). Nothing is synchronised.
 * ------------------------------------------------------------------------------------ */
int64_t ctdk_sample_workspace_bytes(int64_t B, int64_t V);
int ctdk_sample(const float* logits, int64_t B, int64_t V, float temperature, int top_k, float top_p,
                const double* u, void* workspace, int64_t* out_tokens, void* stream);

/* ------------------------------------------------------------------------------------
 * KV-cache greedy decoding, batch 1. Replaces the cached inference path: Model::forward with a
 * KVCache (include/ctd/nn/model.h:155-167), Attention::forward (include/ctd/nn/attention.h:43-97),
 * write_kv_inplace / read_kv_expanded (src/ops/kv_cache.cu:49-109) and the greedy sampler
 * (src/core/sampling.cpp:13-20, first index of the maximum) used by tools/ctd_generate/main.cpp.
 * The caller owns the parameter arena (same layout as the training engine) and a workspace of
 * ctdk_decode_workspace_bytes(cfg, max_seq) bytes holding the K/V cache [layer][kv head][max_seq][D].
 *   prefill : runs the prompt (ids int64 [T], 1 <= T < max_seq) and fills the cache;
 *   greedy  : appends n_new tokens to out_tokens (device int64), continuing where the last call
 *             stopped; token ids stay on the device, one CUDA graph launch per token when `stream`
 *             is not the legacy default stream;
 *   step    : feeds ONE token chosen by the caller (a sampler, a forced token) at the next
 *             position and leaves the logits of that position behind; not to be mixed with
 *             greedy after the same prefill;
 *   logits  : device pointer to the [vocab] logits of the last processed position.
 * ------------------------------------------------------------------------------------ */
int64_t ctdk_decode_workspace_bytes(const ctdk_model_config* cfg, int64_t max_seq);
int ctdk_decode_create(const ctdk_model_config* cfg, const float* params, void* workspace,
                       int64_t workspace_bytes, int64_t max_seq, void** decoder);
int ctdk_decode_destroy(void* decoder);
int ctdk_decode_prefill(void* decoder, const int64_t* ids, int64_t T, void* stream);
int ctdk_decode_greedy(void* decoder, int64_t n_new, int64_t* out_tokens, void* stream);
int ctdk_decode_step(void* decoder, int64_t token, void* stream);
int ctdk_decode_logits(void* decoder, const float** logits);

#ifdef __cplusplus
}
#endif
#endif /* CTDK_H_ */
