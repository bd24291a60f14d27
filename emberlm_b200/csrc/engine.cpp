// Training-step engine: a fixed per-layer forward/backward schedule over the ctdk kernels.
//
// It computes what the reference computes by walking its autograd tape
// (emberlm include/ctd/nn/model.h:170-206, include/ctd/nn/transformer_block.h:28-35,
// include/ctd/nn/attention.h:100-143, include/ctd/nn/mlp.h:16-21,
// src/core/autograd.cu:158-237), but with the schedule known ahead of time:
//   - q/k/v and gate/up projections run as one GEMM each (weights are adjacent in the arena),
//   - residual adds live in GEMM epilogues, the residual-stream gradient in one buffer,
//   - attention never materialises scores, the LM head never materialises all logits:
//     rows are processed in blocks, each block going logits -> loss + dlogits (in place)
//     -> dH and dE immediately, so forward and backward of the head are one pass,
//   - with gradient_checkpointing only layer inputs are kept and the layer forward is
//     re-run inside the backward (the reference's CheckpointNode, autograd.cu:324-363).
// All device memory belongs to the caller; this object only holds pointers into it.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"

namespace ctdk {
namespace {

constexpr int64_t kAlignFloats = 64;  // every arena tensor starts on a 256-byte boundary

inline int64_t pad64(int64_t n) { return (n + kAlignFloats - 1) / kAlignFloats * kAlignFloats; }

struct TensorSlot {
  int64_t offset, numel;
  int decay;
};

struct LayerSlots {
  int64_t w_in, wq, wk, wv, wo, wqn, wkn, w_post, wg, wu, wd;
};

struct Layout {
  std::vector<TensorSlot> slots;
  std::vector<LayerSlots> layers;
  int64_t embed = 0, norm = 0, total = 0;
};

int validate(const ctdk_model_config* c) {
  CTDK_REQUIRE(c != nullptr, "model config: null");
  CTDK_REQUIRE(c->vocab_size > 0 && c->hidden_size > 0 && c->intermediate_size > 0 &&
                   c->num_hidden_layers >= 0 && c->num_attention_heads > 0 &&
                   c->num_key_value_heads > 0 && c->head_dim > 0,
               "model config: non-positive dimension");
  CTDK_REQUIRE(c->num_attention_heads % c->num_key_value_heads == 0,
               "model config: heads must be a multiple of kv heads");
  CTDK_REQUIRE(c->head_dim == 64 || c->head_dim == 128,
               "model config: head_dim must be 64 or 128");
  CTDK_REQUIRE(c->hidden_size % 4 == 0 && c->intermediate_size % 4 == 0,
               "model config: hidden and intermediate sizes must be multiples of 4");
  // gate_proj and up_proj (and q/k/v) are used as one stacked weight, so no padding may
  // separate them in the arena.
  CTDK_REQUIRE((static_cast<int64_t>(c->hidden_size) * c->intermediate_size) % kAlignFloats == 0 &&
                   (static_cast<int64_t>(c->hidden_size) * c->head_dim) % kAlignFloats == 0,
               "model config: hidden*intermediate and hidden*head_dim must be multiples of 64");
  return CTDK_OK;
}

Layout make_layout(const ctdk_model_config& c) {
  Layout L;
  int64_t off = 0;
  auto add = [&](int64_t numel, int decay) {
    const int64_t o = off;
    L.slots.push_back({o, numel, decay});
    off += pad64(numel);
    return o;
  };
  const int64_t hid = c.hidden_size, I = c.intermediate_size, D = c.head_dim;
  const int64_t H = c.num_attention_heads, Hk = c.num_key_value_heads;
  L.embed = add(static_cast<int64_t>(c.vocab_size) * hid, 1);
  for (int i = 0; i < c.num_hidden_layers; ++i) {
    LayerSlots s{};
    s.w_in = add(hid, 0);
    s.wq = add(H * D * hid, 1);
    s.wk = add(Hk * D * hid, 1);
    s.wv = add(Hk * D * hid, 1);
    s.wo = add(hid * H * D, 1);
    if (c.qk_norm) {
      s.wqn = add(D, 0);
      s.wkn = add(D, 0);
    } else {
      s.wqn = s.wkn = -1;
    }
    s.w_post = add(hid, 0);
    s.wg = add(I * hid, 1);
    s.wu = add(I * hid, 1);
    s.wd = add(hid * I, 1);
    L.layers.push_back(s);
  }
  L.norm = add(hid, 0);
  L.total = off;
  return L;
}

// Bump allocator over the caller's workspace; with base == nullptr it only measures.
struct Bump {
  char* base;
  int64_t used = 0;
  explicit Bump(void* b) : base(static_cast<char*>(b)) {}
  float* floats(int64_t n) {
    const int64_t bytes = (n * 4 + 255) / 256 * 256;
    float* p = base ? reinterpret_cast<float*>(base + used) : nullptr;
    used += bytes;
    return p;
  }
};

struct LayerActs {
  float *h1, *qkv_pre, *qkv, *rstd_q, *rstd_k, *attn, *lse, *hm, *h2, *gu, *act;
};

struct Engine {
  ctdk_model_config cfg;
  Layout layout;
  float *params, *grads;
  int64_t maxB, maxT, tok_cap;
  int QKVN;
  int64_t head_rows;  // rows of the LM-head block
  // workspace
  float* rope_table;
  int64_t rope_T = -1;
  std::vector<float*> xs;         // L+1 residual-stream tensors [tok,hid]
  std::vector<LayerActs> acts;    // L entries (all alias entry 0 when checkpointing)
  float *hf, *dh, *dtmp, *dgu, *dact, *dqkv, *dattn, *delta, *norm_scratch, *qk_scratch;
  float* logits;
  float *hfc, *dhfc, *mask_c, *w_c;  // compacted LM-head inputs (supervised rows only)
  int64_t* tgt_c;
  const int32_t* active_rows = nullptr;
  const int32_t* active_rows_last = nullptr;
  int64_t n_active = 0;
  float* ws3 = nullptr;       // operand-split workspace of the 3xTF32 GEMMs
  int64_t ws3_floats = 0;
  ctdk_layer_callback cb = nullptr;
  void* cb_user = nullptr;
  ctdk_layer_callback fcb = nullptr;   // before each part of the forward pass
  void* fcb_user = nullptr;
  // Weight-gradient GEMMs on a second stream. In the backward pass dW = dY^T X of a linear layer
  // feeds nothing before the optimizer, while dX = dY W is the next link of the dependency chain.
  // The kernels of the chain leave SMs idle — most with few rows per GPU: a 64-tile GEMM on 74 CTA
  // pairs, set-up and last-epilogue phases, small attention grids — and the dW GEMMs of a layer, on
  // their own stream, fill those gaps. slot: 0 down-proj, 1 gate|up, 2 o-proj, 3 qkv; done[slot] is
  // recorded behind the GEMM and the main stream waits for it only where a buffer the GEMM reads is
  // about to be overwritten.
  cudaStream_t side = nullptr;
  cudaEvent_t side_ready = nullptr;
  cudaEvent_t side_done[4] = {nullptr, nullptr, nullptr, nullptr};
  bool side_pending[4] = {false, false, false, false};
  bool side_on = false;   // decided per pass
  ~Engine() {
    for (cudaEvent_t ev : side_done)
      if (ev != nullptr) cudaEventDestroy(ev);
    if (side_ready != nullptr) cudaEventDestroy(side_ready);
    if (side != nullptr) cudaStreamDestroy(side);
  }
};

int64_t pick_head_rows(const ctdk_model_config& c, int64_t tok) {
  // Block of LM-head rows whose logits take about 1 GiB, in multiples of 128 rows.
  int64_t rows = (int64_t{1} << 30) / (static_cast<int64_t>(c.vocab_size) * 4);
  rows = rows / 128 * 128;
  if (rows < 128) rows = 128;
  if (rows > tok) rows = tok;
  return rows;
}

void carve(Engine& e, Bump& b) {
  const ctdk_model_config& c = e.cfg;
  const int64_t tok = e.tok_cap, hid = c.hidden_size, I = c.intermediate_size;
  const int64_t D = c.head_dim, H = c.num_attention_heads, Hk = c.num_key_value_heads;
  const int L = c.num_hidden_layers;
  e.rope_table = b.floats(e.maxT * D);
  e.xs.assign(L + 1, nullptr);
  for (int i = 0; i <= L; ++i) e.xs[i] = b.floats(tok * hid);
  const int nsets = c.gradient_checkpointing ? (L > 0 ? 1 : 0) : L;
  std::vector<LayerActs> sets(nsets);
  for (int i = 0; i < nsets; ++i) {
    LayerActs& a = sets[i];
    a.h1 = b.floats(tok * hid);
    a.qkv = b.floats(tok * e.QKVN);
    if (c.qk_norm) {
      a.qkv_pre = b.floats(tok * e.QKVN);
      a.rstd_q = b.floats(tok * H);
      a.rstd_k = b.floats(tok * Hk);
    } else {
      a.qkv_pre = a.qkv;
      a.rstd_q = a.rstd_k = nullptr;
    }
    a.attn = b.floats(tok * H * D);
    a.lse = b.floats(e.maxB * H * e.maxT);
    a.hm = b.floats(tok * hid);
    a.h2 = b.floats(tok * hid);
    a.gu = b.floats(tok * 2 * I);
    a.act = b.floats(tok * I);
  }
  e.acts.resize(L);
  for (int i = 0; i < L; ++i) e.acts[i] = sets[c.gradient_checkpointing ? 0 : i];
  e.hf = b.floats(tok * hid);
  e.dh = b.floats(tok * hid);
  e.dtmp = b.floats(tok * hid);
  e.dgu = b.floats(tok * 2 * I);
  e.dact = b.floats(tok * I);
  e.dqkv = b.floats(tok * e.QKVN);
  e.dattn = b.floats(tok * H * D);
  e.delta = b.floats(e.maxB * H * e.maxT);
  e.norm_scratch = b.floats(ctdk_rmsnorm_bwd_scratch_floats(static_cast<int>(hid)));
  e.qk_scratch = b.floats(ctdk_qk_norm_rope_bwd_scratch_floats(static_cast<int>(D)));
  e.logits = b.floats(e.head_rows * c.vocab_size);
  e.hfc = b.floats(tok * hid);
  e.dhfc = b.floats(tok * hid);
  e.mask_c = b.floats(tok);
  e.w_c = b.floats(tok);
  e.tgt_c = reinterpret_cast<int64_t*>(b.floats(2 * tok));
  if (c.precision == CTDK_GEMM_3XTF32) {
    // largest M*K + K*N over every GEMM (M, N, K) of a step: forward, dX and dW of the four
    // projections of a layer, and the three GEMMs of an LM-head block
    const int64_t V = c.vocab_size, HD = H * D, QN = e.QKVN, R = e.head_rows;
    const int64_t proj[4][2] = {{QN, hid}, {hid, HD}, {2 * I, hid}, {hid, I}};  // {N_out, K_in}
    int64_t mx = 0;
    auto need = [&](int64_t M, int64_t N, int64_t K) {
      const int64_t v = M * K + K * N;
      mx = v > mx ? v : mx;
    };
    for (const auto& p : proj) {
      need(tok, p[0], p[1]);   // Y  = X W^T
      need(tok, p[1], p[0]);   // dX = dY W
      need(p[0], p[1], tok);   // dW = dY^T X
    }
    need(R, V, hid);
    need(R, hid, V);
    need(V, hid, R);
    e.ws3_floats = 2 * mx + 128;
    e.ws3 = b.floats(e.ws3_floats);
  }
}

void init_engine_shape(Engine& e, const ctdk_model_config& c, int64_t B, int64_t T) {
  e.cfg = c;
  e.maxB = B;
  e.maxT = T;
  e.tok_cap = B * T;
  e.QKVN = (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim;
  e.head_rows = pick_head_rows(c, e.tok_cap > 0 ? e.tok_cap : 1);
}

#define TRY(expr)                \
  do {                           \
    int rc_ = (expr);            \
    if (rc_ != CTDK_OK) return rc_; \
  } while (0)

ctdk_rope_params rope_params(const ctdk_model_config& c) {
  ctdk_rope_params p;
  p.theta = c.rope_theta;
  p.scaling_factor = c.rope_scaling_factor;
  p.low_freq_wavelen =
      static_cast<float>(c.rope_scaling_original_max_pos) / c.rope_scaling_low_freq_factor;
  p.high_freq_wavelen =
      static_cast<float>(c.rope_scaling_original_max_pos) / c.rope_scaling_high_freq_factor;
  return p;
}

int gemm(const Engine& e, const float* A, const float* B, float* C, int64_t M, int64_t N,
         int64_t K, int ta, int tb, int epi, const float* aux, void* s) {
  const int64_t lda = ta ? M : K, ldb = tb ? K : N;
  if (e.cfg.precision == CTDK_GEMM_3XTF32)
    return ctdk_gemm_ws(A, B, C, M, N, K, lda, ldb, N, ta, tb, CTDK_GEMM_3XTF32, epi, aux, e.ws3, e.ws3_floats, s);
  return ctdk_gemm(A, B, C, M, N, K, lda, ldb, N, ta, tb, e.cfg.precision, epi, aux, s);
}

// A weight-gradient GEMM: on the side stream when the pass uses it, behind everything enqueued on
// the main stream so far.
int dw_gemm(Engine& e, int slot, const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int epi,
            void* s) {
  if (!e.side_on) return gemm(e, A, B, C, M, N, K, 1, 0, epi, nullptr, s);
  if (cudaEventRecord(e.side_ready, static_cast<cudaStream_t>(s)) != cudaSuccess ||
      cudaStreamWaitEvent(e.side, e.side_ready, 0) != cudaSuccess)
    return fail(CTDK_ELAUNCH, "engine: side-stream dependency failed: %s", cudaGetErrorString(cudaGetLastError()));
  TRY(gemm(e, A, B, C, M, N, K, 1, 0, epi, nullptr, e.side));
  if (cudaEventRecord(e.side_done[slot], e.side) != cudaSuccess)
    return fail(CTDK_ELAUNCH, "engine: side-stream event failed: %s", cudaGetErrorString(cudaGetLastError()));
  e.side_pending[slot] = true;
  return CTDK_OK;
}
// The main stream goes on only after the dW GEMM of `slot` has finished (no-op when none is pending).
int dw_wait(Engine& e, int slot, void* s) {
  if (!e.side_pending[slot]) return CTDK_OK;
  e.side_pending[slot] = false;
  if (cudaStreamWaitEvent(static_cast<cudaStream_t>(s), e.side_done[slot], 0) != cudaSuccess)
    return fail(CTDK_ELAUNCH, "engine: side-stream wait failed: %s", cudaGetErrorString(cudaGetLastError()));
  return CTDK_OK;
}
int dw_wait_all(Engine& e, void* s) {
  for (int slot = 0; slot < 4; ++slot) TRY(dw_wait(e, slot, s));
  return CTDK_OK;
}

// Forward of layer l: reads xs[l], writes xs[l+1] and the activation set `a`.
int layer_forward(Engine& e, int l, int64_t B, int64_t T, void* s) {
  const ctdk_model_config& c = e.cfg;
  const LayerSlots& w = e.layout.layers[l];
  const LayerActs& a = e.acts[l];
  const int64_t tok = B * T, hid = c.hidden_size, I = c.intermediate_size;
  const int D = c.head_dim, H = c.num_attention_heads, Hk = c.num_key_value_heads;
  const float* P = e.params;
  const float* x = e.xs[l];
  TRY(ctdk_rmsnorm_fwd(x, P + w.w_in, a.h1, nullptr, tok, static_cast<int>(hid), c.rms_norm_eps, s));
  TRY(gemm(e, a.h1, P + w.wq, a.qkv_pre, tok, e.QKVN, hid, 0, 1, CTDK_EPI_STORE, nullptr, s));
  TRY(ctdk_qk_norm_rope_fwd(a.qkv_pre, a.qkv, c.qk_norm ? P + w.wqn : nullptr,
                            c.qk_norm ? P + w.wkn : nullptr, a.rstd_q, a.rstd_k, e.rope_table, B,
                            T, H, Hk, D, c.rms_norm_eps, s));
  TRY(ctdk_attn_fwd_p(a.qkv, a.attn, a.lse, B, T, H, Hk, D, c.precision, s));
  TRY(gemm(e, a.attn, P + w.wo, a.hm, tok, hid, static_cast<int64_t>(H) * D, 0, 1,
           CTDK_EPI_RESIDUAL, x, s));
  TRY(ctdk_rmsnorm_fwd(a.hm, P + w.w_post, a.h2, nullptr, tok, static_cast<int>(hid),
                       c.rms_norm_eps, s));
  if (c.precision == CTDK_GEMM_TF32) {
    TRY(ctdk_gemm_swiglu(a.h2, P + w.wg, a.gu, a.act, tok, I, hid, CTDK_GEMM_TF32, s));
  } else {
    TRY(gemm(e, a.h2, P + w.wg, a.gu, tok, 2 * I, hid, 0, 1, CTDK_EPI_STORE, nullptr, s));
    TRY(ctdk_swiglu_fwd(a.gu, a.act, tok, static_cast<int>(I), s));
  }
  TRY(gemm(e, a.act, P + w.wd, e.xs[l + 1], tok, hid, I, 0, 1, CTDK_EPI_RESIDUAL, a.hm, s));
  return CTDK_OK;
}

// Backward of layer l: e.dh holds d(xs[l+1]) on entry and d(xs[l]) on exit.
int layer_backward(Engine& e, int l, int64_t B, int64_t T, int accumulate, void* s) {
  const ctdk_model_config& c = e.cfg;
  const LayerSlots& w = e.layout.layers[l];
  const LayerActs& a = e.acts[l];
  const int64_t tok = B * T, hid = c.hidden_size, I = c.intermediate_size;
  const int D = c.head_dim, H = c.num_attention_heads, Hk = c.num_key_value_heads;
  const int64_t HD = static_cast<int64_t>(H) * D;
  const float* P = e.params;
  float* G = e.grads;
  const int wepi = accumulate ? CTDK_EPI_ACCUMULATE : CTDK_EPI_STORE;

  // MLP: y = hm + act Wd^T
  TRY(dw_wait(e, 1, s));   // the layer above's gate|up dW still reads dgu
  if (c.precision == CTDK_GEMM_TF32) {
    TRY(ctdk_gemm_swiglu_bwd(e.dh, P + w.wd, a.gu, e.dgu, e.dact, tok, I, hid, CTDK_GEMM_TF32, s));
    TRY(dw_gemm(e, 0, e.dh, a.act, G + w.wd, hid, I, tok, wepi, s));
  } else {
    TRY(gemm(e, e.dh, P + w.wd, e.dact, tok, I, hid, 0, 0, CTDK_EPI_STORE, nullptr, s));
    TRY(gemm(e, e.dh, a.act, G + w.wd, hid, I, tok, 1, 0, wepi, nullptr, s));
    TRY(ctdk_swiglu_bwd(a.gu, e.dact, e.dgu, tok, static_cast<int>(I), s));
  }
  TRY(gemm(e, e.dgu, P + w.wg, e.dtmp, tok, hid, 2 * I, 0, 0, CTDK_EPI_STORE, nullptr, s));
  TRY(dw_gemm(e, 1, e.dgu, a.h2, G + w.wg, 2 * I, hid, tok, wepi, s));
  TRY(dw_wait(e, 0, s));   // dh is rewritten next; the down-proj dW reads it
  TRY(ctdk_rmsnorm_bwd(e.dtmp, a.hm, P + w.w_post, e.dh, G + w.w_post, e.norm_scratch, tok,
                       static_cast<int>(hid), c.rms_norm_eps, accumulate, 1, s));
  // attention: hm = x + attn Wo^T
  // (the o-proj dX GEMM also forms delta = rowsum(dattn * attn) in its epilogue; the attention backward is told so)
  if (c.precision == CTDK_GEMM_TF32) {
    TRY(ctdk_gemm_dattn_delta(e.dh, P + w.wo, a.attn, e.dattn, e.delta, B, T, H, D, hid, CTDK_GEMM_TF32, s));
  } else {
    TRY(gemm(e, e.dh, P + w.wo, e.dattn, tok, HD, hid, 0, 0, CTDK_EPI_STORE, nullptr, s));
  }
  TRY(dw_gemm(e, 2, e.dh, a.attn, G + w.wo, hid, HD, tok, wepi, s));
  TRY(dw_wait(e, 3, s));   // the layer above's qkv dW still reads dqkv
  TRY(ctdk_attn_bwd_p(a.qkv, c.precision == CTDK_GEMM_TF32 ? nullptr : a.attn, e.dattn, a.lse, e.delta, e.dqkv, B, T, H, Hk, D,
                      c.precision, s));
  TRY(ctdk_qk_norm_rope_bwd(e.dqkv, a.qkv_pre, c.qk_norm ? P + w.wqn : nullptr,
                            c.qk_norm ? P + w.wkn : nullptr, a.rstd_q, a.rstd_k,
                            c.qk_norm ? G + w.wqn : nullptr, c.qk_norm ? G + w.wkn : nullptr,
                            e.qk_scratch, e.rope_table, B, T, H, Hk, D, accumulate, s));
  TRY(gemm(e, e.dqkv, P + w.wq, e.dtmp, tok, hid, e.QKVN, 0, 0, CTDK_EPI_STORE, nullptr, s));
  TRY(dw_gemm(e, 3, e.dqkv, a.h1, G + w.wq, e.QKVN, hid, tok, wepi, s));
  TRY(dw_wait(e, 2, s));   // dh is rewritten next; the o-proj dW reads it
  TRY(ctdk_rmsnorm_bwd(e.dtmp, e.xs[l], P + w.w_in, e.dh, G + w.w_in, e.norm_scratch, tok,
                       static_cast<int>(hid), c.rms_norm_eps, accumulate, 1, s));
  return CTDK_OK;
}

// Measured on SmolLM2-360M: 4 x 1023 rows per GPU 26.6 -> 25.7 ms per pass + update, 32 x 1023 rows
// 168.2 -> 166.3 ms. Off while launches are being timed one by one (ctdk_prof_enable): kernels that
// share the GPU would each be charged the other's time. CTDK_ENGINE_SIDE_STREAM=0 turns it off.
bool use_side_stream(Engine& e) {
  static const bool off = [] {
    const char* v = std::getenv("CTDK_ENGINE_SIDE_STREAM");
    return v != nullptr && v[0] == '0';
  }();
  if (e.cfg.precision != CTDK_GEMM_TF32) return false;   // the operand-split workspace of 3xTF32 is one per engine
  if (off || prof_enabled()) return false;
  if (e.side == nullptr) {
    if (cudaStreamCreateWithFlags(&e.side, cudaStreamNonBlocking) != cudaSuccess) {
      e.side = nullptr;
      cudaGetLastError();
      return false;
    }
    bool ok = cudaEventCreateWithFlags(&e.side_ready, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < 4 && ok; ++i) ok = cudaEventCreateWithFlags(&e.side_done[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
      cudaGetLastError();
      return false;
    }
  }
  return e.side_ready != nullptr && e.side_done[3] != nullptr;
}

int prepare(Engine& e, int64_t B, int64_t T, void* s) {
  CTDK_REQUIRE(B > 0 && T > 0, "engine: empty batch");
  CTDK_REQUIRE(B <= e.maxB && T <= e.maxT && B * T <= e.tok_cap,
               "engine: batch %lld x %lld exceeds the workspace (%lld x %lld)",
               static_cast<long long>(B), static_cast<long long>(T),
               static_cast<long long>(e.maxB), static_cast<long long>(e.maxT));
  if (e.rope_T < T) {
    const ctdk_rope_params rp = rope_params(e.cfg);
    TRY(ctdk_rope_table(e.rope_table, e.maxT, e.cfg.head_dim, 0, &rp, s));
    e.rope_T = e.maxT;
  }
  return CTDK_OK;
}

int run(Engine& e, const int64_t* ids, const int64_t* targets, const float* loss_mask,
        const float* row_weight, int64_t B, int64_t T, int accumulate, float* loss_sums,
        bool backward, void* s) {
  TRY(prepare(e, B, T, s));
  const ctdk_model_config& c = e.cfg;
  const int L = c.num_hidden_layers;
  const int64_t tok = B * T, hid = c.hidden_size, V = c.vocab_size;
  const float* P = e.params;
  float* G = e.grads;
  CTDK_REQUIRE(ids && targets && loss_sums, "engine: null input");
  CTDK_REQUIRE(!backward || row_weight, "engine: row_weight required for the backward");

  if (e.fcb) e.fcb(-1, e.fcb_user);
  TRY(ctdk_embedding_fwd(ids, P + e.layout.embed, e.xs[0], tok, static_cast<int>(hid), V, s));
  for (int l = 0; l < L; ++l) {
    if (e.fcb) e.fcb(l, e.fcb_user);
    TRY(layer_forward(e, l, B, T, s));
  }
  if (e.fcb) e.fcb(L, e.fcb_user);
  TRY(ctdk_rmsnorm_fwd(e.xs[L], P + e.layout.norm, e.hf, nullptr, tok, static_cast<int>(hid),
                       c.rms_norm_eps, s));

  // LM head + masked CE (+ its backward) in row blocks. dhf goes to dtmp. When the caller named the
  // supervised rows, only those are run through the head: hf, targets, mask and weights are
  // compacted first and d(hf) is scattered back into a zeroed buffer afterwards.
  const float* E = P + e.layout.embed;
  float* dE = G + e.layout.embed;
  const bool compact = e.active_rows != nullptr && e.n_active > 0 && e.n_active < tok;
  const int64_t head_n = compact ? e.n_active : tok;
  const float* hf = e.hf;
  const int64_t* tg = targets;
  const float* mk = loss_mask;
  const float* rw = row_weight;
  float* dhf = e.dtmp;
  if (compact) {
    TRY(ctdk_gather_rows(e.hf, e.active_rows, e.hfc, head_n, static_cast<int>(hid), s));
    TRY(ctdk_gather_ce_inputs(targets, loss_mask, row_weight, e.active_rows, e.tgt_c, e.mask_c,
                              backward ? e.w_c : nullptr, head_n, s));
    hf = e.hfc;
    tg = e.tgt_c;
    mk = e.mask_c;
    rw = e.w_c;
    dhf = e.dhfc;
  }
  e.active_rows_last = e.active_rows;
  e.active_rows = nullptr;  // one call only
  e.n_active = 0;
  bool first_block = true;
  for (int64_t r0 = 0; r0 < head_n; r0 += e.head_rows) {
    const int64_t n = (head_n - r0 < e.head_rows) ? head_n - r0 : e.head_rows;
    TRY(gemm(e, hf + r0 * hid, E, e.logits, n, V, hid, 0, 1, CTDK_EPI_STORE, nullptr, s));
    TRY(ctdk_ce_masked(e.logits, tg + r0, mk ? mk + r0 : nullptr, backward ? rw + r0 : nullptr, loss_sums,
                       nullptr, n, V, backward ? 1 : 0, s));
    if (backward) {
      TRY(gemm(e, e.logits, E, dhf + r0 * hid, n, hid, V, 0, 0, CTDK_EPI_STORE, nullptr, s));
      const int epi = (accumulate || !first_block) ? CTDK_EPI_ACCUMULATE : CTDK_EPI_STORE;
      TRY(gemm(e, e.logits, hf + r0 * hid, dE, V, hid, n, 1, 0, epi, nullptr, s));
    }
    first_block = false;
  }
  if (backward && compact) {
    if (cudaMemsetAsync(e.dtmp, 0, sizeof(float) * tok * hid, static_cast<cudaStream_t>(s)) != cudaSuccess)
      return fail(CTDK_ELAUNCH, "engine: memset failed");
    TRY(ctdk_scatter_rows(e.dhfc, e.active_rows_last, e.dtmp, head_n, static_cast<int>(hid), s));
  }
  if (!backward) return CTDK_OK;

  TRY(ctdk_rmsnorm_bwd(e.dtmp, e.xs[L], P + e.layout.norm, e.dh, G + e.layout.norm,
                       e.norm_scratch, tok, static_cast<int>(hid), c.rms_norm_eps, accumulate, 0,
                       s));
  if (e.cb) e.cb(L, e.cb_user);
  e.side_on = use_side_stream(e);
  for (int l = L - 1; l >= 0; --l) {
    if (c.gradient_checkpointing) {
      TRY(dw_wait_all(e, s));   // the recomputation overwrites the one activation set the dW GEMMs read
      TRY(layer_forward(e, l, B, T, s));
    }
    TRY(layer_backward(e, l, B, T, accumulate, s));
    // With the side stream, layer l's weight gradients are ordered before the main stream only one
    // layer later (layer l-1 waits for each of them before it reuses a buffer), so the callback of a
    // layer is made then.
    if (e.cb) {
      if (!e.side_on) e.cb(l, e.cb_user);
      else if (l + 1 < L) e.cb(l + 1, e.cb_user);
    }
  }
  TRY(dw_wait_all(e, s));
  if (e.cb && e.side_on) e.cb(0, e.cb_user);
  e.side_on = false;
  TRY(ctdk_embedding_bwd(ids, e.dh, dE, tok, static_cast<int>(hid), V, s));
  if (e.cb) e.cb(-1, e.cb_user);
  return CTDK_OK;
}

}  // namespace
}  // namespace ctdk

using namespace ctdk;

extern "C" {

int64_t ctdk_model_num_tensors(const ctdk_model_config* cfg) {
  if (validate(cfg) != CTDK_OK) return -1;
  return 2 + static_cast<int64_t>(cfg->num_hidden_layers) * (cfg->qk_norm ? 11 : 9);
}

int ctdk_model_layout(const ctdk_model_config* cfg, int64_t* offsets, int64_t* numels,
                      int* decay, int64_t* total) {
  TRY(validate(cfg));
  const Layout L = make_layout(*cfg);
  for (size_t i = 0; i < L.slots.size(); ++i) {
    if (offsets) offsets[i] = L.slots[i].offset;
    if (numels) numels[i] = L.slots[i].numel;
    if (decay) decay[i] = L.slots[i].decay;
  }
  if (total) *total = L.total;
  return CTDK_OK;
}

int64_t ctdk_engine_workspace_bytes(const ctdk_model_config* cfg, int64_t B, int64_t T) {
  if (validate(cfg) != CTDK_OK || B <= 0 || T <= 0) return -1;
  Engine e;
  init_engine_shape(e, *cfg, B, T);
  e.layout = make_layout(*cfg);
  Bump b(nullptr);
  carve(e, b);
  return b.used;
}

int ctdk_engine_create(const ctdk_model_config* cfg, float* params, float* grads,
                       void* workspace, int64_t workspace_bytes, int64_t B, int64_t T,
                       void** engine) {
  TRY(validate(cfg));
  CTDK_REQUIRE(engine != nullptr, "ctdk_engine_create: null out pointer");
  CTDK_REQUIRE(params && workspace, "ctdk_engine_create: null arena");
  CTDK_REQUIRE(B > 0 && T > 0, "ctdk_engine_create: empty shape");
  CTDK_REQUIRE((reinterpret_cast<uintptr_t>(params) & 255u) == 0 &&
                   (reinterpret_cast<uintptr_t>(grads) & 255u) == 0 &&
                   (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
               "ctdk_engine_create: arenas must be 256-byte aligned");
  Engine* e = new (std::nothrow) Engine();
  if (e == nullptr) return fail(CTDK_ENOMEM, "ctdk_engine_create: out of host memory");
  init_engine_shape(*e, *cfg, B, T);
  e->layout = make_layout(*cfg);
  e->params = params;
  e->grads = grads;
  Bump b(workspace);
  carve(*e, b);
  if (b.used > workspace_bytes) {
    const long long need = b.used;
    delete e;
    return fail(CTDK_EINVAL, "ctdk_engine_create: workspace too small (%lld < %lld bytes)",
                static_cast<long long>(workspace_bytes), need);
  }
  *engine = e;
  return CTDK_OK;
}

int ctdk_engine_destroy(void* engine) {
  delete static_cast<Engine*>(engine);
  return CTDK_OK;
}

int ctdk_engine_set_layer_callback(void* engine, ctdk_layer_callback cb, void* user) {
  CTDK_REQUIRE(engine != nullptr, "ctdk_engine_set_layer_callback: null engine");
  Engine* e = static_cast<Engine*>(engine);
  e->cb = cb;
  e->cb_user = user;
  return CTDK_OK;
}

int ctdk_engine_set_forward_callback(void* engine, ctdk_layer_callback cb, void* user) {
  CTDK_REQUIRE(engine != nullptr, "ctdk_engine_set_forward_callback: null engine");
  Engine* e = static_cast<Engine*>(engine);
  e->fcb = cb;
  e->fcb_user = user;
  return CTDK_OK;
}

int ctdk_engine_set_active_rows(void* engine, const int32_t* rows, int64_t n) {
  CTDK_REQUIRE(engine != nullptr, "ctdk_engine_set_active_rows: null engine");
  Engine* e = static_cast<Engine*>(engine);
  CTDK_REQUIRE(n >= 0 && n <= e->tok_cap, "ctdk_engine_set_active_rows: bad row count");
  e->active_rows = n > 0 ? rows : nullptr;
  e->n_active = n;
  return CTDK_OK;
}

int ctdk_engine_forward_backward(void* engine, const int64_t* ids, const int64_t* targets,
                                 const float* loss_mask, const float* row_weight, int64_t B,
                                 int64_t T, int accumulate, float* loss_sums, void* stream) {
  CTDK_REQUIRE(engine != nullptr, "ctdk_engine_forward_backward: null engine");
  Engine* e = static_cast<Engine*>(engine);
  CTDK_REQUIRE(e->grads != nullptr, "ctdk_engine_forward_backward: engine has no gradient arena");
  return run(*e, ids, targets, loss_mask, row_weight, B, T, accumulate, loss_sums, true, stream);
}

int ctdk_engine_forward_loss(void* engine, const int64_t* ids, const int64_t* targets,
                             const float* loss_mask, int64_t B, int64_t T, float* loss_sums,
                             void* stream) {
  CTDK_REQUIRE(engine != nullptr, "ctdk_engine_forward_loss: null engine");
  return run(*static_cast<Engine*>(engine), ids, targets, loss_mask, nullptr, B, T, 0, loss_sums,
             false, stream);
}

}  // extern "C"
