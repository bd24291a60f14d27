// Data-parallel trainer: one process per GPU, ZeRO-1 over buckets of the parameter arena.
//
// It owns the part of the reference's step loop that follows the backward pass
// (emberlm tools/ctd_train/main.cpp:362-373: clip_grad_norm_, AdamW::step, zero_grad) and adds what a
// multi-GPU run needs around it:
//   - the step's micro-batches are dealt to the ranks by the caller (each row weighted by
//     mask / (A * sum(mask of its micro-batch)), so the summed gradient does not depend on the
//     number of ranks);
//   - the gradient arena is cut into contiguous buckets (the embedding, then groups of decoder
//     layers); rank r owns slice r of every bucket: of the reduced gradients, of AdamW's m and v
//     (which exist only for the slices: 8*P/R bytes per rank instead of the reference's host
//     offload, src/core/optim.cu:94-130) and of the parameter update;
//   - ncclReduceScatter of a bucket is issued from the engine's layer callback, on a communication
//     stream behind an event on the compute stream, as soon as the last layer the bucket needs has
//     been enqueued, so it runs underneath the backward pass of the layers below;
//   - sum of squares per slice -> one scalar ncclAllReduce (with the loss sums) -> clip scale ->
//     fused AdamW per slice -> ncclAllGather of the bucket, left in flight: the next forward pass
//     waits for a bucket only where it first reads it (the engine's forward callback).
// There is no host synchronisation in a step. NCCL is resolved with dlopen at the first
// multi-rank create, so single-GPU users need no NCCL at all and a process that already loaded
// one (PyTorch's) shares it.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"

namespace ctdk {
namespace {

// ---- NCCL entry points, looked up at run time ----------------------------------------------
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                                cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*GetVersion)(int*) = nullptr;
};
NcclApi g_nccl;
std::mutex g_nccl_mu;

int load_nccl() {
  std::lock_guard<std::mutex> lk(g_nccl_mu);
  if (g_nccl.handle != nullptr) return CTDK_OK;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* n : names) {
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h != nullptr) break;
  }
  if (h == nullptr) return fail(CTDK_ELAUNCH, "NCCL not found (libnccl.so.2): %s", dlerror());
  NcclApi api;
  api.handle = h;
  bool ok = true;
  auto sym = [&](const char* name) {
    void* p = dlsym(h, name);
    if (p == nullptr) ok = false;
    return p;
  };
  api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
  api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
  api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
  api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(sym("ncclReduceScatter"));
  api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
  api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
  api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
  api.GetVersion = reinterpret_cast<decltype(api.GetVersion)>(sym("ncclGetVersion"));
  if (!ok) return fail(CTDK_ELAUNCH, "NCCL library lacks an entry point the trainer needs");
  g_nccl = api;
  return CTDK_OK;
}

#define NCCL_TRY(expr)                                                                         \
  do {                                                                                         \
    const ncclResult_t r_ = (expr);                                                            \
    if (r_ != ncclSuccess) return fail(CTDK_ELAUNCH, "%s: %s", #expr, g_nccl.GetErrorString(r_)); \
  } while (0)
#define CUDA_TRY(expr)                                                                      \
  do {                                                                                      \
    const cudaError_t e_ = (expr);                                                          \
    if (e_ != cudaSuccess) return fail(CTDK_ELAUNCH, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)
#define TRY(expr)                   \
  do {                              \
    const int rc_ = (expr);         \
    if (rc_ != CTDK_OK) return rc_; \
  } while (0)

// ---- plan: buckets and weight-decay segments -------------------------------------------------
struct Tensors {
  std::vector<int64_t> off, num;
  std::vector<int> decay, layer;   // layer: -1 embedding, 0..L-1, L final norm
  int64_t total = 0;
};

int describe(const ctdk_model_config* cfg, Tensors* t) {
  const int64_t n = ctdk_model_num_tensors(cfg);
  if (n < 0) return CTDK_EINVAL;
  t->off.resize(n);
  t->num.resize(n);
  t->decay.resize(n);
  TRY(ctdk_model_layout(cfg, t->off.data(), t->num.data(), t->decay.data(), &t->total));
  const int L = cfg->num_hidden_layers, per = cfg->qk_norm ? 11 : 9;
  t->layer.resize(n);
  t->layer[0] = -1;
  for (int64_t i = 1; i + 1 < n; ++i) t->layer[i] = static_cast<int>((i - 1) / per);
  t->layer[n - 1] = L;
  return CTDK_OK;
}

struct BucketPlan {
  int64_t lo, hi;   // arena range, length a multiple of 64 * world
  int ready;        // lowest completion index of the tensors it overlaps (see ctdk_dp_buckets)
};

int64_t padded_total(int64_t total, int world) {
  const int64_t unit = 64 * static_cast<int64_t>(world);
  return (total + unit - 1) / unit * unit;
}

std::vector<BucketPlan> plan_buckets(const Tensors& t, int L, int world, int layers_per_bucket) {
  const int64_t unit = 64 * static_cast<int64_t>(world);
  const int64_t total = padded_total(t.total, world);
  std::vector<int64_t> cuts{0};
  if (layers_per_bucket > 0) {
    for (int l = 0; l < L; l += layers_per_bucket) {
      int64_t first = -1;
      for (size_t i = 0; i < t.off.size(); ++i)
        if (t.layer[i] == l && (first < 0 || t.off[i] < first)) first = t.off[i];
      if (first < 0) continue;
      const int64_t c = first / unit * unit;
      if (c > cuts.back()) cuts.push_back(c);
    }
  }
  cuts.push_back(total);
  std::vector<BucketPlan> out;
  for (size_t k = 0; k + 1 < cuts.size(); ++k) {
    const int64_t lo = cuts[k], hi = cuts[k + 1];
    if (hi <= lo) continue;
    int ready = L;
    bool any = false;
    for (size_t i = 0; i < t.off.size(); ++i)
      if (t.off[i] < hi && t.off[i] + t.num[i] > lo) {
        ready = any ? std::min(ready, t.layer[i]) : t.layer[i];
        any = true;
      }
    out.push_back({lo, hi, any ? ready : L});
  }
  return out;
}

// Runs of equal weight decay inside the arena range [lo, hi): the decay group gets `wd`, norm
// weights and padding 0 (the two ParamGroups of tools/ctd_train/main.cpp:304-311). A tensor's
// padding belongs to it. Ends are exclusive and relative to lo.
void plan_segments(const Tensors& t, float wd, int64_t lo, int64_t hi, std::vector<int64_t>* ends,
                   std::vector<float>* wds) {
  ends->clear();
  wds->clear();
  int64_t pos = lo;
  for (size_t i = 0; i < t.off.size(); ++i) {
    const int64_t o = t.off[i], padded_end = o + (t.num[i] + 63) / 64 * 64;
    if (padded_end <= lo || o >= hi) continue;
    const int64_t end = std::min(padded_end, hi);
    const float w = t.decay[i] ? wd : 0.0f;
    if (!ends->empty() && wds->back() == w) ends->back() = end - lo;
    else {
      ends->push_back(end - lo);
      wds->push_back(w);
    }
    pos = end;
  }
  if (pos < hi) {
    if (!ends->empty() && wds->back() == 0.0f) ends->back() = hi - lo;
    else {
      ends->push_back(hi - lo);
      wds->push_back(0.0f);
    }
  }
  if (ends->empty()) {
    ends->push_back(hi - lo);
    wds->push_back(0.0f);
  }
  ends->back() = hi - lo;
}

// ---- trainer ---------------------------------------------------------------------------------
struct Bucket {
  int64_t lo, hi, a, b, state;
  int ready;
  int64_t* d_seg_end = nullptr;
  float* d_seg_wd = nullptr;
  int nseg = 0;
  cudaEvent_t rs_done = nullptr, ag_done = nullptr;
  bool rs_issued = false, ag_pending = false;
};

struct Trainer {
  ctdk_model_config cfg;
  ctdk_trainer_hparams hp;
  Tensors tensors;
  void* engine = nullptr;
  float *params = nullptr, *grads = nullptr, *m = nullptr, *v = nullptr;
  int rank = 0, world = 1;
  int64_t total = 0, shard = 0;
  ncclComm_t comm = nullptr;
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ev_compute = nullptr, ev_comm = nullptr;
  std::vector<Bucket> buckets;
  std::vector<int> completion_order;   // bucket indices in the order the backward pass completes them
  float* d_small = nullptr;            // [0] sum mask*loss [1] sum mask [2] sum g^2 [3] clip scale [4] norm
  char* d_tables = nullptr;            // segment tables of all buckets
  int64_t step_count = 0;
  bool reduce_in_backward = false;
  cudaStream_t cur = nullptr;          // the caller's stream of the pass in flight (for the callbacks)
  int cb_error = CTDK_OK;
  ctdk_layer_callback user_cb = nullptr;
  void* user_cb_arg = nullptr;
};

int issue_reduce_scatter(Trainer& t, Bucket& bk, cudaStream_t s) {
  CUDA_TRY(cudaEventRecord(t.ev_compute, s));
  CUDA_TRY(cudaStreamWaitEvent(t.comm_stream, t.ev_compute, 0));
  // In place: rank r's output is slice r of the input (recvbuff == sendbuff + rank * recvcount).
  NCCL_TRY(g_nccl.ReduceScatter(t.grads + bk.lo, t.grads + bk.a, static_cast<size_t>(bk.b - bk.a), ncclFloat, ncclSum,
                                t.comm, t.comm_stream));
  CUDA_TRY(cudaEventRecord(bk.rs_done, t.comm_stream));
  bk.rs_issued = true;
  return CTDK_OK;
}

void on_layer(int layer, void* user) {
  Trainer& t = *static_cast<Trainer*>(user);
  if (t.user_cb != nullptr) t.user_cb(layer, t.user_cb_arg);
  if (!t.reduce_in_backward || t.cb_error != CTDK_OK) return;
  for (Bucket& bk : t.buckets)
    if (bk.ready == layer && !bk.rs_issued) {
      const int rc = issue_reduce_scatter(t, bk, t.cur);
      if (rc != CTDK_OK) {
        t.cb_error = rc;
        return;
      }
    }
}

void on_forward(int layer, void* user) {
  Trainer& t = *static_cast<Trainer*>(user);
  for (Bucket& bk : t.buckets)
    if (bk.ag_pending && bk.ready <= layer) {
      if (cudaStreamWaitEvent(t.cur, bk.ag_done, 0) != cudaSuccess && t.cb_error == CTDK_OK)
        t.cb_error = fail(CTDK_ELAUNCH, "trainer: wait for the parameter all-gather failed");
      bk.ag_pending = false;
    }
}

int wait_parameters(Trainer& t, cudaStream_t s) {
  for (Bucket& bk : t.buckets)
    if (bk.ag_pending) {
      CUDA_TRY(cudaStreamWaitEvent(s, bk.ag_done, 0));
      bk.ag_pending = false;
    }
  return CTDK_OK;
}

void destroy(Trainer* t) {
  if (t == nullptr) return;
  if (t->comm_stream != nullptr) cudaStreamSynchronize(t->comm_stream);
  if (t->engine != nullptr) ctdk_engine_destroy(t->engine);
  if (t->comm != nullptr) g_nccl.CommDestroy(t->comm);
  for (Bucket& bk : t->buckets) {
    if (bk.rs_done != nullptr) cudaEventDestroy(bk.rs_done);
    if (bk.ag_done != nullptr) cudaEventDestroy(bk.ag_done);
  }
  if (t->ev_compute != nullptr) cudaEventDestroy(t->ev_compute);
  if (t->ev_comm != nullptr) cudaEventDestroy(t->ev_comm);
  if (t->comm_stream != nullptr) cudaStreamDestroy(t->comm_stream);
  if (t->d_small != nullptr) cudaFree(t->d_small);
  if (t->d_tables != nullptr) cudaFree(t->d_tables);
  delete t;
}

int optimizer_step(Trainer& t, float lr, cudaStream_t s) {
  float* sc = t.d_small;
  CUDA_TRY(cudaMemsetAsync(sc + 2, 0, 3 * sizeof(float), s));
  if (t.world > 1) {
    for (int i : t.completion_order)
      if (!t.buckets[i].rs_issued) TRY(issue_reduce_scatter(t, t.buckets[i], s));
    for (int i : t.completion_order) {
      Bucket& bk = t.buckets[i];
      CUDA_TRY(cudaStreamWaitEvent(s, bk.rs_done, 0));
      bk.rs_issued = false;
      TRY(ctdk_sumsq(t.grads + bk.a, bk.b - bk.a, sc + 2, s));
    }
    // one scalar all-reduce: {sum mask*loss, sum mask, sum g^2}
    CUDA_TRY(cudaEventRecord(t.ev_compute, s));
    CUDA_TRY(cudaStreamWaitEvent(t.comm_stream, t.ev_compute, 0));
    NCCL_TRY(g_nccl.AllReduce(sc, sc, 3, ncclFloat, ncclSum, t.comm, t.comm_stream));
    CUDA_TRY(cudaEventRecord(t.ev_comm, t.comm_stream));
    CUDA_TRY(cudaStreamWaitEvent(s, t.ev_comm, 0));
  } else {
    TRY(ctdk_sumsq(t.grads, t.shard, sc + 2, s));
  }
  TRY(ctdk_clip_scale(sc + 2, t.hp.clip, 1e-6f, sc + 3, sc + 4, s));
  ++t.step_count;
  ctdk_adamw_params ap{};
  ap.lr = lr;
  ap.beta1 = t.hp.beta1;
  ap.beta2 = t.hp.beta2;
  ap.eps = t.hp.eps;
  ap.wd = 0.0f;
  // bias corrections as AdamW::step, src/core/optim.cu:142-143
  ap.bc1 = 1.0f - powf(t.hp.beta1, static_cast<float>(t.step_count));
  ap.bc2 = 1.0f - powf(t.hp.beta2, static_cast<float>(t.step_count));
  for (Bucket& bk : t.buckets) {   // arena order = the order the next forward pass reads them
    const int64_t n = bk.b - bk.a;
    TRY(ctdk_adamw(t.params + bk.a, t.grads + bk.a, t.m + bk.state, t.v + bk.state, n, &ap, sc + 3, bk.d_seg_end,
                   bk.d_seg_wd, bk.nseg, s));
    if (t.world > 1) {
      CUDA_TRY(cudaEventRecord(t.ev_compute, s));
      CUDA_TRY(cudaStreamWaitEvent(t.comm_stream, t.ev_compute, 0));
      NCCL_TRY(g_nccl.AllGather(t.params + bk.a, t.params + bk.lo, static_cast<size_t>(n), ncclFloat, t.comm,
                                t.comm_stream));
      CUDA_TRY(cudaEventRecord(bk.ag_done, t.comm_stream));
      bk.ag_pending = true;
    }
  }
  return CTDK_OK;
}

int forward_backward(Trainer& t, const int64_t* ids, const int64_t* targets, const float* mask, const float* weight,
                     int64_t B, int64_t T, int accumulate, int last, cudaStream_t s) {
  t.cur = s;
  t.cb_error = CTDK_OK;
  t.reduce_in_backward = last != 0 && t.world > 1;
  const int rc = ctdk_engine_forward_backward(t.engine, ids, targets, mask, weight, B, T, accumulate, t.d_small, s);
  t.reduce_in_backward = false;
  if (rc != CTDK_OK) return rc;
  return t.cb_error;
}

}  // namespace
}  // namespace ctdk

using namespace ctdk;

extern "C" {

int64_t ctdk_dp_arena_floats(const ctdk_model_config* cfg, int world) {
  Tensors t;
  if (world < 1 || describe(cfg, &t) != CTDK_OK) return -1;
  return padded_total(t.total, world);
}

int ctdk_dp_num_buckets(const ctdk_model_config* cfg, int world, int layers_per_bucket) {
  Tensors t;
  if (world < 1 || describe(cfg, &t) != CTDK_OK) return -1;
  return static_cast<int>(plan_buckets(t, cfg->num_hidden_layers, world, layers_per_bucket).size());
}

int ctdk_dp_buckets(const ctdk_model_config* cfg, int world, int rank, int layers_per_bucket, int64_t* lo,
                    int64_t* hi, int64_t* own_lo, int64_t* own_hi, int64_t* state_offset, int* ready) {
  Tensors t;
  CTDK_REQUIRE(world >= 1 && rank >= 0 && rank < world, "ctdk_dp_buckets: bad rank / world");
  TRY(describe(cfg, &t));
  int64_t pos = 0;
  const std::vector<BucketPlan> plan = plan_buckets(t, cfg->num_hidden_layers, world, layers_per_bucket);
  for (size_t i = 0; i < plan.size(); ++i) {
    const int64_t n = (plan[i].hi - plan[i].lo) / world;
    if (lo) lo[i] = plan[i].lo;
    if (hi) hi[i] = plan[i].hi;
    if (own_lo) own_lo[i] = plan[i].lo + rank * n;
    if (own_hi) own_hi[i] = plan[i].lo + (rank + 1) * n;
    if (state_offset) state_offset[i] = pos;
    if (ready) ready[i] = plan[i].ready;
    pos += n;
  }
  return CTDK_OK;
}

int ctdk_dp_segments(const ctdk_model_config* cfg, float weight_decay, int64_t lo, int64_t hi, int64_t* seg_end,
                     float* seg_wd, int capacity) {
  Tensors t;
  if (describe(cfg, &t) != CTDK_OK) return -1;
  if (lo < 0 || hi <= lo) {
    fail(CTDK_EINVAL, "ctdk_dp_segments: empty range");
    return -1;
  }
  std::vector<int64_t> ends;
  std::vector<float> wds;
  plan_segments(t, weight_decay, lo, hi, &ends, &wds);
  const int n = static_cast<int>(ends.size());
  if (seg_end != nullptr && seg_wd != nullptr)
    for (int i = 0; i < n && i < capacity; ++i) {
      seg_end[i] = ends[i];
      seg_wd[i] = wds[i];
    }
  return n;
}

int ctdk_trainer_unique_id(void* id128) {
  CTDK_REQUIRE(id128 != nullptr, "ctdk_trainer_unique_id: null pointer");
  TRY(load_nccl());
  ncclUniqueId id;
  NCCL_TRY(g_nccl.GetUniqueId(&id));
  static_assert(sizeof(id) == 128, "ncclUniqueId is 128 bytes");
  std::memcpy(id128, &id, sizeof(id));
  return CTDK_OK;
}

int ctdk_trainer_create(const ctdk_model_config* cfg, float* params, float* grads, float* m, float* v,
                        void* workspace, int64_t workspace_bytes, int64_t B, int64_t T, int rank, int world,
                        const void* nccl_id, const ctdk_trainer_hparams* hp, void** trainer) {
  CTDK_REQUIRE(trainer != nullptr && hp != nullptr, "ctdk_trainer_create: null pointer");
  CTDK_REQUIRE(world >= 1 && rank >= 0 && rank < world, "ctdk_trainer_create: bad rank / world");
  CTDK_REQUIRE(world == 1 || nccl_id != nullptr, "ctdk_trainer_create: several ranks need the NCCL unique id");
  CTDK_REQUIRE(params && grads && m && v, "ctdk_trainer_create: null arena");
  Trainer* t = new (std::nothrow) Trainer();
  if (t == nullptr) return fail(CTDK_ENOMEM, "ctdk_trainer_create: out of host memory");
  t->cfg = *cfg;
  t->hp = *hp;
  t->params = params;
  t->grads = grads;
  t->m = m;
  t->v = v;
  t->rank = rank;
  t->world = world;
  auto bail = [&](int rc) {
    destroy(t);
    return rc;
  };
  if (describe(cfg, &t->tensors) != CTDK_OK) return bail(CTDK_EINVAL);
  t->total = padded_total(t->tensors.total, world);
  t->shard = t->total / world;
  int rc = ctdk_engine_create(cfg, params, grads, workspace, workspace_bytes, B, T, &t->engine);
  if (rc != CTDK_OK) return bail(rc);

  // buckets (one bucket = the whole arena on a single rank) and their weight-decay segments
  const int per = world > 1 ? (hp->layers_per_bucket < 0 ? 4 : hp->layers_per_bucket) : 0;
  const std::vector<BucketPlan> plan = plan_buckets(t->tensors, cfg->num_hidden_layers, world, per);
  std::vector<std::vector<int64_t>> ends(plan.size());
  std::vector<std::vector<float>> wds(plan.size());
  int64_t pos = 0;
  size_t table_bytes = 0;
  for (size_t i = 0; i < plan.size(); ++i) {
    Bucket bk;
    bk.lo = plan[i].lo;
    bk.hi = plan[i].hi;
    bk.ready = plan[i].ready;
    const int64_t n = (bk.hi - bk.lo) / world;
    bk.a = bk.lo + rank * n;
    bk.b = bk.a + n;
    bk.state = pos;
    pos += n;
    plan_segments(t->tensors, hp->weight_decay, bk.a, bk.b, &ends[i], &wds[i]);
    bk.nseg = static_cast<int>(ends[i].size());
    table_bytes += (static_cast<size_t>(bk.nseg) * 12 + 255) / 256 * 256;
    t->buckets.push_back(bk);
  }
  if (cudaMalloc(reinterpret_cast<void**>(&t->d_small), 256) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&t->d_tables), table_bytes + 256) != cudaSuccess)
    return bail(fail(CTDK_ENOMEM, "ctdk_trainer_create: cudaMalloc of the small tables failed"));
  cudaMemset(t->d_small, 0, 256);
  size_t cursor = 0;
  for (size_t i = 0; i < plan.size(); ++i) {
    Bucket& bk = t->buckets[i];
    bk.d_seg_end = reinterpret_cast<int64_t*>(t->d_tables + cursor);
    bk.d_seg_wd = reinterpret_cast<float*>(t->d_tables + cursor + static_cast<size_t>(bk.nseg) * 8);
    cursor += (static_cast<size_t>(bk.nseg) * 12 + 255) / 256 * 256;
    if (cudaMemcpy(bk.d_seg_end, ends[i].data(), static_cast<size_t>(bk.nseg) * 8, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(bk.d_seg_wd, wds[i].data(), static_cast<size_t>(bk.nseg) * 4, cudaMemcpyHostToDevice) != cudaSuccess)
      return bail(fail(CTDK_ELAUNCH, "ctdk_trainer_create: copying the segment tables failed"));
  }
  t->completion_order.resize(t->buckets.size());
  for (size_t i = 0; i < t->buckets.size(); ++i) t->completion_order[i] = static_cast<int>(i);
  std::stable_sort(t->completion_order.begin(), t->completion_order.end(),
                   [&](int x, int y) { return t->buckets[x].ready > t->buckets[y].ready; });

  if (world > 1) {
    if (load_nccl() != CTDK_OK) return bail(CTDK_ELAUNCH);
    ncclUniqueId id;
    std::memcpy(&id, nccl_id, sizeof(id));
    const ncclResult_t nr = g_nccl.CommInitRank(&t->comm, world, id, rank);
    if (nr != ncclSuccess) {
      t->comm = nullptr;
      return bail(fail(CTDK_ELAUNCH, "ncclCommInitRank: %s", g_nccl.GetErrorString(nr)));
    }
    bool ok = cudaStreamCreateWithFlags(&t->comm_stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&t->ev_compute, cudaEventDisableTiming) == cudaSuccess &&
              cudaEventCreateWithFlags(&t->ev_comm, cudaEventDisableTiming) == cudaSuccess;
    for (Bucket& bk : t->buckets)
      ok = ok && cudaEventCreateWithFlags(&bk.rs_done, cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&bk.ag_done, cudaEventDisableTiming) == cudaSuccess;
    if (!ok) return bail(fail(CTDK_ELAUNCH, "ctdk_trainer_create: stream / event creation failed"));
    ctdk_engine_set_forward_callback(t->engine, on_forward, t);
  }
  ctdk_engine_set_layer_callback(t->engine, on_layer, t);
  *trainer = t;
  return CTDK_OK;
}

int ctdk_trainer_destroy(void* trainer) {
  destroy(static_cast<Trainer*>(trainer));
  return CTDK_OK;
}

void* ctdk_trainer_engine(void* trainer) { return trainer ? static_cast<Trainer*>(trainer)->engine : nullptr; }

int ctdk_trainer_set_layer_callback(void* trainer, ctdk_layer_callback cb, void* user) {
  CTDK_REQUIRE(trainer != nullptr, "ctdk_trainer_set_layer_callback: null trainer");
  Trainer* t = static_cast<Trainer*>(trainer);
  t->user_cb = cb;
  t->user_cb_arg = user;
  return CTDK_OK;
}

int ctdk_trainer_zero_loss(void* trainer, void* stream) {
  CTDK_REQUIRE(trainer != nullptr, "ctdk_trainer_zero_loss: null trainer");
  CUDA_TRY(cudaMemsetAsync(static_cast<Trainer*>(trainer)->d_small, 0, 2 * sizeof(float), static_cast<cudaStream_t>(stream)));
  return CTDK_OK;
}

int ctdk_trainer_forward_backward(void* trainer, const int64_t* ids, const int64_t* targets, const float* loss_mask,
                                  const float* row_weight, int64_t B, int64_t T, int accumulate, int last,
                                  void* stream) {
  CTDK_REQUIRE(trainer != nullptr, "ctdk_trainer_forward_backward: null trainer");
  return forward_backward(*static_cast<Trainer*>(trainer), ids, targets, loss_mask, row_weight, B, T, accumulate, last,
                          static_cast<cudaStream_t>(stream));
}

int ctdk_trainer_forward_loss(void* trainer, const int64_t* ids, const int64_t* targets, const float* loss_mask,
                              int64_t B, int64_t T, void* stream) {
  CTDK_REQUIRE(trainer != nullptr, "ctdk_trainer_forward_loss: null trainer");
  Trainer& t = *static_cast<Trainer*>(trainer);
  t.cur = static_cast<cudaStream_t>(stream);
  t.cb_error = CTDK_OK;
  TRY(ctdk_engine_forward_loss(t.engine, ids, targets, loss_mask, B, T, t.d_small, stream));
  return t.cb_error;
}

int ctdk_trainer_allreduce_loss(void* trainer, void* stream) {
  CTDK_REQUIRE(trainer != nullptr, "ctdk_trainer_allreduce_loss: null trainer");
  Trainer& t = *static_cast<Trainer*>(trainer);
  if (t.world == 1) return CTDK_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUDA_TRY(cudaEventRecord(t.ev_compute, s));
  CUDA_TRY(cudaStreamWaitEvent(t.comm_stream, t.ev_compute, 0));
  NCCL_TRY(g_nccl.AllReduce(t.d_small, t.d_small, 2, ncclFloat, ncclSum, t.comm, t.comm_stream));
  CUDA_TRY(cudaEventRecord(t.ev_comm, t.comm_stream));
  CUDA_TRY(cudaStreamWaitEvent(s, t.ev_comm, 0));
  return CTDK_OK;
}

int ctdk_trainer_optimizer_step(void* trainer, float lr, void* stream) {
  CTDK_REQUIRE(trainer != nullptr, "ctdk_trainer_optimizer_step: null trainer");
  return optimizer_step(*static_cast<Trainer*>(trainer), lr, static_cast<cudaStream_t>(stream));
}

int ctdk_trainer_step(void* trainer, const int64_t* ids, const int64_t* targets, const float* loss_mask,
                      const float* row_weight, int64_t B, int64_t T, const int32_t* active_rows, int64_t n_active,
                      float lr, void* stream) {
  CTDK_REQUIRE(trainer != nullptr, "ctdk_trainer_step: null trainer");
  Trainer& t = *static_cast<Trainer*>(trainer);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUDA_TRY(cudaMemsetAsync(t.d_small, 0, 2 * sizeof(float), s));
  if (active_rows != nullptr && n_active > 0) TRY(ctdk_engine_set_active_rows(t.engine, active_rows, n_active));
  TRY(forward_backward(t, ids, targets, loss_mask, row_weight, B, T, 0, 1, s));
  return optimizer_step(t, lr, s);
}

int ctdk_trainer_wait_parameters(void* trainer, void* stream) {
  CTDK_REQUIRE(trainer != nullptr, "ctdk_trainer_wait_parameters: null trainer");
  return wait_parameters(*static_cast<Trainer*>(trainer), static_cast<cudaStream_t>(stream));
}

int ctdk_trainer_read_metrics(void* trainer, float* out5, void* stream) {
  CTDK_REQUIRE(trainer != nullptr && out5 != nullptr, "ctdk_trainer_read_metrics: null pointer");
  Trainer& t = *static_cast<Trainer*>(trainer);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUDA_TRY(cudaMemcpyAsync(out5, t.d_small, 5 * sizeof(float), cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  return ctdk_device_status(stream, nullptr);
}

const float* ctdk_trainer_loss_sums(void* trainer) { return trainer ? static_cast<Trainer*>(trainer)->d_small : nullptr; }

int64_t ctdk_trainer_step_count(void* trainer) { return trainer ? static_cast<Trainer*>(trainer)->step_count : -1; }

int ctdk_trainer_set_step_count(void* trainer, int64_t n) {
  CTDK_REQUIRE(trainer != nullptr && n >= 0, "ctdk_trainer_set_step_count: bad argument");
  static_cast<Trainer*>(trainer)->step_count = n;
  return CTDK_OK;
}

int ctdk_trainer_gather_state(void* trainer, const float* shard_state, float* full, void* stream) {
  CTDK_REQUIRE(trainer != nullptr && shard_state && full, "ctdk_trainer_gather_state: null pointer");
  Trainer& t = *static_cast<Trainer*>(trainer);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (t.world == 1) {
    CUDA_TRY(cudaMemcpyAsync(full, shard_state, static_cast<size_t>(t.total) * sizeof(float), cudaMemcpyDeviceToDevice, s));
    return CTDK_OK;
  }
  CUDA_TRY(cudaEventRecord(t.ev_compute, s));
  CUDA_TRY(cudaStreamWaitEvent(t.comm_stream, t.ev_compute, 0));
  for (const Bucket& bk : t.buckets)
    NCCL_TRY(g_nccl.AllGather(shard_state + bk.state, full + bk.lo, static_cast<size_t>(bk.b - bk.a), ncclFloat, t.comm,
                              t.comm_stream));
  CUDA_TRY(cudaEventRecord(t.ev_comm, t.comm_stream));
  CUDA_TRY(cudaStreamWaitEvent(s, t.ev_comm, 0));
  return CTDK_OK;
}

int ctdk_trainer_scatter_state(void* trainer, const float* full, float* shard_state, void* stream) {
  CTDK_REQUIRE(trainer != nullptr && shard_state && full, "ctdk_trainer_scatter_state: null pointer");
  Trainer& t = *static_cast<Trainer*>(trainer);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (const Bucket& bk : t.buckets)
    CUDA_TRY(cudaMemcpyAsync(shard_state + bk.state, full + bk.a, static_cast<size_t>(bk.b - bk.a) * sizeof(float),
                             cudaMemcpyDeviceToDevice, s));
  return CTDK_OK;
}

}  // extern "C"
