// ctd_train: the reference's SFT trainer (emberlm tools/ctd_train/main.cpp) on the B200 step engine.
//
//   ctd_train --config runs/<name>/config.json
//
// Same config keys and defaults (main.cpp:45-103), same data bins (train.bin int32 [docs, seq_len],
// train_mask.bin int8, val.bin / val_mask.bin; main.cpp:120-138), same document sampling
// (mt19937_64(seed + start_step), one uniform pick per row, main.cpp:327-328, 347-349), same
// shifted batches (main.cpp:145-174), warm-up + cosine schedule (main.cpp:177-188), loss.jsonl events
// (main.cpp:375-407), checkpoints every save_every steps plus final.safetensors with the optimizer
// state in a sibling .opt.safetensors (main.cpp:211-235, 409-420) and resume (main.cpp:300-315).
// Messages go to stderr with the "[ctd_train]" prefix; errors exit 1, usage errors exit 2.
//
// What differs: the grad_accum_steps micro-batches of a step run as fused passes through the
// library's trainer (ctdk_trainer_*; per-row weights mask / (A * sum(mask of the row's micro-batch))
// reproduce mul_scalar(loss, 1/A) + backward per micro-batch); clip and AdamW are fused kernels;
// there is one host sync per step (to log). "offload_optimizer" is accepted and ignored (m / v stay
// in HBM, sharded over the ranks).
//
// Several GPUs: start one process per GPU with RANK, WORLD_SIZE and LOCAL_RANK in the environment
// (what torchrun / torch.distributed.run set). Every rank draws the same document sequence and keeps
// micro-batches rank, rank + WORLD_SIZE, ... (grad_accum_steps must divide by WORLD_SIZE); gradients
// are reduce-scattered, AdamW's m / v are sharded ZeRO-1 style, parameters all-gathered (NCCL). Rank 0
// makes the NCCL unique id and leaves it in a file the others wait for (CTDK_NCCL_ID_FILE, default
// <run dir>/.nccl_id.<parent pid>); rank 0 alone writes loss.jsonl and the checkpoints, with the
// m / v slices gathered for it.
//
// Data feed: the step's rows go to pinned memory as they are in the bins (int32 tokens, int8 masks:
// 5 bytes per token instead of the 24 of int64 ids / targets and fp32 masks), are copied on a copy
// stream and widened on the device (ctdk_batch_widen); the next step's rows are staged and copied
// while the current step runs. Checkpoints move through two pinned buffers so that the file and
// the PCIe link work at the same time (include/ctdk_util/device_io.hpp).
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <filesystem>
#include <memory>
#include <fstream>
#include <iostream>
#include <random>
#include <sstream>
#include <thread>
#include <string>
#include <vector>

#include <cuda_runtime.h>
#include <unistd.h>

#include "../../include/ctdk.h"
#include "../../include/ctdk_util/minijson.hpp"
#include "model_desc.hpp"
#include "../../include/ctdk_util/device_io.hpp"
#include "../../include/ctdk_util/safetensors.hpp"

namespace fs = std::filesystem;

namespace {

#define CUDA_OK(expr)                                                                          \
  do {                                                                                         \
    const cudaError_t e_ = (expr);                                                             \
    if (e_ != cudaSuccess) throw std::runtime_error(std::string(#expr) + ": " + cudaGetErrorString(e_)); \
  } while (0)
#define CTDK_OK_OR_THROW(expr)                                                     \
  do {                                                                             \
    if ((expr) != CTDK_OK) throw std::runtime_error(std::string(ctdk_last_error())); \
  } while (0)

struct Config {
  std::string run_name;
  fs::path run_dir, init_weights, resume_from, data_dir;
  int seq_len = 1024, batch_size = 1, grad_accum_steps = 8, total_steps = 2800, warmup_steps = 100;
  float lr = 3e-4f, min_lr_ratio = 0.1f, weight_decay = 0.1f, beta1 = 0.9f, beta2 = 0.95f, eps = 1e-8f;
  float clip_grad_norm = 1.0f;
  int val_every = 100, save_every = 500, log_every = 1;
  uint64_t seed = 42;
  bool offload_optimizer = false, gradient_checkpointing = false;
  int precision = CTDK_GEMM_TF32;   // extra key "precision": "tf32" (default) or "3xtf32"
};

std::string slurp(const fs::path& p) {
  std::ifstream f(p, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open config " + p.string());
  std::ostringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

Config load_config(const fs::path& path) {
  const minijson::Value j = minijson::parse(slurp(path));
  Config c;
  c.run_dir = path.parent_path();
  c.run_name = j.value("run_name", c.run_dir.filename().string());
  c.init_weights = j.at("init_weights").string();
  if (j.contains("resume_from")) c.resume_from = j.at("resume_from").string();
  c.data_dir = j.at("data_dir").string();
  auto geti = [&](const char* k, int d) { return static_cast<int>(j.value(k, static_cast<double>(d))); };
  auto getf = [&](const char* k, float d) { return static_cast<float>(j.value(k, static_cast<double>(d))); };
  c.seq_len = geti("seq_len", c.seq_len);
  c.batch_size = geti("batch_size", c.batch_size);
  c.grad_accum_steps = geti("grad_accum_steps", c.grad_accum_steps);
  c.total_steps = geti("total_steps", c.total_steps);
  c.warmup_steps = geti("warmup_steps", c.warmup_steps);
  c.lr = getf("lr", c.lr);
  c.min_lr_ratio = getf("min_lr_ratio", c.min_lr_ratio);
  c.weight_decay = getf("weight_decay", c.weight_decay);
  c.beta1 = getf("beta1", c.beta1);
  c.beta2 = getf("beta2", c.beta2);
  c.eps = getf("eps", c.eps);
  c.clip_grad_norm = getf("clip_grad_norm", c.clip_grad_norm);
  c.val_every = geti("val_every", c.val_every);
  c.save_every = geti("save_every", c.save_every);
  c.log_every = geti("log_every", c.log_every);
  if (j.contains("seed")) c.seed = j.at("seed").as_uint64();
  c.offload_optimizer = j.value("offload_optimizer", c.offload_optimizer);
  c.gradient_checkpointing = j.value("gradient_checkpointing", c.gradient_checkpointing);
  const std::string prec = j.value("precision", std::string("tf32"));
  if (prec == "3xtf32") c.precision = CTDK_GEMM_3XTF32;
  else if (prec != "tf32") throw std::runtime_error("config: precision must be \"tf32\" or \"3xtf32\"");
  if (c.seq_len < 2 || c.batch_size < 1 || c.grad_accum_steps < 1) throw std::runtime_error("config: seq_len >= 2, batch_size >= 1, grad_accum_steps >= 1 required");
  return c;
}

std::vector<unsigned char> read_file(const fs::path& p) {
  std::ifstream f(p, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + p.string());
  f.seekg(0, std::ios::end);
  const size_t n = static_cast<size_t>(f.tellg());
  f.seekg(0, std::ios::beg);
  std::vector<unsigned char> buf(n);
  if (n > 0 && !f.read(reinterpret_cast<char*>(buf.data()), static_cast<std::streamsize>(n))) throw std::runtime_error("short read " + p.string());
  return buf;
}

struct Split {
  std::vector<int32_t> tokens;   // [docs, seq_len]
  std::vector<int8_t> masks;     // [docs, seq_len]
  int64_t docs = 0;
};

Split load_split(const fs::path& tok, const fs::path& mask, int seq_len) {
  const auto tb = read_file(tok);
  const auto mb = read_file(mask);
  const size_t row = static_cast<size_t>(seq_len) * 4;
  if (tb.size() % row != 0) throw std::runtime_error("token bin size not multiple of seq_len*4: " + tok.string());
  Split s;
  s.docs = static_cast<int64_t>(tb.size() / row);
  if (static_cast<int64_t>(mb.size()) != s.docs * seq_len) throw std::runtime_error("mask size mismatch for " + mask.string());
  s.tokens.resize(tb.size() / 4);
  std::memcpy(s.tokens.data(), tb.data(), tb.size());
  s.masks.resize(mb.size());
  std::memcpy(s.masks.data(), mb.data(), mb.size());
  return s;
}

float lr_at_step(int step, const Config& c) {
  if (step < c.warmup_steps) return c.lr * (static_cast<float>(step) / static_cast<float>(std::max(1, c.warmup_steps)));
  const int decay = std::max(1, c.total_steps - c.warmup_steps);
  const int s = std::min(step - c.warmup_steps, decay);
  const float t = static_cast<float>(s) / static_cast<float>(decay);
  const float cosf_ = 0.5f * (1.0f + std::cos(static_cast<float>(M_PI) * t));
  const float lo = c.lr * c.min_lr_ratio;
  return lo + (c.lr - lo) * cosf_;
}

template <typename T>
struct DeviceBuf {
  T* p = nullptr;
  size_t n = 0;
  DeviceBuf() = default;
  explicit DeviceBuf(size_t count) { alloc(count); }
  DeviceBuf(const DeviceBuf&) = delete;
  DeviceBuf& operator=(const DeviceBuf&) = delete;
  void alloc(size_t count) {   // zero-filled
    n = count;
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&p), std::max<size_t>(count, 1) * sizeof(T)));
    CUDA_OK(cudaMemset(p, 0, std::max<size_t>(count, 1) * sizeof(T)));
  }
  ~DeviceBuf() {
    if (p) cudaFree(p);
  }
};

template <typename T>
struct PinnedBuf {
  T* p = nullptr;
  explicit PinnedBuf(size_t count) {
    CUDA_OK(cudaMallocHost(reinterpret_cast<void**>(&p), std::max<size_t>(count, 1) * sizeof(T)));
  }
  PinnedBuf(const PinnedBuf&) = delete;
  PinnedBuf& operator=(const PinnedBuf&) = delete;
  ~PinnedBuf() {
    if (p) cudaFreeHost(p);
  }
};

// One fused pass inside a staged set of rows.
struct Pass {
  int64_t row0 = 0, rows = 0;       // rows of the staging buffers
  int64_t act0 = 0, n_active = 0;   // its supervised positions (relative to the pass) in the active list
};

// The rows of one step (or one block of validation rows) of this rank as they lie in the bins, in
// pinned memory and, after copy(), on the device.
struct Staging {
  PinnedBuf<int32_t> h_tok;
  PinnedBuf<int8_t> h_msk;
  PinnedBuf<int32_t> h_act;
  DeviceBuf<int32_t> d_tok, d_act;
  DeviceBuf<int8_t> d_msk;
  std::vector<Pass> passes;
  cudaEvent_t ready = nullptr;
  int64_t rows = 0, n_act = 0;
  Staging(int64_t max_rows, int S)
      : h_tok(max_rows * S), h_msk(max_rows * S), h_act(max_rows * S), d_tok(max_rows * S), d_act(max_rows * S),
        d_msk(max_rows * S) {
    CUDA_OK(cudaEventCreateWithFlags(&ready, cudaEventDisableTiming));
  }
  Staging(const Staging&) = delete;
  Staging& operator=(const Staging&) = delete;
  ~Staging() {
    if (ready) cudaEventDestroy(ready);
  }
  // docs: the documents of consecutive passes of at most pass_rows rows each. A pass whose mask is
  // empty is dropped (main.cpp:350: such a micro-batch contributes nothing).
  void fill(const Split& split, const std::vector<int64_t>& docs, int64_t pass_rows, int S) {
    const int T = S - 1;
    passes.clear();
    rows = static_cast<int64_t>(docs.size());
    n_act = 0;
    for (int64_t r = 0; r < rows; ++r) {
      std::memcpy(h_tok.p + r * S, split.tokens.data() + docs[r] * S, static_cast<size_t>(S) * 4);
      std::memcpy(h_msk.p + r * S, split.masks.data() + docs[r] * S, static_cast<size_t>(S));
    }
    for (int64_t r0 = 0; r0 < rows; r0 += pass_rows) {
      Pass ps;
      ps.row0 = r0;
      ps.rows = std::min(pass_rows, rows - r0);
      ps.act0 = n_act;
      for (int64_t r = 0; r < ps.rows; ++r) {
        const int8_t* m = h_msk.p + (r0 + r) * S;
        for (int t = 0; t < T; ++t)
          if (m[t + 1] != 0) h_act.p[n_act++] = static_cast<int32_t>(r * T + t);
      }
      ps.n_active = n_act - ps.act0;
      if (ps.n_active > 0) passes.push_back(ps);
    }
  }
  void copy(int S, cudaStream_t copy_stream) {
    if (rows > 0) {
      CUDA_OK(cudaMemcpyAsync(d_tok.p, h_tok.p, static_cast<size_t>(rows) * S * 4, cudaMemcpyHostToDevice, copy_stream));
      CUDA_OK(cudaMemcpyAsync(d_msk.p, h_msk.p, static_cast<size_t>(rows) * S, cudaMemcpyHostToDevice, copy_stream));
    }
    if (n_act > 0)
      CUDA_OK(cudaMemcpyAsync(d_act.p, h_act.p, static_cast<size_t>(n_act) * 4, cudaMemcpyHostToDevice, copy_stream));
    CUDA_OK(cudaEventRecord(ready, copy_stream));
  }
};

fs::path opt_path_for(const fs::path& weights) { return weights.string() + ".opt.safetensors"; }

std::string parse_config_path(int argc, char** argv) {
  std::string cfg;
  for (int i = 1; i < argc; ++i) {
    if (std::string(argv[i]) == "--config" && i + 1 < argc) cfg = argv[++i];
  }
  if (cfg.empty()) {
    std::cerr << "usage: " << argv[0] << " --config <path-to-config.json>\n";
    std::exit(2);
  }
  return cfg;
}

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return (v != nullptr && *v != '\0') ? std::atoi(v) : fallback;
}

// Rank 0 writes the 128-byte NCCL unique id to `path` (through a temporary name, so a reader never
// sees half of it); the other ranks wait for the file.
void exchange_nccl_id(const fs::path& path, int rank, unsigned char id[128]) {
  if (rank == 0) {
    CTDK_OK_OR_THROW(ctdk_trainer_unique_id(id));
    const fs::path tmp = path.string() + ".tmp";
    {
      std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
      f.write(reinterpret_cast<const char*>(id), 128);
      if (!f) throw std::runtime_error("cannot write " + tmp.string());
    }
    fs::rename(tmp, path);
    return;
  }
  for (int tries = 0; tries < 1200; ++tries) {   // up to two minutes
    std::error_code ec;
    if (fs::exists(path, ec) && fs::file_size(path, ec) == 128) {
      std::ifstream f(path, std::ios::binary);
      if (f.read(reinterpret_cast<char*>(id), 128)) return;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
  }
  throw std::runtime_error("rank 0's NCCL id never appeared at " + path.string());
}

}  // namespace

int main(int argc, char** argv) try {
  const std::string cfg_path = parse_config_path(argc, argv);
  const Config cfg = load_config(cfg_path);
  const int rank = env_int("RANK", 0), world = std::max(1, env_int("WORLD_SIZE", 1)), local = env_int("LOCAL_RANK", rank);
  if (rank < 0 || rank >= world) throw std::runtime_error("RANK must be in [0, WORLD_SIZE)");
  if (cfg.grad_accum_steps % world != 0)
    throw std::runtime_error("grad_accum_steps (" + std::to_string(cfg.grad_accum_steps) + ") must divide by WORLD_SIZE (" +
                             std::to_string(world) + "): whole micro-batches are dealt to the ranks");
  const bool chief = rank == 0;
  auto say = [&](const std::string& msg) {
    if (chief) std::cerr << "[ctd_train] " << msg << "\n";
  };
  if (chief) fs::create_directories(cfg.run_dir);
  say("run=" + cfg.run_name + " dir=\"" + cfg.run_dir.string() + "\"" + (world > 1 ? " ranks=" + std::to_string(world) : ""));
  const bool resuming = !cfg.resume_from.empty();
  const fs::path weights_path = resuming ? cfg.resume_from : cfg.init_weights;
  say(std::string(resuming ? "resuming from " : "loading init weights ") + "\"" + weights_path.string() + "\"");

  st::File wfile(weights_path.string());
  const st::Entry& emb = wfile.entry("model.embed_tokens.weight");
  if (emb.shape.size() != 2) throw std::runtime_error("autodetect_config: model.embed_tokens.weight must be 2-D");
  ctdk_model_config mc = cli::autodetect_config(emb.shape[0], emb.shape[1]);
  mc.gradient_checkpointing = cfg.gradient_checkpointing ? 1 : 0;
  mc.precision = cfg.precision;
  say("arch: hidden=" + std::to_string(mc.hidden_size) + " layers=" + std::to_string(mc.num_hidden_layers) +
      " heads=" + std::to_string(mc.num_attention_heads));
  if (cfg.gradient_checkpointing) say("gradient checkpointing enabled");
  if (cfg.offload_optimizer) say("offload_optimizer ignored: optimizer state stays in HBM");

  int64_t layout_floats = 0;
  const std::vector<cli::ParamDesc> params = cli::describe_parameters(mc, &layout_floats);
  size_t n_decay = 0;
  for (const auto& p : params) n_decay += p.decay ? 1 : 0;
  say("parameters: " + std::to_string(n_decay) + " decay + " + std::to_string(params.size() - n_decay) + " no_decay");

  // ---- device state: parameter / gradient arenas, this rank's slices of AdamW's moments ----
  CUDA_OK(cudaSetDevice(local));
  cudaStream_t stream, copy_stream;
  CUDA_OK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  CUDA_OK(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));
  const int64_t arena = ctdk_dp_arena_floats(&mc, world);
  if (arena < layout_floats) throw std::runtime_error(ctdk_last_error());
  const int64_t shard = arena / world;
  DeviceBuf<float> d_params(arena), d_grads(arena), d_m(shard), d_v(shard);   // all zero-filled
  st::PinnedPipe pipe;
  {
    std::FILE* f = std::fopen(weights_path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open " + weights_path.string());
    for (const auto& p : params)
      st::read_f32_to_device(wfile, weights_path.string(), f, p.name, d_params.p + p.offset, p.numel, pipe);
    pipe.synchronize();
    std::fclose(f);
  }

  say("loading data from \"" + cfg.data_dir.string() + "\"");
  const Split train = load_split(cfg.data_dir / "train.bin", cfg.data_dir / "train_mask.bin", cfg.seq_len);
  const Split val = load_split(cfg.data_dir / "val.bin", cfg.data_dir / "val_mask.bin", cfg.seq_len);
  say("train=" + std::to_string(train.docs) + " val=" + std::to_string(val.docs));
  if (train.docs < 1) throw std::runtime_error("train split is empty");

  // Micro-batches of this rank fused per pass: all of them if the workspace fits in free memory, else halved.
  const int T = cfg.seq_len - 1, S = cfg.seq_len;
  const int my_accum = cfg.grad_accum_steps / world;
  int fused = my_accum;
  int64_t ws_bytes = 0;
  for (;; fused = (fused + 1) / 2) {
    ws_bytes = ctdk_engine_workspace_bytes(&mc, static_cast<int64_t>(fused) * cfg.batch_size, T);
    if (ws_bytes < 0) throw std::runtime_error(ctdk_last_error());
    size_t free_b = 0, total_b = 0;
    CUDA_OK(cudaMemGetInfo(&free_b, &total_b));
    if (static_cast<double>(ws_bytes) < 0.9 * static_cast<double>(free_b) || fused == 1) break;
  }
  const int64_t pass_rows = static_cast<int64_t>(fused) * cfg.batch_size;
  const int64_t step_rows = static_cast<int64_t>(my_accum) * cfg.batch_size;
  say(std::to_string(fused) + " of " + std::to_string(my_accum) + " micro-batches per pass, workspace " +
      std::to_string(ws_bytes >> 20) + " MiB");
  unsigned char* d_ws = nullptr;   // scratch: not zero-filled
  CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_ws), static_cast<size_t>(ws_bytes)));

  unsigned char nccl_id[128] = {0};
  fs::path id_file;
  if (world > 1) {
    const char* named = std::getenv("CTDK_NCCL_ID_FILE");
    id_file = named != nullptr ? fs::path(named)
                               : cfg.run_dir / (".nccl_id." + std::to_string(static_cast<long>(getppid())));
    exchange_nccl_id(id_file, rank, nccl_id);
  }
  ctdk_trainer_hparams hp{};
  hp.lr = cfg.lr;
  hp.beta1 = cfg.beta1;
  hp.beta2 = cfg.beta2;
  hp.eps = cfg.eps;
  hp.weight_decay = cfg.weight_decay;
  hp.clip = cfg.clip_grad_norm;
  hp.layers_per_bucket = -1;
  void* trainer = nullptr;
  CTDK_OK_OR_THROW(ctdk_trainer_create(&mc, d_params.p, d_grads.p, d_m.p, d_v.p, d_ws, ws_bytes, pass_rows, T, rank, world,
                                       world > 1 ? nccl_id : nullptr, &hp, &trainer));
  void* engine = ctdk_trainer_engine(trainer);

  int64_t step_count = 0;
  if (resuming) {
    const fs::path op = opt_path_for(cfg.resume_from);
    if (fs::exists(op)) {
      say("loading optimizer state \"" + op.string() + "\"");
      st::File ofile(op.string());
      std::FILE* f = std::fopen(op.c_str(), "rb");
      if (!f) throw std::runtime_error("cannot open " + op.string());
      // each of m, v: the whole arena-order array into the gradient arena, then this rank's slices out of it
      for (int which = 0; which < 2; ++which) {
        const std::string prefix = which == 0 ? "optimizer.m." : "optimizer.v.";
        CUDA_OK(cudaMemsetAsync(d_grads.p, 0, static_cast<size_t>(arena) * sizeof(float), pipe.stream()));
        for (const auto& p : params) {
          if (!ofile.has(prefix + p.name)) throw std::runtime_error("resume: missing " + prefix + p.name);
          st::read_f32_to_device(ofile, op.string(), f, prefix + p.name, d_grads.p + p.offset, p.numel, pipe);
        }
        pipe.synchronize();
        CTDK_OK_OR_THROW(ctdk_trainer_scatter_state(trainer, d_grads.p, which == 0 ? d_m.p : d_v.p, stream));
        CUDA_OK(cudaStreamSynchronize(stream));
      }
      std::fclose(f);
      if (!ofile.has("optimizer.step")) throw std::runtime_error("resume: missing optimizer.step");
      float sf = 0.0f;
      ofile.read_f32("optimizer.step", &sf, 1);
      step_count = static_cast<int64_t>(sf);
      CTDK_OK_OR_THROW(ctdk_trainer_set_step_count(trainer, step_count));
      say("resumed at step " + std::to_string(step_count));
    } else {
      say("no optimizer state at \"" + op.string() + "\" — continuing with fresh m/v (warmup will restart)");
    }
  }
  const int64_t start_step = step_count;

  const size_t pass_n = static_cast<size_t>(pass_rows) * static_cast<size_t>(T);
  DeviceBuf<int64_t> d_ids(pass_n), d_tgt(pass_n);
  DeviceBuf<float> d_mask(pass_n), d_w(pass_n), d_sums(static_cast<size_t>(pass_rows) + 1);
  const int64_t stage_rows = std::max<int64_t>(step_rows, pass_rows);
  Staging slot_a(stage_rows, S), slot_b(stage_rows, S);
  Staging* slots[2] = {&slot_a, &slot_b};

  // Widens one staged pass on the device and names its supervised rows to the engine.
  auto widen_pass = [&](const Staging& st, const Pass& ps, int micro_rows, int accum_total) {
    CTDK_OK_OR_THROW(ctdk_batch_widen(st.d_tok.p + ps.row0 * S, st.d_msk.p + ps.row0 * S, ps.rows, S, micro_rows,
                                      accum_total, d_ids.p, d_tgt.p, d_mask.p, d_w.p, d_sums.p, stream));
    CTDK_OK_OR_THROW(ctdk_engine_set_active_rows(engine, st.d_act.p + ps.act0, ps.n_active));
  };

  auto save_checkpoint = [&](const fs::path& ckpt) {
    // the all-gathers of the last step must have landed before the parameters are read
    CTDK_OK_OR_THROW(ctdk_trainer_wait_parameters(trainer, stream));
    CUDA_OK(cudaStreamSynchronize(stream));
    std::vector<st::Item> witems, oitems;
    for (const auto& p : params) witems.push_back({p.name, p.shape, nullptr});
    // optimizer file: all m tensors (decay group first, then no-decay, main.cpp:218-226), then all v
    // tensors, then the step counter; offsets are in the header, so any reader finds them by name
    std::vector<const cli::ParamDesc*> order;
    for (int pass = 0; pass < 2; ++pass)
      for (const auto& p : params)
        if (p.decay == (pass == 0)) order.push_back(&p);
    for (const char* prefix : {"optimizer.m.", "optimizer.v."})
      for (const cli::ParamDesc* p : order) oitems.push_back({prefix + p->name, p->shape, nullptr});
    oitems.push_back({"optimizer.step", {1}, nullptr});
    if (chief) {
      st::DeviceWriter w(ckpt.string(), witems, pipe);
      for (const auto& p : params) w.append_device(d_params.p + p.offset);
      w.close();
    }
    std::unique_ptr<st::DeviceWriter> ow;
    if (chief) ow = std::make_unique<st::DeviceWriter>(opt_path_for(ckpt).string(), oitems, pipe);
    for (int which = 0; which < 2; ++which) {
      // every rank's slices, assembled in arena order in the gradient arena (free between steps)
      CTDK_OK_OR_THROW(ctdk_trainer_gather_state(trainer, which == 0 ? d_m.p : d_v.p, d_grads.p, stream));
      CUDA_OK(cudaStreamSynchronize(stream));
      if (chief)
        for (const cli::ParamDesc* p : order) ow->append_device(d_grads.p + p->offset);
    }
    if (chief) {
      const float sf = static_cast<float>(step_count);
      ow->append_host(&sf);
      ow->close();
    }
  };

  auto run_val = [&]() -> float {
    // validation rows in blocks of pass_rows; block k belongs to rank k % world; one all-reduce at the end
    CTDK_OK_OR_THROW(ctdk_trainer_zero_loss(trainer, stream));
    Staging& st = *slots[0];
    int64_t block = 0;
    for (int64_t d0 = 0; d0 < val.docs; d0 += pass_rows, ++block) {
      if (block % world != rank) continue;
      std::vector<int64_t> docs;
      for (int64_t d = d0; d < std::min(val.docs, d0 + pass_rows); ++d) docs.push_back(d);
      CUDA_OK(cudaStreamSynchronize(stream));   // the previous block has consumed the staging buffers
      st.fill(val, docs, pass_rows, S);
      st.copy(S, copy_stream);
      CUDA_OK(cudaStreamWaitEvent(stream, st.ready, 0));
      for (const Pass& ps : st.passes) {
        widen_pass(st, ps, 1, 1);
        CTDK_OK_OR_THROW(ctdk_trainer_forward_loss(trainer, d_ids.p, d_tgt.p, d_mask.p, ps.rows, T, stream));
      }
    }
    CTDK_OK_OR_THROW(ctdk_trainer_allreduce_loss(trainer, stream));
    float m5[5];
    CTDK_OK_OR_THROW(ctdk_trainer_read_metrics(trainer, m5, stream));
    return m5[1] > 0.0f ? m5[0] / m5[1] : 0.0f;
  };

  std::mt19937_64 rng(cfg.seed + static_cast<uint64_t>(start_step));
  std::uniform_int_distribution<int64_t> pick(0, train.docs - 1);
  // The step's documents, drawn micro-batch by micro-batch, row by row, identically on every rank
  // (main.cpp:347-349); this rank keeps micro-batches rank, rank + world, ...
  auto stage_step = [&](Staging& st) {
    std::vector<int64_t> mine;
    for (int mb = 0; mb < cfg.grad_accum_steps; ++mb)
      for (int r = 0; r < cfg.batch_size; ++r) {
        const int64_t d = pick(rng);
        if (mb % world == rank) mine.push_back(d);
      }
    st.fill(train, mine, pass_rows, S);
    st.copy(S, copy_stream);
  };

  const fs::path log_path = cfg.run_dir / "loss.jsonl";
  std::ofstream log;
  if (chief) {
    log.open(log_path, resuming ? (std::ios::out | std::ios::app) : (std::ios::out | std::ios::trunc));
    if (!log) throw std::runtime_error("cannot open log " + log_path.string());
  }
  const auto t_run = std::chrono::steady_clock::now();

  const int first_step = static_cast<int>(start_step) + 1;
  if (first_step <= cfg.total_steps) stage_step(*slots[first_step & 1]);
  for (int step = first_step; step <= cfg.total_steps; ++step) {
    const auto t_step = std::chrono::steady_clock::now();
    Staging& st = *slots[step & 1];
    CUDA_OK(cudaStreamWaitEvent(stream, st.ready, 0));
    CTDK_OK_OR_THROW(ctdk_trainer_zero_loss(trainer, stream));
    for (size_t i = 0; i < st.passes.size(); ++i) {
      widen_pass(st, st.passes[i], cfg.batch_size, cfg.grad_accum_steps);
      CTDK_OK_OR_THROW(ctdk_trainer_forward_backward(trainer, d_ids.p, d_tgt.p, d_mask.p, d_w.p, st.passes[i].rows, T,
                                                     i == 0 ? 0 : 1, i + 1 == st.passes.size() ? 1 : 0, stream));
    }
    if (st.passes.empty())   // every mask of this rank's rows was empty
      CUDA_OK(cudaMemsetAsync(d_grads.p, 0, static_cast<size_t>(arena) * sizeof(float), stream));
    const float lr = lr_at_step(step, cfg);
    CTDK_OK_OR_THROW(ctdk_trainer_optimizer_step(trainer, lr, stream));
    ++step_count;
    // the next step's rows are staged and copied while this step runs
    const bool val_now = cfg.val_every > 0 && step % cfg.val_every == 0;
    if (step < cfg.total_steps && !val_now) stage_step(*slots[(step + 1) & 1]);
    float m5[5];
    CTDK_OK_OR_THROW(ctdk_trainer_read_metrics(trainer, m5, stream));   // the step's one host sync

    const auto t_end = std::chrono::steady_clock::now();
    const double step_s = std::chrono::duration<double>(t_end - t_step).count();
    const double wall_s = std::chrono::duration<double>(t_end - t_run).count();
    const float train_loss = m5[1] > 0.0f ? m5[0] / m5[1] : 0.0f;
    const double tps = static_cast<double>(m5[1]) / std::max(step_s, 1e-9);
    if (chief && cfg.log_every > 0 && step % cfg.log_every == 0) {
      log << minijson::Line().add("step", static_cast<long long>(step)).add("phase", std::string("train")).add("loss", train_loss)
                 .add("lr", lr).add("grad_norm", m5[4]).add("tokens_per_sec", tps).add("wall_s", wall_s).dump()
          << "\n";
      log.flush();
      std::cerr << "[step " << step << "/" << cfg.total_steps << "] loss=" << train_loss << " lr=" << lr << " |g|=" << m5[4]
                << " tok/s=" << static_cast<long long>(tps) << "\n";
    }
    if (val_now) {
      const auto t_val = std::chrono::steady_clock::now();
      const float vl = run_val();
      const auto now = std::chrono::steady_clock::now();
      if (chief) {
        log << minijson::Line().add("step", static_cast<long long>(step)).add("phase", std::string("val")).add("loss", vl)
                   .add("wall_s", std::chrono::duration<double>(now - t_run).count()).dump()
            << "\n";
        log.flush();
        std::cerr << "[step " << step << "] val_loss=" << vl << " (" << std::chrono::duration<double>(now - t_val).count() << "s)\n";
      }
      if (step < cfg.total_steps) stage_step(*slots[(step + 1) & 1]);   // validation used a staging slot
    }
    if (cfg.save_every > 0 && step % cfg.save_every == 0) {
      const fs::path ckpt = cfg.run_dir / ("ckpt_step_" + std::to_string(step) + ".safetensors");
      save_checkpoint(ckpt);
      if (chief) std::cerr << "[step " << step << "] saved " << ckpt << " (+ optimizer)\n";
    }
  }

  const fs::path final_ckpt = cfg.run_dir / "final.safetensors";
  save_checkpoint(final_ckpt);
  say("done. final → \"" + final_ckpt.string() + "\" (+ optimizer)");
  ctdk_trainer_destroy(trainer);
  if (chief && !id_file.empty()) {
    std::error_code ec;
    fs::remove(id_file, ec);
  }
  cudaFree(d_ws);
  cudaStreamDestroy(copy_stream);
  cudaStreamDestroy(stream);
  return 0;
} catch (const std::exception& e) {
  std::cerr << "[ctd_train] error: " << e.what() << "\n";
  return 1;
}
