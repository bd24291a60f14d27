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
// What differs: the grad_accum_steps micro-batches of a step run as ONE fused pass through
// ctdk_engine_forward_backward (per-row weights mask / (A * sum(mask of the row's micro-batch))
// reproduce mul_scalar(loss, 1/A) + backward per micro-batch); clip and AdamW are the fused
// kernels behind ctdk_sumsq / ctdk_clip_scale / ctdk_adamw; there is one host sync per step (to log).
// "offload_optimizer" is accepted and ignored (m / v stay in HBM).
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <iostream>
#include <random>
#include <sstream>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/ctdk.h"
#include "../../include/ctdk_util/minijson.hpp"
#include "model_desc.hpp"
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
  c.seed = static_cast<uint64_t>(j.value("seed", static_cast<double>(c.seed)));
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
  void alloc(size_t count) {
    n = count;
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&p), std::max<size_t>(count, 1) * sizeof(T)));
  }
  ~DeviceBuf() {
    if (p) cudaFree(p);
  }
};

// Host-built device inputs of one fused pass over `rows` documents.
struct HostBatch {
  std::vector<int64_t> ids, targets;
  std::vector<float> mask, weight;
  std::vector<int32_t> active;   // flattened positions whose mask is 1
  double sum_mask = 0.0;
};

// rows_docs: the documents of consecutive micro-batches of `micro` rows each; a micro-batch whose
// mask is empty contributes nothing (main.cpp:350). accum = micro-batches in the whole step.
void build_batch(const Split& split, const std::vector<int64_t>& rows_docs, int micro, int accum, int seq_len,
                 HostBatch* out) {
  const int T = seq_len - 1;
  const size_t rows = rows_docs.size(), n = rows * static_cast<size_t>(T);
  out->ids.resize(n);
  out->targets.resize(n);
  out->mask.resize(n);
  out->weight.assign(n, 0.0f);
  out->active.clear();
  out->sum_mask = 0.0;
  for (size_t r0 = 0; r0 < rows; r0 += static_cast<size_t>(micro)) {
    double sm = 0.0;
    const size_t r1 = std::min(rows, r0 + static_cast<size_t>(micro));
    for (size_t r = r0; r < r1; ++r) {
      const int32_t* tok = split.tokens.data() + rows_docs[r] * seq_len;
      const int8_t* msk = split.masks.data() + rows_docs[r] * seq_len;
      for (int t = 0; t < T; ++t) {
        const size_t i = r * static_cast<size_t>(T) + static_cast<size_t>(t);
        out->ids[i] = tok[t];
        out->targets[i] = tok[t + 1];
        out->mask[i] = static_cast<float>(msk[t + 1]);
        sm += out->mask[i];
      }
    }
    if (sm <= 0.0) {   // skipped micro-batch: no loss, no gradient, not counted in the logged mean
      for (size_t i = r0 * static_cast<size_t>(T); i < r1 * static_cast<size_t>(T); ++i) out->mask[i] = 0.0f;
      continue;
    }
    const float w = static_cast<float>(1.0 / (static_cast<double>(accum) * sm));
    for (size_t i = r0 * static_cast<size_t>(T); i < r1 * static_cast<size_t>(T); ++i) {
      if (out->mask[i] != 0.0f) {
        out->weight[i] = out->mask[i] * w;
        out->active.push_back(static_cast<int32_t>(i));
      }
    }
    out->sum_mask += sm;
  }
}

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

}  // namespace

int main(int argc, char** argv) try {
  const std::string cfg_path = parse_config_path(argc, argv);
  const Config cfg = load_config(cfg_path);
  fs::create_directories(cfg.run_dir);
  std::cerr << "[ctd_train] run=" << cfg.run_name << " dir=" << cfg.run_dir << "\n";
  const bool resuming = !cfg.resume_from.empty();
  const fs::path weights_path = resuming ? cfg.resume_from : cfg.init_weights;
  std::cerr << "[ctd_train] " << (resuming ? "resuming from " : "loading init weights ") << weights_path << "\n";

  st::File wfile(weights_path.string());
  const st::Entry& emb = wfile.entry("model.embed_tokens.weight");
  if (emb.shape.size() != 2) throw std::runtime_error("autodetect_config: model.embed_tokens.weight must be 2-D");
  ctdk_model_config mc = cli::autodetect_config(emb.shape[0], emb.shape[1]);
  mc.gradient_checkpointing = cfg.gradient_checkpointing ? 1 : 0;
  mc.precision = cfg.precision;
  std::cerr << "[ctd_train] arch: hidden=" << mc.hidden_size << " layers=" << mc.num_hidden_layers
            << " heads=" << mc.num_attention_heads << "\n";
  if (cfg.gradient_checkpointing) std::cerr << "[ctd_train] gradient checkpointing enabled\n";
  if (cfg.offload_optimizer) std::cerr << "[ctd_train] offload_optimizer ignored: optimizer state stays in HBM\n";

  int64_t arena = 0;
  const std::vector<cli::ParamDesc> params = cli::describe_parameters(mc, &arena);
  size_t n_decay = 0;
  for (const auto& p : params) n_decay += p.decay ? 1 : 0;
  std::cerr << "[ctd_train] parameters: " << n_decay << " decay + " << (params.size() - n_decay) << " no_decay\n";

  // ---- device state: parameter / gradient arenas, AdamW moments, workspace ----
  CUDA_OK(cudaSetDevice(0));
  cudaStream_t stream;
  CUDA_OK(cudaStreamCreate(&stream));
  DeviceBuf<float> d_params(arena), d_grads(arena), d_m(arena), d_v(arena);
  CUDA_OK(cudaMemset(d_params.p, 0, arena * sizeof(float)));
  CUDA_OK(cudaMemset(d_m.p, 0, arena * sizeof(float)));
  CUDA_OK(cudaMemset(d_v.p, 0, arena * sizeof(float)));
  std::vector<float> h_arena(static_cast<size_t>(arena), 0.0f);
  for (const auto& p : params) wfile.read_f32(p.name, h_arena.data() + p.offset, p.numel);
  CUDA_OK(cudaMemcpy(d_params.p, h_arena.data(), arena * sizeof(float), cudaMemcpyHostToDevice));

  int64_t step_count = 0;
  if (resuming) {
    const fs::path op = opt_path_for(cfg.resume_from);
    if (fs::exists(op)) {
      std::cerr << "[ctd_train] loading optimizer state " << op << "\n";
      st::File ofile(op.string());
      std::vector<float> hm(static_cast<size_t>(arena), 0.0f), hv(static_cast<size_t>(arena), 0.0f);
      for (const auto& p : params) {
        if (!ofile.has("optimizer.m." + p.name) || !ofile.has("optimizer.v." + p.name))
          throw std::runtime_error("resume: missing optimizer.m." + p.name + " or optimizer.v." + p.name);
        ofile.read_f32("optimizer.m." + p.name, hm.data() + p.offset, p.numel);
        ofile.read_f32("optimizer.v." + p.name, hv.data() + p.offset, p.numel);
      }
      if (!ofile.has("optimizer.step")) throw std::runtime_error("resume: missing optimizer.step");
      float sf = 0.0f;
      ofile.read_f32("optimizer.step", &sf, 1);
      step_count = static_cast<int64_t>(sf);
      CUDA_OK(cudaMemcpy(d_m.p, hm.data(), arena * sizeof(float), cudaMemcpyHostToDevice));
      CUDA_OK(cudaMemcpy(d_v.p, hv.data(), arena * sizeof(float), cudaMemcpyHostToDevice));
      std::cerr << "[ctd_train] resumed at step " << step_count << "\n";
    } else {
      std::cerr << "[ctd_train] no optimizer state at " << op << " — continuing with fresh m/v (warmup will restart)\n";
    }
  }
  const int64_t start_step = step_count;

  std::cerr << "[ctd_train] loading data from " << cfg.data_dir << "\n";
  const Split train = load_split(cfg.data_dir / "train.bin", cfg.data_dir / "train_mask.bin", cfg.seq_len);
  const Split val = load_split(cfg.data_dir / "val.bin", cfg.data_dir / "val_mask.bin", cfg.seq_len);
  std::cerr << "[ctd_train] train=" << train.docs << " val=" << val.docs << "\n";
  if (train.docs < 1) throw std::runtime_error("train split is empty");

  // Micro-batches fused per pass: all of the step's if the workspace fits in free memory, else halved.
  const int T = cfg.seq_len - 1;
  int fused = cfg.grad_accum_steps;
  int64_t ws_bytes = 0;
  for (;; fused = (fused + 1) / 2) {
    ws_bytes = ctdk_engine_workspace_bytes(&mc, static_cast<int64_t>(fused) * cfg.batch_size, T);
    if (ws_bytes < 0) throw std::runtime_error(ctdk_last_error());
    size_t free_b = 0, total_b = 0;
    CUDA_OK(cudaMemGetInfo(&free_b, &total_b));
    if (static_cast<double>(ws_bytes) < 0.9 * static_cast<double>(free_b) || fused == 1) break;
  }
  const int64_t pass_rows = static_cast<int64_t>(fused) * cfg.batch_size;
  std::cerr << "[ctd_train] " << fused << " of " << cfg.grad_accum_steps << " micro-batches per pass, workspace "
            << (ws_bytes >> 20) << " MiB\n";
  DeviceBuf<unsigned char> d_ws(static_cast<size_t>(ws_bytes));
  void* engine = nullptr;
  CTDK_OK_OR_THROW(ctdk_engine_create(&mc, d_params.p, d_grads.p, d_ws.p, ws_bytes, pass_rows, T, &engine));

  const size_t pass_n = static_cast<size_t>(pass_rows) * static_cast<size_t>(T);
  DeviceBuf<int64_t> d_ids(pass_n), d_tgt(pass_n);
  DeviceBuf<float> d_mask(pass_n), d_w(pass_n), d_scal(8);   // scal: [0..1] loss sums, [2] sumsq, [3] scale, [4] norm
  DeviceBuf<int32_t> d_active(pass_n);

  // weight-decay segments of the arena: runs of equal decay in parameter order, padding with its tensor
  std::vector<int64_t> seg_end;
  std::vector<float> seg_wd;
  for (size_t i = 0; i < params.size(); ++i) {
    const float wd = params[i].decay ? cfg.weight_decay : 0.0f;
    const int64_t end = i + 1 < params.size() ? params[i + 1].offset : arena;
    if (!seg_wd.empty() && seg_wd.back() == wd) seg_end.back() = end;
    else {
      seg_end.push_back(end);
      seg_wd.push_back(wd);
    }
  }
  DeviceBuf<int64_t> d_seg_end(seg_end.size());
  DeviceBuf<float> d_seg_wd(seg_wd.size());
  CUDA_OK(cudaMemcpy(d_seg_end.p, seg_end.data(), seg_end.size() * sizeof(int64_t), cudaMemcpyHostToDevice));
  CUDA_OK(cudaMemcpy(d_seg_wd.p, seg_wd.data(), seg_wd.size() * sizeof(float), cudaMemcpyHostToDevice));

  HostBatch hb;
  auto upload = [&](const HostBatch& b) {
    const size_t n = b.ids.size();
    CUDA_OK(cudaMemcpyAsync(d_ids.p, b.ids.data(), n * sizeof(int64_t), cudaMemcpyHostToDevice, stream));
    CUDA_OK(cudaMemcpyAsync(d_tgt.p, b.targets.data(), n * sizeof(int64_t), cudaMemcpyHostToDevice, stream));
    CUDA_OK(cudaMemcpyAsync(d_mask.p, b.mask.data(), n * sizeof(float), cudaMemcpyHostToDevice, stream));
    CUDA_OK(cudaMemcpyAsync(d_w.p, b.weight.data(), n * sizeof(float), cudaMemcpyHostToDevice, stream));
    if (!b.active.empty())
      CUDA_OK(cudaMemcpyAsync(d_active.p, b.active.data(), b.active.size() * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
    CUDA_OK(cudaStreamSynchronize(stream));   // the host vectors are reused by the next pass
  };

  auto save_checkpoint = [&](const fs::path& ckpt) {
    CUDA_OK(cudaMemcpy(h_arena.data(), d_params.p, arena * sizeof(float), cudaMemcpyDeviceToHost));
    std::vector<st::Item> items;
    for (const auto& p : params) items.push_back({p.name, p.shape, h_arena.data() + p.offset});
    st::save(items, ckpt.string());
    std::vector<float> hm(static_cast<size_t>(arena)), hv(static_cast<size_t>(arena));
    CUDA_OK(cudaMemcpy(hm.data(), d_m.p, arena * sizeof(float), cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(hv.data(), d_v.p, arena * sizeof(float), cudaMemcpyDeviceToHost));
    std::vector<st::Item> opt;
    for (int pass = 0; pass < 2; ++pass)   // decay group first, then no-decay (main.cpp:218-226)
      for (const auto& p : params) {
        if (p.decay != (pass == 0)) continue;
        opt.push_back({"optimizer.m." + p.name, p.shape, hm.data() + p.offset});
        opt.push_back({"optimizer.v." + p.name, p.shape, hv.data() + p.offset});
      }
    const float sf = static_cast<float>(step_count);
    opt.push_back({"optimizer.step", {1}, &sf});
    st::save(opt, opt_path_for(ckpt).string());
  };

  auto run_val = [&]() -> float {
    double sum_loss = 0.0, sum_mask = 0.0;
    for (int64_t d0 = 0; d0 < val.docs; d0 += pass_rows) {
      std::vector<int64_t> docs;
      for (int64_t d = d0; d < std::min(val.docs, d0 + pass_rows); ++d) docs.push_back(d);
      build_batch(val, docs, 1, 1, cfg.seq_len, &hb);
      if (hb.sum_mask <= 0.0) continue;
      upload(hb);
      CUDA_OK(cudaMemsetAsync(d_scal.p, 0, 2 * sizeof(float), stream));
      CTDK_OK_OR_THROW(ctdk_engine_set_active_rows(engine, d_active.p, static_cast<int64_t>(hb.active.size())));
      CTDK_OK_OR_THROW(ctdk_engine_forward_loss(engine, d_ids.p, d_tgt.p, d_mask.p, static_cast<int64_t>(docs.size()), T, d_scal.p, stream));
      float ls[2];
      CUDA_OK(cudaMemcpyAsync(ls, d_scal.p, sizeof ls, cudaMemcpyDeviceToHost, stream));
      CUDA_OK(cudaStreamSynchronize(stream));
      sum_loss += ls[0];
      sum_mask += ls[1];
    }
    return sum_mask > 0.0 ? static_cast<float>(sum_loss / sum_mask) : 0.0f;
  };

  std::mt19937_64 rng(cfg.seed + static_cast<uint64_t>(start_step));
  std::uniform_int_distribution<int64_t> pick(0, train.docs - 1);
  const fs::path log_path = cfg.run_dir / "loss.jsonl";
  std::ofstream log(log_path, resuming ? (std::ios::out | std::ios::app) : (std::ios::out | std::ios::trunc));
  if (!log) throw std::runtime_error("cannot open log " + log_path.string());
  const auto t_run = std::chrono::steady_clock::now();

  for (int step = static_cast<int>(start_step) + 1; step <= cfg.total_steps; ++step) {
    const auto t_step = std::chrono::steady_clock::now();
    // the step's documents, drawn micro-batch by micro-batch, row by row
    std::vector<int64_t> docs(static_cast<size_t>(cfg.grad_accum_steps) * cfg.batch_size);
    for (auto& d : docs) d = pick(rng);
    CUDA_OK(cudaMemsetAsync(d_scal.p, 0, 8 * sizeof(float), stream));
    bool first_pass = true;
    for (int mb0 = 0; mb0 < cfg.grad_accum_steps; mb0 += fused) {
      const int nmb = std::min(fused, cfg.grad_accum_steps - mb0);
      const std::vector<int64_t> sub(docs.begin() + static_cast<int64_t>(mb0) * cfg.batch_size,
                                     docs.begin() + static_cast<int64_t>(mb0 + nmb) * cfg.batch_size);
      build_batch(train, sub, cfg.batch_size, cfg.grad_accum_steps, cfg.seq_len, &hb);
      if (hb.sum_mask <= 0.0) continue;
      upload(hb);
      CTDK_OK_OR_THROW(ctdk_engine_set_active_rows(engine, d_active.p, static_cast<int64_t>(hb.active.size())));
      CTDK_OK_OR_THROW(ctdk_engine_forward_backward(engine, d_ids.p, d_tgt.p, d_mask.p, d_w.p, static_cast<int64_t>(sub.size()), T,
                                                    first_pass ? 0 : 1, d_scal.p, stream));
      first_pass = false;
    }
    if (first_pass) CUDA_OK(cudaMemsetAsync(d_grads.p, 0, arena * sizeof(float), stream));   // every mask was empty

    const float lr = lr_at_step(step, cfg);
    CTDK_OK_OR_THROW(ctdk_sumsq(d_grads.p, arena, d_scal.p + 2, stream));
    CTDK_OK_OR_THROW(ctdk_clip_scale(d_scal.p + 2, cfg.clip_grad_norm, 1e-6f, d_scal.p + 3, d_scal.p + 4, stream));
    ++step_count;
    ctdk_adamw_params hp{};
    hp.lr = lr;
    hp.beta1 = cfg.beta1;
    hp.beta2 = cfg.beta2;
    hp.eps = cfg.eps;
    hp.wd = 0.0f;
    hp.bc1 = 1.0f - std::pow(cfg.beta1, static_cast<float>(step_count));
    hp.bc2 = 1.0f - std::pow(cfg.beta2, static_cast<float>(step_count));
    CTDK_OK_OR_THROW(ctdk_adamw(d_params.p, d_grads.p, d_m.p, d_v.p, arena, &hp, d_scal.p + 3, d_seg_end.p, d_seg_wd.p,
                                static_cast<int>(seg_end.size()), stream));
    float sc[5];
    CUDA_OK(cudaMemcpyAsync(sc, d_scal.p, sizeof sc, cudaMemcpyDeviceToHost, stream));
    CUDA_OK(cudaStreamSynchronize(stream));
    int dev_status[4] = {0, 0, 0, 0};
    if (ctdk_device_status(stream, dev_status) != CTDK_OK) throw std::runtime_error(ctdk_last_error());

    const auto t_end = std::chrono::steady_clock::now();
    const double step_s = std::chrono::duration<double>(t_end - t_step).count();
    const double wall_s = std::chrono::duration<double>(t_end - t_run).count();
    const float train_loss = sc[1] > 0.0f ? sc[0] / sc[1] : 0.0f;
    const double tps = static_cast<double>(sc[1]) / std::max(step_s, 1e-9);
    if (cfg.log_every > 0 && step % cfg.log_every == 0) {
      log << minijson::Line().add("step", static_cast<long long>(step)).add("phase", std::string("train")).add("loss", train_loss)
                 .add("lr", lr).add("grad_norm", sc[4]).add("tokens_per_sec", tps).add("wall_s", wall_s).dump()
          << "\n";
      log.flush();
      std::cerr << "[step " << step << "/" << cfg.total_steps << "] loss=" << train_loss << " lr=" << lr << " |g|=" << sc[4]
                << " tok/s=" << static_cast<long long>(tps) << "\n";
    }
    if (cfg.val_every > 0 && step % cfg.val_every == 0) {
      const auto t_val = std::chrono::steady_clock::now();
      const float vl = run_val();
      const auto now = std::chrono::steady_clock::now();
      log << minijson::Line().add("step", static_cast<long long>(step)).add("phase", std::string("val")).add("loss", vl)
                 .add("wall_s", std::chrono::duration<double>(now - t_run).count()).dump()
          << "\n";
      log.flush();
      std::cerr << "[step " << step << "] val_loss=" << vl << " (" << std::chrono::duration<double>(now - t_val).count() << "s)\n";
    }
    if (cfg.save_every > 0 && step % cfg.save_every == 0) {
      const fs::path ckpt = cfg.run_dir / ("ckpt_step_" + std::to_string(step) + ".safetensors");
      save_checkpoint(ckpt);
      std::cerr << "[step " << step << "] saved " << ckpt << " (+ optimizer)\n";
    }
  }

  const fs::path final_ckpt = cfg.run_dir / "final.safetensors";
  save_checkpoint(final_ckpt);
  std::cerr << "[ctd_train] done. final → " << final_ckpt << " (+ optimizer)\n";
  ctdk_engine_destroy(engine);
  cudaStreamDestroy(stream);
  return 0;
} catch (const std::exception& e) {
  std::cerr << "[ctd_train] error: " << e.what() << "\n";
  return 1;
}
