// Drives the UNMODIFIED reference (KyleCr4ne/emberlm, compiled from its own sources by
// oracle/Makefile) through its public C++ API for the training step, so that its results and
// its step time can be put beside the ctdk engine's. TEST / BENCH INFRASTRUCTURE ONLY: nothing
// in the product links or runs this.
//
// The loop is the body of the reference's ctd_train (tools/ctd_train/main.cpp:346-373):
//   for each micro-batch: loss = model.forward_train_masked(ids, targets, mask);
//                         mul_scalar(loss, 1/A).backward();
//   clip_grad_norm_(all params, clip); opt.step(); opt.zero_grad();
// with an explicit LlamaConfig passed to build_model (include/ctd/nn/model.h:220) and documents
// taken in order (micro-batch j of step s uses rows [(s*A+j)*b, (s*A+j+1)*b)) instead of random
// draws, so both sides see the same rows without sharing an RNG.
//
// usage: ref_harness <spec.json>
// spec keys: weights, tokens (int32 [docs,S]), mask (int8 [docs,S]), seq_len, batch_size,
//   grad_accum_steps, steps, warmup, lr, beta1, beta2, eps, weight_decay, clip,
//   gradient_checkpointing, dump_grads (path or ""), dump_params (path or ""), config{...}
// stdout: one JSON line {"loss":[...], "grad_norm":[...], "step_ms":[...]}.
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_runtime.h>
#include <nlohmann/json.hpp>

#include "ctd/autograd.h"
#include "ctd/nn/model.h"
#include "ctd/ops/repeat_kv.h"
#include "ctd/optim.h"
#include "ctd/safetensors.h"
#include "ctd/tensor.h"

using namespace ctd;
using json = nlohmann::json;

static std::vector<char> read_all(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  f.seekg(0, std::ios::end);
  std::vector<char> buf(static_cast<size_t>(f.tellg()));
  f.seekg(0);
  f.read(buf.data(), static_cast<std::streamsize>(buf.size()));
  return buf;
}

int main(int argc, char** argv) try {
  if (argc != 2) {
    std::fprintf(stderr, "usage: ref_harness <spec.json>\n");
    return 2;
  }
  json spec;
  {
    std::ifstream f(argv[1]);
    f >> spec;
  }
  const int S = spec.at("seq_len"), b = spec.at("batch_size"), A = spec.at("grad_accum_steps");
  const int steps = spec.at("steps"), warmup = spec.value("warmup", 0);
  const float lr = spec.at("lr"), beta1 = spec.at("beta1"), beta2 = spec.at("beta2");
  const float eps = spec.at("eps"), wd = spec.at("weight_decay"), clip = spec.at("clip");
  const json& c = spec.at("config");
  nn::LlamaConfig cfg{};
  cfg.vocab_size = c.at("vocab_size");
  cfg.hidden_size = c.at("hidden_size");
  cfg.intermediate_size = c.at("intermediate_size");
  cfg.num_hidden_layers = c.at("num_hidden_layers");
  cfg.num_attention_heads = c.at("num_attention_heads");
  cfg.num_key_value_heads = c.at("num_key_value_heads");
  cfg.head_dim = c.at("head_dim");
  cfg.max_position_embeddings = c.value("max_position_embeddings", 8192);
  cfg.rms_norm_eps = c.at("rms_norm_eps");
  cfg.rope_theta = c.at("rope_theta");
  cfg.tie_word_embeddings = true;
  cfg.qk_norm = c.value("qk_norm", false);
  cfg.rope_scaling_factor = c.value("rope_scaling_factor", 0.0f);
  cfg.rope_scaling_low_freq_factor = c.value("rope_scaling_low_freq_factor", 1.0f);
  cfg.rope_scaling_high_freq_factor = c.value("rope_scaling_high_freq_factor", 4.0f);
  cfg.rope_scaling_original_max_pos = c.value("rope_scaling_original_max_pos", 8192);

  TensorDict w = load_safetensors(spec.at("weights").get<std::string>(), kCUDA0);
  nn::Model model = nn::build_model(w, cfg);
  model.gradient_checkpointing = spec.value("gradient_checkpointing", false);
  auto named = model.collect_parameters();
  std::vector<Tensor> all_params;
  for (auto& kv : named.all) all_params.push_back(kv.second);
  std::vector<optim::ParamGroup> groups;
  groups.push_back({named.decay, lr, wd});
  groups.push_back({named.no_decay, lr, 0.0f});
  optim::AdamW opt(groups, beta1, beta2, eps, false);

  const std::vector<char> tok_bytes = read_all(spec.at("tokens").get<std::string>());
  const std::vector<char> msk_bytes = read_all(spec.at("mask").get<std::string>());
  const int32_t* tok = reinterpret_cast<const int32_t*>(tok_bytes.data());
  const int8_t* msk = reinterpret_cast<const int8_t*>(msk_bytes.data());
  const int64_t docs = static_cast<int64_t>(tok_bytes.size() / 4 / S);
  const int T = S - 1;

  const std::string dump_grads = spec.value("dump_grads", std::string());
  const std::string dump_params = spec.value("dump_params", std::string());
  std::vector<float> losses, norms;
  std::vector<double> step_ms;
  const float inv_accum = 1.0f / static_cast<float>(A);

  for (int s = 0; s < warmup + steps; ++s) {
    cudaDeviceSynchronize();
    const auto t0 = std::chrono::steady_clock::now();
    double acc_loss = 0.0, acc_active = 0.0;
    for (int j = 0; j < A; ++j) {
      const int64_t first = (static_cast<int64_t>(s) * A + j) * b;
      std::vector<int64_t> ids(static_cast<size_t>(b) * T), tgt(ids.size());
      std::vector<float> mk(ids.size());
      float sum_mask = 0.0f;
      for (int r = 0; r < b; ++r) {
        const int64_t doc = (first + r) % docs;
        for (int t = 0; t < T; ++t) {
          ids[static_cast<size_t>(r) * T + t] = tok[doc * S + t];
          tgt[static_cast<size_t>(r) * T + t] = tok[doc * S + t + 1];
          const float m = static_cast<float>(msk[doc * S + t + 1]);
          mk[static_cast<size_t>(r) * T + t] = m;
          sum_mask += m;
        }
      }
      if (sum_mask <= 0.0f) continue;
      const std::vector<int64_t> shape = {b, T};
      Tensor d_ids = Tensor::from_host(ids.data(), shape, DType::kInt64, kCUDA0);
      Tensor d_tgt = Tensor::from_host(tgt.data(), shape, DType::kInt64, kCUDA0);
      Tensor d_mk = Tensor::from_host(mk.data(), shape, DType::kFloat32, kCUDA0);
      Tensor loss = model.forward_train_masked(d_ids, d_tgt, d_mk);
      Tensor scaled = ops::mul_scalar(loss, inv_accum);
      scaled.backward();
      float l = 0.0f;
      loss.copy_to_host(&l);
      acc_loss += static_cast<double>(l) * sum_mask;
      acc_active += sum_mask;
    }
    if (s == 0 && !dump_grads.empty()) {
      std::vector<std::pair<std::string, Tensor>> items;
      for (auto& kv : named.all) items.emplace_back(kv.first, kv.second.grad());
      save_safetensors(items, dump_grads);
    }
    const float gn = optim::clip_grad_norm_(all_params, clip);
    opt.step();
    opt.zero_grad();
    cudaDeviceSynchronize();
    const auto t1 = std::chrono::steady_clock::now();
    if (s >= warmup) {
      losses.push_back(acc_active > 0 ? static_cast<float>(acc_loss / acc_active) : 0.0f);
      norms.push_back(gn);
      step_ms.push_back(std::chrono::duration<double, std::milli>(t1 - t0).count());
    }
  }
  if (!dump_params.empty()) {
    std::vector<std::pair<std::string, Tensor>> items;
    for (auto& kv : named.all) items.emplace_back(kv.first, kv.second);
    save_safetensors(items, dump_params);
  }
  json out;
  out["loss"] = losses;
  out["grad_norm"] = norms;
  out["step_ms"] = step_ms;
  out["positions_per_step"] = static_cast<int64_t>(A) * b * T;
  std::cout << out.dump() << std::endl;
  return 0;
} catch (const std::exception& e) {
  std::fprintf(stderr, "[ref_harness] error: %s\n", e.what());
  return 1;
}
