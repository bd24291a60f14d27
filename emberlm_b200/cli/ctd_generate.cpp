// ctd_generate: the reference's token generation subprocess (emberlm tools/ctd_generate/main.cpp) on
// the B200 decode path.
//
//   ctd_generate --model <path-to-fp32.safetensors>
//
// Protocol as there: one JSON request on stdin ({"input_ids": [...], "max_new_tokens", "max_seq_len",
// "temperature", "top_k", "top_p", "seed", "eos_ids", "thinking_token_budget", "think_open_ids",
// "think_close_ids"}), one {"token": id} line per generated token on stdout, then
// {"done": true, "reason": "eos" | "max_tokens" | "max_seq_len" | ..., "generated_tokens": n}.
// Errors: "[ctd_generate] error: ..." on stderr, a {"done": true, "reason": "error"} line, exit 1;
// usage errors exit 2. The sampler follows src/core/sampling.cpp: temperature <= 0 is the first
// index of the maximum, otherwise temperature, top-k threshold, softmax, top-p nucleus and one
// uniform draw from mt19937_64(seed). Greedy requests without a thinking budget run on the device
// in chunks (ctdk_decode_greedy: one CUDA graph launch per token); everything else feeds one chosen
// token at a time (ctdk_decode_step) and samples on the device (ctdk_sample), one draw per token.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <iostream>
#include <limits>
#include <numeric>
#include <random>
#include <set>
#include <sstream>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/ctdk.h"
#include "../../include/ctdk_util/minijson.hpp"
#include "model_desc.hpp"
#include "../../include/ctdk_util/safetensors.hpp"

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

struct Sampler {
  float temperature = 1.0f;
  int top_k = 0;
  float top_p = 0.0f;
};

std::vector<int64_t> id_list(const minijson::Value& req, const char* key) {
  std::vector<int64_t> out;
  if (req.contains(key))
    for (const auto& v : req.at(key).array()) out.push_back(static_cast<int64_t>(v.number()));
  return out;
}

void emit(const std::string& line) { std::cout << line << "\n" << std::flush; }

std::string parse_model_path(int argc, char** argv) {
  std::string model;
  for (int i = 1; i < argc; ++i)
    if (std::string(argv[i]) == "--model" && i + 1 < argc) model = argv[++i];
  if (model.empty()) {
    std::cerr << "usage: " << argv[0] << " --model <path-to-fp32.safetensors> [--precision fp32|tf32]\n";
    std::exit(2);
  }
  return model;
}

// The prompt pass: exact fp32 products by default, like the reference's generator (the token steps are
// fp32 GEMVs in either case), so that a request draws the same tokens; --precision tf32 runs the prompt
// on the TF32 tensor cores (long prompts, where a rounding difference of 1e-3 in the cache is acceptable).
int parse_precision(int argc, char** argv) {
  for (int i = 1; i + 1 < argc; ++i)
    if (std::string(argv[i]) == "--precision") {
      const std::string v = argv[i + 1];
      if (v == "tf32") return CTDK_GEMM_TF32;
      if (v == "fp32" || v == "3xtf32") return CTDK_GEMM_3XTF32;
      std::cerr << "--precision: expected fp32 or tf32\n";
      std::exit(2);
    }
  return CTDK_GEMM_3XTF32;
}

}  // namespace

int main(int argc, char** argv) try {
  const std::string model_path = parse_model_path(argc, argv);
  std::ostringstream in;
  in << std::cin.rdbuf();
  const minijson::Value req = minijson::parse(in.str());
  const std::vector<int64_t> input_ids = id_list(req, "input_ids");
  if (!req.contains("input_ids")) throw std::runtime_error("json: key 'input_ids' not found");
  const int max_new = static_cast<int>(req.value("max_new_tokens", 64.0));
  const int max_seq = static_cast<int>(req.value("max_seq_len", 2048.0));
  Sampler sampler;
  sampler.temperature = static_cast<float>(req.value("temperature", 1.0));
  sampler.top_k = static_cast<int>(req.value("top_k", 0.0));
  sampler.top_p = static_cast<float>(req.value("top_p", 0.0));
  const uint64_t seed = req.contains("seed") ? req.at("seed").as_uint64() : 0;
  const std::vector<int64_t> eos_list = id_list(req, "eos_ids");
  const std::set<int64_t> eos(eos_list.begin(), eos_list.end());
  const int budget = static_cast<int>(req.value("thinking_token_budget", 0.0));
  const std::vector<int64_t> open_ids = id_list(req, "think_open_ids"), close_ids = id_list(req, "think_close_ids");
  const bool budget_active = budget > 0 && !open_ids.empty() && !close_ids.empty();

  const auto t0 = std::chrono::steady_clock::now();
  std::cerr << "[ctd_generate] loading " << model_path << "\n";
  st::File wfile(model_path);
  const st::Entry& emb = wfile.entry("model.embed_tokens.weight");
  if (emb.shape.size() != 2) throw std::runtime_error("autodetect_config: model.embed_tokens.weight must be 2-D");
  ctdk_model_config mc = cli::autodetect_config(emb.shape[0], emb.shape[1]);
  mc.precision = parse_precision(argc, argv);
  std::cerr << "[ctd_generate] arch: hidden=" << mc.hidden_size << " layers=" << mc.num_hidden_layers << "\n";
  const int prompt_len = static_cast<int>(input_ids.size());
  for (const int64_t id : input_ids)
    if (id < 0 || id >= mc.vocab_size) throw std::runtime_error("input_ids: token id out of range");

  int64_t arena = 0;
  const std::vector<cli::ParamDesc> params = cli::describe_parameters(mc, &arena);
  std::vector<float> h_arena(static_cast<size_t>(arena), 0.0f);
  for (const auto& p : params) wfile.read_f32(p.name, h_arena.data() + p.offset, p.numel);
  CUDA_OK(cudaSetDevice(0));
  cudaStream_t stream;
  CUDA_OK(cudaStreamCreate(&stream));
  float* d_params = nullptr;
  CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_params), arena * sizeof(float)));
  CUDA_OK(cudaMemcpy(d_params, h_arena.data(), arena * sizeof(float), cudaMemcpyHostToDevice));
  std::cerr << "[ctd_generate] model ready in " << std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count()
            << " s\n";

  if (prompt_len == 0) {
    emit(minijson::Line().add_bool("done", true).add("reason", std::string("empty_prompt")).dump());
    return 0;
  }
  if (prompt_len >= max_seq) {
    emit(minijson::Line().add_bool("done", true).add("reason", std::string("max_seq_len")).dump());
    return 0;
  }

  const int64_t ws_bytes = ctdk_decode_workspace_bytes(&mc, max_seq);
  if (ws_bytes < 0) throw std::runtime_error(ctdk_last_error());
  void* d_ws = nullptr;
  CUDA_OK(cudaMalloc(&d_ws, static_cast<size_t>(ws_bytes)));
  void* dec = nullptr;
  CTDK_OK_OR_THROW(ctdk_decode_create(&mc, d_params, d_ws, ws_bytes, max_seq, &dec));
  int64_t* d_ids = nullptr;
  CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_ids), static_cast<size_t>(std::max(max_seq, 16)) * sizeof(int64_t)));
  CUDA_OK(cudaMemcpy(d_ids, input_ids.data(), static_cast<size_t>(prompt_len) * sizeof(int64_t), cudaMemcpyHostToDevice));
  const auto t1 = std::chrono::steady_clock::now();
  CTDK_OK_OR_THROW(ctdk_decode_prefill(dec, d_ids, prompt_len, stream));
  CUDA_OK(cudaStreamSynchronize(stream));
  std::cerr << "[ctd_generate] prefill (" << prompt_len << " tok) in "
            << std::chrono::duration<double>(std::chrono::steady_clock::now() - t1).count() << " s\n";

  const int64_t V = mc.vocab_size;
  std::mt19937_64 rng(seed);
  int generated = 0;
  std::string stop = "max_tokens";
  const auto t2 = std::chrono::steady_clock::now();

  if (sampler.temperature <= 0.0f && !budget_active) {
    // greedy on the device, 16 tokens per round trip; tokens after an end-of-sequence id are dropped
    std::vector<int64_t> chunk(16);
    bool done = false;
    while (!done && generated < max_new) {
      int n = std::min<int>(16, max_new - generated);
      n = std::min<int>(n, max_seq + 1 - (prompt_len + generated));   // cache positions left (the last token needs none)
      if (n <= 0) {
        stop = "max_seq_len";
        break;
      }
      CTDK_OK_OR_THROW(ctdk_decode_greedy(dec, n, d_ids, stream));
      CUDA_OK(cudaMemcpyAsync(chunk.data(), d_ids + generated, static_cast<size_t>(n) * sizeof(int64_t), cudaMemcpyDeviceToHost, stream));
      CUDA_OK(cudaStreamSynchronize(stream));
      for (int i = 0; i < n; ++i) {
        emit(minijson::Line().add("token", static_cast<long long>(chunk[i])).dump());
        ++generated;
        if (eos.count(chunk[i])) {
          stop = "eos";
          done = true;
          break;
        }
        if (prompt_len + generated > max_seq) {
          stop = "max_seq_len";
          done = true;
          break;
        }
      }
    }
  } else {
    // Sampling on the device (ctdk_sample: the reference sampler's semantics and draw order): the
    // uniform draw goes there, the token id comes back; the V logits never leave the GPU.
    const float* d_logits = nullptr;
    CTDK_OK_OR_THROW(ctdk_decode_logits(dec, &d_logits));
    void* d_sample_ws = nullptr;
    double* d_u = nullptr;
    int64_t* d_tok = nullptr;
    CUDA_OK(cudaMalloc(&d_sample_ws, static_cast<size_t>(ctdk_sample_workspace_bytes(1, V))));
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_u), sizeof(double)));
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d_tok), sizeof(int64_t)));
    std::uniform_real_distribution<double> uniform(0.0, 1.0);
    std::vector<int64_t> window, force_queue;
    bool in_think = false;
    int think_tokens = 0;
    const size_t window_cap = budget_active ? std::max(open_ids.size(), close_ids.size()) : 0;
    auto window_ends_with = [&](const std::vector<int64_t>& seq) {
      return window.size() >= seq.size() && std::equal(window.end() - seq.size(), window.end(), seq.begin());
    };
    int fed = 0;
    while (generated < max_new) {
      int64_t tok;
      if (budget_active && !force_queue.empty()) {
        tok = force_queue.front();
        force_queue.erase(force_queue.begin());
      } else {
        const double u = sampler.temperature > 0.0f ? uniform(rng) : 0.0;   // greedy takes no draw (sampling.cpp:33)
        CUDA_OK(cudaMemcpyAsync(d_u, &u, sizeof u, cudaMemcpyHostToDevice, stream));
        CTDK_OK_OR_THROW(ctdk_sample(d_logits, 1, V, sampler.temperature, sampler.top_k, sampler.top_p, d_u, d_sample_ws, d_tok, stream));
        CUDA_OK(cudaMemcpyAsync(&tok, d_tok, sizeof tok, cudaMemcpyDeviceToHost, stream));
        CUDA_OK(cudaStreamSynchronize(stream));
      }
      emit(minijson::Line().add("token", static_cast<long long>(tok)).dump());
      ++generated;
      if (budget_active) {
        window.push_back(tok);
        if (window.size() > window_cap) window.erase(window.begin());
        if (window_ends_with(open_ids)) {
          in_think = true;
          think_tokens = 0;
        } else if (window_ends_with(close_ids)) {
          in_think = false;
        } else if (in_think) {
          ++think_tokens;
        }
        if (in_think && force_queue.empty() && think_tokens >= budget) force_queue = close_ids;
      }
      if (eos.count(tok)) {
        stop = "eos";
        break;
      }
      if (prompt_len + fed + 1 > max_seq) {   // no cache position left for this token
        stop = "max_seq_len";
        break;
      }
      CTDK_OK_OR_THROW(ctdk_decode_step(dec, tok, stream));
      ++fed;
    }
    CUDA_OK(cudaStreamSynchronize(stream));
    cudaFree(d_sample_ws);
    cudaFree(d_u);
    cudaFree(d_tok);
  }
  const double decode_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t2).count();
  std::cerr << "[ctd_generate] generated " << generated << " tok in " << decode_s << " s  ("
            << (generated / std::max(decode_s, 1e-9)) << " tok/s)\n";
  emit(minijson::Line().add_bool("done", true).add("reason", stop).add("generated_tokens", static_cast<long long>(generated)).dump());
  ctdk_decode_destroy(dec);
  return 0;
} catch (const std::exception& e) {
  std::cerr << "[ctd_generate] error: " << e.what() << "\n";
  std::cout << minijson::Line().add_bool("done", true).add("reason", std::string("error")).add("error", std::string(e.what())).dump() << "\n";
  return 1;
}
