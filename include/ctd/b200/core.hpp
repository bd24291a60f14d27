// Core of the ctd:: C++ surface on top of the C-ABI in ctdk.h: Device, DType, the allocators,
// Storage, Tensor and the autograd tape. Names, argument order and error behaviour are those of the
// reference's include/ctd/{device,dtype,allocator,storage,tensor,autograd,cuda_utils}.h (emberlm),
// which the small headers at those paths in this tree forward to, so a translation unit written
// against the reference compiles against this tree unchanged and links with -lctdk -lcudart.
//
// What is different underneath:
//   - device memory comes from a caching arena allocator (size-bucketed free lists over blocks that
//     are never returned to the driver while the process runs), not from a cudaMalloc / cudaFree
//     pair per tensor (the reference's allocator, src/core/allocator.cpp:14-30, whose calls
//     synchronise the device). Every op of this surface enqueues on the legacy default stream, so a
//     block handed back by a destroyed tensor can be reused by the next op at once: the kernels
//     that still read it are ordered before the kernels that will write it;
//   - a tensor may be a view into a larger storage (the parameters and gradients of a built model
//     are slices of two arenas);
//   - a tensor may carry a deferred value: the loss of a fused model pass is computed when it is
//     first read or when backward() reaches it (one fused pass instead of two).
// Header-only.
#pragma once

#include <cstdlib>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include <cuda_runtime.h>

#include "ctdk.h"

// ---- cuda_utils.h ---------------------------------------------------------------------------
#define CTD_CUDA_CHECK(expr)                                                                       \
  do {                                                                                             \
    const cudaError_t ctd_err_ = (expr);                                                           \
    if (ctd_err_ != cudaSuccess)                                                                   \
      throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(ctd_err_) + " at " \
                               __FILE__ ":" + std::to_string(__LINE__));                           \
  } while (0)
#define CTD_CUDA_CHECK_KERNEL() CTD_CUDA_CHECK(cudaGetLastError())

namespace ctd {

// ---- device.h / dtype.h ---------------------------------------------------------------------
enum class DeviceType : uint8_t { kCPU = 0, kCUDA = 1 };

struct Device {
  DeviceType type = DeviceType::kCPU;
  int index = 0;
  constexpr Device() = default;
  constexpr Device(DeviceType t, int i = 0) : type(t), index(i) {}
  bool is_cpu() const { return type == DeviceType::kCPU; }
  bool is_cuda() const { return type == DeviceType::kCUDA; }
  bool operator==(const Device& o) const { return type == o.type && index == o.index; }
  bool operator!=(const Device& o) const { return !(*this == o); }
};
constexpr Device kCPU{DeviceType::kCPU, 0};
constexpr Device kCUDA0{DeviceType::kCUDA, 0};

enum class DType : uint8_t { kFloat32 = 0, kFloat16 = 1, kBFloat16 = 2, kInt32 = 3, kInt64 = 4 };

constexpr size_t dtype_size(DType dt) {
  return (dt == DType::kFloat32 || dt == DType::kInt32) ? 4 : (dt == DType::kInt64 ? 8 : 2);
}
inline const char* dtype_name(DType dt) {
  static const char* const names[] = {"float32", "float16", "bfloat16", "int32", "int64"};
  const unsigned i = static_cast<unsigned>(dt);
  return i < 5 ? names[i] : "?";
}

namespace detail {
inline void require(bool ok, const char* msg) {
  if (!ok) throw std::runtime_error(msg);
}
inline void require(bool ok, const std::string& msg) {
  if (!ok) throw std::runtime_error(msg);
}
// Precision of the per-op matrix products (matmul, bmm, Linear): TF32 tensor cores by default; with
// CTD_MATMUL_PRECISION=fp32 in the environment they are exact fp32 products like the reference's
// cublasSgemm (src/ops/matmul.cpp:38-47), at a fraction of the speed. The fused training engine has
// its own setting (LlamaConfig / the "precision" key of ctd_train).
inline int matmul_precision() {
  static const int p = [] {
    const char* e = std::getenv("CTD_MATMUL_PRECISION");
    return (e != nullptr && (std::string(e) == "fp32" || std::string(e) == "3xtf32")) ? CTDK_GEMM_3XTF32 : CTDK_GEMM_TF32;
  }();
  return p;
}
inline void ctdk_ok(int rc) {
  if (rc != CTDK_OK) throw std::runtime_error(ctdk_last_error());
}
}  // namespace detail

// ---- allocator.h ----------------------------------------------------------------------------
class Allocator {
 public:
  virtual ~Allocator() = default;
  virtual void* allocate(size_t nbytes) = 0;
  virtual void deallocate(void* ptr) noexcept = 0;
  virtual Device device() const = 0;
};

namespace detail {

// Caching device allocator. Requests are rounded up (512 B steps below 1 MiB, 2 MiB steps above)
// and served from a free list of that exact rounded size; a miss takes a new block from the
// driver. Blocks go back to their list on deallocate and to the driver only in release_all().
class ArenaAllocator final : public Allocator {
 public:
  void* allocate(size_t nbytes) override {
    const size_t size = rounded(nbytes);
    {
      std::lock_guard<std::mutex> lk(mu_);
      auto it = free_.find(size);
      if (it != free_.end() && !it->second.empty()) {
        void* p = it->second.back();
        it->second.pop_back();
        live_[p] = size;
        return p;
      }
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, size);
    if (e != cudaSuccess) {   // give cached blocks back to the driver and try once more
      cudaGetLastError();
      release_all();
      e = cudaMalloc(&p, size);
    }
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(e) + " (cudaMalloc of " + std::to_string(size) + " bytes)");
    std::lock_guard<std::mutex> lk(mu_);
    live_[p] = size;
    reserved_ += size;
    return p;
  }
  void deallocate(void* ptr) noexcept override {
    if (ptr == nullptr) return;
    std::lock_guard<std::mutex> lk(mu_);
    auto it = live_.find(ptr);
    if (it == live_.end()) return;
    free_[it->second].push_back(ptr);
    live_.erase(it);
  }
  Device device() const override { return kCUDA0; }
  // Returns every cached (unused) block to the driver.
  void release_all() noexcept {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& kv : free_) {
      for (void* p : kv.second) {
        cudaFree(p);
        reserved_ -= kv.first;
      }
      kv.second.clear();
    }
  }
  size_t reserved_bytes() const { return reserved_; }
  size_t driver_allocations() const { return live_.size(); }

 private:
  static size_t rounded(size_t n) {
    if (n == 0) n = 1;
    const size_t step = n < (size_t{1} << 20) ? 512 : (size_t{2} << 20);
    return (n + step - 1) / step * step;
  }
  std::mutex mu_;
  std::map<size_t, std::vector<void*>> free_;
  std::unordered_map<void*, size_t> live_;
  size_t reserved_ = 0;
};

class HostAllocator final : public Allocator {
 public:
  explicit HostAllocator(bool pinned) : pinned_(pinned) {}
  void* allocate(size_t nbytes) override {
    if (nbytes == 0) nbytes = 1;
    void* p = nullptr;
    if (pinned_) {
      const cudaError_t e = cudaMallocHost(&p, nbytes);
      if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(e) + " (cudaMallocHost)");
    } else {
      p = ::operator new(nbytes);
    }
    return p;
  }
  void deallocate(void* ptr) noexcept override {
    if (ptr == nullptr) return;
    if (pinned_) cudaFreeHost(ptr);
    else ::operator delete(ptr);
  }
  Device device() const override { return kCPU; }

 private:
  bool pinned_;
};

}  // namespace detail

inline detail::ArenaAllocator& cuda_arena() {
  static detail::ArenaAllocator* a = new detail::ArenaAllocator();   // never destroyed: tensors with static lifetime may outlive main()
  return *a;
}
inline Allocator& cuda_allocator() { return cuda_arena(); }
inline Allocator& cpu_allocator() {
  static detail::HostAllocator a(false);
  return a;
}
inline Allocator& pinned_cpu_allocator() {
  static detail::HostAllocator a(true);
  return a;
}
inline Allocator& allocator_for(const Device& device) { return device.is_cuda() ? cuda_allocator() : cpu_allocator(); }

// ---- storage.h ------------------------------------------------------------------------------
class Storage {
 public:
  Storage(size_t nbytes, Allocator& allocator)
      : allocator_(&allocator), data_(allocator.allocate(nbytes)), nbytes_(nbytes), device_(allocator.device()) {}
  Storage(const Storage&) = delete;
  Storage& operator=(const Storage&) = delete;
  Storage(Storage&& o) noexcept { steal(o); }
  Storage& operator=(Storage&& o) noexcept {
    if (this != &o) {
      release();
      steal(o);
    }
    return *this;
  }
  ~Storage() { release(); }
  void* data() { return data_; }
  const void* data() const { return data_; }
  size_t nbytes() const { return nbytes_; }
  const Device& device() const { return device_; }

 private:
  void release() noexcept {
    if (data_ != nullptr && allocator_ != nullptr) allocator_->deallocate(data_);
    data_ = nullptr;
  }
  void steal(Storage& o) noexcept {
    allocator_ = o.allocator_;
    data_ = o.data_;
    nbytes_ = o.nbytes_;
    device_ = o.device_;
    o.data_ = nullptr;
    o.nbytes_ = 0;
  }
  Allocator* allocator_ = nullptr;
  void* data_ = nullptr;
  size_t nbytes_ = 0;
  Device device_{};
};
using StoragePtr = std::shared_ptr<Storage>;
inline StoragePtr make_storage(size_t nbytes, Allocator& alloc) { return std::make_shared<Storage>(nbytes, alloc); }

// ---- tensor.h -------------------------------------------------------------------------------
namespace autograd {
struct AutogradMeta;
}
namespace detail {
// A value that is computed on first use (see the header comment).
struct Deferred {
  std::function<void()> compute;
  bool done = false;
  void ensure() {
    if (!done) {
      done = true;   // set first: compute() may read the tensor it fills
      compute();
    }
  }
};
}  // namespace detail

inline std::vector<int64_t> contiguous_strides(const std::vector<int64_t>& shape) {
  std::vector<int64_t> s(shape.size(), 1);
  for (size_t i = shape.size(); i-- > 1;) s[i - 1] = s[i] * shape[i];
  return s;
}

class Tensor {
 public:
  Tensor() = default;

  static Tensor empty(std::vector<int64_t> shape, DType dtype, Device device) {
    Tensor t;
    t.shape_ = std::move(shape);
    t.strides_ = contiguous_strides(t.shape_);
    t.dtype_ = dtype;
    t.device_ = device;
    t.storage_ = make_storage(t.nbytes(), allocator_for(device));
    return t;
  }
  static Tensor zeros(std::vector<int64_t> shape, DType dtype, Device device) {
    Tensor t = empty(std::move(shape), dtype, device);
    if (t.nbytes() == 0) return t;
    if (device.is_cuda()) CTD_CUDA_CHECK(cudaMemsetAsync(t.storage_->data(), 0, t.nbytes(), nullptr));
    else std::memset(t.storage_->data(), 0, t.nbytes());
    return t;
  }
  static Tensor zeros_pinned(std::vector<int64_t> shape, DType dtype) {
    Tensor t;
    t.shape_ = std::move(shape);
    t.strides_ = contiguous_strides(t.shape_);
    t.dtype_ = dtype;
    t.device_ = kCPU;
    t.storage_ = make_storage(t.nbytes(), pinned_cpu_allocator());
    std::memset(t.storage_->data(), 0, t.nbytes());
    return t;
  }
  static Tensor from_host(const void* host_data, std::vector<int64_t> shape, DType dtype, Device device) {
    Tensor t = empty(std::move(shape), dtype, device);
    if (t.nbytes() == 0) return t;
    if (device.is_cuda()) CTD_CUDA_CHECK(cudaMemcpy(t.storage_->data(), host_data, t.nbytes(), cudaMemcpyHostToDevice));
    else std::memcpy(t.storage_->data(), host_data, t.nbytes());
    return t;
  }
  // A contiguous tensor over `numel(shape)` elements of `storage` starting `offset` elements in.
  static Tensor view_of(StoragePtr storage, int64_t offset, std::vector<int64_t> shape, DType dtype) {
    Tensor t;
    t.device_ = storage->device();
    t.storage_ = std::move(storage);
    t.storage_offset_ = offset;
    t.shape_ = std::move(shape);
    t.strides_ = contiguous_strides(t.shape_);
    t.dtype_ = dtype;
    return t;
  }

  void copy_to_host(void* dst) const {
    if (nbytes() == 0) return;
    detail::require(is_contiguous(), "Tensor::copy_to_host: non-contiguous tensors not yet supported");
    if (device_.is_cuda()) CTD_CUDA_CHECK(cudaMemcpy(dst, data_ptr(), nbytes(), cudaMemcpyDeviceToHost));
    else std::memcpy(dst, data_ptr(), nbytes());
  }

  inline Tensor reshape(std::vector<int64_t> new_shape) const;   // zero-copy; keeps the autograd history

  const std::vector<int64_t>& shape() const { return shape_; }
  const std::vector<int64_t>& strides() const { return strides_; }
  int64_t dim() const { return static_cast<int64_t>(shape_.size()); }
  int64_t numel() const {
    int64_t n = 1;
    for (const int64_t d : shape_) n *= d;
    return n;
  }
  size_t nbytes() const { return static_cast<size_t>(numel()) * dtype_size(dtype_); }
  DType dtype() const { return dtype_; }
  const Device& device() const { return device_; }
  bool is_contiguous() const { return strides_ == contiguous_strides(shape_); }

  void* data_ptr() {
    if (deferred_) deferred_->ensure();
    return storage_ ? static_cast<char*>(storage_->data()) + storage_offset_ * static_cast<int64_t>(dtype_size(dtype_)) : nullptr;
  }
  const void* data_ptr() const { return const_cast<Tensor*>(this)->data_ptr(); }
  const StoragePtr& storage() const { return storage_; }
  int64_t storage_offset() const { return storage_offset_; }

  // ---- autograd interface ----
  inline Tensor& requires_grad_(bool v = true);
  inline bool requires_grad() const;
  inline Tensor grad() const;
  inline void zero_grad_();
  inline void backward();
  inline void backward(const Tensor& grad_output);
  Tensor detach() const {
    Tensor t = *this;
    t.autograd_meta_.reset();
    return t;
  }
  const std::shared_ptr<autograd::AutogradMeta>& autograd_meta() const { return autograd_meta_; }
  std::shared_ptr<autograd::AutogradMeta>& mutable_autograd_meta() { return autograd_meta_; }

  // ---- this build only ----
  void set_deferred(std::shared_ptr<detail::Deferred> d) { deferred_ = std::move(d); }
  const std::shared_ptr<detail::Deferred>& deferred() const { return deferred_; }

 private:
  StoragePtr storage_;
  std::vector<int64_t> shape_;
  std::vector<int64_t> strides_;
  int64_t storage_offset_ = 0;
  DType dtype_ = DType::kFloat32;
  Device device_{};
  std::shared_ptr<autograd::AutogradMeta> autograd_meta_;
  std::shared_ptr<detail::Deferred> deferred_;
};

// ---- autograd.h -----------------------------------------------------------------------------
namespace autograd {

class Node;
struct Edge {
  std::shared_ptr<Node> node;
  uint32_t input_nr = 0;
};

class Node {
 public:
  virtual ~Node() = default;
  virtual std::vector<Tensor> backward(const std::vector<Tensor>& grads_out) = 0;
  virtual const char* name() const { return "Node"; }
  std::vector<Edge> next_edges;
};

struct AutogradMeta {
  bool requires_grad = false;
  Tensor grad;
  std::shared_ptr<Node> grad_fn;
  uint32_t output_nr = 0;
  std::shared_ptr<Node> grad_accumulator;
};

namespace detail {
inline bool& grad_mode() {
  thread_local bool enabled = true;
  return enabled;
}
}  // namespace detail

inline bool is_grad_enabled() { return detail::grad_mode(); }

class NoGradGuard {
 public:
  NoGradGuard() : prev_(detail::grad_mode()) { detail::grad_mode() = false; }
  ~NoGradGuard() { detail::grad_mode() = prev_; }
  NoGradGuard(const NoGradGuard&) = delete;
  NoGradGuard& operator=(const NoGradGuard&) = delete;

 private:
  bool prev_;
};

inline bool any_requires_grad(const std::vector<Tensor>& inputs) {
  if (!is_grad_enabled()) return false;
  for (const Tensor& t : inputs)
    if (t.requires_grad()) return true;
  return false;
}

// dst += src (fp32, CUDA, equal shapes).
inline void accumulate_inplace(Tensor& dst, const Tensor& src) {
  if (dst.shape() != src.shape()) {
    auto show = [](const std::vector<int64_t>& s) {
      std::string m = "[";
      for (const int64_t d : s) m += std::to_string(d) + ",";
      return m + "]";
    };
    throw std::runtime_error("accumulate: shape mismatch: dst=" + show(dst.shape()) + " src=" + show(src.shape()));
  }
  ::ctd::detail::require(dst.dtype() == DType::kFloat32 && src.dtype() == DType::kFloat32, "accumulate: only fp32");
  ::ctd::detail::require(dst.device().is_cuda() && src.device().is_cuda(), "accumulate: only CUDA");
  if (dst.numel() == 0) return;
  float* d = static_cast<float*>(dst.data_ptr());
  ::ctd::detail::ctdk_ok(ctdk_add(d, static_cast<const float*>(src.data_ptr()), d, dst.numel(), nullptr));
}

namespace detail {
// Leaf end of the tape: stores the first gradient that arrives and adds the later ones.
struct AccumulateGrad final : Node {
  std::weak_ptr<AutogradMeta> leaf;
  const char* name() const override { return "AccumulateGrad"; }
  std::vector<Tensor> backward(const std::vector<Tensor>& grads_out) override {
    ::ctd::detail::require(grads_out.size() == 1, "AccumulateGrad: expected 1 grad");
    if (std::shared_ptr<AutogradMeta> m = leaf.lock()) {
      if (!m->grad.storage()) m->grad = grads_out[0];
      else accumulate_inplace(m->grad, grads_out[0]);
    }
    return {};
  }
};
}  // namespace detail

inline std::vector<Edge> collect_next_edges(const std::vector<Tensor>& inputs) {
  std::vector<Edge> edges;
  edges.reserve(inputs.size());
  for (const Tensor& t : inputs) {
    const std::shared_ptr<AutogradMeta>& meta = t.autograd_meta();
    if (meta && meta->grad_fn) {
      edges.push_back(Edge{meta->grad_fn, meta->output_nr});
    } else if (meta && meta->requires_grad) {
      if (!meta->grad_accumulator) {
        auto acc = std::make_shared<detail::AccumulateGrad>();
        acc->leaf = meta;
        meta->grad_accumulator = acc;
      }
      edges.push_back(Edge{meta->grad_accumulator, 0});
    } else {
      edges.push_back(Edge{nullptr, 0});
    }
  }
  return edges;
}

inline void set_history(Tensor& out, std::shared_ptr<Node> node, uint32_t output_nr = 0) {
  std::shared_ptr<AutogradMeta>& meta = out.mutable_autograd_meta();
  if (!meta) meta = std::make_shared<AutogradMeta>();
  meta->requires_grad = true;
  meta->grad_fn = std::move(node);
  meta->output_nr = output_nr;
}

namespace detail {

// A tape node whose backward is a closure: what every op of this surface records.
struct FnNode final : Node {
  const char* label;
  std::function<std::vector<Tensor>(const std::vector<Tensor>&)> fn;
  FnNode(const char* l, std::function<std::vector<Tensor>(const std::vector<Tensor>&)> f) : label(l), fn(std::move(f)) {}
  const char* name() const override { return label; }
  std::vector<Tensor> backward(const std::vector<Tensor>& g) override { return fn(g); }
};

// Attaches `backward` to `out` if any input needs a gradient (and recording is on).
inline void record(Tensor& out, const std::vector<Tensor>& inputs, const char* label,
                   std::function<std::vector<Tensor>(const std::vector<Tensor>&)> backward) {
  if (!any_requires_grad(inputs)) return;
  auto node = std::make_shared<FnNode>(label, std::move(backward));
  node->next_edges = collect_next_edges(inputs);
  set_history(out, std::move(node));
}

// Walks the tape from `root`: nodes run once all their consumers have delivered (dependency
// counts from a first sweep), gradients meeting at one input slot are summed.
inline void run_backward(const std::shared_ptr<Node>& root, uint32_t root_slot, Tensor seed) {
  std::unordered_map<Node*, int> pending;
  std::unordered_map<Node*, std::shared_ptr<Node>> owner;
  std::vector<Node*> stack{root.get()};
  pending[root.get()] = 0;
  owner[root.get()] = root;
  while (!stack.empty()) {
    Node* n = stack.back();
    stack.pop_back();
    for (const Edge& e : n->next_edges) {
      if (!e.node) continue;
      auto it = pending.find(e.node.get());
      if (it == pending.end()) {
        pending[e.node.get()] = 1;
        owner[e.node.get()] = e.node;
        stack.push_back(e.node.get());
      } else {
        ++it->second;
      }
    }
  }
  std::unordered_map<Node*, std::vector<Tensor>> inbox;
  inbox[root.get()].resize(root_slot + 1);
  inbox[root.get()][root_slot] = std::move(seed);
  std::vector<Node*> ready{root.get()};
  size_t head = 0;
  while (head < ready.size()) {
    Node* n = ready[head++];
    std::vector<Tensor> grads = std::move(inbox[n]);
    inbox.erase(n);
    std::vector<Tensor> out = n->backward(grads);
    if (out.size() != n->next_edges.size())
      throw std::runtime_error(std::string("backward: node ") + n->name() + " returned wrong number of grads");
    for (size_t i = 0; i < out.size(); ++i) {
      const Edge& e = n->next_edges[i];
      if (!e.node) continue;
      Node* p = e.node.get();
      if (out[i].storage()) {
        std::vector<Tensor>& slots = inbox[p];
        if (slots.size() <= e.input_nr) slots.resize(e.input_nr + 1);
        if (!slots[e.input_nr].storage()) slots[e.input_nr] = std::move(out[i]);
        else accumulate_inplace(slots[e.input_nr], out[i]);
      }
      auto it = pending.find(p);
      if (it != pending.end() && --it->second == 0) ready.push_back(p);
    }
  }
}

}  // namespace detail

// Activation checkpointing: fn(input) runs without a tape; the backward re-runs it with one and
// walks that local graph (parameters reached inside fn receive their gradients there).
inline Tensor checkpoint(std::function<Tensor(const Tensor&)> fn, const Tensor& input) {
  if (!is_grad_enabled()) return fn(input);
  Tensor out;
  {
    NoGradGuard ng;
    out = fn(input);
  }
  Tensor saved = input.detach();
  const bool input_needs = input.requires_grad();
  auto node = std::make_shared<detail::FnNode>("CheckpointBackward", [fn, saved, input_needs](const std::vector<Tensor>& g) {
    Tensor x = saved;
    x.requires_grad_(true);
    Tensor y = fn(x);
    ::ctd::detail::require(y.autograd_meta() && y.autograd_meta()->grad_fn, "checkpoint: fn produced no graph on recompute");
    y.backward(g.at(0));
    std::vector<Tensor> r;
    r.push_back(input_needs ? x.grad() : Tensor{});
    return r;
  });
  node->next_edges = collect_next_edges({input});
  set_history(out, std::move(node));
  return out;
}

}  // namespace autograd

// ---- Tensor members that need the autograd types ----------------------------------------------
inline Tensor& Tensor::requires_grad_(bool v) {
  if (!autograd_meta_) autograd_meta_ = std::make_shared<autograd::AutogradMeta>();
  if (v && autograd_meta_->grad_fn) throw std::runtime_error("requires_grad_: cannot mark a non-leaf as requires_grad");
  autograd_meta_->requires_grad = v;
  return *this;
}
inline bool Tensor::requires_grad() const { return autograd_meta_ && autograd_meta_->requires_grad; }
inline Tensor Tensor::grad() const { return autograd_meta_ ? autograd_meta_->grad : Tensor{}; }
inline void Tensor::zero_grad_() {
  if (autograd_meta_) autograd_meta_->grad = Tensor{};
}
inline void Tensor::backward() {
  if (!autograd_meta_ || !autograd_meta_->grad_fn) throw std::runtime_error("backward: this tensor has no grad_fn");
  detail::require(dtype_ == DType::kFloat32, "backward: fp32 only");
  detail::require(numel() == 1, "backward: only scalar loss is supported");
  const float one = 1.0f;
  autograd::detail::run_backward(autograd_meta_->grad_fn, autograd_meta_->output_nr, Tensor::from_host(&one, shape_, dtype_, device_));
}
inline void Tensor::backward(const Tensor& grad_output) {
  if (!autograd_meta_ || !autograd_meta_->grad_fn) throw std::runtime_error("backward: this tensor has no grad_fn");
  detail::require(grad_output.shape() == shape_, "backward: grad_output shape mismatch");
  autograd::detail::run_backward(autograd_meta_->grad_fn, autograd_meta_->output_nr, grad_output);
}
inline Tensor Tensor::reshape(std::vector<int64_t> new_shape) const {
  detail::require(is_contiguous(), "reshape: input must be contiguous");
  int64_t n = 1;
  for (const int64_t d : new_shape) n *= d;
  detail::require(n == numel(), "reshape: numel mismatch");
  Tensor out;
  out.storage_ = storage_;
  out.storage_offset_ = storage_offset_;
  out.dtype_ = dtype_;
  out.device_ = device_;
  out.deferred_ = deferred_;
  out.shape_ = std::move(new_shape);
  out.strides_ = contiguous_strides(out.shape_);
  const std::vector<int64_t> back = shape_;
  autograd::detail::record(out, {*this}, "ReshapeBackward",
                           [back](const std::vector<Tensor>& g) { return std::vector<Tensor>{g.at(0).reshape(back)}; });
  return out;
}

}  // namespace ctd
