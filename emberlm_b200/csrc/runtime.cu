// Error reporting, device properties and the device status word of the ctdk library.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace ctdk {

namespace {
thread_local char g_err[512] = "";
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices] = {0};

// The status word lives in device global memory that belongs to the library image, so
// kernels can report a bounded wait that ran out without any allocation.
__device__ int g_status_word[4];
int* g_status_ptr[kMaxDevices] = {nullptr};
std::mutex g_mu;
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

std::atomic<long long> g_launches{0};

// ---- optional per-class kernel timing with CUDA events on the launching stream ----
struct ProfRec {
  cudaEvent_t a, b;
  int cls;
  double work;
};
std::mutex g_prof_mu;
bool g_prof_on = false;
std::vector<ProfRec> g_prof;
std::vector<cudaEvent_t> g_event_pool;

cudaEvent_t take_event() {
  if (!g_event_pool.empty()) {
    cudaEvent_t e = g_event_pool.back();
    g_event_pool.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}

bool prof_enabled() { return g_prof_on; }

void* prof_begin(int cls, double work, cudaStream_t s) {
  if (!g_prof_on) return nullptr;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  ProfRec r{take_event(), take_event(), cls, work};
  cudaEventRecord(r.a, s);
  g_prof.push_back(r);
  return reinterpret_cast<void*>(g_prof.size());
}

void prof_end(void* token, cudaStream_t s) {
  if (token == nullptr) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  const size_t i = reinterpret_cast<size_t>(token) - 1;
  if (i < g_prof.size()) cudaEventRecord(g_prof[i].b, s);
}

int check_launch(const char* what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return CTDK_OK;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

// SMs left to the persistent tensor-core kernels (one CTA, or one CTA pair, per SM): all of them,
// less what ctdk_reserve_sms() set aside for kernels of other streams.
static int g_reserved_sms = 0;
int sm_budget() {
  const int n = sm_count() - g_reserved_sms;
  return n < 2 ? 2 : n;
}

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

int read_device_status(cudaStream_t stream) {
  int* p = device_status_word();
  if (p == nullptr) return fail(CTDK_ELAUNCH, "status word unavailable");
  int h[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyAsync(h, p, sizeof(h), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(CTDK_ELAUNCH, "status read: %s", cudaGetErrorString(e));
  if (h[0] != 0) {
    cudaMemsetAsync(p, 0, sizeof(h), stream);
    return fail(h[0], "device status %d at site %d (block %d, detail %d)", h[0], h[1], h[2],
                h[3]);
  }
  return CTDK_OK;
}

}  // namespace ctdk

extern "C" {

const char* ctdk_last_error(void) { return ctdk::g_err; }

int ctdk_sm_count(void) { return ctdk::sm_count(); }
int ctdk_reserve_sms(int n) {
  if (n < 0 || n >= ctdk::sm_count()) return ctdk::fail(CTDK_EINVAL, "ctdk_reserve_sms: n out of range");
  ctdk::g_reserved_sms = n & ~1;   // whole CTA pairs
  return CTDK_OK;
}

long long ctdk_launch_count(void) { return ctdk::g_launches.load(); }

int ctdk_prof_enable(int on) {
  std::lock_guard<std::mutex> lk(ctdk::g_prof_mu);
  ctdk::g_prof_on = on != 0;
  return CTDK_OK;
}

int ctdk_prof_collect(int cls, double* total_ms, double* total_work, long long* launches) {
  cudaDeviceSynchronize();
  std::lock_guard<std::mutex> lk(ctdk::g_prof_mu);
  double ms = 0.0, work = 0.0;
  long long n = 0;
  std::vector<ctdk::ProfRec> keep;
  for (auto& r : ctdk::g_prof) {
    if (r.cls != cls) {
      keep.push_back(r);
      continue;
    }
    float t = 0.0f;
    if (cudaEventElapsedTime(&t, r.a, r.b) == cudaSuccess) {
      ms += t;
      work += r.work;
      ++n;
    }
    ctdk::g_event_pool.push_back(r.a);
    ctdk::g_event_pool.push_back(r.b);
  }
  ctdk::g_prof.swap(keep);
  if (total_ms) *total_ms = ms;
  if (total_work) *total_work = work;
  if (launches) *launches = n;
  return CTDK_OK;
}

int ctdk_device_status(void* stream, int* where) {
  int* p = ctdk::device_status_word();
  if (p == nullptr) return ctdk::fail(CTDK_ELAUNCH, "status word unavailable");
  int h[4] = {0, 0, 0, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(h, p, sizeof(h), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return ctdk::fail(CTDK_ELAUNCH, "status read: %s", cudaGetErrorString(e));
  if (where != nullptr)
    for (int i = 0; i < 4; ++i) where[i] = h[i];
  if (h[0] != 0) {
    cudaMemsetAsync(p, 0, sizeof(h), s);
    cudaStreamSynchronize(s);
    return ctdk::fail(h[0], "device status %d at site %d (block %d, detail %d)", h[0], h[1],
                      h[2], h[3]);
  }
  return CTDK_OK;
}

}  // extern "C"
