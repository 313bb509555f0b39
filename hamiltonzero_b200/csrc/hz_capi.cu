// Status strings, version and error bookkeeping of the C ABI.
#include "hz_internal.h"

#include <map>
#include <mutex>
#include <utility>
#include <vector>

namespace hz {
namespace {
thread_local int g_last_cuda_error = 0;

struct Span { int stage; cudaEvent_t a, b; double flops; int launches; };
std::mutex g_mu;
bool g_timing = false;
std::vector<Span> g_spans;
std::vector<cudaEvent_t> g_pool;
cudaEvent_t g_open[kStCount];
double g_ms[kStCount], g_flops[kStCount];
long long g_launches[kStCount];

cudaEvent_t take_event() {
  if (!g_pool.empty()) { cudaEvent_t e = g_pool.back(); g_pool.pop_back(); return e; }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}

// Resolves finished spans into the per-stage totals. Caller holds g_mu.
void drain() {
  for (const Span& s : g_spans) {
    if (!s.a || !s.b) continue;
    float ms = 0.f;
    if (cudaEventSynchronize(s.b) == cudaSuccess && cudaEventElapsedTime(&ms, s.a, s.b) == cudaSuccess) {
      g_ms[s.stage] += ms; g_flops[s.stage] += s.flops; g_launches[s.stage] += s.launches;
    }
    g_pool.push_back(s.a); g_pool.push_back(s.b);
  }
  g_spans.clear();
}
}  // namespace

void set_last_cuda_error(int err) { g_last_cuda_error = err; }

int ensure_kernel_attributes(const void* kernel, int bytes, bool max_carveout) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, std::pair<int, bool>> done;   // (kernel, device)
  int dev = 0;
  HZ_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  std::pair<int, bool>& have = done[std::make_pair(kernel, dev)];
  if (bytes > 48 * 1024 && have.first < bytes) {
    HZ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    have.first = bytes;
  }
  if (max_carveout && !have.second) {
    HZ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared));
    have.second = true;
  }
  return HZ_OK;
}

bool stage_timing_on() { return g_timing; }

void stage_begin(int stage, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_open[stage] = take_event();
  if (g_open[stage]) cudaEventRecord(g_open[stage], stream);
}

void stage_end(int stage, cudaStream_t stream, double flops, int launches) {
  std::lock_guard<std::mutex> lock(g_mu);
  cudaEvent_t b = take_event();
  if (b) cudaEventRecord(b, stream);
  g_spans.push_back(Span{stage, g_open[stage], b, flops, launches});
  g_open[stage] = nullptr;
  if (g_spans.size() > 4096) drain();   // bounds the number of live events
}
}  // namespace hz

extern "C" int hz_stage_count(void) { return hz::kStCount; }

extern "C" const char* hz_stage_name(int stage) {
  static const char* names[hz::kStCount] = {"leaf_map", "leaf_kernel", "merge_tc_kernel",
                                            "factor_gemm<V>", "factor_gemm<U>",
                                            "norm_reduce_kernel", "norm_apply_kernel",
                                            "factor_gemm<readout>", "root_kernel",
                                            "level1_prepare", "l1_coeff_kernel",
                                            "l1_expand_kernel", "level2_prepare",
                                            "l2_coeff_kernel", "level2_gram_gemm",
                                            "l2_norm_kernel", "level2_expand_gemm",
                                            "merge_cross_kernel"};
  return (stage >= 0 && stage < hz::kStCount) ? names[stage] : "";
}

extern "C" int hz_stage_timing_enable(int on) {
  std::lock_guard<std::mutex> lock(hz::g_mu);
  hz::g_timing = on != 0;
  return HZ_OK;
}

extern "C" int hz_stage_timing_read(double* ms, double* flops, long long* launches, int n,
                                    int reset) {
  if (!ms || !flops || !launches) return HZ_ERR_NULL_POINTER;
  if (n < hz::kStCount) return HZ_ERR_BAD_SHAPE;
  std::lock_guard<std::mutex> lock(hz::g_mu);
  hz::drain();
  for (int i = 0; i < hz::kStCount; ++i) {
    ms[i] = hz::g_ms[i]; flops[i] = hz::g_flops[i]; launches[i] = hz::g_launches[i];
    if (reset) { hz::g_ms[i] = 0; hz::g_flops[i] = 0; hz::g_launches[i] = 0; }
  }
  return HZ_OK;
}

extern "C" const char* hz_status_string(int status) {
  switch (status) {
    case HZ_OK: return "ok";
    case HZ_ERR_NULL_POINTER: return "a required pointer is NULL";
    case HZ_ERR_BAD_SHAPE: return "non-positive or inconsistent extent";
    case HZ_ERR_UNSUPPORTED: return "extent outside what the kernels implement";
    case HZ_ERR_MISALIGNED: return "pointer not aligned as required";
    case HZ_ERR_CUDA: return "a CUDA runtime call failed";
    case HZ_ERR_NO_DEVICE: return "no usable sm_100 device";
    case HZ_ERR_WORKSPACE: return "caller-provided workspace is too small";
    case HZ_ERR_STATIC_SCRATCH:
      return "one walker of this wavefunction needs more scratch than the library's built-in "
             "32 MiB array; use hz_logpsi with a caller-provided workspace";
    case HZ_ERR_TIMEOUT: return "a bounded device-side wait ran out; the call's outputs are NaN";
    case HZ_ERR_WRONG_DEVICE: return "a buffer lives on another device than the current one";
    default: return "unknown status";
  }
}

extern "C" int hz_last_cuda_error(void) { return hz::g_last_cuda_error; }

extern "C" int hz_version(void) { return 100; }
