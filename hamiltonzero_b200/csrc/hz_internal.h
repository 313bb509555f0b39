// Internal helpers shared by the translation units of libhz_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>


#include "../../include/hz_b200.h"

namespace hz {
// Records the failing cudaError_t for hz_last_cuda_error() (thread local).
void set_last_cuda_error(int err);

// Optional per-stage device timing of the walker pipeline (hz_stage_timing_*): when
// enabled, every stage launch is bracketed by CUDA events on the launching stream.
enum Stage {
  kStLeafMap = 0, kStLeaf, kStMerge, kStGemmV, kStGemmU, kStNormReduce, kStNormApply,
  kStRootGemm, kStRoot, kStL1Prep, kStL1Coeff, kStL1Expand,
  kStL2Prep, kStL2Coeff, kStL2Gram, kStL2Norm, kStL2Expand, kStMergeCross, kStCount
};
bool stage_timing_on();
void stage_begin(int stage, cudaStream_t stream);
void stage_end(int stage, cudaStream_t stream, double flops, int launches);
struct StageScope {
  int stage; cudaStream_t stream; double flops; int launches; bool on;
  // `n_launches`: kernels launched inside the scope (counted by hz_stage_timing_read)
  StageScope(int st, cudaStream_t s, double f, int n_launches = 1)
      : stage(st), stream(s), flops(f), launches(n_launches), on(stage_timing_on()) {
    if (on) stage_begin(stage, stream);
  }
  ~StageScope() { if (on) stage_end(stage, stream, flops, launches); }
};
}  // namespace hz

namespace hz {
// True when the environment variable `name` equals `value`. Callers keep the answer in a
// function-local `static const`, whose initialisation the language makes thread-safe.
inline bool env_equals(const char* name, const char* value) {
  const char* e = getenv(name);
  return e != nullptr && strcmp(e, value) == 0;
}
inline int env_int(const char* name, int fallback) {
  const char* e = getenv(name);
  return e != nullptr ? atoi(e) : fallback;
}
constexpr int kMaxDevicesTracked = 64;
}  // namespace hz

namespace hz {
// One-time function attributes per (kernel, device): raises the kernel's dynamic shared-memory
// limit to `bytes` (and, with max_carveout, asks for the largest shared-memory carve-out) the
// first time it is needed on the current device, under a lock; later launches only look the
// kernel up. Returns an HZ_* status.
int ensure_kernel_attributes(const void* kernel, int bytes, bool max_carveout = false);
}  // namespace hz

#define HZ_CUDA_TRY(expr)                          \
  do {                                             \
    cudaError_t hz_err__ = (expr);                 \
    if (hz_err__ != cudaSuccess) {                 \
      ::hz::set_last_cuda_error((int)hz_err__);    \
      return HZ_ERR_CUDA;                          \
    }                                              \
  } while (0)
