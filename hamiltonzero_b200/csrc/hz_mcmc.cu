// Replica-exchange MALA sweep on SU(2)^N for sm_100a.
//
// Reference semantics: src/hamiltonzero/mcmc/langevin.py:25-135 (MALA move with a
// wrapped-normal proposal density, 17 images), src/hamiltonzero/mcmc/replica_exchange.py
// :96-303 (refresh, global Haar move, deterministic even-odd swaps, sweep loop) and
// src/hamiltonzero/mcmc/quaternion.py (exp / log / product). log p = 2 log|psi|
// (src/hamiltonzero/mcmc/runtime.py:66-72).
//
// The reference caches grad_q log p [N,4] and only ever uses its projection on the frame
// e_1..e_3 (langevin.py:25-40). That projection is the derivative of log p along the
// right-SU(2) chart, which the forward-jet pipeline of hz_walker.cu delivers; the sweep
// therefore carries "drift" [N,3] instead of the 4-vector, and one value-and-gradient is
// one jet pass with a zero energy frame.
// Random numbers: Philox4x32-10 keyed by (seed, offset); every draw can be overridden by
// caller-provided arrays (hz_mcmc_noise) so that single steps can be checked bit for bit
// against a host restatement.
#include "hz_internal.h"

#include <math.h>

namespace hz {
// defined in hz_walker.cu
int chart_value_and_grad(const hz_wavefunction* w, const float* q, long long n, float* log_abs, float* phase, float* grad, void* workspace,
                         long long workspace_bytes, cudaStream_t stream, bool prepared);
long long chart_workspace_bytes(const hz_wavefunction* w, long long walkers_per_chunk);

namespace {

constexpr int kWrap = 8;
constexpr float kTwoPi = 6.28318530717958647692f;

// ---------------------------------------------------------------- Philox4x32-10
struct Philox {
  uint32_t key[2];
  __device__ Philox(uint64_t seed) { key[0] = (uint32_t)seed; key[1] = (uint32_t)(seed >> 32); }
  __device__ uint4 operator()(uint64_t index, uint32_t stream, uint32_t sub) const {
    uint32_t c[4] = {(uint32_t)index, (uint32_t)(index >> 32), stream, sub};
    uint32_t k0 = key[0], k1 = key[1];
#pragma unroll
    for (int r = 0; r < 10; ++r) {
      const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
      const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
      c[0] = hi1 ^ c[1] ^ k0; c[1] = lo1; c[2] = hi0 ^ c[3] ^ k1; c[3] = lo0;
      k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return make_uint4(c[0], c[1], c[2], c[3]);
  }
};
__device__ __forceinline__ float u01(uint32_t x) { return ((float)x + 0.5f) * 2.3283064365386963e-10f; }
__device__ __forceinline__ void box_muller(uint32_t a, uint32_t b, float& n0, float& n1) {
  const float r = sqrtf(-2.f * logf(u01(a)));
  float s, c;
  sincosf(kTwoPi * u01(b), &s, &c);
  n0 = r * c; n1 = r * s;
}
enum Stream { kStreamLocalNoise = 1, kStreamLocalU = 2, kStreamSwapU = 3, kStreamHaarScore = 4,
              kStreamHaarRaw = 5, kStreamHaarU = 6 };

// ---------------------------------------------------------------- quaternion algebra
struct Q4 { float w, x, y, z; };
__device__ __forceinline__ Q4 qmul(const Q4& a, const Q4& b) {
  return Q4{a.w * b.w - a.x * b.x - a.y * b.y - a.z * b.z, a.w * b.x + a.x * b.w + a.y * b.z - a.z * b.y,
            a.w * b.y - a.x * b.z + a.y * b.w + a.z * b.x, a.w * b.z + a.x * b.y - a.y * b.x + a.z * b.w};
}
__device__ __forceinline__ Q4 qexp(float vx, float vy, float vz) {     // quaternion.py:43-58
  const float t2 = vx * vx + vy * vy + vz * vz, t = sqrtf(t2);
  const bool small = t2 < 1e-12f;
  const float s = small ? 1.f - t2 / 6.f + t2 * t2 / 120.f : sinf(t) / t;
  const float r = small ? 1.f - t2 / 2.f + t2 * t2 / 24.f : cosf(t);
  return Q4{r, s * vx, s * vy, s * vz};
}
__device__ __forceinline__ Q4 qnormalize(const Q4& q) {                // quaternion.py:61-65
  const float inv = 1.f / sqrtf(q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z + 1e-12f);
  return Q4{q.w * inv, q.x * inv, q.y * inv, q.z * inv};
}
__device__ __forceinline__ void qlog(const Q4& q, float& vx, float& vy, float& vz) {  // :74-90
  const float sn2 = q.x * q.x + q.y * q.y + q.z * q.z, sn = sqrtf(sn2);
  const float factor = (sn < 1e-8f) ? 1.f + sn2 / 6.f : atan2f(sn, q.w) / sn;
  vx = q.x * factor; vy = q.y * factor; vz = q.z * factor;
}
__device__ __forceinline__ float log_jacobian_su2(float norm) {       // langevin.py:43-53
  const float ns = fmaxf(norm, 1e-9f);
  const float full = logf(fmaxf(fabsf(sinf(ns)), 1e-9f)) - logf(ns);
  return 2.f * ((norm < 1e-3f) ? -norm * norm / 6.f : full);
}
// log of the wrapped proposal density of one site (langevin.py:56-81)
__device__ float wrapped_log_q_site(const float xi[3], const float mu[3], float sigma_sq) {
  const float norm = sqrtf(xi[0] * xi[0] + xi[1] * xi[1] + xi[2] * xi[2]);
  float u[3] = {1.f, 0.f, 0.f};
  if (!(norm < 1e-9f)) { u[0] = xi[0] / norm; u[1] = xi[1] / norm; u[2] = xi[2] / norm; }
  float lk[2 * kWrap + 1], mx = -INFINITY;
#pragma unroll
  for (int i = 0; i <= 2 * kWrap; ++i) {
    const float sh = kTwoPi * (float)(i - kWrap);
    const float b0 = xi[0] + sh * u[0], b1 = xi[1] + sh * u[1], b2 = xi[2] + sh * u[2];
    const float d0 = b0 - mu[0], d1 = b1 - mu[1], d2 = b2 - mu[2];
    lk[i] = -(d0 * d0 + d1 * d1 + d2 * d2) / (2.f * sigma_sq) -
            log_jacobian_su2(sqrtf(b0 * b0 + b1 * b1 + b2 * b2));
    mx = fmaxf(mx, lk[i]);
  }
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i <= 2 * kWrap; ++i) sum += expf(lk[i] - mx);
  return mx + logf(sum);
}

struct Dims { int B, R, N; };

// ---------------------------------------------------------------- kernels
// One thread per (walker, replica, site): forward proposal and the chart coordinate of the
// reverse move.
__global__ void mala_propose_kernel(Dims dm, const float* __restrict__ q, const float* __restrict__ drift,
                                    const float* __restrict__ beta, const float* __restrict__ sigma,
                                    const int32_t* __restrict__ mask, const float* __restrict__ noise_in,
                                    uint64_t seed, uint32_t step_id, float* __restrict__ q_prop,
                                    float* __restrict__ xi_fwd_out, float* __restrict__ mu_fwd_out) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)dm.B * dm.R * dm.N;
  if (idx >= total) return;
  const int site = (int)(idx % dm.N), r = (int)((idx / dm.N) % dm.R);
  const float mf = mask[site] ? 1.f : 0.f;
  float n[3];
  if (noise_in) { n[0] = noise_in[idx * 3]; n[1] = noise_in[idx * 3 + 1]; n[2] = noise_in[idx * 3 + 2]; }
  else {
    const uint4 x = Philox(seed)((uint64_t)idx, kStreamLocalNoise, step_id);
    float dummy;
    box_muller(x.x, x.y, n[0], n[1]);
    box_muller(x.z, x.w, n[2], dummy);
  }
  const float s = sigma[r], s2 = s * s, b = beta[r];
  float mu[3], xi[3];
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    mu[a] = 0.5f * s2 * b * (drift[idx * 3 + a] * mf);
    xi[a] = mu[a] + s * (n[a] * mf);
  }
  const Q4 q0{q[idx * 4], q[idx * 4 + 1], q[idx * 4 + 2], q[idx * 4 + 3]};
  const Q4 qp = qnormalize(qmul(q0, qexp(xi[0], xi[1], xi[2])));
  const Q4 back = qmul(Q4{qp.w, -qp.x, -qp.y, -qp.z}, q0);
  float bx, by, bz;
  qlog(back, bx, by, bz);
  q_prop[idx * 4] = qp.w; q_prop[idx * 4 + 1] = qp.x; q_prop[idx * 4 + 2] = qp.y; q_prop[idx * 4 + 3] = qp.z;
  xi_fwd_out[idx * 3] = -bx * mf; xi_fwd_out[idx * 3 + 1] = -by * mf; xi_fwd_out[idx * 3 + 2] = -bz * mf;
  mu_fwd_out[idx * 3] = mu[0]; mu_fwd_out[idx * 3 + 1] = mu[1]; mu_fwd_out[idx * 3 + 2] = mu[2];
}

__device__ __forceinline__ float warp_sum_f(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// drift (e1, e2, e3) of a site from the chart gradient grad [3N][2] (rows x, y, z; column 0 =
// d log|psi|): log p = 2 log|psi| and (e1, e2, e3) = d/d(z, y, x).
__device__ __forceinline__ float drift_from_grad(const float* g, int site, int a) {
  return 2.f * g[(size_t)(3 * site + (2 - a)) * 2];
}

// One warp per (walker, replica): Metropolis-Hastings test of a MALA proposal and state update.
// mode 0: MALA (uses xi_fwd, mu_fwd); mode 1: Haar move (log alpha = min(0, beta dlogp)).
__global__ void accept_kernel(Dims dm, int mode, float* __restrict__ q, float* __restrict__ log_p,
                              float* __restrict__ drift, const float* __restrict__ beta,
                              const float* __restrict__ sigma, const int32_t* __restrict__ mask,
                              const float* __restrict__ q_prop, const float* __restrict__ la_prop,
                              const float* __restrict__ grad_prop, const float* __restrict__ xi_fwd,
                              const float* __restrict__ mu_fwd, const float* __restrict__ logu_in,
                              uint64_t seed, uint32_t step_id, float* __restrict__ n_accept,
                              float* __restrict__ log_alpha_out) {
  const long long wr = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wr >= (long long)dm.B * dm.R) return;
  const int r = (int)(wr % dm.R), N = dm.N;
  const float b = beta[r], s = sigma[r], s2 = s * s;
  const float* g = grad_prop + (size_t)wr * 3 * N * 2;
  const float lp_new = 2.f * la_prop[wr], lp_old = log_p[wr];
  float lq = 0.f;
  if (mode == 0) {
    for (int site = lane; site < N; site += 32) {
      if (!mask[site]) continue;
      const size_t o = ((size_t)wr * N + site) * 3;
      const float xi[3] = {xi_fwd[o], xi_fwd[o + 1], xi_fwd[o + 2]};
      const float mf[3] = {mu_fwd[o], mu_fwd[o + 1], mu_fwd[o + 2]};
      float mb[3];
#pragma unroll
      for (int a = 0; a < 3; ++a) mb[a] = -0.5f * s2 * b * drift_from_grad(g, site, a);
      lq += wrapped_log_q_site(xi, mb, s2) - wrapped_log_q_site(xi, mf, s2);
    }
    lq = warp_sum_f(lq);
  }
  float log_alpha = b * (lp_new - lp_old) + lq;
  if (mode == 1) log_alpha = fminf(0.f, log_alpha);
  float logu;
  if (logu_in) logu = logu_in[wr];
  else logu = logf(u01(Philox(seed)((uint64_t)wr, mode == 0 ? kStreamLocalU : kStreamHaarU, step_id).x));
  bool accept = (mode == 0) ? (logu < log_alpha) : (logu <= log_alpha);
  if (mode == 0) accept = accept || (isnan(lp_old) && !isnan(lp_new));
  if (log_alpha_out && lane == 0) log_alpha_out[wr] = log_alpha;
  if (!accept) return;
  for (int site = lane; site < N; site += 32) {
    const size_t o = (size_t)wr * N + site;
    if (mode == 1 || mask[site]) {
#pragma unroll
      for (int c = 0; c < 4; ++c) q[o * 4 + c] = q_prop[o * 4 + c];
    }
#pragma unroll
    for (int a = 0; a < 3; ++a) drift[o * 3 + a] = drift_from_grad(g, site, a);
  }
  if (lane == 0) {
    log_p[wr] = lp_new;
    n_accept[wr] += 1.f;
  }
}

// log_p and drift of the current state (refresh at the start of a sweep)
__global__ void refresh_kernel(Dims dm, const float* __restrict__ la, const float* __restrict__ grad,
                               float* __restrict__ log_p, float* __restrict__ drift) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)dm.B * dm.R * dm.N;
  if (idx >= total) return;
  const long long wr = idx / dm.N;
  const int site = (int)(idx % dm.N);
  const float* g = grad + (size_t)wr * 3 * dm.N * 2;
#pragma unroll
  for (int a = 0; a < 3; ++a) drift[idx * 3 + a] = drift_from_grad(g, site, a);
  if (site == 0) log_p[wr] = 2.f * la[wr];
}

// One CTA per walker: deterministic even-odd neighbour swaps (replica_exchange.py:112-152).
__global__ void swap_kernel(Dims dm, float* __restrict__ q, float* __restrict__ log_p,
                            float* __restrict__ drift, const float* __restrict__ beta, int step,
                            const float* __restrict__ logu_in, uint64_t seed, uint32_t step_id,
                            float* __restrict__ n_swap_accept, int32_t* __restrict__ n_swap) {
  __shared__ int acc_s[64];
  const int b = blockIdx.x, R = dm.R, N = dm.N;
  for (int e = threadIdx.x; e < R - 1; e += blockDim.x) {
    const bool eligible = (e % 2) == (step % 2);
    const float lpi = log_p[(size_t)b * R + e], lpj = log_p[(size_t)b * R + e + 1];
    const float log_alpha = (beta[e + 1] - beta[e]) * (lpi - lpj);
    const size_t o = (size_t)b * (R - 1) + e;
    const float logu = logu_in ? logu_in[o] : logf(u01(Philox(seed)((uint64_t)o, kStreamSwapU, step_id).x));
    const bool a = eligible && ((logu < log_alpha) || (isnan(lpj) && !isnan(lpi)));
    acc_s[e] = a ? 1 : 0;
    if (eligible) n_swap[o] += 1;
    if (a) n_swap_accept[o] += 1.f;
  }
  __syncthreads();
  for (int e = (step % 2); e < R - 1; e += 2) {      // eligible edges are disjoint
    if (!acc_s[e]) continue;
    float* qa = q + ((size_t)b * R + e) * N * 4;
    float* da = drift + ((size_t)b * R + e) * N * 3;
    for (int i = threadIdx.x; i < N * 4; i += blockDim.x) { const float t = qa[i]; qa[i] = qa[N * 4 + i]; qa[N * 4 + i] = t; }
    for (int i = threadIdx.x; i < N * 3; i += blockDim.x) { const float t = da[i]; da[i] = da[N * 3 + i]; da[N * 3 + i] = t; }
    if (threadIdx.x == 0) {
      const float t = log_p[(size_t)b * R + e];
      log_p[(size_t)b * R + e] = log_p[(size_t)b * R + e + 1];
      log_p[(size_t)b * R + e + 1] = t;
    }
  }
}

// One CTA per (walker, replica): Haar proposal on the m[r] real sites with the smallest scores
// (replica_exchange.py:155-180). N <= 256.
__global__ void haar_propose_kernel(Dims dm, const float* __restrict__ q, const int32_t* __restrict__ mask,
                                    const int32_t* __restrict__ m, const float* __restrict__ scores_in,
                                    const float* __restrict__ raw_in, uint64_t seed, uint32_t step_id,
                                    float* __restrict__ q_prop) {
  __shared__ float sc[256];
  const long long wr = blockIdx.x;
  const int r = (int)(wr % dm.R), N = dm.N, site = threadIdx.x;
  if (site < N) {
    const size_t o = (size_t)wr * N + site;
    float v = scores_in ? scores_in[o] : u01(Philox(seed)((uint64_t)o, kStreamHaarScore, step_id).x);
    sc[site] = mask[site] ? v : INFINITY;
  }
  __syncthreads();
  if (site >= N) return;
  int rank = 0;
  for (int j = 0; j < N; ++j) rank += (sc[j] < sc[site]) || (sc[j] == sc[site] && j < site);
  const bool move = mask[site] && rank < m[r];
  const size_t o = (size_t)wr * N + site;
  Q4 out{q[o * 4], q[o * 4 + 1], q[o * 4 + 2], q[o * 4 + 3]};
  if (move) {
    Q4 raw;
    if (raw_in) raw = Q4{raw_in[o * 4], raw_in[o * 4 + 1], raw_in[o * 4 + 2], raw_in[o * 4 + 3]};
    else {
      const uint4 x = Philox(seed)((uint64_t)o, kStreamHaarRaw, step_id);
      box_muller(x.x, x.y, raw.w, raw.x);
      box_muller(x.z, x.w, raw.y, raw.z);
    }
    out = qnormalize(raw);
  }
  q_prop[o * 4] = out.w; q_prop[o * 4 + 1] = out.x; q_prop[o * 4 + 2] = out.y; q_prop[o * 4 + 3] = out.z;
}

size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

struct McmcWs {
  float *q_prop, *xi, *mu, *la, *ph, *grad;
  char* rest;
  size_t fixed;
};
McmcWs carve(long long B, long long R, long long N, char* base) {
  McmcWs w{};
  size_t off = 0;
  auto take = [&](size_t nfloats) {
    float* p = base ? reinterpret_cast<float*>(base + off) : nullptr;
    off += align_up(nfloats * sizeof(float));
    return p;
  };
  w.q_prop = take((size_t)(B * R * N * 4));
  w.xi = take((size_t)(B * R * N * 3));
  w.mu = take((size_t)(B * R * N * 3));
  w.la = take((size_t)(B * R));
  w.ph = take((size_t)(B * R));
  w.grad = take((size_t)(B * R * N * 6));
  w.rest = base ? base + off : nullptr;
  w.fixed = off;
  return w;
}

}  // namespace
}  // namespace hz

using namespace hz;

extern "C" long long hz_mcmc_workspace_bytes(const hz_wavefunction* wf, int n_walkers,
                                             int n_replicas, long long replicas_per_chunk) {
  if (!wf || n_walkers <= 0 || n_replicas < 2 || replicas_per_chunk <= 0) return -1;
  const long long inner = chart_workspace_bytes(wf, replicas_per_chunk);
  if (inner < 0) return -1;
  return (long long)carve(n_walkers, n_replicas, wf->n_sites, nullptr).fixed + inner;
}

extern "C" int hz_mcmc_sweep(const hz_wavefunction* wf, hz_mcmc_state* st, int n_steps,
                             const hz_mcmc_noise* noise, float* log_alpha_out, void* workspace,
                             long long workspace_bytes, void* stream) {
  if (!wf || !st || !workspace) return HZ_ERR_NULL_POINTER;
  const int B = st->n_walkers, R = st->n_replicas, N = st->n_sites;
  if (B <= 0 || R < 2 || R > 64 || N != wf->n_sites || n_steps < 0) return HZ_ERR_BAD_SHAPE;
  if (N > 256) return HZ_ERR_UNSUPPORTED;
  if (!st->q || !st->log_p || !st->drift || !st->beta || !st->sigma || !st->mask || !st->m ||
      !st->n_local_accept || !st->n_swap_accept || !st->n_swap || !st->n_haar_accept)
    return HZ_ERR_NULL_POINTER;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return HZ_ERR_MISALIGNED;
  // layout: [scratch of the value-and-gradient passes (status word first) | sweep arrays]
  const long long fixed = (long long)carve(B, R, N, nullptr).fixed;
  if (fixed >= workspace_bytes) return HZ_ERR_WORKSPACE;
  const long long inner_bytes = (workspace_bytes - fixed) & ~255ll;
  McmcWs ws = carve(B, R, N, static_cast<char*>(workspace) + inner_bytes);
  ws.rest = static_cast<char*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const Dims dm{B, R, N};
  const long long BR = (long long)B * R, BRN = BR * N;
  const unsigned site_blocks = (unsigned)((BRN + 255) / 256);
  const unsigned warp_blocks = (unsigned)((BR + 3) / 4);

  // the once-per-call arrays of the value-and-gradient pass (weight splits, level bases) are built
  // by the first evaluation of the sweep and reused by the others
  bool prepared = false;
  auto eval = [&](const float* q) {
    const int rc = chart_value_and_grad(wf, q, BR, ws.la, ws.ph, ws.grad, ws.rest,
                                        inner_bytes, s, prepared);
    prepared = true;
    return rc;
  };
  // refresh the cached log p and drift (replica_exchange.py:96-109)
  int rc = eval(st->q);
  if (rc != HZ_OK) return rc;
  refresh_kernel<<<site_blocks, 256, 0, s>>>(dm, ws.la, ws.grad, st->log_p, st->drift);
  // global Haar move (replica_exchange.py:155-230)
  const uint32_t base_id = (uint32_t)(st->offset * 4099u);
  haar_propose_kernel<<<(unsigned)BR, 256, 0, s>>>(dm, st->q, st->mask, st->m,
                                                   noise ? noise->haar_scores : nullptr,
                                                   noise ? noise->haar_raw : nullptr, st->seed, base_id,
                                                   ws.q_prop);
  HZ_CUDA_TRY(cudaGetLastError());
  rc = eval(ws.q_prop);
  if (rc != HZ_OK) return rc;
  accept_kernel<<<warp_blocks, 128, 0, s>>>(dm, 1, st->q, st->log_p, st->drift, st->beta, st->sigma,
                                            st->mask, ws.q_prop, ws.la, ws.grad, nullptr, nullptr,
                                            noise ? noise->haar_logu : nullptr, st->seed, base_id,
                                            st->n_haar_accept, nullptr);
  HZ_CUDA_TRY(cudaGetLastError());
  for (int i = 0; i < n_steps; ++i) {
    const uint32_t id = base_id + 1u + (uint32_t)i;
    mala_propose_kernel<<<site_blocks, 256, 0, s>>>(
        dm, st->q, st->drift, st->beta, st->sigma, st->mask,
        noise && noise->local_noise ? noise->local_noise + (size_t)i * BRN * 3 : nullptr, st->seed, id,
        ws.q_prop, ws.xi, ws.mu);
    HZ_CUDA_TRY(cudaGetLastError());
    rc = eval(ws.q_prop);
    if (rc != HZ_OK) return rc;
    accept_kernel<<<warp_blocks, 128, 0, s>>>(
        dm, 0, st->q, st->log_p, st->drift, st->beta, st->sigma, st->mask, ws.q_prop, ws.la, ws.grad,
        ws.xi, ws.mu, noise && noise->local_logu ? noise->local_logu + (size_t)i * BR : nullptr,
        st->seed, id, st->n_local_accept, log_alpha_out ? log_alpha_out + (size_t)i * BR : nullptr);
    swap_kernel<<<(unsigned)B, 128, 0, s>>>(
        dm, st->q, st->log_p, st->drift, st->beta, st->step + i,
        noise && noise->swap_logu ? noise->swap_logu + (size_t)i * B * (R - 1) : nullptr, st->seed, id,
        st->n_swap_accept, st->n_swap);
    HZ_CUDA_TRY(cudaGetLastError());
  }
  return HZ_OK;
}
