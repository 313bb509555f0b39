// Masked multi-head softmax attention with additive edge bias: forward,
// forward-mode tangent and backward, for sm_100a.
//
// Semantics follow the reference's Pallas kernels
// (src/hamiltonzero/model/_pallas_attn/mhsea.py:13-31, mhsea_tuned_jvp.py:20-91,
// custom_gradients.py:231-347) and, in HZ_MASK_KEYS mode, its einsum twin
// (src/hamiltonzero/model/pallas_attention.py:22-37).
//
// Tiling: one CTA of 4 warps owns one (batch, head) pair and a block of 64
// query rows; each warp owns 16 of them. Keys are visited in chunks of 64 that
// are staged in shared memory, so for N <= 64 the whole sequence of a
// (batch, head) pair is on chip and every HBM byte is read exactly once.
// Contractions run on the tensor cores as 3xTF32 split products (hz_mma.cuh).
#include "hz_gemm_tc.cuh"
#include "hz_internal.h"
#include "hz_mma.cuh"

#include <math.h>
#include <stdlib.h>

#include <mutex>
#include <string.h>

namespace hz {
namespace {

constexpr int kThreads = 128;
constexpr int kTile = 64;        // query rows per CTA and keys per chunk
constexpr float kBigNegative = -10000.0f;   // utils.py:52-53
constexpr float kKeyMask = -1e9f;           // pallas_attention.py:33

struct AttnArgs {
  int B, N, H, mode;
  int D;               // head dimension (the fast path pads 8 and 16 to 32 on chip)
  const float* q;
  const float* k;
  const float* e;
  const float* v;
  const uint8_t* mask;
  // forward
  float* out;
  float* lse;
  // tangent
  const float* out_in;
  const float* lse_in;
  const float* qt;
  const float* kt;
  const float* et;
  const float* vt;
  float* tangent;
  // backward
  const float* dout;
  float* dq;
  float* dk;
  float* de;
  float* dv;
};

__device__ __forceinline__ float4 ldg4(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}

// Stage `rows` rows (global row index row0 + r, zero beyond N or where the row
// is masked out) of a [B,N,H,D] tensor's (b,h) slice into shared memory with
// leading dimension D+4.
template <int D>
__device__ __forceinline__ void stage_rows(float* dst, const float* src, size_t base,
                                           size_t rowstride, int row0, int N,
                                           const uint8_t* keep) {
  constexpr int LD = D + 4;
  constexpr int C4 = D / 4;
  for (int idx = threadIdx.x; idx < kTile * C4; idx += kThreads) {
    const int r = idx / C4;
    const int c = (idx % C4) * 4;
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    const int row = row0 + r;
    if (row < N && keep[r]) val = ldg4(src + base + (size_t)row * rowstride + c);
    *reinterpret_cast<float4*>(dst + r * LD + c) = val;
  }
}

// keep flags for 64 rows starting at row0: 1 = load the row, 0 = zero it.
__device__ __forceinline__ void stage_mask(uint8_t* real, uint8_t* keep, const uint8_t* mask,
                                           int b, int row0, int N, int mode) {
  for (int r = threadIdx.x; r < kTile; r += kThreads) {
    const int row = row0 + r;
    uint8_t m = 0;
    if (row < N) m = mask ? (mask[(size_t)b * N + row] != 0) : 1;
    real[r] = m;
    keep[r] = (mode == HZ_MASK_SQUARE) ? m : (row < N ? 1 : 0);
  }
}

// score post-processing shared by the three kernels
__device__ __forceinline__ float finish_score(float s, bool row_ok, bool key_real, bool key_in,
                                              int mode) {
  if (!key_in) return -INFINITY;
  if (mode == HZ_MASK_SQUARE) return (row_ok && key_real) ? s : kBigNegative;
  return key_real ? s : s + kKeyMask;
}

// ------------------------------------------------------------------ forward
template <int D>
__global__ void __launch_bounds__(kThreads) attn_fwd_kernel(AttnArgs a) {
  constexpr int LD = D + 4;
  constexpr int ND = D / 8;
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;
  float* Ks = Qs + kTile * LD;
  float* Vs = Ks + kTile * LD;
  uint8_t* q_real = reinterpret_cast<uint8_t*>(Vs + kTile * LD);
  uint8_t* q_keep = q_real + kTile;
  uint8_t* k_real = q_keep + kTile;
  uint8_t* k_keep = k_real + kTile;

  const int N = a.N, H = a.H, mode = a.mode;
  const int qblocks = (N + kTile - 1) / kTile;
  const int bh = blockIdx.x / qblocks;
  const int qb = blockIdx.x % qblocks;
  const int b = bh / H, h = bh % H;
  const size_t base = ((size_t)b * N * H + h) * D;
  const size_t rowstride = (size_t)H * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int q0 = qb * kTile;

  stage_mask(q_real, q_keep, a.mask, b, q0, N, mode);
  __syncthreads();
  stage_rows<D>(Qs, a.q, base, rowstride, q0, N, q_keep);

  const int lr0 = warp * 16 + g, lr1 = lr0 + 8;   // local query rows of this lane
  const int row0 = q0 + lr0, row1 = q0 + lr1;
  const bool warp_active = (q0 + warp * 16) < N;

  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float acc[ND][4];
#pragma unroll
  for (int i = 0; i < ND; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;

  for (int kc = 0; kc < N; kc += kTile) {
    __syncthreads();   // previous chunk fully consumed
    stage_mask(k_real, k_keep, a.mask, b, kc, N, mode);
    __syncthreads();
    stage_rows<D>(Ks, a.k, base, rowstride, kc, N, k_keep);
    stage_rows<D>(Vs, a.v, base, rowstride, kc, N, k_keep);
    __syncthreads();
    if (!warp_active) continue;
    const int nkt = min(8, (N - kc + 7) >> 3);

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[i][c] = 0.f;

#pragma unroll
    for (int ks = 0; ks < ND; ++ks) {
      FragA fa;
      fa.set(Qs[lr0 * LD + ks * 8 + t], Qs[lr1 * LD + ks * 8 + t],
             Qs[lr0 * LD + ks * 8 + t + 4], Qs[lr1 * LD + ks * 8 + t + 4]);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (nt < nkt) {
          FragB fb;
          fb.set(Ks[(nt * 8 + g) * LD + ks * 8 + t], Ks[(nt * 8 + g) * LD + ks * 8 + t + 4]);
          mma3(s[nt], fa, fb);
        }
      }
    }

    const bool rok0 = q_real[lr0] != 0, rok1 = q_real[lr1] != 0;
    float cmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int lk = nt * 8 + 2 * t + (c & 1);
        const int key = kc + lk;
        const int row = (c < 2) ? row0 : row1;
        float val = s[nt][c];
        const bool key_in = (nt < nkt) && key < N;
        if (a.e != nullptr && key_in && row < N)
          val += __ldg(a.e + (((size_t)b * N + row) * H + h) * N + key);
        val = finish_score(val, (c < 2) ? rok0 : rok1, key_in && k_real[lk], key_in, mode);
        s[nt][c] = val;
        cmax[c >> 1] = fmaxf(cmax[c >> 1], val);
      }
    }
    float scale[2], m_new[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      cmax[r] = quad_max(cmax[r]);
      m_new[r] = fmaxf(m_run[r], cmax[r]);
      scale[r] = __expf(m_run[r] - m_new[r]);
      m_run[r] = m_new[r];
    }
    float csum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = __expf(s[nt][c] - m_new[c >> 1]);
        s[nt][c] = p;
        csum[c >> 1] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * scale[r] + quad_sum(csum[r]);
#pragma unroll
    for (int nd = 0; nd < ND; ++nd) {
      acc[nd][0] *= scale[0];
      acc[nd][1] *= scale[0];
      acc[nd][2] *= scale[1];
      acc[nd][3] *= scale[1];
    }
    // O += P V. The k-slots of the A fragment are mapped to keys (2t, 2t+1) so
    // that the score accumulators can be used as the A operand without shuffles.
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      if (kk < nkt) {
        FragA fa;
        fa.set(s[kk][0], s[kk][2], s[kk][1], s[kk][3]);
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) {
          FragB fb;
          fb.set(Vs[(kk * 8 + 2 * t) * LD + nd * 8 + g], Vs[(kk * 8 + 2 * t + 1) * LD + nd * 8 + g]);
          mma3(acc[nd], fa, fb);
        }
      }
    }
  }

  if (!warp_active) return;
  const bool zero0 = (mode == HZ_MASK_SQUARE) && !q_real[lr0];
  const bool zero1 = (mode == HZ_MASK_SQUARE) && !q_real[lr1];
  const float inv0 = 1.f / l_run[0], inv1 = 1.f / l_run[1];
#pragma unroll
  for (int nd = 0; nd < ND; ++nd) {
    const int col = nd * 8 + 2 * t;
    if (row0 < N) {
      float2 o = zero0 ? make_float2(0.f, 0.f) : make_float2(acc[nd][0] * inv0, acc[nd][1] * inv0);
      *reinterpret_cast<float2*>(a.out + base + (size_t)row0 * rowstride + col) = o;
    }
    if (row1 < N) {
      float2 o = zero1 ? make_float2(0.f, 0.f) : make_float2(acc[nd][2] * inv1, acc[nd][3] * inv1);
      *reinterpret_cast<float2*>(a.out + base + (size_t)row1 * rowstride + col) = o;
    }
  }
  if (t == 0) {
    if (row0 < N) a.lse[((size_t)b * N + row0) * H + h] = m_run[0] + logf(l_run[0]);
    if (row1 < N) a.lse[((size_t)b * N + row1) * H + h] = m_run[1] + logf(l_run[1]);
  }
}

// ------------------------------------------------------------------ tangent
template <int D>
__global__ void __launch_bounds__(kThreads) attn_jvp_kernel(AttnArgs a) {
  constexpr int LD = D + 4;
  constexpr int ND = D / 8;
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;
  float* Qts = Qs + kTile * LD;
  float* Ks = Qts + kTile * LD;
  float* Kts = Ks + kTile * LD;
  float* Vs = Kts + kTile * LD;
  float* Vts = Vs + kTile * LD;
  uint8_t* q_real = reinterpret_cast<uint8_t*>(Vts + kTile * LD);
  uint8_t* q_keep = q_real + kTile;
  uint8_t* k_real = q_keep + kTile;
  uint8_t* k_keep = k_real + kTile;

  const int N = a.N, H = a.H, mode = a.mode;
  const int qblocks = (N + kTile - 1) / kTile;
  const int bh = blockIdx.x / qblocks;
  const int qb = blockIdx.x % qblocks;
  const int b = bh / H, h = bh % H;
  const size_t base = ((size_t)b * N * H + h) * D;
  const size_t rowstride = (size_t)H * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int q0 = qb * kTile;

  stage_mask(q_real, q_keep, a.mask, b, q0, N, mode);
  __syncthreads();
  stage_rows<D>(Qs, a.q, base, rowstride, q0, N, q_keep);
  stage_rows<D>(Qts, a.qt, base, rowstride, q0, N, q_keep);

  const int lr0 = warp * 16 + g, lr1 = lr0 + 8;
  const int row0 = q0 + lr0, row1 = q0 + lr1;
  const bool warp_active = (q0 + warp * 16) < N;

  float lse_r[2] = {0.f, 0.f};
  if (row0 < N) lse_r[0] = __ldg(a.lse_in + ((size_t)b * N + row0) * H + h);
  if (row1 < N) lse_r[1] = __ldg(a.lse_in + ((size_t)b * N + row1) * H + h);

  float mean[2] = {0.f, 0.f};
  float accA[ND][4], accB[ND][4];
#pragma unroll
  for (int i = 0; i < ND; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) accA[i][c] = accB[i][c] = 0.f;

  for (int kc = 0; kc < N; kc += kTile) {
    __syncthreads();
    stage_mask(k_real, k_keep, a.mask, b, kc, N, mode);
    __syncthreads();
    stage_rows<D>(Ks, a.k, base, rowstride, kc, N, k_keep);
    stage_rows<D>(Kts, a.kt, base, rowstride, kc, N, k_keep);
    stage_rows<D>(Vs, a.v, base, rowstride, kc, N, k_keep);
    stage_rows<D>(Vts, a.vt, base, rowstride, kc, N, k_keep);
    __syncthreads();
    if (!warp_active) continue;
    const int nkt = min(8, (N - kc + 7) >> 3);

    float s[8][4], sd[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[i][c] = sd[i][c] = 0.f;

#pragma unroll
    for (int ks = 0; ks < ND; ++ks) {
      FragA fq, fqt;
      fq.set(Qs[lr0 * LD + ks * 8 + t], Qs[lr1 * LD + ks * 8 + t],
             Qs[lr0 * LD + ks * 8 + t + 4], Qs[lr1 * LD + ks * 8 + t + 4]);
      fqt.set(Qts[lr0 * LD + ks * 8 + t], Qts[lr1 * LD + ks * 8 + t],
              Qts[lr0 * LD + ks * 8 + t + 4], Qts[lr1 * LD + ks * 8 + t + 4]);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (nt < nkt) {
          FragB fk, fkt;
          fk.set(Ks[(nt * 8 + g) * LD + ks * 8 + t], Ks[(nt * 8 + g) * LD + ks * 8 + t + 4]);
          fkt.set(Kts[(nt * 8 + g) * LD + ks * 8 + t], Kts[(nt * 8 + g) * LD + ks * 8 + t + 4]);
          mma3(s[nt], fq, fk);
          mma3(sd[nt], fqt, fk);
          mma3(sd[nt], fq, fkt);
        }
      }
    }

    const bool rok0 = q_real[lr0] != 0, rok1 = q_real[lr1] != 0;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int lk = nt * 8 + 2 * t + (c & 1);
        const int key = kc + lk;
        const int row = (c < 2) ? row0 : row1;
        const bool rok = (c < 2) ? rok0 : rok1;
        const bool key_in = (nt < nkt) && key < N;
        const bool key_real = key_in && k_real[lk];
        float val = s[nt][c];
        float dval = sd[nt][c];
        if (key_in && row < N) {
          const size_t eoff = (((size_t)b * N + row) * H + h) * N + key;
          if (a.e != nullptr) val += __ldg(a.e + eoff);
          if (a.et != nullptr) dval += __ldg(a.et + eoff);
        }
        val = finish_score(val, rok, key_real, key_in, mode);
        const float p = (row < N) ? __expf(val - lse_r[c >> 1]) : 0.f;
        // tangent of the score: zero wherever the score is the masked constant
        const bool live = key_in && (mode == HZ_MASK_SQUARE ? (rok && key_real) : true);
        const float psd = live ? p * dval : 0.f;
        s[nt][c] = p;
        sd[nt][c] = psd;
        mean[c >> 1] += psd;
      }
    }
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      if (kk < nkt) {
        FragA fp, fpsd;
        fp.set(s[kk][0], s[kk][2], s[kk][1], s[kk][3]);
        fpsd.set(sd[kk][0], sd[kk][2], sd[kk][1], sd[kk][3]);
#pragma unroll
        for (int nd = 0; nd < ND; ++nd) {
          FragB fv, fvt;
          fv.set(Vs[(kk * 8 + 2 * t) * LD + nd * 8 + g], Vs[(kk * 8 + 2 * t + 1) * LD + nd * 8 + g]);
          fvt.set(Vts[(kk * 8 + 2 * t) * LD + nd * 8 + g], Vts[(kk * 8 + 2 * t + 1) * LD + nd * 8 + g]);
          mma3(accA[nd], fpsd, fv);
          mma3(accB[nd], fp, fvt);
        }
      }
    }
  }

  if (!warp_active) return;
  mean[0] = quad_sum(mean[0]);
  mean[1] = quad_sum(mean[1]);
  const bool zero0 = (mode == HZ_MASK_SQUARE) && !q_real[lr0];
  const bool zero1 = (mode == HZ_MASK_SQUARE) && !q_real[lr1];
#pragma unroll
  for (int nd = 0; nd < ND; ++nd) {
    const int col = nd * 8 + 2 * t;
    if (row0 < N) {
      const size_t off = base + (size_t)row0 * rowstride + col;
      const float2 o = __ldg(reinterpret_cast<const float2*>(a.out_in + off));
      float2 r = make_float2(accA[nd][0] + accB[nd][0] - mean[0] * o.x,
                             accA[nd][1] + accB[nd][1] - mean[0] * o.y);
      if (zero0) r = make_float2(0.f, 0.f);
      *reinterpret_cast<float2*>(a.tangent + off) = r;
    }
    if (row1 < N) {
      const size_t off = base + (size_t)row1 * rowstride + col;
      const float2 o = __ldg(reinterpret_cast<const float2*>(a.out_in + off));
      float2 r = make_float2(accA[nd][2] + accB[nd][2] - mean[1] * o.x,
                             accA[nd][3] + accB[nd][3] - mean[1] * o.y);
      if (zero1) r = make_float2(0.f, 0.f);
      *reinterpret_cast<float2*>(a.tangent + off) = r;
    }
  }
}

// ------------------------------------------------------------------ backward
// One CTA per (batch, head). Outer loop over key blocks (dK, dV of the block in
// registers), inner loop over query blocks. P and dS of a 64x64 tile go through
// shared memory once so that the same tile feeds dQ (row-major use) and dK, dV
// (transposed use) without recomputing the scores.
constexpr int kPLD = kTile + 4;   // leading dimension of the P / dS tiles

template <int D, bool SINGLE>
__global__ void __launch_bounds__(kThreads) attn_bwd_kernel(AttnArgs a) {
  constexpr int LD = D + 4;
  constexpr int ND = D / 8;
  extern __shared__ __align__(16) float smem[];
  const int N = a.N, H = a.H, mode = a.mode;
  const int Np = (N + kTile - 1) / kTile * kTile;
  float* Qs = smem;
  float* dOs = Qs + kTile * LD;
  float* Ks = dOs + kTile * LD;
  float* Vs = Ks + kTile * LD;
  float* Ps = Vs + kTile * LD;
  float* dSs = Ps + kTile * kPLD;
  float* lse_s = dSs + kTile * kPLD;     // [Np]
  float* delta_s = lse_s + Np;           // [Np]
  float* dQs = delta_s + Np;             // [Np][LD] unless SINGLE
  uint8_t* q_real = reinterpret_cast<uint8_t*>(dQs + (SINGLE ? 0 : Np * LD));
  uint8_t* q_keep = q_real + kTile;
  uint8_t* k_real = q_keep + kTile;
  uint8_t* k_keep = k_real + kTile;

  const int b = blockIdx.x / H, h = blockIdx.x % H;
  const size_t base = ((size_t)b * N * H + h) * D;
  const size_t rowstride = (size_t)H * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int lr0 = warp * 16 + g, lr1 = lr0 + 8;

  for (int r = threadIdx.x; r < Np; r += kThreads)
    lse_s[r] = (r < N) ? __ldg(a.lse_in + ((size_t)b * N + r) * H + h) : 0.f;
  if (!SINGLE)
    for (int i = threadIdx.x; i < Np * LD; i += kThreads) dQs[i] = 0.f;

  float dq_acc[ND][4];
#pragma unroll
  for (int i = 0; i < ND; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) dq_acc[i][c] = 0.f;

  for (int kc = 0; kc < N; kc += kTile) {
    __syncthreads();
    stage_mask(k_real, k_keep, a.mask, b, kc, N, mode);
    __syncthreads();
    stage_rows<D>(Ks, a.k, base, rowstride, kc, N, k_keep);
    stage_rows<D>(Vs, a.v, base, rowstride, kc, N, k_keep);
    const int nkt = min(8, (N - kc + 7) >> 3);
    const bool kwarp_active = (kc + warp * 16) < N;

    float dk_acc[ND][4], dv_acc[ND][4];
#pragma unroll
    for (int i = 0; i < ND; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) dk_acc[i][c] = dv_acc[i][c] = 0.f;

    for (int q0 = 0; q0 < N; q0 += kTile) {
      __syncthreads();   // previous tile's Qs/dOs/Ps/dSs fully consumed
      stage_mask(q_real, q_keep, a.mask, b, q0, N, mode);
      __syncthreads();
      stage_rows<D>(Qs, a.q, base, rowstride, q0, N, q_keep);
      // dO rows (masked like q) and, on the first key block, delta = sum_d O*dO
      {
        constexpr int C4 = D / 4;
        for (int idx = threadIdx.x; idx < kTile * C4; idx += kThreads) {
          const int r = idx / C4;
          const int c = (idx % C4) * 4;
          const int row = q0 + r;
          float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
          float part = 0.f;
          if (row < N && q_keep[r]) {
            val = ldg4(a.dout + base + (size_t)row * rowstride + c);
            if (kc == 0) {
              const float4 o = ldg4(a.out_in + base + (size_t)row * rowstride + c);
              part = o.x * val.x + o.y * val.y + o.z * val.z + o.w * val.w;
            }
          }
          *reinterpret_cast<float4*>(dOs + r * LD + c) = val;
          if (kc == 0) {
#pragma unroll
            for (int off = C4 / 2; off > 0; off >>= 1)
              part += __shfl_xor_sync(0xffffffffu, part, off);
            if ((idx % C4) == 0) delta_s[row] = part;
          }
        }
      }
      __syncthreads();

      const int row0 = q0 + lr0, row1 = q0 + lr1;
      const bool qwarp_active = (q0 + warp * 16) < N;
      if (qwarp_active) {
        float s[8][4], dp[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) s[i][c] = dp[i][c] = 0.f;
#pragma unroll
        for (int ks = 0; ks < ND; ++ks) {
          FragA fq, fdo;
          fq.set(Qs[lr0 * LD + ks * 8 + t], Qs[lr1 * LD + ks * 8 + t],
                 Qs[lr0 * LD + ks * 8 + t + 4], Qs[lr1 * LD + ks * 8 + t + 4]);
          fdo.set(dOs[lr0 * LD + ks * 8 + t], dOs[lr1 * LD + ks * 8 + t],
                  dOs[lr0 * LD + ks * 8 + t + 4], dOs[lr1 * LD + ks * 8 + t + 4]);
#pragma unroll
          for (int nt = 0; nt < 8; ++nt) {
            if (nt < nkt) {
              FragB fk, fv;
              fk.set(Ks[(nt * 8 + g) * LD + ks * 8 + t], Ks[(nt * 8 + g) * LD + ks * 8 + t + 4]);
              fv.set(Vs[(nt * 8 + g) * LD + ks * 8 + t], Vs[(nt * 8 + g) * LD + ks * 8 + t + 4]);
              mma3(s[nt], fq, fk);
              mma3(dp[nt], fdo, fv);
            }
          }
        }
        const bool rok0 = q_real[lr0] != 0, rok1 = q_real[lr1] != 0;
        const float lse0 = lse_s[q0 + lr0], lse1 = lse_s[q0 + lr1];
        const float del0 = delta_s[q0 + lr0], del1 = delta_s[q0 + lr1];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int lk = nt * 8 + 2 * t + (c & 1);
            const int key = kc + lk;
            const int row = (c < 2) ? row0 : row1;
            const bool rok = (c < 2) ? rok0 : rok1;
            const bool key_in = (nt < nkt) && key < N;
            const bool key_real = key_in && k_real[lk];
            float val = s[nt][c];
            if (a.e != nullptr && key_in && row < N)
              val += __ldg(a.e + (((size_t)b * N + row) * H + h) * N + key);
            val = finish_score(val, rok, key_real, key_in, mode);
            const float p = (row < N) ? __expf(val - ((c < 2) ? lse0 : lse1)) : 0.f;
            const bool live = key_in && row < N &&
                              (mode == HZ_MASK_SQUARE ? (rok && key_real) : true);
            const float ds = live ? (dp[nt][c] - ((c < 2) ? del0 : del1)) * p : 0.f;
            s[nt][c] = p;
            dp[nt][c] = ds;
          }
          const int lk0 = nt * 8 + 2 * t;
          *reinterpret_cast<float2*>(Ps + lr0 * kPLD + lk0) = make_float2(s[nt][0], s[nt][1]);
          *reinterpret_cast<float2*>(Ps + lr1 * kPLD + lk0) = make_float2(s[nt][2], s[nt][3]);
          *reinterpret_cast<float2*>(dSs + lr0 * kPLD + lk0) = make_float2(dp[nt][0], dp[nt][1]);
          *reinterpret_cast<float2*>(dSs + lr1 * kPLD + lk0) = make_float2(dp[nt][2], dp[nt][3]);
          if (a.de != nullptr && nt < nkt) {
            const int key = kc + lk0;
            if (row0 < N) {
              float* dst = a.de + (((size_t)b * N + row0) * H + h) * N + key;
              if (key < N) dst[0] = dp[nt][0];
              if (key + 1 < N) dst[1] = dp[nt][1];
            }
            if (row1 < N) {
              float* dst = a.de + (((size_t)b * N + row1) * H + h) * N + key;
              if (key < N) dst[0] = dp[nt][2];
              if (key + 1 < N) dst[1] = dp[nt][3];
            }
          }
        }
        // dQ += dS K
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          if (kk < nkt) {
            FragA fds;
            fds.set(dp[kk][0], dp[kk][2], dp[kk][1], dp[kk][3]);
#pragma unroll
            for (int nd = 0; nd < ND; ++nd) {
              FragB fk;
              fk.set(Ks[(kk * 8 + 2 * t) * LD + nd * 8 + g],
                     Ks[(kk * 8 + 2 * t + 1) * LD + nd * 8 + g]);
              mma3(dq_acc[nd], fds, fk);
            }
          }
        }
        if (!SINGLE) {
#pragma unroll
          for (int nd = 0; nd < ND; ++nd) {
            float* d0 = dQs + (q0 + lr0) * LD + nd * 8 + 2 * t;
            float* d1 = dQs + (q0 + lr1) * LD + nd * 8 + 2 * t;
            d0[0] += dq_acc[nd][0];
            d0[1] += dq_acc[nd][1];
            d1[0] += dq_acc[nd][2];
            d1[1] += dq_acc[nd][3];
#pragma unroll
            for (int c = 0; c < 4; ++c) dq_acc[nd][c] = 0.f;
          }
        }
      } else {
        // rows beyond N in this tile contribute nothing: publish zeros
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const int lk0 = nt * 8 + 2 * t;
          const float2 z = make_float2(0.f, 0.f);
          *reinterpret_cast<float2*>(Ps + lr0 * kPLD + lk0) = z;
          *reinterpret_cast<float2*>(Ps + lr1 * kPLD + lk0) = z;
          *reinterpret_cast<float2*>(dSs + lr0 * kPLD + lk0) = z;
          *reinterpret_cast<float2*>(dSs + lr1 * kPLD + lk0) = z;
        }
      }
      __syncthreads();

      // dV += P^T dO, dK += dS^T Q for the 16 keys owned by this warp. The
      // contraction index (query) uses slots (2t, 2t+1), consistently in A and B.
      if (kwarp_active) {
        const int nqt = min(8, (N - q0 + 7) >> 3);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          if (ks < nqt) {
            const int qa = ks * 8 + 2 * t, qb2 = qa + 1;
            FragA fp, fds;
            fp.set(Ps[qa * kPLD + lr0], Ps[qa * kPLD + lr1], Ps[qb2 * kPLD + lr0],
                   Ps[qb2 * kPLD + lr1]);
            fds.set(dSs[qa * kPLD + lr0], dSs[qa * kPLD + lr1], dSs[qb2 * kPLD + lr0],
                    dSs[qb2 * kPLD + lr1]);
#pragma unroll
            for (int nd = 0; nd < ND; ++nd) {
              FragB fdo, fq;
              fdo.set(dOs[qa * LD + nd * 8 + g], dOs[qb2 * LD + nd * 8 + g]);
              fq.set(Qs[qa * LD + nd * 8 + g], Qs[qb2 * LD + nd * 8 + g]);
              mma3(dv_acc[nd], fp, fdo);
              mma3(dk_acc[nd], fds, fq);
            }
          }
        }
      }
    }  // query blocks

    if (kwarp_active) {
      const int key0 = kc + lr0, key1 = kc + lr1;
#pragma unroll
      for (int nd = 0; nd < ND; ++nd) {
        const int col = nd * 8 + 2 * t;
        if (key0 < N) {
          const size_t off = base + (size_t)key0 * rowstride + col;
          *reinterpret_cast<float2*>(a.dk + off) = make_float2(dk_acc[nd][0], dk_acc[nd][1]);
          *reinterpret_cast<float2*>(a.dv + off) = make_float2(dv_acc[nd][0], dv_acc[nd][1]);
        }
        if (key1 < N) {
          const size_t off = base + (size_t)key1 * rowstride + col;
          *reinterpret_cast<float2*>(a.dk + off) = make_float2(dk_acc[nd][2], dk_acc[nd][3]);
          *reinterpret_cast<float2*>(a.dv + off) = make_float2(dv_acc[nd][2], dv_acc[nd][3]);
        }
      }
    }
  }  // key blocks

  if (SINGLE) {
    const int row0 = lr0, row1 = lr1;
#pragma unroll
    for (int nd = 0; nd < ND; ++nd) {
      const int col = nd * 8 + 2 * t;
      if (row0 < N)
        *reinterpret_cast<float2*>(a.dq + base + (size_t)row0 * rowstride + col) =
            make_float2(dq_acc[nd][0], dq_acc[nd][1]);
      if (row1 < N)
        *reinterpret_cast<float2*>(a.dq + base + (size_t)row1 * rowstride + col) =
            make_float2(dq_acc[nd][2], dq_acc[nd][3]);
    }
  } else {
    __syncthreads();
    constexpr int C4 = D / 4;
    for (int idx = threadIdx.x; idx < N * C4; idx += kThreads) {
      const int r = idx / C4, c = (idx % C4) * 4;
      *reinterpret_cast<float4*>(a.dq + base + (size_t)r * rowstride + c) =
          *reinterpret_cast<const float4*>(dQs + r * LD + c);
    }
  }
}

#include "hz_attn_fast.cuh"
#include "hz_attn_tc.cuh"

// ------------------------------------------------------------------ host side
int persistent_grid(int tiles, int ctas_per_sm) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int cap = sms * ctas_per_sm;
  return tiles < cap ? tiles : cap;
}

// Error word of the tcgen05 kernel's bounded waits, one per device (the attention entry points
// have no workspace to put it in). It is cleared before every launch of that kernel; when a wait
// ran out, attn_tc_poison_kernel overwrites the call's outputs with NaN, so that a timeout can
// never pass as a result.
__device__ int g_attn_tc_status;

int attn_tc_status_word(int** out) {
  static std::mutex mu;
  static int* cached[kMaxDevicesTracked] = {nullptr};
  int dev = 0;
  HZ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevicesTracked) return HZ_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    HZ_CUDA_TRY(cudaGetSymbolAddress(&p, g_attn_tc_status));
    cached[dev] = static_cast<int*>(p);
  }
  *out = cached[dev];
  return HZ_OK;
}

__global__ void attn_tc_poison_kernel(const int* __restrict__ status, float* __restrict__ out,
                                      long long n_out, float* __restrict__ lse, long long n_lse) {
  if (*status == 0) return;
  const float bad = __int_as_float(0x7fc00000);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_out;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = bad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_lse;
       i += (long long)gridDim.x * blockDim.x)
    lse[i] = bad;
}

// The tcgen05 forward kernel is opt-in: flag HZ_ATTN_TCGEN05 in mask_mode, or HZ_ATTN_FWD=tc for
// every call of the process.
bool use_attn_tc() {
  static const bool on = env_equals("HZ_ATTN_FWD", "tc");
  return on;
}

// Arithmetic of the fast path's contractions, from the flags in mask_mode. Without a flag the
// contractions run on the two-term BF16 split (three BF16 products per fp32 product): it has the
// range of fp32, keeps every output within 1e-4 of its scale (about 1e-5 on operands of order
// one), and lets the three passes run at the HBM rate. HZ_ATTN_TF32X3 asks for the three-term
// TF32 split (fp32-faithful to about 1e-6, half the tensor rate). HZ_ATTN=tf32x3, bf16x3, fp16x3 or
// tf32 in the environment sets the arithmetic of calls that carry no flag.
int attn_arith(int mask_mode) {
  if (mask_mode & HZ_ATTN_TF32) return kArTf32;
  if (mask_mode & (HZ_ATTN_TF32X3 | HZ_ATTN_TCGEN05)) return kArTf32x3;
  if (mask_mode & HZ_ATTN_BF16X3) return kArBf16x3;
  if (mask_mode & HZ_ATTN_FP16X3) return kArFp16x3;
  static const int env = env_equals("HZ_ATTN", "tf32x3")   ? kArTf32x3
                         : env_equals("HZ_ATTN", "fp16x3") ? kArFp16x3
                         : env_equals("HZ_ATTN", "tf32")   ? kArTf32
                                                           : kArBf16x3;
  return env;
}

// N = 64 with D = 32, or D = 8 / 16 (zero-padded to 32 columns in shared memory: the loads and
// stores move the real bytes, the contractions run over 32 columns; HZ_ATTN_PAD=off sends
// those head dimensions to the generic kernels)
bool fast_shape(const hz_attn_shape* s) {
  static const bool pad = !env_equals("HZ_ATTN_PAD", "off");
  const bool d_ok = s->D == kFD || (pad && (s->D == 8 || s->D == 16));
  return s->N == kFN && d_ok && (s->mask_mode & 0xff) == HZ_MASK_SQUARE;
}

int check_shape(const hz_attn_shape* s) {
  if (s == nullptr) return HZ_ERR_NULL_POINTER;
  if (s->B <= 0 || s->N <= 0 || s->H <= 0 || s->D <= 0) return HZ_ERR_BAD_SHAPE;
  const int mm = s->mask_mode & ~(HZ_ATTN_TF32 | HZ_ATTN_TCGEN05 | HZ_ATTN_BF16X3 | HZ_ATTN_FP16X3 |
                                  HZ_ATTN_TF32X3);
  if (mm != HZ_MASK_SQUARE && mm != HZ_MASK_KEYS) return HZ_ERR_BAD_SHAPE;
  if (s->N > 256) return HZ_ERR_UNSUPPORTED;
  if (!(s->D == 8 || s->D == 16 || s->D == 32 || s->D == 64)) return HZ_ERR_UNSUPPORTED;
  const long long ctas = (long long)s->B * s->H * ((s->N + kTile - 1) / kTile);
  if (ctas > 0x7fffffffLL) return HZ_ERR_UNSUPPORTED;
  return HZ_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename K>
int launch(K kernel, int grid, size_t smem, const AttnArgs& args, cudaStream_t stream) {
  // several CTAs per SM hide the staging latency: ask for the largest shared-memory carve-out
  const int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(kernel), (int)smem, true);
  if (rc != HZ_OK) return rc;
  kernel<<<grid, kThreads, smem, stream>>>(args);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

}  // namespace
}  // namespace hz

using namespace hz;

extern "C" int hz_mhsea_fwd(const hz_attn_shape* shape, const float* q, const float* k,
                            const float* e, const float* v, const uint8_t* mask, float* out,
                            float* lse, void* stream) {
  int st = check_shape(shape);
  if (st != HZ_OK) return st;
  if (!q || !k || !v || !out || !lse) return HZ_ERR_NULL_POINTER;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) ||
      (e && !aligned16(e)))
    return HZ_ERR_MISALIGNED;
  AttnArgs a{};
  a.B = shape->B; a.N = shape->N; a.H = shape->H; a.mode = shape->mask_mode & 0xff;
  a.D = shape->D;
  const int ar = attn_arith(shape->mask_mode);
  a.q = q; a.k = k; a.e = e; a.v = v; a.mask = mask; a.out = out; a.lse = lse;
  const int grid = shape->B * shape->H * ((shape->N + kTile - 1) / kTile);
  const int D = shape->D;
  const size_t smem = (size_t)3 * kTile * (D + 4) * sizeof(float) + 4 * kTile;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (fast_shape(shape) && shape->D == kFD && ar == kArTf32x3 && (use_attn_tc() || (shape->mask_mode & HZ_ATTN_TCGEN05)) &&
      shape->H % 2 == 0 && encode_tiled_fn() != nullptr &&
      aligned16(out)) {
    int* status = nullptr;
    st = attn_tc_status_word(&status);
    if (st != HZ_OK) return st;
    AttnTcMaps maps;
    if (!make_attn_map(&maps.q, q, shape->B, kFN, shape->H, kFD, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_attn_map(&maps.k, k, shape->B, kFN, shape->H, kFD, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_attn_map(&maps.v, v, shape->B, kFN, shape->H, kFD, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
      return HZ_ERR_CUDA;
    const int items = shape->B * (shape->H / 2);
    const int sms = tc_sm_count();
    const int tgrid = items < sms ? items : sms;
    constexpr size_t tsm = (size_t)2 * kAtBuf + 1024;
#define HZ_FWD_TC(E, M)                                                                        \
  do {                                                                                         \
    st = ensure_kernel_attributes(reinterpret_cast<const void*>(attn_fwd_tc_kernel<E, M>),     \
                                  (int)tsm);                                                   \
    if (st != HZ_OK) return st;                                                                \
    attn_fwd_tc_kernel<E, M><<<tgrid, kAtThreads, tsm, s>>>(maps, a, items, status);           \
  } while (0)
    HZ_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), s));
    if (e && mask) HZ_FWD_TC(true, true);
    else if (e) HZ_FWD_TC(true, false);
    else if (mask) HZ_FWD_TC(false, true);
    else HZ_FWD_TC(false, false);
#undef HZ_FWD_TC
    HZ_CUDA_TRY(cudaGetLastError());
    const long long n_lse = (long long)shape->B * shape->N * shape->H;
    attn_tc_poison_kernel<<<148, 256, 0, s>>>(status, out, n_lse * shape->D, lse, n_lse);
    HZ_CUDA_TRY(cudaGetLastError());
    return HZ_OK;
  }
  if (fast_shape(shape)) {
    const int tiles = shape->B * shape->H;
    const size_t fsm = (size_t)2 * 3 * kFTile * sizeof(float) + 2 * kFN;
    const int fgrid = persistent_grid(tiles, 4);
    // two load stages and four CTAs per SM (measured faster), or (HZ_ATTN_FWD_STAGES=1) one
    // stage and five CTAs
    const size_t fsm1 = (size_t)3 * kFTile * sizeof(float) + 2 * kFN;
    const int fgrid1 = persistent_grid(tiles, 5);
    static const bool one_stage = env_int("HZ_ATTN_FWD_STAGES", 2) == 1;
#define HZ_FWD_FAST_XS(E, M, X, S)                                                             \
  do {                                                                                      \
    st = ensure_kernel_attributes(reinterpret_cast<const void*>(attn_fwd_fast<E, M, X, S>),    \
                                  (int)(S == 1 ? fsm1 : fsm), true);                        \
    if (st != HZ_OK) return st;                                                             \
    attn_fwd_fast<E, M, X, S><<<S == 1 ? fgrid1 : fgrid, 128, S == 1 ? fsm1 : fsm, s>>>(a, tiles); \
  } while (0)
#define HZ_FWD_FAST_X(E, M, X)                                                                 \
  do {                                                                                      \
    if (one_stage) HZ_FWD_FAST_XS(E, M, X, 1);                                              \
    else HZ_FWD_FAST_XS(E, M, X, 2);                                                        \
  } while (0)
#define HZ_FWD_FAST(E, M)                                                   \
  do {                                                                       \
    if (ar == kArTf32) HZ_FWD_FAST_X(E, M, kArTf32);                        \
    else if (ar == kArBf16x3) HZ_FWD_FAST_X(E, M, kArBf16x3);               \
    else if (ar == kArFp16x3) HZ_FWD_FAST_X(E, M, kArFp16x3);               \
    else HZ_FWD_FAST_X(E, M, kArTf32x3);                                    \
  } while (0)
    if (e && mask) HZ_FWD_FAST(true, true);
    else if (e) HZ_FWD_FAST(true, false);
    else if (mask) HZ_FWD_FAST(false, true);
    else HZ_FWD_FAST(false, false);
#undef HZ_FWD_FAST
#undef HZ_FWD_FAST_X
#undef HZ_FWD_FAST_XS
    HZ_CUDA_TRY(cudaGetLastError());
    return HZ_OK;
  }
  switch (D) {
    case 8:  return launch(attn_fwd_kernel<8>, grid, smem, a, s);
    case 16: return launch(attn_fwd_kernel<16>, grid, smem, a, s);
    case 32: return launch(attn_fwd_kernel<32>, grid, smem, a, s);
    default: return launch(attn_fwd_kernel<64>, grid, smem, a, s);
  }
}

extern "C" int hz_mhsea_jvp(const hz_attn_shape* shape, const float* q, const float* k,
                            const float* e, const float* v, const uint8_t* mask,
                            const float* out, const float* lse, const float* qt,
                            const float* kt, const float* et, const float* vt, float* tangent,
                            void* stream) {
  int st = check_shape(shape);
  if (st != HZ_OK) return st;
  if (!q || !k || !v || !out || !lse || !qt || !kt || !vt || !tangent)
    return HZ_ERR_NULL_POINTER;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(qt) ||
      !aligned16(kt) || !aligned16(vt) || !aligned16(tangent) || (e && !aligned16(e)) ||
      (et && !aligned16(et)))
    return HZ_ERR_MISALIGNED;
  AttnArgs a{};
  a.B = shape->B; a.N = shape->N; a.H = shape->H; a.mode = shape->mask_mode & 0xff;
  a.D = shape->D;
  const int ar = attn_arith(shape->mask_mode);
  a.q = q; a.k = k; a.e = e; a.v = v; a.mask = mask;
  a.out_in = out; a.lse_in = lse; a.qt = qt; a.kt = kt; a.et = et; a.vt = vt;
  a.tangent = tangent;
  const int grid = shape->B * shape->H * ((shape->N + kTile - 1) / kTile);
  const int D = shape->D;
  const size_t smem = (size_t)6 * kTile * (D + 4) * sizeof(float) + 4 * kTile;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (fast_shape(shape)) {
    const int tiles = shape->B * shape->H;
    const size_t fsm = (size_t)2 * 6 * kFTile * sizeof(float) + 2 * kFN;
    const int fgrid = persistent_grid(tiles, 2);
#define HZ_JVP_FAST_XS(E, M, X, S)                                                             \
  do {                                                                                      \
    st = ensure_kernel_attributes(reinterpret_cast<const void*>(attn_jvp_fast<E, M, X, S>),    \
                                  (int)(S == 1 ? fsm1 : fsm), true);                        \
    if (st != HZ_OK) return st;                                                             \
    attn_jvp_fast<E, M, X, S><<<S == 1 ? fgrid1 : fgrid, 128, S == 1 ? fsm1 : fsm, s>>>(a, tiles); \
  } while (0)
#define HZ_JVP_FAST_X(E, M, X)                                                                 \
  do {                                                                                      \
    if (one_stage) HZ_JVP_FAST_XS(E, M, X, 1);                                              \
    else HZ_JVP_FAST_XS(E, M, X, 2);                                                        \
  } while (0)
#define HZ_JVP_FAST(E, M)                                                   \
  do {                                                                       \
    if (ar == kArTf32) HZ_JVP_FAST_X(E, M, kArTf32);                        \
    else if (ar == kArBf16x3) HZ_JVP_FAST_X(E, M, kArBf16x3);               \
    else if (ar == kArFp16x3) HZ_JVP_FAST_X(E, M, kArFp16x3);               \
    else HZ_JVP_FAST_X(E, M, kArTf32x3);                                    \
  } while (0)
    // one load stage and three CTAs per SM, or (HZ_ATTN_JVP=2stage) two stages and two CTAs
    const size_t fsm1 = (size_t)6 * kFTile * sizeof(float) + 2 * kFN;
    const int fgrid1 = persistent_grid(tiles, 3);
    static const bool one_stage = !env_equals("HZ_ATTN_JVP", "2stage");
    const bool has_e = (e != nullptr) || (et != nullptr);
    if (has_e && mask) HZ_JVP_FAST(true, true);
    else if (has_e) HZ_JVP_FAST(true, false);
    else if (mask) HZ_JVP_FAST(false, true);
    else HZ_JVP_FAST(false, false);
#undef HZ_JVP_FAST
#undef HZ_JVP_FAST_X
#undef HZ_JVP_FAST_XS
    HZ_CUDA_TRY(cudaGetLastError());
    return HZ_OK;
  }
  switch (D) {
    case 8:  return launch(attn_jvp_kernel<8>, grid, smem, a, s);
    case 16: return launch(attn_jvp_kernel<16>, grid, smem, a, s);
    case 32: return launch(attn_jvp_kernel<32>, grid, smem, a, s);
    default: return launch(attn_jvp_kernel<64>, grid, smem, a, s);
  }
}

extern "C" int hz_mhsea_bwd(const hz_attn_shape* shape, const float* q, const float* k,
                            const float* e, const float* v, const uint8_t* mask,
                            const float* lse, const float* out, const float* dout, float* dq,
                            float* dk, float* de, float* dv, void* stream) {
  int st = check_shape(shape);
  if (st != HZ_OK) return st;
  if (!q || !k || !v || !out || !lse || !dout || !dq || !dk || !dv) return HZ_ERR_NULL_POINTER;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(dout) ||
      !aligned16(dq) || !aligned16(dk) || !aligned16(dv) || (e && !aligned16(e)) ||
      (de && !aligned16(de)))
    return HZ_ERR_MISALIGNED;
  AttnArgs a{};
  a.B = shape->B; a.N = shape->N; a.H = shape->H; a.mode = shape->mask_mode & 0xff;
  a.D = shape->D;
  const int ar = attn_arith(shape->mask_mode);
  a.q = q; a.k = k; a.e = e; a.v = v; a.mask = mask;
  a.out_in = out; a.lse_in = lse; a.dout = dout;
  a.dq = dq; a.dk = dk; a.de = de; a.dv = dv;
  const int grid = shape->B * shape->H;
  const int D = shape->D, N = shape->N;
  const bool single = N <= kTile;
  const int Np = (N + kTile - 1) / kTile * kTile;
  const size_t smem = ((size_t)4 * kTile * (D + 4) + 2 * kTile * kPLD + 2 * Np +
                       (single ? 0 : (size_t)Np * (D + 4))) * sizeof(float) + 4 * kTile;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (fast_shape(shape)) {
    const int tiles = shape->B * shape->H;
    const size_t fsm = (size_t)(2 * 4 * kFTile + 2 * 64 * 64) * sizeof(float) + 2 * kFN;
    const int fgrid = persistent_grid(tiles, 2);
#define HZ_BWD_FAST_XS(E, M, W, X, S)                                                          \
  do {                                                                                      \
    st = ensure_kernel_attributes(reinterpret_cast<const void*>(attn_bwd_fast<E, M, W, X, S>), \
                                  (int)(S == 1 ? fsm1 : fsm), true);                        \
    if (st != HZ_OK) return st;                                                             \
    attn_bwd_fast<E, M, W, X, S><<<S == 1 ? fgrid1 : fgrid, 128, S == 1 ? fsm1 : fsm, s>>>(a, tiles); \
  } while (0)
#define HZ_BWD_FAST_X(E, M, W, X)                                                              \
  do {                                                                                      \
    if (one_stage) HZ_BWD_FAST_XS(E, M, W, X, 1);                                           \
    else HZ_BWD_FAST_XS(E, M, W, X, 2);                                                     \
  } while (0)
#define HZ_BWD_FAST(E, M, W)                                                   \
  do {                                                                       \
    if (ar == kArTf32) HZ_BWD_FAST_X(E, M, W, kArTf32);                        \
    else if (ar == kArBf16x3) HZ_BWD_FAST_X(E, M, W, kArBf16x3);               \
    else if (ar == kArFp16x3) HZ_BWD_FAST_X(E, M, W, kArFp16x3);               \
    else HZ_BWD_FAST_X(E, M, W, kArTf32x3);                                    \
  } while (0)
    // one load stage and three CTAs per SM, or (HZ_ATTN_BWD=2stage) two stages and two CTAs
    const size_t fsm1 = (size_t)(4 * kFTile + 2 * 64 * 64) * sizeof(float) + 2 * kFN;
    const int fgrid1 = persistent_grid(tiles, 3);
    static const bool one_stage = !env_equals("HZ_ATTN_BWD", "2stage");
    const int sel = (e ? 4 : 0) | (mask ? 2 : 0) | (de ? 1 : 0);
    switch (sel) {
      case 0: HZ_BWD_FAST(false, false, false); break;
      case 1: HZ_BWD_FAST(false, false, true); break;
      case 2: HZ_BWD_FAST(false, true, false); break;
      case 3: HZ_BWD_FAST(false, true, true); break;
      case 4: HZ_BWD_FAST(true, false, false); break;
      case 5: HZ_BWD_FAST(true, false, true); break;
      case 6: HZ_BWD_FAST(true, true, false); break;
      default: HZ_BWD_FAST(true, true, true); break;
    }
#undef HZ_BWD_FAST
#undef HZ_BWD_FAST_X
#undef HZ_BWD_FAST_XS
    HZ_CUDA_TRY(cudaGetLastError());
    return HZ_OK;
  }
#define HZ_BWD_CASE(DD)                                                             \
  case DD:                                                                          \
    return single ? launch(attn_bwd_kernel<DD, true>, grid, smem, a, s)             \
                  : launch(attn_bwd_kernel<DD, false>, grid, smem, a, s);
  switch (D) {
    HZ_BWD_CASE(8)
    HZ_BWD_CASE(16)
    HZ_BWD_CASE(32)
    default:
      return single ? launch(attn_bwd_kernel<64, true>, grid, smem, a, s)
                    : launch(attn_bwd_kernel<64, false>, grid, smem, a, s);
  }
#undef HZ_BWD_CASE
}
