// Quadrilinear contraction of the merge with two carrier vectors, values only, on tcgen05:
//
//   Z[p][g, n] = sum_(k,l) B_g[n][(k, l)] X[p][g, k] Y[p][g, l]        (g = group of 32 channels)
//
// for all (walker, node) pairs p of a tree level. With B_g = T_g[j][(k, l)] this is the raw merge
// raw = T(u_L, u_R) (src/hamiltonzero/compiled/execute.py:48-66, the einsum over the carrier
// halves); with the two other arrangements of T_g, B_g = T_g[k][(j, l)] and T_g[l][(j, k)], it is
// the merge's two carrier cotangents du_L = T(d raw, ., u_R), du_R = T(d raw, u_L, .). Written as
// one GEMM per group with M = pairs, K = 1024, N = 32, the A operand is the outer product
// X_g (x) Y_g of a pair, which never exists in memory: the rewriter warps form it in registers,
// 32 entries (one k, all l) per k-tile, split it into FP16 head and tail and store it straight
// into TMEM; B_g (FP16 head/tail, 128 KB) stays in shared memory for the whole kernel; the two
// accumulators (head x head; tail x head + head x tail) live in TMEM over all 32 k-tiles and are
// added in the epilogue.
//
// Ranges: every pair's X and Y are scaled by powers of two so that their largest entries lie in
// [1/2, 1) and the products in [0, 2^15); B's rows are scaled into [2^14, 2^15) when packed
// (prepare_weights_f16); the epilogue multiplies the scales back in (exact).
//
// Roles of the 512 threads (register budgets as in gemm_tcf_kernel): warp 0 loads B once by TMA,
// warp 1 issues the UMMAs, warps 4-11 are two rewriter groups that alternate k-tiles (thread =
// pair = TMEM lane), warps 12-15 run the epilogue (thread = pair). Every wait is bounded; a wait
// that runs out sets the status word, makes the other roles leave and the CTA frees its TMEM.
#pragma once
#include "hz_gemm_tc.cuh"

namespace hz {

struct TprodArgs {
  const float* X;            // rows of d floats; row of pair p: p * xm + xa
  const float* Y;
  float* Z;
  int xm, xa, ym, ya, zm, za;
  long long pairs;
  int nodes;                 // node of pair p: p % nodes
  const uint8_t* opcodes;    // nullable: Z is written only where opcodes[node] == 0
  int d;
  const float* b_scale;      // [G * 32] row scales of the packed B
};

constexpr int kTpThreads = 512, kTpStages = 4, kTpKT = 32, kTpScaleRing = 4;
constexpr int kTpBTile = 32 * 128;                 // one k-tile of B_g: 32 rows x (head | tail)
constexpr uint32_t kTpTmemCols = 256;              // 2 x (32 main + 32 small) + 4 stages x 32
constexpr uint32_t kTpColA = 128;
constexpr int kTpXsLd = 33;
constexpr size_t kTpSmem = (size_t)kTpKT * kTpBTile + 2 * 128 * kTpXsLd * sizeof(float) +
                           kTpScaleRing * 128 * sizeof(float) + 1024;
static_assert(kTpStages % 2 == 0, "two rewriter groups need an even number of stages");

__global__ void __launch_bounds__(kTpThreads, 1)
tprod_tc_kernel(const __grid_constant__ CUtensorMap bmap, TprodArgs a, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* Bs = smem;
  float* xs = reinterpret_cast<float*>(smem + (size_t)kTpKT * kTpBTile);     // [2][128][33]
  float* sc = xs + 2 * 128 * kTpXsLd;                                         // [ring][128]
  __shared__ __align__(8) uint64_t b_bar, conv_bar[kTpStages], afree_bar[kTpStages];
  __shared__ __align__(8) uint64_t tfull_bar[2], tfree_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = blockIdx.x;
  const long long tiles = (a.pairs + 127) / 128;

  if (tid == 0) {
    mbar_init(&b_bar, 1);
    for (int s = 0; s < kTpStages; ++s) { mbar_init(&conv_bar[s], 128); mbar_init(&afree_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tfree_bar[b], 128); }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kTpTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  auto fail = [&](int code) { atomicExch(status, code); abort_s = 1; };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      // ---------------- B_g: 32 k-tiles of 4 KB, once
      if (lane == 0) {
        mbar_expect_tx(&b_bar, kTpKT * kTpBTile);
        for (int kt = 0; kt < kTpKT; ++kt)
          tma_load_2d(Bs + (size_t)kt * kTpBTile, &bmap, kt * 32, g * 32, &b_bar);
        // this thread's copies must have landed before the CTA may exit
        if (!mbar_wait(&b_bar, 0)) fail(kTcTimeoutLoad);
      }
    } else if (warp == 1) {
      // ---------------- issuer
      if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_f16_n(32);
        bool alive = mbar_wait_abortable(&b_bar, 0, &abort_s);
        if (!alive) fail(kTcTimeoutLoad);
        long long it = 0, ti = 0;
        for (long long tile = blockIdx.y; tile < tiles && alive; tile += gridDim.y, ++ti) {
          const int buf = (int)(ti & 1);
          for (int kt = 0; kt < kTpKT; ++kt, ++it) {
            const int s = (int)(it % kTpStages);
            if (!mbar_wait_abortable(&conv_bar[s], (uint32_t)(it / kTpStages) & 1, &abort_s) ||
                (kt == 0 && ti >= 2 &&
                 !mbar_wait_abortable(&tfree_bar[buf], (uint32_t)((ti >> 1) - 1) & 1, &abort_s))) {
              fail(kTcTimeoutMma);
              alive = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t b = smem_u32(Bs) + (uint32_t)(kt * kTpBTile);
            const uint32_t tmain = tmem_base + (uint32_t)(buf * 64), tsmall = tmain + 32;
            const uint32_t ta = tmem_base + kTpColA + (uint32_t)(s * 32);
            const uint32_t acc0 = kt > 0 ? 1u : 0u;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)      // tail x head
              umma_f16_ts(tsmall, ta + 16 + ks * 8, umma_desc_sw128(b + ks * 32), idesc, ks > 0 ? 1u : acc0);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)      // head x tail
              umma_f16_ts(tsmall, ta + ks * 8, umma_desc_sw128(b + 64 + ks * 32), idesc, 1u);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)      // head x head
              umma_f16_ts(tmain, ta + ks * 8, umma_desc_sw128(b + ks * 32), idesc, ks > 0 ? 1u : acc0);
            umma_commit(&afree_bar[s]);
            if (kt == kTpKT - 1) umma_commit(&tfull_bar[buf]);
          }
        }
      }
    }
  } else if (warp < 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    // ---------------- rewriters: thread = pair of the tile = TMEM lane; group rgrp takes the
    // k-tiles with it % 2 == rgrp. Both groups load the pair's X and Y.
    const int row = (warp & 3) * 32 + lane, rgrp = (warp - 4) >> 2;
    float* myx = xs + (size_t)(rgrp * 128 + row) * kTpXsLd;
    long long it = 0, ti = 0;
    bool alive = true;
    for (long long tile = blockIdx.y; tile < tiles && alive; tile += gridDim.y, ++ti) {
      const long long pair = tile * 128 + row;
      float y[32];
      {
        float x[32];
        if (pair < a.pairs) {
          const float4* xp = reinterpret_cast<const float4*>(a.X + (size_t)(pair * a.xm + a.xa) * a.d + g * 32);
          const float4* yp = reinterpret_cast<const float4*>(a.Y + (size_t)(pair * a.ym + a.ya) * a.d + g * 32);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 v = xp[c], u = yp[c];
            x[4 * c] = v.x; x[4 * c + 1] = v.y; x[4 * c + 2] = v.z; x[4 * c + 3] = v.w;
            y[4 * c] = u.x; y[4 * c + 1] = u.y; y[4 * c + 2] = u.z; y[4 * c + 3] = u.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = y[i] = 0.f;
        }
        float mx = 0.f, my = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) { mx = fmaxf(mx, fabsf(x[i])); my = fmaxf(my, fabsf(y[i])); }
        // exponents that bring the largest entries into [1/2, 1); 0 for zero or non-finite rows
        int ex = 0, ey = 0;
        if (mx > 0.f && isfinite(mx)) ex = max(min((int)((__float_as_uint(mx) >> 23) & 0xff) - 126, 100), -100);
        if (my > 0.f && isfinite(my)) ey = max(min((int)((__float_as_uint(my) >> 23) & 0xff) - 126, 100), -100);
        const float sx = __uint_as_float((uint32_t)(127 - ex) << 23);
        const float sy = __uint_as_float((uint32_t)(127 + 15 - ey) << 23);
#pragma unroll
        for (int i = 0; i < 32; ++i) { myx[i] = x[i] * sx; y[i] *= sy; }
        if (rgrp == 0) sc[(int)(ti & (kTpScaleRing - 1)) * 128 + row] = ldexpf(1.f, ex + ey - 15);
      }
      for (int kt = 0; kt < kTpKT; ++kt, ++it) {
        if ((int)(it & 1) != rgrp) continue;
        const int s = (int)(it % kTpStages);
        if (it >= kTpStages &&
            !__all_sync(0xffffffffu, mbar_wait_abortable(&afree_bar[s], (uint32_t)((it / kTpStages) - 1) & 1,
                                                         &abort_s))) {
          if (lane == 0) fail(kTcTimeoutMma);
          alive = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float xk = myx[kt];
        uint32_t av[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float v0 = xk * y[2 * i], v1 = xk * y[2 * i + 1];
          const __half2 hi = __floats2half2_rn(v0, v1);
          const float2 hf = __half22float2(hi);
          const __half2 lo = __floats2half2_rn(v0 - hf.x, v1 - hf.y);
          av[i] = *reinterpret_cast<const uint32_t*>(&hi);
          av[16 + i] = *reinterpret_cast<const uint32_t*>(&lo);
        }
        tmem_st32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + kTpColA + (uint32_t)(s * 32), av);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(&conv_bar[s]);
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ---------------- epilogue: thread = pair, 32 output channels
    const int q = warp & 3, row = q * 32 + lane;
    long long ti = 0;
    bool ok = true;
    for (long long tile = blockIdx.y; tile < tiles && ok; tile += gridDim.y, ++ti) {
      const int buf = (int)(ti & 1);
      if (!mbar_wait_abortable(&tfull_bar[buf], (uint32_t)(ti >> 1) & 1, &abort_s)) {
        if (lane == 0) fail(kTcTimeoutMma);
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 64);
      uint32_t vm[32], vs[32];
      tmem_ld32(vm, t0);
      tmem_ld32(vs, t0 + 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&tfree_bar[buf]);
      const float scale = sc[(int)(ti & (kTpScaleRing - 1)) * 128 + row];
      const long long pair = tile * 128 + row;
      if (pair < a.pairs && (a.opcodes == nullptr || a.opcodes[pair % a.nodes] == 0)) {
        float4* z = reinterpret_cast<float4*>(a.Z + (size_t)(pair * a.zm + a.za) * a.d + g * 32);
        const float4* w = reinterpret_cast<const float4*>(a.b_scale + g * 32);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float4 w4 = w[c];
          z[c] = make_float4((__uint_as_float(vm[4 * c]) + __uint_as_float(vs[4 * c])) * scale * w4.x,
                             (__uint_as_float(vm[4 * c + 1]) + __uint_as_float(vs[4 * c + 1])) * scale * w4.y,
                             (__uint_as_float(vm[4 * c + 2]) + __uint_as_float(vs[4 * c + 2])) * scale * w4.z,
                             (__uint_as_float(vm[4 * c + 3]) + __uint_as_float(vs[4 * c + 3])) * scale * w4.w);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTpTmemCols)
                 : "memory");
  }
}

// T [G][j][k][l] -> arrangement 1: [G][k][(j, l)], arrangement 2: [G][l][(j, k)]
static __global__ void tprod_permute_kernel(const float* __restrict__ T, float* __restrict__ out, long long n,
                                            int arrangement) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const int l = (int)(idx & 31), k = (int)((idx >> 5) & 31), j = (int)((idx >> 10) & 31);
  const long long gbase = (idx >> 15) << 15;
  const long long dst = arrangement == 1 ? gbase + ((long long)k << 10) + (j << 5) + l
                                         : gbase + ((long long)l << 10) + (j << 5) + k;
  out[dst] = T[idx];
}

// packed [G*32][1024] halves (the bytes of one fp32 matrix of that shape) and scales [2 * G*32]
inline int tprod_prepare(const float* T, int G, int arrangement, float* scratch, float* packed, float* scales,
                         cudaStream_t stream) {
  const float* src = T;
  if (arrangement != 0) {
    const long long n = (long long)G * 32768;
    tprod_permute_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(T, scratch, n, arrangement);
    HZ_CUDA_TRY(cudaGetLastError());
    src = scratch;
  }
  return prepare_weights_f16(src, packed, scales, 1024, G * 32, false, stream);
}

inline int launch_tprod(const TprodArgs& a, int G, const float* packed, int* status, cudaStream_t stream) {
  if (a.pairs <= 0) return HZ_OK;
  CUtensorMap bmap;
  if (!make_map(&bmap, packed, (long long)G * 32, 1024, 1024, 32)) return HZ_ERR_CUDA;
  const int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(tprod_tc_kernel), (int)kTpSmem);
  if (rc != HZ_OK) return rc;
  const long long tiles = (a.pairs + 127) / 128;
  int slices = tc_sm_count() / G;
  if (slices < 1) slices = 1;
  if (slices > tiles) slices = (int)tiles;
  tprod_tc_kernel<<<dim3(G, slices), kTpThreads, kTpSmem, stream>>>(bmap, a, status);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// HZ_TPROD=legacy keeps the value-only merge and its carrier cotangents on the mma.sync kernels.
inline bool use_tprod_tc() {
  static const bool on = !env_equals("HZ_TPROD", "legacy") && use_persistent_tc();
  return on;
}


// ------------------------------------------------------------------ tensor application form
// The same three products with far fewer, wider UMMAs (a tcgen05.mma of M = 128 costs about 120
// cycles however narrow it is, so N = 32 wastes most of each): first the tensor application
//   D[p][(j, x)] = sum_y B_g[(j, x)][y] A[p][g, y]          (M = 128 pairs, N = 128 per UMMA, K = 32)
// with the carrier A as the TMEM operand (FP16 head/tail of one 32-vector per pair: the rewriters'
// work is one store per tile) and all 1024 rows of the group's view of T as B, then the second
// contraction with the pair's other vector V on the CUDA cores, straight from the accumulator
// columns in TMEM:
//   mode 0: Z[p][j] = sum_x D[(j, x)] V[x]      (raw = A_R u_L with B = T[(j,k)][l], A = u_R)
//   mode 1: Z[p][x] = sum_j V[j] D[(j, x)]      (du_L = A_R^T d raw; du_R = A_L^T d raw with
//                                                B = T[(j,l)][k], A = u_L)
// V enters in fp32 only, so a cotangent of any magnitude needs no scaling. Three accumulators of
// 128 columns rotate between the issuer and the four consumer warps.
struct TapplyArgs {
  const float* A;            // TMEM operand rows; row of pair p: p * am + aa
  const float* V;            // second vector
  float* Z;
  int am, aa, vm, va, zm, za;
  long long pairs;
  int nodes;
  const uint8_t* opcodes;    // nullable: Z is written only where opcodes[node] == 0
  int d;
  const float* t_scale;      // [G] power of two by which the group's T was divided
  int brow0;                 // first row of this arrangement in the packed T (arrangement * G * 1024)
};

constexpr uint32_t kTaTmemCols = 512;              // 3 x 128 accumulators, 2 x 32 carrier columns
constexpr uint32_t kTaColA = 384;
constexpr size_t kTaSmem = (size_t)1024 * 128 + kTpScaleRing * 128 * sizeof(float) + 1024;

// packed[(arr * G + g) * 1024 + row][head(32) | tail(32)] halves of T_g * 2^-e_g, e_g such that
// the group's largest entry lands in [2^14, 2^15); arr 0: row = (j, k), column l; arr 1: row =
// (j, l), column k. t_scale[g] = 2^e_g.
static __global__ void __launch_bounds__(256)
tapply_pack_kernel(const float* __restrict__ T, __half* __restrict__ packed, float* __restrict__ t_scale, int G,
                   int arrangements) {
  __shared__ float red[8];
  __shared__ int expo_s;
  const int grp = blockIdx.x, tid = threadIdx.x;
  const float* Tg = T + (size_t)grp * 32768;
  float mx = 0.f;
  for (int i = tid; i < 32768; i += 256) mx = fmaxf(mx, fabsf(Tg[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  if (tid == 0) {
    float m = 0.f;
    for (int i = 0; i < 8; ++i) m = fmaxf(m, red[i]);
    int e = 0;
    if (m > 0.f && isfinite(m)) { frexpf(m, &e); e -= 15; }
    expo_s = e;
    t_scale[grp] = ldexpf(1.f, e);
  }
  __syncthreads();
  const int e = expo_s;
  for (int rr = tid; rr < 1024 * arrangements; rr += 256) {
    const int arr = rr >> 10, row = rr & 1023, j = row >> 5, x = row & 31;
    __half* dst = packed + ((size_t)(arr * G + grp) * 1024 + row) * 64;
    for (int y = 0; y < 32; ++y) {
      const float val = arr == 0 ? Tg[(j * 32 + x) * 32 + y] : Tg[(j * 32 + y) * 32 + x];
      const float ts = ldexpf(val, -e);
      const __half hi = __float2half_rn(ts);
      dst[y] = hi;
      dst[32 + y] = __float2half_rn(ts - __half2float(hi));
    }
  }
}

template <int MODE>
__global__ void __launch_bounds__(kTpThreads, 1)
tapply_tc_kernel(const __grid_constant__ CUtensorMap bmap, TapplyArgs a, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* Bs = smem;                                                         // 1024 rows x 128 B
  float* sc = reinterpret_cast<float*>(smem + (size_t)1024 * 128);           // [ring][128]
  __shared__ __align__(8) uint64_t b_bar, conv_bar[2], afree_bar[2], tfull_bar[3], tfree_bar[3];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = blockIdx.x;
  const long long tiles = (a.pairs + 127) / 128;

  if (tid == 0) {
    mbar_init(&b_bar, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&conv_bar[s], 128); mbar_init(&afree_bar[s], 1); }
    for (int b = 0; b < 3; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tfree_bar[b], 128); }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kTaTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  auto fail = [&](int code) { atomicExch(status, code); abort_s = 1; };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      // ---------------- the group's view of T: four boxes of 256 rows, once
      if (lane == 0) {
        mbar_expect_tx(&b_bar, 1024 * 128);
        for (int i = 0; i < 4; ++i)
          tma_load_2d(Bs + (size_t)i * 256 * 128, &bmap, 0, a.brow0 + g * 1024 + i * 256, &b_bar);
        if (!mbar_wait(&b_bar, 0)) fail(kTcTimeoutLoad);      // own copies landed before the CTA may exit
      }
    } else if (warp == 1) {
      // ---------------- issuer: 8 chunks of 128 rows of T per tile, six UMMAs each
      if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_f16_n(128);
        bool alive = mbar_wait_abortable(&b_bar, 0, &abort_s);
        if (!alive) fail(kTcTimeoutLoad);
        long long ti = 0, cc = 0;
        for (long long tile = blockIdx.y; tile < tiles && alive; tile += gridDim.y, ++ti) {
          const int ab = (int)(ti & 1);
          if (!mbar_wait_abortable(&conv_bar[ab], (uint32_t)(ti >> 1) & 1, &abort_s)) {
            fail(kTcTimeoutMma);
            break;
          }
          const uint32_t ta = tmem_base + kTaColA + (uint32_t)(ab * 32);
          for (int c = 0; c < 8; ++c, ++cc) {
            const int buf = (int)(cc % 3);
            if (cc >= 3 && !mbar_wait_abortable(&tfree_bar[buf], (uint32_t)((cc / 3) - 1) & 1, &abort_s)) {
              fail(kTcTimeoutMma);
              alive = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t b = smem_u32(Bs) + (uint32_t)(c * 128 * 128);
            const uint32_t tacc = tmem_base + (uint32_t)(buf * 128);
            // small terms first: tail x head, head x tail, then head x head
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
              umma_f16_ts(tacc, ta + 16 + ks * 8, umma_desc_sw128(b + ks * 32), idesc, ks > 0 ? 1u : 0u);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
              umma_f16_ts(tacc, ta + ks * 8, umma_desc_sw128(b + 64 + ks * 32), idesc, 1u);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
              umma_f16_ts(tacc, ta + ks * 8, umma_desc_sw128(b + ks * 32), idesc, 1u);
            umma_commit(&tfull_bar[buf]);
          }
          if (alive) umma_commit(&afree_bar[ab]);
        }
      }
    }
  } else if (warp < 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    if (warp < 8) {
      // ---------------- carrier rows -> FP16 head/tail in TMEM: thread = pair = TMEM lane
      const int row = (warp & 3) * 32 + lane;
      long long ti = 0;
      for (long long tile = blockIdx.y; tile < tiles; tile += gridDim.y, ++ti) {
        const int ab = (int)(ti & 1);
        const long long pair = tile * 128 + row;
        float4 x[8];
        if (pair < a.pairs) {
          const float4* xp = reinterpret_cast<const float4*>(a.A + (size_t)(pair * a.am + a.aa) * a.d + g * 32);
#pragma unroll
          for (int c = 0; c < 8; ++c) x[c] = xp[c];
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) x[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float mx = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          mx = fmaxf(fmaxf(mx, fmaxf(fabsf(x[c].x), fabsf(x[c].y))), fmaxf(fabsf(x[c].z), fabsf(x[c].w)));
        // power of two that brings the largest entry into [2^14, 2^15)
        int e = 0;
        if (mx > 0.f && isfinite(mx)) e = max((int)((__float_as_uint(mx) >> 23) & 0xff) - 141, -126);
        const float down = __uint_as_float((uint32_t)(127 - e) << 23);
        uint32_t av[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float v[4] = {x[c].x * down, x[c].y * down, x[c].z * down, x[c].w * down};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const __half2 hi = __floats2half2_rn(v[2 * h], v[2 * h + 1]);
            const float2 hf = __half22float2(hi);
            const __half2 lo = __floats2half2_rn(v[2 * h] - hf.x, v[2 * h + 1] - hf.y);
            av[2 * c + h] = *reinterpret_cast<const uint32_t*>(&hi);
            av[16 + 2 * c + h] = *reinterpret_cast<const uint32_t*>(&lo);
          }
        }
        if (ti >= 2 &&
            !__all_sync(0xffffffffu, mbar_wait_abortable(&afree_bar[ab], (uint32_t)((ti >> 1) - 1) & 1, &abort_s))) {
          if (lane == 0) fail(kTcTimeoutMma);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        sc[(int)(ti & (kTpScaleRing - 1)) * 128 + row] = __uint_as_float((uint32_t)(127 + e) << 23);
        tmem_st32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + kTaColA + (uint32_t)(ab * 32), av);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(&conv_bar[ab]);
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ---------------- consumers: thread = pair; second contraction from the accumulator columns
    const int q = warp & 3, row = q * 32 + lane;
    long long ti = 0, cc = 0;
    bool ok = true;
    for (long long tile = blockIdx.y; tile < tiles && ok; tile += gridDim.y, ++ti) {
      const long long pair = tile * 128 + row;
      const bool valid = pair < a.pairs;
      float v[32], out[32];
      if (valid) {
        const float4* vp = reinterpret_cast<const float4*>(a.V + (size_t)(pair * a.vm + a.va) * a.d + g * 32);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float4 u = vp[c];
          v[4 * c] = u.x; v[4 * c + 1] = u.y; v[4 * c + 2] = u.z; v[4 * c + 3] = u.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) out[i] = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c, ++cc) {
        if (!ok) continue;
        const int buf = (int)(cc % 3);
        if (!mbar_wait_abortable(&tfull_bar[buf], (uint32_t)(cc / 3) & 1, &abort_s)) {
          if (lane == 0) fail(kTcTimeoutMma);
          ok = false;
          continue;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 128);
#pragma unroll
        for (int jj = 0; jj < 4; jj += 2) {
          uint32_t d0[32], d1[32];
          tmem_ld32(d0, t0 + jj * 32);
          tmem_ld32(d1, t0 + jj * 32 + 32);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (jj == 2) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&tfree_bar[buf]);
          }
          if (MODE == 0) {
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int x = 0; x < 32; ++x) {
              s0 = fmaf(__uint_as_float(d0[x]), v[x], s0);
              s1 = fmaf(__uint_as_float(d1[x]), v[x], s1);
            }
            out[4 * c + jj] = s0;
            out[4 * c + jj + 1] = s1;
          } else {
            const float w0 = v[4 * c + jj], w1 = v[4 * c + jj + 1];
#pragma unroll
            for (int x = 0; x < 32; ++x)
              out[x] = fmaf(w1, __uint_as_float(d1[x]), fmaf(w0, __uint_as_float(d0[x]), out[x]));
          }
        }
      }
      if (!ok) break;
      const float scale = sc[(int)(ti & (kTpScaleRing - 1)) * 128 + row] * a.t_scale[g];
      if (valid && (a.opcodes == nullptr || a.opcodes[pair % a.nodes] == 0)) {
        float4* z = reinterpret_cast<float4*>(a.Z + (size_t)(pair * a.zm + a.za) * a.d + g * 32);
#pragma unroll
        for (int c = 0; c < 8; ++c)
          z[c] = make_float4(out[4 * c] * scale, out[4 * c + 1] * scale, out[4 * c + 2] * scale,
                             out[4 * c + 3] * scale);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTaTmemCols)
                 : "memory");
  }
}

// arrangements: 2 packs both views of T (packed holds 2 G 1024 rows of 128 bytes), 1 only the
// first (G 1024 rows), which is all the raw merge needs
inline int tapply_prepare(const float* T, int G, float* packed, float* t_scale, cudaStream_t stream,
                          int arrangements = 2) {
  tapply_pack_kernel<<<G, 256, 0, stream>>>(T, reinterpret_cast<__half*>(packed), t_scale, G, arrangements);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

inline int launch_tapply(int mode, const TapplyArgs& a, int G, const float* packed, int* status,
                         cudaStream_t stream, int arrangements = 2) {
  if (a.pairs <= 0) return HZ_OK;
  CUtensorMap bmap;
  if (!make_map(&bmap, packed, (long long)arrangements * G * 1024, 32, 32, 256)) return HZ_ERR_CUDA;
  const long long tiles = (a.pairs + 127) / 128;
  int slices = tc_sm_count() / G;
  if (slices < 1) slices = 1;
  if (slices > tiles) slices = (int)tiles;
  const dim3 grid(G, slices);
  if (mode == 0) {
    const int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(tapply_tc_kernel<0>), (int)kTaSmem);
    if (rc != HZ_OK) return rc;
    tapply_tc_kernel<0><<<grid, kTpThreads, kTaSmem, stream>>>(bmap, a, status);
  } else {
    const int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(tapply_tc_kernel<1>), (int)kTaSmem);
    if (rc != HZ_OK) return rc;
    tapply_tc_kernel<1><<<grid, kTpThreads, kTaSmem, stream>>>(bmap, a, status);
  }
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// HZ_TPROD=outer keeps the outer-product form above (A/B timing).
inline bool use_tapply_tc() {
  static const bool on = !env_equals("HZ_TPROD", "outer");
  return on && use_tprod_tc();
}

}  // namespace hz
