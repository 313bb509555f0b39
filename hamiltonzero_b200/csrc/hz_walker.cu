// Walker-batch operators for sm_100a: log-psi of the compiled binary-merge-tree
// wavefunction and its forward-Laplacian local energy.
//
// Reference semantics: src/hamiltonzero/compiled/execute.py:79-118 (executor),
// src/hamiltonzero/energy/kernel.py:20-37,80-119 (chart, energy assembly) and the
// jet calculus of src/hamiltonzero/energy/custom_lap.py (linear maps :630-725,
// unary ops :136-181, products :408-483, quadrilinear merge :1318-1389).
//
// For every tree node the pipeline carries the value u, the Jacobian rows of the
// node's own 3k chart coordinates and the J_eff-weighted Laplacian ("jets").
// One level of the tree is four launches over a chunk of walkers:
//   merge_tstage   quadrilinear merge of the two children's jets (tensor cores)
//   gemm x2        out = raw + ((raw V) * h) U for all jet rows (hz_gemm.cuh)
//   norm_reduce    row statistics of out: |out|^2, J.out, tr(W J J^T), scalars
//   norm_apply     u = out/sigma with its jets, opcode gating, in place
// Jet rows of a walker are packed as [3N Jacobian rows | nodes values | nodes
// Laplacians], each row d_m floats, so that a level is one [rows, d_m] matrix.
#include <cuda_fp16.h>

#include "hz_gemm_tc.cuh"
#include "hz_syrk_tc.cuh"
#include "hz_tprod_tc.cuh"

#include <stdlib.h>
#include <string.h>

#include <math.h>

#include <mutex>

namespace hz {
namespace {

constexpr int kDr = 32;                 // group width of the merge tensor
constexpr float kLeafEps = 1e-30f;      // src/hamiltonzero/model/model.py:32

struct Level {
  int N, d, G;
  int nodes;          // nodes at this (output) level
  int m;              // Jacobian rows of ONE child (3k); output node has 2m
  int jets;           // 0: values only
  int rows_in, rows_out;   // packed rows per walker at the input / output level
  int Bc;             // walkers in the chunk
};

__host__ __device__ inline int packed_rows(int N, int nodes, int jets) {
  return jets ? 3 * N + 2 * nodes : nodes;
}
__device__ __forceinline__ size_t row_u(const Level& L, int rows, int nodes, int b, int n) {
  return (size_t)b * rows + (L.jets ? 3 * L.N : 0) + n;
}
__device__ __forceinline__ size_t row_l(const Level& L, int rows, int nodes, int b, int n) {
  return (size_t)b * rows + 3 * L.N + nodes + n;
}
__device__ __forceinline__ size_t row_j(int rows, int b, int a) { return (size_t)b * rows + a; }

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Block-wide sum of NV values per thread; result valid in every thread.
template <int NV, int THREADS>
__device__ __forceinline__ void block_sum(float (&v)[NV], float* scratch /* NV*THREADS/32 */) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = warp_sum(v[i]);
  __syncthreads();
  if (lane == 0)
#pragma unroll
    for (int i = 0; i < NV; ++i) scratch[warp * NV + i] = v[i];
  __syncthreads();
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float s = 0.f;
    for (int w = 0; w < THREADS / 32; ++w) s += scratch[w * NV + i];
    v[i] = s;
  }
}

// ------------------------------------------------------------------ leaf map
// tmp[n*4+o][r] = (q_weight @ leaf_V)[o][r] * leaf_h[n][r]; leaf_map = tmp @ leaf_U by GEMM.
__global__ void leaf_tmp_kernel(const float* Wq, const float* V, const float* h, float* tmp,
                                int N, int d_o, int r) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= N * 4 * r) return;
  const int c = idx % r, o = (idx / r) % 4, n = idx / (4 * r);
  float acc = 0.f;
  for (int k = 0; k < d_o; ++k) acc = fmaf(Wq[o * d_o + k], V[k * r + c], acc);
  tmp[idx] = acc * h[n * r + c];
}

// ------------------------------------------------------------------ leaves
// One CTA per (site, walker): u_raw and its chart jets are linear in the
// quaternion (leaf_map[n] is 4 x d), followed by the RMS normalisation.
constexpr int kLeafThreads = 128;

__global__ void __launch_bounds__(kLeafThreads)
leaf_kernel(Level L, const float* __restrict__ q, const float* __restrict__ leaf_map,
            const float* __restrict__ J_eff, float* __restrict__ buf, float* __restrict__ s_out,
            float* __restrict__ js_out, float* __restrict__ ls_out,
            const uint8_t* __restrict__ skip_merged = nullptr /* first-level opcodes: leaves of merged
                                                                 parents are not materialised */) {
  __shared__ float scratch[10 * kLeafThreads / 32];
  const int n = blockIdx.x, b = blockIdx.y;
  if (skip_merged != nullptr && skip_merged[n >> 1] == 0) return;
  const int N = L.N, d = L.d;
  const float* qq = q + ((size_t)b * N + n) * 4;
  const float q0 = qq[0], q1 = qq[1], q2 = qq[2], q3 = qq[3];
  // rows x, y, z of d(chart)/dz at z = 0 (energy/kernel.py:20-37)
  const float dq[3][4] = {{-q3, q2, -q1, q0}, {-q2, -q3, q0, q1}, {-q1, q0, q3, -q2}};
  const float* M = leaf_map + (size_t)n * 4 * d;

  float red[10];
#pragma unroll
  for (int i = 0; i < 10; ++i) red[i] = 0.f;
  for (int c = threadIdx.x; c < d; c += kLeafThreads) {
    const float m0 = M[c], m1 = M[d + c], m2 = M[2 * d + c], m3 = M[3 * d + c];
    const float v = q0 * m0 + q1 * m1 + q2 * m2 + q3 * m3;
    red[0] += v * v;
    if (L.jets) {
      float j[3];
#pragma unroll
      for (int a = 0; a < 3; ++a) j[a] = dq[a][0] * m0 + dq[a][1] * m1 + dq[a][2] * m2 + dq[a][3] * m3;
      red[1] += j[0] * v; red[2] += j[1] * v; red[3] += j[2] * v;
      red[4] += j[0] * j[0]; red[5] += j[0] * j[1]; red[6] += j[0] * j[2];
      red[7] += j[1] * j[1]; red[8] += j[1] * j[2]; red[9] += j[2] * j[2];
    }
  }
  block_sum<10, kLeafThreads>(red, scratch);

  const float inv_d = 1.f / (float)d;
  const float y = red[0] * inv_d + kLeafEps;
  const float r = rsqrtf(y);
  float dr[3] = {0.f, 0.f, 0.f}, wdr[3] = {0.f, 0.f, 0.f}, lap_r = 0.f, trW = 0.f;
  if (L.jets) {
    float W[3][3];
#pragma unroll
    for (int a = 0; a < 3; ++a)
#pragma unroll
      for (int c = 0; c < 3; ++c) W[a][c] = J_eff[(size_t)(3 * n + a) * (3 * N) + 3 * n + c];
    trW = W[0][0] + W[1][1] + W[2][2];
    const float dy[3] = {2.f * inv_d * red[1], 2.f * inv_d * red[2], 2.f * inv_d * red[3]};
    const float gram = W[0][0] * red[4] + W[1][1] * red[7] + W[2][2] * red[9] +
                       (W[0][1] + W[1][0]) * red[5] + (W[0][2] + W[2][0]) * red[6] +
                       (W[1][2] + W[2][1]) * red[8];
    const float oL = -trW * red[0];
    const float lap_y = 2.f * inv_d * (oL + gram);
    float wdy[3], dywdy = 0.f;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
      wdy[a] = W[a][0] * dy[0] + W[a][1] * dy[1] + W[a][2] * dy[2];
      dywdy += dy[a] * wdy[a];
    }
    const float y15 = r * r * r;            // y^-1.5
    const float y25 = y15 * r * r;          // y^-2.5
    lap_r = -0.5f * y15 * lap_y + 0.75f * y25 * dywdy;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
      dr[a] = -0.5f * y15 * dy[a];
      wdr[a] = -0.5f * y15 * wdy[a];
    }
    if (threadIdx.x == 0) {
      ls_out[(size_t)b * N + n] = 0.5f * (lap_y / y - dywdy / (y * y));
#pragma unroll
      for (int a = 0; a < 3; ++a) js_out[(size_t)b * 3 * N + 3 * n + a] = 0.5f * dy[a] / y;
    }
  }
  if (threadIdx.x == 0) s_out[(size_t)b * N + n] = 0.5f * logf(y);

  const int rows = L.rows_out;
  float* urow = buf + row_u(L, rows, N, b, n) * d;
  float* lrow = L.jets ? buf + row_l(L, rows, N, b, n) * d : nullptr;
  float* jrow = L.jets ? buf + row_j(rows, b, 3 * n) * d : nullptr;
  for (int c = threadIdx.x; c < d; c += kLeafThreads) {
    const float m0 = M[c], m1 = M[d + c], m2 = M[2 * d + c], m3 = M[3 * d + c];
    const float v = q0 * m0 + q1 * m1 + q2 * m2 + q3 * m3;
    urow[c] = v * r;
    if (L.jets) {
      float acc = 0.f;
#pragma unroll
      for (int a = 0; a < 3; ++a) {
        const float j = dq[a][0] * m0 + dq[a][1] * m1 + dq[a][2] * m2 + dq[a][3] * m3;
        jrow[(size_t)a * d + c] = j * r + dr[a] * v;
        acc += wdr[a] * j;
      }
      lrow[c] = (-trW * v) * r + v * lap_r + 2.f * acc;
    }
  }
}

// ------------------------------------------------------------------ merge T-stage
// One CTA owns one group i of the merge tensor, keeps T_i (32x32x32 fp32) in
// shared memory and walks over tiles of 16 (walker, node) pairs:
//   A_R[j,k] = sum_l T[j,k,l] u_R[l]      A_L[j,l] = sum_k T[j,k,l] u_L[k]
//   raw[j]   = sum_k A_R[j,k] u_L[k]
//   Jraw[A]  = A_R J_L[A]  (left rows)    Jraw[m+B] = A_L J_R[B]  (right rows)
//   Lraw     = A_R L_L + A_L L_R + 2 sum_kl T[j,k,l] C[k,l],
//              C = J_L^T (W_off J_R)       (custom_lap.py:1318-1389)
// Shared-memory tiles are XOR-swizzled instead of padded so that T_i (128 KB), the
// A_R / A_L / C tile of 16 pairs (64 KB) and the small vectors fit in 227 KB.
constexpr int kTsThreads = 512;      // 16 warps: warp w owns pair w of a tile
constexpr int kTsPairs = 16;
constexpr int kTsVecLd = 36;
constexpr int kTsWarps = kTsThreads / 32;
// per-warp 16x32 scratch (Y blocks, later the cross partials); it overlays the child vectors,
// which are dead by then
constexpr int kTsScratchFloats = kTsWarps * 16 * 32;
constexpr size_t kTsSmemFloats = 32768 + kTsPairs * 1024 + kTsScratchFloats + kTsPairs * 32;
static_assert(4 * kTsPairs * kTsVecLd <= kTsScratchFloats, "child vectors must fit the scratch");

// T_i element (j,k,l); the l index is XORed with a multiple of 4 that depends on k + j.
__device__ __forceinline__ int t_idx(int j, int k, int l) {
  return ((j * 32 + k) << 5) + (l ^ (((k + j) & 7) << 2));
}
// element (r, c) of a pair's 32x32 tile (A_R: r=j,c=k; A_L: r=j,c=l; C: r=k,c=l)
__device__ __forceinline__ int ax_idx(int p, int r, int c) {
  return (p << 10) + (r << 5) + (c ^ (((r + p) & 7) << 2));
}

// head/tail split for mma.sync operands: the tail keeps its low bits (the tensor core
// ignores them), which costs 2^-22 relative at most.
__device__ __forceinline__ void split2(float x, uint32_t& hi, uint32_t& lo) {
  hi = to_tf32(x);
  lo = __float_as_uint(x - __uint_as_float(hi));
}
struct FA2 { uint32_t hi[4], lo[4];
  __device__ __forceinline__ void set(float a0, float a1, float a2, float a3) {
    split2(a0, hi[0], lo[0]); split2(a1, hi[1], lo[1]); split2(a2, hi[2], lo[2]); split2(a3, hi[3], lo[3]); } };
struct FB2 { uint32_t hi[2], lo[2];
  __device__ __forceinline__ void set(float b0, float b1) { split2(b0, hi[0], lo[0]); split2(b1, hi[1], lo[1]); } };
// main += hi*hi ; small += lo*hi + hi*lo : two independent accumulator chains
__device__ __forceinline__ void mma3x(float (&main_acc)[4], float (&small_acc)[4], const FA2& a,
                                      const FB2& b) {
  mma_tf32(small_acc, a.lo, b.hi);
  mma_tf32(main_acc, a.hi, b.hi);
  mma_tf32(small_acc, a.hi, b.lo);
}

// T-application with the contraction over l (A_R) or over k (A_L); rows are (j, x)
// with x the index that survives, 16 per m-tile; columns are the 16 pairs. Ts: swizzled T_i,
// u: the contracted child vectors [16][kTsVecLd], AX: the [16][32][32] swizzled result tile.
// Arithmetic: both operands are range-safe by construction (T_i entries are weights of order
// 1/d_r, the child vectors are RMS-normalised carriers), so the contraction runs on a two-term
// FP16 split with scaled tails on m16n8k16: two k8 steps of the TF32 layout fuse into one k16
// instruction (k index 2t, 2t+1 <-> slots t, t+4 of the first step; 2t+8, 2t+9 <-> the second),
// three instructions per product pair instead of six, each product exact to about 3 * 2^-22.
__device__ __forceinline__ void ts_t_apply(const float* __restrict__ Ts, float* __restrict__ AX,
                                           const float* __restrict__ u, const bool over_l,
                                           const int warp, const int g, const int t) {
  uint32_t bh[2][2][2], bl[2][2][2];      // [n-tile][pair of k-steps][register]
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      split_f16x2_scaled(u[(nt * 8 + g) * kTsVecLd + ks * 8 + t],
                         u[(nt * 8 + g) * kTsVecLd + ks * 8 + t + 4], bh[nt][ks >> 1][ks & 1],
                         bl[nt][ks >> 1][ks & 1]);
#pragma unroll 2
  for (int i = 0; i < 4; ++i) {
    const int mt = warp * 4 + i;
    const int j = mt >> 1, x0 = (mt & 1) * 16 + g;     // surviving index of rows g / g+8
    float am[2][4], as[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) am[nt][c] = as[nt][c] = 0.f;
#pragma unroll
    for (int kp = 0; kp < 2; ++kp) {
      uint32_t ah[4], al[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int ks = 2 * kp + h;
        float a0, a1, a2, a3;     // (g, t) (g+8, t) (g, t+4) (g+8, t+4) of step ks
        if (over_l) {
          // element (row (j,k=x), col l): fixed swizzle per row
          const int sw = ((x0 + j) & 7) << 2;              // same for x0 and x0 + 8
          const int base0 = ((j * 32 + x0) << 5) + t, base1 = base0 + (8 << 5);
          const int c0 = (ks * 8) ^ sw, c1 = (ks * 8 + 4) ^ sw;
          a0 = Ts[base0 + c0]; a1 = Ts[base1 + c0]; a2 = Ts[base0 + c1]; a3 = Ts[base1 + c1];
        } else {
          // element (row (j,l=x), col k): swizzle depends on the column k
          const int ka = ks * 8 + t, kb = ka + 4;
          const int swa = ((ka + j) & 7) << 2, swb = ((kb + j) & 7) << 2;
          const int ra = (j * 32 + ka) << 5, rb = (j * 32 + kb) << 5;
          a0 = Ts[ra + (x0 ^ swa)]; a1 = Ts[ra + ((x0 + 8) ^ swa)];
          a2 = Ts[rb + (x0 ^ swb)]; a3 = Ts[rb + ((x0 + 8) ^ swb)];
        }
        split_f16x2_scaled(a0, a2, ah[2 * h], al[2 * h]);
        split_f16x2_scaled(a1, a3, ah[2 * h + 1], al[2 * h + 1]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        mma_f16(as[nt], al, bh[nt][kp]);
        mma_f16(am[nt], ah, bh[nt][kp]);
        mma_f16(as[nt], ah, bl[nt][kp]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int p0 = nt * 8 + 2 * t, p1 = p0 + 1;
      constexpr float w = 1.f / 2048.f;
      AX[ax_idx(p0, j, x0)] = fmaf(as[nt][0], w, am[nt][0]);
      AX[ax_idx(p1, j, x0)] = fmaf(as[nt][1], w, am[nt][1]);
      AX[ax_idx(p0, j, x0 + 8)] = fmaf(as[nt][2], w, am[nt][2]);
      AX[ax_idx(p1, j, x0 + 8)] = fmaf(as[nt][3], w, am[nt][3]);
    }
  }
}

// kCrossOnly: only the cross term 2 T : (J_L^T W_off J_R) of the Laplacian row; everything else
// of the merge has been written by merge_tc_kernel (the row holds A_R L_L, lap_b holds A_L L_R),
// and the three terms are added here in a fixed order.
template <bool kCrossOnly>
__global__ void __launch_bounds__(kTsThreads, 1)
merge_tstage_kernel(Level L, const float* __restrict__ T, const float* __restrict__ J_eff,
                    const float* __restrict__ in, float* __restrict__ out,
                    const float* __restrict__ lap_b) {
  extern __shared__ __align__(16) float sm[];
  float* Ts = sm;
  float* AX = Ts + 32768;                       // [16][32][32] swizzled; later C, same layout
  float* vec = AX + kTsPairs * 1024;            // uL, uR, LL, LR : [4][16][36] (until S6)
  float* Ys = vec;                              // per warp [16][32] swizzled (S7), then
  float* red = vec;                             // cross partials [16 warps][16][32]
  float* lap_s = vec + kTsScratchFloats;        // [16][32]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int grp = blockIdx.x;
  const int N = L.N, d = L.d, m = L.m, nodes = L.nodes, nodes_in = 2 * L.nodes;
  const int col0 = grp * kDr;
  const int threeN = 3 * N;

  {  // T_i -> shared, swizzled
    const float* Tg = T + (size_t)grp * 32768;
    for (int idx = tid * 4; idx < 32768; idx += kTsThreads * 4) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(Tg + idx));
      const int l = idx & 31, k = (idx >> 5) & 31, j = idx >> 10;
      *reinterpret_cast<float4*>(Ts + t_idx(j, k, l)) = v;   // l multiple of 4: stays 16B aligned
    }
  }

  const long long total_pairs = (long long)L.Bc * nodes;
  const long long tiles = (total_pairs + kTsPairs - 1) / kTsPairs;
  for (long long tile = blockIdx.y; tile < tiles; tile += gridDim.y) {
    __syncthreads();
    const int mtiles = (m + 15) >> 4;
    // global rows of pair p (warp w owns pairs w and w + 8)
    auto pair_rows = [&](int p, bool& ok, int& pn, const float*& JLg, float*& OLg) {
      const long long pair = tile * kTsPairs + p;
      ok = pair < total_pairs;
      const int pb = ok ? (int)(pair / nodes) : 0;
      pn = ok ? (int)(pair % nodes) : 0;
      JLg = in + (row_j(L.rows_in, pb, pn * 2 * m)) * d + col0;
      OLg = out + (row_j(L.rows_out, pb, pn * 2 * m)) * d + col0;
    };
    if (!kCrossOnly) {
    // ---- S0: child vectors of the 16 pairs
    for (int idx = tid; idx < 4 * kTsPairs * 32; idx += kTsThreads) {
      const int c = idx & 31, p = (idx >> 5) & 15, which = idx >> 9;
      const long long pair = tile * kTsPairs + p;
      float v = 0.f;
      if (pair < total_pairs && (L.jets || which < 2)) {
        const int b = (int)(pair / nodes), n = (int)(pair % nodes);
        const int child = 2 * n + (which & 1);
        const size_t row = (which < 2) ? row_u(L, L.rows_in, nodes_in, b, child)
                                       : row_l(L, L.rows_in, nodes_in, b, child);
        v = in[row * d + col0 + c];
      }
      vec[(which * kTsPairs + p) * kTsVecLd + c] = v;
    }
    __syncthreads();
    const float* uL = vec;
    const float* uR = vec + kTsPairs * kTsVecLd;
    const float* LL = vec + 2 * kTsPairs * kTsVecLd;
    const float* LR = vec + 3 * kTsPairs * kTsVecLd;

    // ---- S1: A_R
    ts_t_apply(Ts, AX, uR, true, warp, g, t);
    __syncthreads();
    // ---- S2: raw = A_R uL, first Laplacian term A_R L_L
    {
      const int p = tid >> 5, j = tid & 31;
      const long long pair = tile * kTsPairs + p;
      float raw = 0.f, l1 = 0.f;
#pragma unroll 8
      for (int k = 0; k < 32; ++k) {
        const float ax = AX[ax_idx(p, j, k)];
        raw = fmaf(ax, uL[p * kTsVecLd + k], raw);
        l1 = fmaf(ax, LL[p * kTsVecLd + k], l1);
      }
      lap_s[p * 32 + j] = l1;
      if (pair < total_pairs) {
        const int b = (int)(pair / nodes), n = (int)(pair % nodes);
        out[row_u(L, L.rows_out, nodes, b, n) * d + col0 + j] = raw;
      }
    }
    if (!L.jets) continue;

    // Og[A][j] = sum_k Jg[A][k] * AX[p][j][k]; the contraction index uses slots
    // (t, t+4) <-> k = (16kk + 4t + 2h, +1) so that both operands load as float4.
    auto apply = [&](int p, const float* Jg, float* Og) {
      for (int mt = 0; mt < mtiles; ++mt) {
        const int A0 = mt * 16 + g, A1 = A0 + 8;
        float am[4][4], as[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) am[i][c] = as[i][c] = 0.f;
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
          const float4 r0 = A0 < m ? *reinterpret_cast<const float4*>(Jg + (size_t)A0 * d + kk * 16 + 4 * t) : z4;
          const float4 r1 = A1 < m ? *reinterpret_cast<const float4*>(Jg + (size_t)A1 * d + kk * 16 + 4 * t) : z4;
          FA2 fa0, fa1;
          fa0.set(r0.x, r1.x, r0.y, r1.y);
          fa1.set(r0.z, r1.z, r0.w, r1.w);
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            const int j = nt * 8 + g;
            const float4 bv = *reinterpret_cast<const float4*>(AX + ax_idx(p, j, kk * 16 + 4 * t));
            FB2 fb0, fb1;
            fb0.set(bv.x, bv.y);
            fb1.set(bv.z, bv.w);
            mma3x(am[nt], as[nt], fa0, fb0);
            mma3x(am[nt], as[nt], fa1, fb1);
          }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int col = nt * 8 + 2 * t;
          if (A0 < m)
            *reinterpret_cast<float2*>(Og + (size_t)A0 * d + col) =
                make_float2(am[nt][0] + as[nt][0], am[nt][1] + as[nt][1]);
          if (A1 < m)
            *reinterpret_cast<float2*>(Og + (size_t)A1 * d + col) =
                make_float2(am[nt][2] + as[nt][2], am[nt][3] + as[nt][3]);
        }
      }
    };

    // ---- S3: left Jacobian rows through A_R
    {
      bool ok; int pn; const float* JLg; float* OLg;
      pair_rows(warp, ok, pn, JLg, OLg);
      if (ok) apply(warp, JLg, OLg);
    }
    __syncthreads();
    // ---- S4: A_L
    ts_t_apply(Ts, AX, uL, false, warp, g, t);
    __syncthreads();
    // ---- S5: second Laplacian term A_L L_R
    {
      const int p = tid >> 5, j = tid & 31;
      float l2 = 0.f;
#pragma unroll 8
      for (int l = 0; l < 32; ++l) l2 = fmaf(AX[ax_idx(p, j, l)], LR[p * kTsVecLd + l], l2);
      lap_s[p * 32 + j] += l2;
    }
    // ---- S6: right Jacobian rows through A_L
    {
      bool ok; int pn; const float* JLg; float* OLg;
      pair_rows(warp, ok, pn, JLg, OLg);
      if (ok) apply(warp, JLg + (size_t)m * d, OLg + (size_t)m * d);
    }
    __syncthreads();      // A_L and the child vectors are dead: their space becomes C / Y
    }   // !kCrossOnly

    // ---- S7: C[k,l] = sum_A J_L[A][k] Y[A][l],  Y = W_off J_R
    float* Yw = Ys + warp * 16 * 32;       // element (r, c) at r*32 + (c ^ ((r & 3) << 3))
    {
      const int p = warp;
      bool ok; int pn; const float* JLg; float* OLg;
      pair_rows(p, ok, pn, JLg, OLg);
      const float* JRg = JLg + (size_t)m * d;
      float cacc[2][4][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) cacc[i][j][c] = 0.f;
      if (ok) {
        const float* Woff = J_eff + (size_t)(pn * 2 * m) * threeN + pn * 2 * m + m;
        const int ksB = (m + 7) >> 3;
        for (int ab = 0; ab < mtiles; ++ab) {
          const int A0 = ab * 16 + g, A1 = A0 + 8;
          float y[4][4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) y[i][c] = 0.f;
          {
            // loads of step kb + 1 are in flight while the MMAs of step kb run
            const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
            auto load_w = [&](int kb, float (&w)[4]) {
              const int B0 = kb * 8 + t, B1 = B0 + 4;
              w[0] = (A0 < m && B0 < m) ? Woff[(size_t)A0 * threeN + B0] : 0.f;
              w[1] = (A1 < m && B0 < m) ? Woff[(size_t)A1 * threeN + B0] : 0.f;
              w[2] = (A0 < m && B1 < m) ? Woff[(size_t)A0 * threeN + B1] : 0.f;
              w[3] = (A1 < m && B1 < m) ? Woff[(size_t)A1 * threeN + B1] : 0.f;
            };
            // column slot g of n-tile nt <-> channel 4g + nt: one 128-bit load per row feeds
            // all four n-tiles
            auto load_j = [&](int kb, float4& v0, float4& v1) {
              const int B0 = kb * 8 + t, B1 = B0 + 4;
              v0 = B0 < m ? *reinterpret_cast<const float4*>(JRg + (size_t)B0 * d + 4 * g) : z4;
              v1 = B1 < m ? *reinterpret_cast<const float4*>(JRg + (size_t)B1 * d + 4 * g) : z4;
            };
            float wn[4];
            float4 n0, n1;
            load_w(0, wn);
            load_j(0, n0, n1);
            for (int kb = 0; kb < ksB; ++kb) {
              FragA fa;
              fa.set(wn[0], wn[1], wn[2], wn[3]);
              const float4 v0 = n0, v1 = n1;
              if (kb + 1 < ksB) {
                load_w(kb + 1, wn);
                load_j(kb + 1, n0, n1);
              }
              FragB fb;
              fb.set(v0.x, v1.x); mma3(y[0], fa, fb);
              fb.set(v0.y, v1.y); mma3(y[1], fa, fb);
              fb.set(v0.z, v1.z); mma3(y[2], fa, fb);
              fb.set(v0.w, v1.w); mma3(y[3], fa, fb);
            }
          }
          __syncwarp();
          {
            // accumulator column slots 2t, 2t+1 of n-tile nt are channels 8t + nt, 8t + 4 + nt
            const int cs = (8 * t) ^ ((g & 3) << 3);              // rows g and g+8 share g & 3
            *reinterpret_cast<float4*>(Yw + g * 32 + cs) = make_float4(y[0][0], y[1][0], y[2][0], y[3][0]);
            *reinterpret_cast<float4*>(Yw + g * 32 + cs + 4) = make_float4(y[0][1], y[1][1], y[2][1], y[3][1]);
            *reinterpret_cast<float4*>(Yw + (g + 8) * 32 + cs) = make_float4(y[0][2], y[1][2], y[2][2], y[3][2]);
            *reinterpret_cast<float4*>(Yw + (g + 8) * 32 + cs + 4) = make_float4(y[0][3], y[1][3], y[2][3], y[3][3]);
          }
          __syncwarp();
          // C += J_L[block]^T Y[block]: rows k, cols l, contraction over the 16 rows A
#pragma unroll
          for (int ks2 = 0; ks2 < 2; ++ks2) {
            const int Aa = ab * 16 + ks2 * 8 + t, Ab = Aa + 4;
            FragB fb[4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
              fb[nt].set(Yw[(ks2 * 8 + t) * 32 + ((nt * 8 + g) ^ (t << 3))],
                         Yw[(ks2 * 8 + t + 4) * 32 + ((nt * 8 + g) ^ (t << 3))]);
            // row slots g, g+8 of m-tile mk <-> channels 4g + 2mk, 4g + 2mk + 1: one 128-bit load
            // per Jacobian row feeds both m-tiles
            const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 u0 = Aa < m ? *reinterpret_cast<const float4*>(JLg + (size_t)Aa * d + 4 * g) : z4;
            const float4 u1 = Ab < m ? *reinterpret_cast<const float4*>(JLg + (size_t)Ab * d + 4 * g) : z4;
            {
              FragA fa;
              fa.set(u0.x, u0.y, u1.x, u1.y);
#pragma unroll
              for (int nt = 0; nt < 4; ++nt) mma3(cacc[0][nt], fa, fb[nt]);
              fa.set(u0.z, u0.w, u1.z, u1.w);
#pragma unroll
              for (int nt = 0; nt < 4; ++nt) mma3(cacc[1][nt], fa, fb[nt]);
            }
          }
        }
      }
#pragma unroll
      for (int mk = 0; mk < 2; ++mk)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int k0 = 4 * g + 2 * mk, l = nt * 8 + 2 * t;      // the row-slot permutation of S7
          *reinterpret_cast<float2*>(AX + ax_idx(p, k0, l)) = make_float2(cacc[mk][nt][0], cacc[mk][nt][1]);
          *reinterpret_cast<float2*>(AX + ax_idx(p, k0 + 1, l)) = make_float2(cacc[mk][nt][2], cacc[mk][nt][3]);
        }
    }
    __syncthreads();
    // ---- cross[j, p] = sum_(k,l) T[j,(k,l)] C[(k,l), p]; warp w contracts k in {2w, 2w+1}
    {
      float acc[2][2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[i][n2][c] = 0.f;
      for (int kq = 0; kq < 2; ++kq) {       // one k per pass: short MMA chains
        const int k = warp * 2 + kq;
        float pm[2][2][4], ps[2][2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
            for (int c = 0; c < 4; ++c) pm[i][n2][c] = ps[i][n2][c] = 0.f;
#pragma unroll
        for (int ks4 = 0; ks4 < 4; ++ks4) {
          const int l = ks4 * 8 + t;
          FB2 fb[2];
#pragma unroll
          for (int n2 = 0; n2 < 2; ++n2)
            fb[n2].set(AX[ax_idx(n2 * 8 + g, k, l)], AX[ax_idx(n2 * 8 + g, k, l + 4)]);
#pragma unroll
          for (int mj = 0; mj < 2; ++mj) {
            const int j0 = mj * 16 + g;
            FA2 fa;
            fa.set(Ts[t_idx(j0, k, l)], Ts[t_idx(j0 + 8, k, l)], Ts[t_idx(j0, k, l + 4)],
                   Ts[t_idx(j0 + 8, k, l + 4)]);
            mma3x(pm[mj][0], ps[mj][0], fa, fb[0]);
            mma3x(pm[mj][1], ps[mj][1], fa, fb[1]);
          }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][n2][c] += pm[i][n2][c] + ps[i][n2][c];
      }
      // red[warp][p][j] overlays the Y scratch: dead, every warp passed the barrier after S7
#pragma unroll
      for (int mj = 0; mj < 2; ++mj)
#pragma unroll
        for (int n2 = 0; n2 < 2; ++n2) {
          const int j0 = mj * 16 + g, p0 = n2 * 8 + 2 * t;
          red[(warp * 16 + p0) * 32 + j0] = acc[mj][n2][0];
          red[(warp * 16 + p0 + 1) * 32 + j0] = acc[mj][n2][1];
          red[(warp * 16 + p0) * 32 + j0 + 8] = acc[mj][n2][2];
          red[(warp * 16 + p0 + 1) * 32 + j0 + 8] = acc[mj][n2][3];
        }
    }
    __syncthreads();
    {
      const int p = tid >> 5, j = tid & 31;
      const long long pair = tile * kTsPairs + p;
      float cross = 0.f;
#pragma unroll
      for (int w = 0; w < kTsWarps; ++w) cross += red[(w * 16 + p) * 32 + j];
      if (pair < total_pairs) {
        const int b = (int)(pair / nodes), n = (int)(pair % nodes);
        float* dst = out + row_l(L, L.rows_out, nodes, b, n) * d + col0 + j;
        if (kCrossOnly) *dst = (*dst + lap_b[(size_t)pair * d + col0 + j]) + 2.f * cross;
        else *dst = lap_s[p * 32 + j] + 2.f * cross;
      }
    }
  }
}

#include "hz_merge_tc.cuh"
#include "hz_cross_tc.cuh"

// ------------------------------------------------------------------ normalisation: reduce
// One CTA per (walker, node): over column tiles of `out`'s Jacobian rows J [2m, d]
//   oo = |out|^2, oL = out.L, a[A] = J_A.out, gram = sum_AB W_AB J_A.J_B
// then the scalar jets of sigma = sqrt(oo/d + eps): r = 1/sigma, dr, W dr, lap r,
// log sigma and the gated scalar carriers s, Js, Ls of the next level.
constexpr int kNrThreads = 256;
constexpr int kNrWarps = kNrThreads / 32;
// column tile of norm_reduce: 64 for the wide upper levels (W fills shared memory), 256 for
// the lower ones (few rows per node, so the per-tile barriers would dominate)
constexpr int kNrColsWide = 256, kNrColsNarrow = 64;
// Nodes with more than 192 Jacobian rows (trees of 128 and 256 sites, upper levels): the W block
// no longer fits shared memory; it is then read from J_eff (L2-resident) and the column tile
// shrinks to 32 so that the Jacobian tile still fits.
constexpr int kNrColsHuge = 32, kNrMaxRowsShared = 192;

struct NormOut {          // per (walker, node)
  float r, lap_r;
};

__host__ __device__ inline int pad16(int x) { return (x + 15) & ~15; }

template <int kNrCols, bool kWGlobal>
__global__ void __launch_bounds__(kNrThreads)
norm_reduce_kernel(Level L, float eps, const float* __restrict__ J_eff,
                   const uint8_t* __restrict__ opcodes, const float* __restrict__ X,
                   const float* __restrict__ s_in, const float* __restrict__ js_in,
                   const float* __restrict__ ls_in, float* __restrict__ s_out,
                   float* __restrict__ js_out, float* __restrict__ ls_out,
                   NormOut* __restrict__ nout, float* __restrict__ dr_out,
                   float* __restrict__ wdr_out,
                   const float* __restrict__ gram_in /* nullable: [Bc, blocks, 3N] partial sums of the tcgen05 kernel */,
                   const float* __restrict__ a_in /* with gram_in: [Bc, 3N] = J_A . out */,
                   const float* __restrict__ oo_in /* nullable, with gram_in: [Bc, nodes] |out|^2 */,
                   const float* __restrict__ oL_in /* with oo_in: [Bc, nodes] out . L */) {
  constexpr int kNrJLd = kNrCols + 8;
  // pre: the quadratic form and the dots J_A . out come from the tcgen05 kernel; only |out|^2 and
  // out . L are taken here (requires kWGlobal, whose W reads need no staging)
  const bool pre = gram_in != nullptr;
  extern __shared__ __align__(16) float sm[];
  const int N = L.N, d = L.d, nodes = L.nodes, m2 = 2 * L.m, threeN = 3 * N;
  const int mp = pad16(m2), wld = kWGlobal ? threeN : mp + 4;
  const int n = blockIdx.x, b = blockIdx.y;
  // W block of the node: staged [mp][mp + 4] in shared memory, or (kWGlobal; m2 is then a
  // multiple of 16, so no padding is read) straight from J_eff
  const float* Ws = kWGlobal ? J_eff + (size_t)(n * m2) * threeN + n * m2 : sm;
  float* Js = sm + ((L.jets && !kWGlobal) ? mp * wld : 0);   // [mp][kNrJLd]
  float* outs = Js + ((L.jets && !pre) ? mp * kNrJLd : 0);   // [kNrCols]
  float* a_s = outs + kNrCols;          // [mp]
  float* v_s = a_s + mp;                // [mp] scratch vector
  float* scratch = v_s + mp;            // [3 * kNrWarps]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rows = L.rows_out;
  const float* urow = X + row_u(L, rows, nodes, b, n) * d;
  const float* lrow = L.jets ? X + row_l(L, rows, nodes, b, n) * d : nullptr;
  const float* jrows = L.jets ? X + row_j(rows, b, n * m2) * d : nullptr;

  float red[3] = {0.f, 0.f, 0.f};       // oo, oL, gram
  if (L.jets) {
    if (!kWGlobal) {
      float* Wst = sm;
      for (int idx = tid; idx < mp * mp; idx += kNrThreads) {
        const int A = idx / mp, Bc = idx % mp;
        Wst[A * wld + Bc] = (A < m2 && Bc < m2)
                                ? J_eff[(size_t)(n * m2 + A) * threeN + n * m2 + Bc] : 0.f;
      }
    }
    for (int A = tid; A < mp; A += kNrThreads) a_s[A] = 0.f;
  }
  // Value-and-gradient pass: only |out|^2, out . L and the dots J_A . out are needed, a
  // matrix-vector product that is bound by the one read of the node's rows. It goes straight
  // from global memory - the value row in registers, every warp a row at a time, twelve 16-byte
  // loads per lane in flight - instead of through the column tiles and their two barriers each.
  const bool direct = L.jets == 2 && !pre && (d & 127) == 0 && d <= 2048;
  if (direct) {
    __syncthreads();                       // a_s is zeroed
    const int nch = d >> 7;                // chunks of 128 floats: one float4 per lane
    float4 o4[16];
#pragma unroll
    for (int c = 0; c < 16; ++c)
      if (c < nch) o4[c] = __ldg(reinterpret_cast<const float4*>(urow) + c * 32 + lane);
    auto dot_row = [&](const float* row) {
      const float4* r4 = reinterpret_cast<const float4*>(row);
      float part = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c)
        if (c < nch) {
          const float4 v = __ldg(r4 + c * 32 + lane);
          part = fmaf(v.x, o4[c].x, part); part = fmaf(v.y, o4[c].y, part);
          part = fmaf(v.z, o4[c].z, part); part = fmaf(v.w, o4[c].w, part);
        }
      return part;
    };
    if (warp == 0) red[0] = dot_row(urow);
    if (warp == 1) red[1] = dot_row(lrow);
    for (int A = warp; A < m2; A += kNrWarps) {
      const float part = warp_sum(dot_row(jrows + (size_t)A * d));
      if (lane == 0) a_s[A] = part;
    }
  }
  for (int c0 = 0; c0 < ((oo_in != nullptr || direct) ? 0 : d); c0 += kNrCols) {
    __syncthreads();
    for (int i = tid; i < kNrCols; i += kNrThreads) {
      const int c = c0 + i;
      const float o = c < d ? urow[c] : 0.f;
      outs[i] = o;
      red[0] += o * o;
      if (L.jets && c < d) red[1] += o * lrow[c];
    }
    if (L.jets && !pre) {
      for (int idx = tid; idx < mp * (kNrCols / 4); idx += kNrThreads) {
        const int A = idx / (kNrCols / 4), c = (idx % (kNrCols / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (A < m2 && c0 + c < d) v = *reinterpret_cast<const float4*>(jrows + (size_t)A * d + c0 + c);
        *reinterpret_cast<float4*>(Js + A * kNrJLd + c) = v;
      }
    }
    __syncthreads();
    if (!L.jets || pre) continue;
    // a[A] += J_A . out over this tile: warp w owns rows w, w + kNrWarps, ...
    for (int A = warp; A < m2; A += kNrWarps) {
      float part = 0.f;
#pragma unroll
      for (int c = lane; c < kNrCols; c += 32) part = fmaf(Js[A * kNrJLd + c], outs[c], part);
      part = warp_sum(part);
      if (lane == 0) a_s[A] += part;
    }
    if (L.jets == 2) continue;      // value-and-gradient pass: no Laplacian, W is never read
    // gram += sum_{A,c} (W J)[A,c] * J[A,c] on the tensor cores. One work item is one
    // 16-row block of W against four 8-column blocks of J, so that a W fragment is split once
    // for twelve MMAs.
    const int mts = mp >> 4, kss = mp >> 3;
    constexpr int kGroups = kNrCols / 32;      // groups of four 8-column blocks
    for (int item = warp; item < mts * kGroups; item += kNrWarps) {
      const int mt = item / kGroups, nt0 = (item % kGroups) * 4;
      float acc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
      // W and J J^T are symmetric: only the blocks on and above the diagonal of this row block
      // are contracted, the blocks above the diagonal with weight two.
      for (int kq = 2 * mt; kq < kss; kq += 4) {      // short MMA chains, folded with fp32 adds
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) part[i][c] = 0.f;
        // the first chain holds exactly the diagonal block (two k-steps)
        const int kend = (kq == 2 * mt) ? kq + 2 : min(kss, kq + 4);
        for (int ks = kq; ks < kend; ++ks) {
          FA2 fa;
          const float* w0 = Ws + (mt * 16 + g) * wld + ks * 8 + t;
          fa.set(w0[0], w0[8 * wld], w0[4], w0[8 * wld + 4]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            FB2 fb;
            fb.set(Js[(ks * 8 + t) * kNrJLd + (nt0 + i) * 8 + g],
                   Js[(ks * 8 + t + 4) * kNrJLd + (nt0 + i) * 8 + g]);
            mma_tf32(part[i], fa.lo, fb.hi);
            mma_tf32(part[i], fa.hi, fb.lo);
            mma_tf32(part[i], fa.hi, fb.hi);
          }
        }
        const float wgt = (kq == 2 * mt) ? 1.f : 2.f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[i][c] += wgt * part[i][c];
        if (kq == 2 * mt) kq -= 2;      // the next chain starts right after the diagonal block
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float* j0 = Js + (mt * 16 + g) * kNrJLd + (nt0 + i) * 8 + 2 * t;
        red[2] += acc[i][0] * j0[0] + acc[i][1] * j0[1] + acc[i][2] * j0[8 * kNrJLd] +
                  acc[i][3] * j0[8 * kNrJLd + 1];
      }
    }
  }
  if (pre) {
    // tr(W J J^T) of the node: its rows' partial sums over the column blocks on and after each
    // row's own block, in a fixed order
    const int blocks = (threeN + 2 * nodes + 127) / 128;
    for (int idx = tid; idx < m2 * blocks; idx += kNrThreads) {
      const int A = n * m2 + idx % m2, bj = idx / m2;
      if (bj >= A / 128) red[2] += gram_in[((size_t)b * blocks + bj) * threeN + A];
    }
  }
  block_sum<3, kNrThreads>(red, scratch);
  if (pre) {
    if (oo_in != nullptr) {
      red[0] = oo_in[(size_t)b * nodes + n];
      red[1] = oL_in[(size_t)b * nodes + n];
    }
    for (int A = tid; A < m2; A += kNrThreads) a_s[A] = a_in[(size_t)b * threeN + n * m2 + A];
    __syncthreads();
  }

  const float inv_d = 1.f / (float)d;
  const float y = red[0] * inv_d + eps;
  const float r = rsqrtf(y);
  const float s_val = 0.5f * logf(y);
  const uint8_t op = opcodes[n];
  const int left = 2 * n, right = 2 * n + 1, nodes_in = 2 * nodes;
  const float sl = s_in[(size_t)b * nodes_in + left], sr = s_in[(size_t)b * nodes_in + right];
  float lap_r = 0.f;
  if (L.jets) {
    // v = W dy with dy = (2/d) a
    for (int A = tid; A < m2; A += kNrThreads) {
      float acc = 0.f;
      if (L.jets != 2)
        for (int Bc = 0; Bc < m2; ++Bc) acc = fmaf(Ws[A * wld + Bc], a_s[Bc], acc);
      v_s[A] = 2.f * inv_d * acc;
    }
    __syncthreads();
    float q[1] = {0.f};
    for (int A = tid; A < m2; A += kNrThreads) q[0] += 2.f * inv_d * a_s[A] * v_s[A];
    block_sum<1, kNrThreads>(q, scratch);
    const float dywdy = q[0];
    const float lap_y = 2.f * inv_d * (red[1] + red[2]);
    const float y15 = r * r * r, y25 = y15 * r * r;
    lap_r = -0.5f * y15 * lap_y + 0.75f * y25 * dywdy;
    const float s_lap = 0.5f * (lap_y / y - dywdy / (y * y));
    const int m = L.m;
    for (int A = tid; A < m2; A += kNrThreads) {
      const float dy = 2.f * inv_d * a_s[A];
      const size_t row = (size_t)b * threeN + n * m2 + A;
      dr_out[row] = -0.5f * y15 * dy;
      wdr_out[row] = -0.5f * y15 * v_s[A];
      const float js_child = js_in[row];
      float js = 0.f;
      if (op == 0) js = js_child + 0.5f * dy / y;
      else if (op == 1) js = (A < m) ? js_child : 0.f;
      else if (op == 2) js = (A >= m) ? js_child : 0.f;
      js_out[row] = js;
    }
    if (tid == 0) {
      const float ll = ls_in[(size_t)b * nodes_in + left], lr = ls_in[(size_t)b * nodes_in + right];
      float ls = 0.f;
      if (op == 0) ls = ll + lr + s_lap;
      else if (op == 1) ls = ll;
      else if (op == 2) ls = lr;
      ls_out[(size_t)b * nodes + n] = ls;
    }
  }
  if (tid == 0) {
    float s = 0.f;
    if (op == 0) s = sl + sr + s_val;
    else if (op == 1) s = sl;
    else if (op == 2) s = sr;
    s_out[(size_t)b * nodes + n] = s;
    nout[(size_t)b * nodes + n] = NormOut{r, lap_r};
  }
}

// ------------------------------------------------------------------ normalisation: apply
// In place on X: u = r out, J_A = r J_A + dr_A out, L = r L + lap_r out + 2 sum_A (W dr)_A J_A,
// then the opcode gate (MERGE / CARRY_LEFT / CARRY_RIGHT / EMPTY, compiled/types.py:15-19);
// carried children come from the previous level's buffer.
constexpr int kNaThreads = 256;

__global__ void __launch_bounds__(kNaThreads)
norm_apply_kernel(Level L, const uint8_t* __restrict__ opcodes, const float* __restrict__ prev,
                  float* __restrict__ X, const NormOut* __restrict__ nout,
                  const float* __restrict__ dr, const float* __restrict__ wdr) {
  extern __shared__ float sm[];
  const int N = L.N, d = L.d, nodes = L.nodes, m = L.m, m2 = 2 * L.m, threeN = 3 * N;
  float* dr_s = sm;
  float* wdr_s = sm + m2;
  const int n = blockIdx.y, b = blockIdx.z;
  const int c = blockIdx.x * kNaThreads + threadIdx.x;
  const uint8_t op = opcodes[n];
  if (L.jets)
    for (int A = threadIdx.x; A < m2; A += kNaThreads) {
      dr_s[A] = dr[(size_t)b * threeN + n * m2 + A];
      wdr_s[A] = wdr[(size_t)b * threeN + n * m2 + A];
    }
  __syncthreads();
  if (c >= d) return;
  const NormOut no = nout[(size_t)b * nodes + n];
  const int rows = L.rows_out, nodes_in = 2 * nodes;
  float* urow = X + row_u(L, rows, nodes, b, n) * d;
  if (op == 0) {
    const float o = urow[c];
    urow[c] = o * no.r;
    if (L.jets) {
      float* lrow = X + row_l(L, rows, nodes, b, n) * d;
      float* jrows = X + row_j(rows, b, n * m2) * d;
      float acc = 0.f;
      int A = 0;
      for (; A + 8 <= m2; A += 8) {       // eight independent row loads in flight per thread
        float j[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) j[i] = jrows[(size_t)(A + i) * d + c];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          jrows[(size_t)(A + i) * d + c] = j[i] * no.r + dr_s[A + i] * o;
          acc = fmaf(wdr_s[A + i], j[i], acc);
        }
      }
      for (; A < m2; ++A) {
        const float j = jrows[(size_t)A * d + c];
        jrows[(size_t)A * d + c] = j * no.r + dr_s[A] * o;
        acc = fmaf(wdr_s[A], j, acc);
      }
      lrow[c] = lrow[c] * no.r + o * no.lap_r + 2.f * acc;
    }
    return;
  }
  // carried or empty node
  const int child = 2 * n + (op == 2 ? 1 : 0);
  const bool carry = (op == 1 || op == 2);
  urow[c] = carry ? prev[row_u(L, L.rows_in, nodes_in, b, child) * d + c] : 0.f;
  if (L.jets) {
    X[row_l(L, rows, nodes, b, n) * d + c] =
        carry ? prev[row_l(L, L.rows_in, nodes_in, b, child) * d + c] : 0.f;
    float* jrows = X + row_j(rows, b, n * m2) * d;
    const float* pj = prev + row_j(L.rows_in, b, n * m2) * d;    // same row indices
    for (int A = 0; A < m2; ++A) {
      const bool keep = carry && ((op == 1) ? (A < m) : (A >= m));
      jrows[(size_t)A * d + c] = keep ? pj[(size_t)A * d + c] : 0.f;
    }
  }
}

// Value-only passes: normalisation and opcode gate of a level in one kernel, one warp per
// (walker, node) row kept in registers between the sum of squares and the scaled store (the
// general pair norm_reduce_kernel + norm_apply_kernel reads the row twice and runs one small CTA
// per row). d <= 2048, a multiple of 4.
constexpr int kNvMaxD = 2048;
__global__ void __launch_bounds__(256)
norm_values_kernel(int d, int nodes, long long rows_total, float eps, const uint8_t* __restrict__ opcodes,
                   const float* __restrict__ prev, float* __restrict__ X, const float* __restrict__ s_in,
                   float* __restrict__ s_out, NormOut* __restrict__ nout) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows_total) return;
  const int lane = threadIdx.x & 31, n = (int)(row % nodes), d4 = d >> 2;
  const uint8_t op = opcodes[n];
  float4* xrow = reinterpret_cast<float4*>(X + (size_t)row * d);
  float4 v[kNvMaxD / 128];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNvMaxD / 128; ++i) {
    const int c = lane + 32 * i;
    if (c < d4) {
      v[i] = xrow[c];
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  ss = warp_sum(ss);
  const float y = ss / (float)d + eps;
  const float r = rsqrtf(y);
  const float sl = s_in[2 * row], sr = s_in[2 * row + 1];
  if (op == 0) {
#pragma unroll
    for (int i = 0; i < kNvMaxD / 128; ++i) {
      const int c = lane + 32 * i;
      if (c < d4) xrow[c] = make_float4(v[i].x * r, v[i].y * r, v[i].z * r, v[i].w * r);
    }
  } else {
    const bool carry = (op == 1 || op == 2);
    const float4* crow = reinterpret_cast<const float4*>(prev + (size_t)(2 * row + (op == 2 ? 1 : 0)) * d);
    for (int c = lane; c < d4; c += 32) xrow[c] = carry ? crow[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (lane == 0) {
    s_out[row] = op == 0 ? sl + sr + 0.5f * logf(y) : (op == 1 ? sl : (op == 2 ? sr : 0.f));
    nout[row] = NormOut{r, 0.f};
  }
}

// the level's block-diagonal W for syrk_tc_kernel: J_eff where both rows belong to one node
__global__ void syrk_w_mask_kernel(const float* __restrict__ J_eff, int three_n, int m2,
                                   float* __restrict__ W) {
  const int A = blockIdx.x;
  for (int B = threadIdx.x; B < three_n; B += blockDim.x)
    W[(size_t)A * three_n + B] = (A / m2 == B / m2) ? J_eff[(size_t)A * three_n + B] : 0.f;
}

// ------------------------------------------------------------------ first tree level in coefficient space
// A leaf carrier is linear in its quaternion: u_raw = q . M_site with M_site [4, d] the leaf
// map. So every jet row of a leaf (value, three Jacobian rows, Laplacian) is a 4-vector of
// coefficients over the rows of M_site, and every jet row of a first-level node - bilinear
// in its two leaves, then through the linear factor map - is a 16-vector over
//   Phi_n[4o+o'] = F_h(T(M_left[o], M_right[o']))           (walker independent).
// The first level, which holds half of the tree's nodes, therefore needs no tensor
// application and no GEMM per walker: Phi_n and its 16x16 Gram matrix are built once per
// call (with the generic kernels, on a fake batch of 16 "walkers"), each (walker, node)
// then costs a few hundred flops of coefficient algebra (l1_coeff_kernel) and one 8 x 24
// by 24 x d product to materialise its rows for the second level (l1_expand_kernel).
// Carried children (CARRY_LEFT / CARRY_RIGHT) use the extra basis rows M_left, M_right.
constexpr int kL1Basis = 24;

__global__ void leaf_gram_kernel(const float* __restrict__ leaf_map, float* __restrict__ Gs, int d) {
  __shared__ float scratch[16 * 4];
  const float* M = leaf_map + (size_t)blockIdx.x * 4 * d;
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  for (int c = threadIdx.x; c < d; c += 128) {
    const float m[4] = {M[c], M[d + c], M[2 * d + c], M[3 * d + c]};
#pragma unroll
    for (int o = 0; o < 4; ++o)
#pragma unroll
      for (int p = 0; p < 4; ++p) acc[o * 4 + p] += m[o] * m[p];
  }
  block_sum<16, 128>(acc, scratch);
  if (threadIdx.x < 16) Gs[blockIdx.x * 16 + threadIdx.x] = acc[threadIdx.x];
}

// The once-per-call bases are built by running the merge and factor kernels on "fake batches"
// whose rows are raw map rows, not RMS-normalised carriers. Their magnitude follows the model's
// leaf weights and is unbounded, while the merge kernel's two-term FP16 split needs operands of
// moderate size. Every fake row is therefore scaled by a power of two that brings its largest
// entry into [1/2, 1) (exact in fp32), and the bilinear result is scaled back by the sum of its
// two children's exponents.
__global__ void row_exponent_kernel(const float* __restrict__ rows, int* __restrict__ expo, int d) {
  __shared__ float scratch[128 / 32];
  float mx[1] = {0.f};
  const float* src = rows + (size_t)blockIdx.x * d;
  for (int c = threadIdx.x; c < d; c += 128) mx[0] = fmaxf(mx[0], fabsf(src[c]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = mx[0];
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = fmaxf(fmaxf(scratch[0], scratch[1]), fmaxf(scratch[2], scratch[3]));
    int e = 0;
    if (m > 0.f && isfinite(m)) frexpf(m, &e);       // m = f * 2^e, f in [1/2, 1)
    expo[blockIdx.x] = e;
  }
}

// rows of the fake batch: walker w = 4o + o', site s -> M_s[o] (s even) or M_s[o'] (s odd)
__global__ void l1_fake_kernel(const float* __restrict__ leaf_map, const int* __restrict__ expo,
                               float* __restrict__ U, int N, int d) {
  const int s = blockIdx.x, wk = blockIdx.y;
  const int o = (s & 1) ? (wk & 3) : (wk >> 2);
  const float* src = leaf_map + ((size_t)s * 4 + o) * d;
  const int e = expo[s * 4 + o];
  float* dst = U + ((size_t)wk * N + s) * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) dst[c] = ldexpf(src[c], -e);
}

// undo the row scaling of a fake batch on the merged rows: row (wk, n) was built from child rows
// with exponents expo[(2n) * per + left(wk)] and expo[(2n + 1) * per + right(wk)]
__global__ void fake_unscale_kernel(float* __restrict__ Phi, const int* __restrict__ expo, int nodes,
                                    int per, int d) {
  const int n = blockIdx.x, wk = blockIdx.y;
  const int e = expo[(2 * n) * per + wk / per] + expo[(2 * n + 1) * per + wk % per];
  float* row = Phi + ((size_t)wk * nodes + n) * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) row[c] = ldexpf(row[c], e);
}

// G16[n][w][w'] = Phi[w][n] . Phi[w'][n]
__global__ void l1_gram_kernel(const float* __restrict__ Phi, float* __restrict__ G16, int nodes, int d) {
  const int n = blockIdx.x, w0 = threadIdx.x >> 4, w1 = threadIdx.x & 15;
  const float4* a = reinterpret_cast<const float4*>(Phi + ((size_t)w0 * nodes + n) * d);
  const float4* b = reinterpret_cast<const float4*>(Phi + ((size_t)w1 * nodes + n) * d);
  float acc = 0.f;
  for (int c = 0; c < d / 4; ++c) {
    const float4 x = a[c], y = b[c];
    acc += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
  }
  G16[(size_t)n * 256 + threadIdx.x] = acc;
}

struct LeafCoef {
  float al[4], be[3][4], ga[4], s, js[3], ls;
};

__device__ __forceinline__ void leaf_coefficients(const float* __restrict__ qq,
                                                  const float* __restrict__ G,
                                                  const float* __restrict__ J_eff, int N, int site,
                                                  int d, int jets, LeafCoef& o) {
  const float q[4] = {qq[0], qq[1], qq[2], qq[3]};
  float Gq[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) Gq[i] = G[i * 4] * q[0] + G[i * 4 + 1] * q[1] + G[i * 4 + 2] * q[2] + G[i * 4 + 3] * q[3];
  const float oo = q[0] * Gq[0] + q[1] * Gq[1] + q[2] * Gq[2] + q[3] * Gq[3];
  const float inv_d = 1.f / (float)d;
  const float y = oo * inv_d + kLeafEps;
  const float r = rsqrtf(y);
  o.s = 0.5f * logf(y);
#pragma unroll
  for (int i = 0; i < 4; ++i) o.al[i] = r * q[i];
  if (!jets) return;
  const float dq[3][4] = {{-q[3], q[2], -q[1], q[0]}, {-q[2], -q[3], q[0], q[1]}, {-q[1], q[0], q[3], -q[2]}};
  float W[3][3];
#pragma unroll
  for (int a = 0; a < 3; ++a)
#pragma unroll
    for (int c = 0; c < 3; ++c) W[a][c] = J_eff[(size_t)(3 * site + a) * (3 * N) + 3 * site + c];
  const float trW = W[0][0] + W[1][1] + W[2][2];
  float Gd[3][4], aA[3], gram = 0.f;
#pragma unroll
  for (int a = 0; a < 3; ++a) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      Gd[a][i] = G[i * 4] * dq[a][0] + G[i * 4 + 1] * dq[a][1] + G[i * 4 + 2] * dq[a][2] + G[i * 4 + 3] * dq[a][3];
    aA[a] = dq[a][0] * Gq[0] + dq[a][1] * Gq[1] + dq[a][2] * Gq[2] + dq[a][3] * Gq[3];
  }
#pragma unroll
  for (int a = 0; a < 3; ++a)
#pragma unroll
    for (int b = 0; b < 3; ++b)
      gram += W[a][b] * (dq[a][0] * Gd[b][0] + dq[a][1] * Gd[b][1] + dq[a][2] * Gd[b][2] + dq[a][3] * Gd[b][3]);
  const float dy[3] = {2.f * inv_d * aA[0], 2.f * inv_d * aA[1], 2.f * inv_d * aA[2]};
  const float lap_y = 2.f * inv_d * (-trW * oo + gram);
  float wdy[3], dywdy = 0.f;
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    wdy[a] = W[a][0] * dy[0] + W[a][1] * dy[1] + W[a][2] * dy[2];
    dywdy += dy[a] * wdy[a];
  }
  const float y15 = r * r * r, y25 = y15 * r * r;
  const float lap_r = -0.5f * y15 * lap_y + 0.75f * y25 * dywdy;
  o.ls = 0.5f * (lap_y / y - dywdy / (y * y));
  float wdr[3];
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    const float dr = -0.5f * y15 * dy[a];
    wdr[a] = -0.5f * y15 * wdy[a];
    o.js[a] = 0.5f * dy[a] / y;
#pragma unroll
    for (int i = 0; i < 4; ++i) o.be[a][i] = r * dq[a][i] + dr * q[i];
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    o.ga[i] = (-trW * r + lap_r) * q[i] + 2.f * (wdr[0] * dq[0][i] + wdr[1] * dq[1][i] + wdr[2] * dq[2][i]);
}

struct L1Args {
  int N, d, nodes, jets, Bc;
  float eps;
  const float* q;        // [Bc, N, 4]
  const float* Gs;       // [N, 16]
  const float* G16;      // [nodes, 256]
  const float* J_eff;
  const uint8_t* opcodes;
  float* coef;           // [Bc, nodes, R, 24], R = 8 (J0..J5, U, L) or 1 (U)
  float* s_out;
  float* js_out;
  float* ls_out;
};

__device__ __forceinline__ void matvec16(const float* __restrict__ G, const float* x, float* y) {
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) acc = fmaf(G[i * 16 + j], x[j], acc);
    y[i] = acc;
  }
}
__device__ __forceinline__ float dot16(const float* a, const float* b) {
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) acc = fmaf(a[j], b[j], acc);
  return acc;
}

__global__ void __launch_bounds__(128) l1_coeff_kernel(L1Args a) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)a.Bc * a.nodes) return;
  const int b = (int)(idx / a.nodes), n = (int)(idx % a.nodes);
  const int N = a.N, d = a.d, jets = a.jets, threeN = 3 * N;
  const int R = jets ? 8 : 1;
  LeafCoef lc, rc;
  leaf_coefficients(a.q + ((size_t)b * N + 2 * n) * 4, a.Gs + (2 * n) * 16, a.J_eff, N, 2 * n, d, jets, lc);
  leaf_coefficients(a.q + ((size_t)b * N + 2 * n + 1) * 4, a.Gs + (2 * n + 1) * 16, a.J_eff, N, 2 * n + 1, d, jets, rc);
  const uint8_t op = a.opcodes[n];
  float* out = a.coef + (size_t)idx * R * kL1Basis;
  float* s_o = a.s_out + (size_t)b * a.nodes + n;

  if (op != 0) {        // carried child or empty node: coefficients over M_left / M_right
    for (int i = 0; i < R * kL1Basis; ++i) out[i] = 0.f;
    const LeafCoef& c = (op == 2) ? rc : lc;
    const int off = (op == 2) ? 20 : 16;
    const bool carry = (op == 1 || op == 2);
    float* urow = out + (jets ? 6 : 0) * kL1Basis;
    if (carry)
      for (int i = 0; i < 4; ++i) urow[off + i] = c.al[i];
    *s_o = carry ? c.s : 0.f;
    if (jets) {
      const int a0 = (op == 2) ? 3 : 0;
      for (int A = 0; A < 6; ++A) {
        const bool keep = carry && A >= a0 && A < a0 + 3;
        a.js_out[(size_t)b * threeN + 6 * n + A] = keep ? c.js[A - a0] : 0.f;
        if (keep)
          for (int i = 0; i < 4; ++i) out[A * kL1Basis + off + i] = c.be[A - a0][i];
      }
      if (carry)
        for (int i = 0; i < 4; ++i) out[7 * kL1Basis + off + i] = c.ga[i];
      a.ls_out[(size_t)b * a.nodes + n] = carry ? c.ls : 0.f;
    }
    return;
  }

  const float* G = a.G16 + (size_t)n * 256;
  float cU[16], gU[16];
#pragma unroll
  for (int o = 0; o < 4; ++o)
#pragma unroll
    for (int p = 0; p < 4; ++p) cU[o * 4 + p] = lc.al[o] * rc.al[p];
  matvec16(G, cU, gU);
  const float inv_d = 1.f / (float)d;
  const float y = dot16(cU, gU) * inv_d + a.eps;
  const float r = rsqrtf(y);
  *s_o = lc.s + rc.s + 0.5f * logf(y);
  if (!jets) {
    for (int i = 0; i < 16; ++i) out[i] = r * cU[i];
    for (int i = 16; i < kL1Basis; ++i) out[i] = 0.f;
    return;
  }
  float cJ[6][16], cL[16];
#pragma unroll
  for (int A = 0; A < 3; ++A)
#pragma unroll
    for (int o = 0; o < 4; ++o)
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        cJ[A][o * 4 + p] = lc.be[A][o] * rc.al[p];
        cJ[3 + A][o * 4 + p] = lc.al[o] * rc.be[A][p];
      }
  float W2[6][6];
  for (int A = 0; A < 6; ++A)
    for (int B = 0; B < 6; ++B) W2[A][B] = a.J_eff[(size_t)(6 * n + A) * threeN + 6 * n + B];
  {
    float wb[3][4];      // sum_B W_off[A][B] beR[B][p]
#pragma unroll
    for (int A = 0; A < 3; ++A)
#pragma unroll
      for (int p = 0; p < 4; ++p)
        wb[A][p] = W2[A][3] * rc.be[0][p] + W2[A][4] * rc.be[1][p] + W2[A][5] * rc.be[2][p];
#pragma unroll
    for (int o = 0; o < 4; ++o)
#pragma unroll
      for (int p = 0; p < 4; ++p)
        cL[o * 4 + p] = lc.ga[o] * rc.al[p] + lc.al[o] * rc.ga[p] +
                        2.f * (lc.be[0][o] * wb[0][p] + lc.be[1][o] * wb[1][p] + lc.be[2][o] * wb[2][p]);
  }
  float aA[6], gram = 0.f;
  {
    float gJ[6][16];
    for (int A = 0; A < 6; ++A) {
      matvec16(G, cJ[A], gJ[A]);
      aA[A] = dot16(cJ[A], gU);
    }
    for (int A = 0; A < 6; ++A)
      for (int B = 0; B < 6; ++B) gram += W2[A][B] * dot16(cJ[A], gJ[B]);
  }
  const float oL = dot16(cL, gU);
  float dy[6], wdy[6], dywdy = 0.f;
  for (int A = 0; A < 6; ++A) dy[A] = 2.f * inv_d * aA[A];
  for (int A = 0; A < 6; ++A) {
    float acc = 0.f;
    for (int B = 0; B < 6; ++B) acc += W2[A][B] * dy[B];
    wdy[A] = acc;
    dywdy += dy[A] * acc;
  }
  const float lap_y = 2.f * inv_d * (oL + gram);
  const float y15 = r * r * r, y25 = y15 * r * r;
  const float lap_r = -0.5f * y15 * lap_y + 0.75f * y25 * dywdy;
  const float s_lap = 0.5f * (lap_y / y - dywdy / (y * y));
  a.ls_out[(size_t)b * a.nodes + n] = lc.ls + rc.ls + s_lap;
  float lacc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) lacc[i] = r * cL[i] + lap_r * cU[i];
  for (int A = 0; A < 6; ++A) {
    const float dr = -0.5f * y15 * dy[A], wdr = -0.5f * y15 * wdy[A];
    a.js_out[(size_t)b * threeN + 6 * n + A] = (A < 3 ? lc.js[A] : rc.js[A - 3]) + 0.5f * dy[A] / y;
    float* row = out + A * kL1Basis;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      row[i] = r * cJ[A][i] + dr * cU[i];
      lacc[i] += 2.f * wdr * cJ[A][i];
    }
    for (int i = 16; i < kL1Basis; ++i) row[i] = 0.f;
  }
  float* urow = out + 6 * kL1Basis;
  float* lrow = out + 7 * kL1Basis;
  for (int i = 0; i < 16; ++i) { urow[i] = r * cU[i]; lrow[i] = lacc[i]; }
  for (int i = 16; i < kL1Basis; ++i) { urow[i] = 0.f; lrow[i] = 0.f; }
}

// rows of first-level node n of every walker: coef [R, 24] x basis [24, d]
constexpr int kL1WalkersPerCta = 32;
__global__ void __launch_bounds__(256)
l1_expand_kernel(Level L, const float* __restrict__ coef, const float* __restrict__ Phi,
                 const float* __restrict__ leaf_map, float* __restrict__ out) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  const int n = blockIdx.y, nodes = L.nodes, d = L.d;
  if (c >= d) return;
  float basis[kL1Basis];
#pragma unroll
  for (int w = 0; w < 16; ++w) basis[w] = Phi[((size_t)w * nodes + n) * d + c];
#pragma unroll
  for (int o = 0; o < 4; ++o) {
    basis[16 + o] = leaf_map[((size_t)(2 * n) * 4 + o) * d + c];
    basis[20 + o] = leaf_map[((size_t)(2 * n + 1) * 4 + o) * d + c];
  }
  const int R = L.jets ? 8 : 1;
  const int b_end = min(L.Bc, (int)(blockIdx.z + 1) * kL1WalkersPerCta);
  for (int b = blockIdx.z * kL1WalkersPerCta; b < b_end; ++b) {
    const float* cf = coef + ((size_t)b * nodes + n) * R * kL1Basis;
    for (int rrow = 0; rrow < R; ++rrow) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < kL1Basis; ++j) acc = fmaf(__ldg(cf + rrow * kL1Basis + j), basis[j], acc);
      size_t row;
      if (!L.jets) row = row_u(L, L.rows_out, nodes, b, n);
      else if (rrow < 6) row = row_j(L.rows_out, b, n * 6 + rrow);
      else if (rrow == 6) row = row_u(L, L.rows_out, nodes, b, n);
      else row = row_l(L, L.rows_out, nodes, b, n);
      out[row * d + c] = acc;
    }
  }
}

// ------------------------------------------------------------------ second tree level in coefficient space
// A first-level carrier is a 16-vector over its effective basis E_m (Phi_m for a merged node,
// the four rows of the carried leaf's map otherwise), so every jet row of a second-level node
// - bilinear in its two children, then through the linear factor map - is a vector over
//   B2_n = [ F_h(T(E_left[i], E_right[j])) (256 rows) ; E_left (16) ; E_right (16) ]
// (the last 32 rows serve carried children). B2_n, its transposed head/tail split and its Gram
// matrix are built once per call with the generic kernels on a fake batch of 256 value-only
// "walkers". Per chunk: l2_coeff_kernel forms the raw coefficient rows, one tcgen05 GEMM per
// node multiplies them by the Gram matrix, l2_norm_kernel normalises them, and a second
// tcgen05 GEMM per node expands them against B2_n straight into the packed jet rows that the
// third level reads. The second level (a quarter of the tree's nodes) thus costs two dense
// GEMMs with K = 288 instead of tensor applications and factor GEMMs on every Jacobian row.
// Coefficient rows of node n are stored as a dense matrix X_n [tiles * 128, 288]; a tile
// holds 8 walkers: rows 12 w + A (Jacobian), 96 + w (value), 104 + w (Laplacian), 112..127 zero.
constexpr int kL2K = 288;
constexpr int kL2GN = 384;      // Gram columns padded to the GEMM's 128-wide tiles

__device__ __forceinline__ int l2_child_col(int op, int i) {
  // column of first-level coefficient i in the 24-wide rows of l1_coeff_kernel, or -1
  if (op == 0) return i;
  if (i >= 4) return -1;
  return op == 1 ? 16 + i : (op == 2 ? 20 + i : -1);
}

// E[m][i][:]: effective basis of first-level node m
__global__ void l2_child_basis_kernel(const float* __restrict__ Phi1, const float* __restrict__ leaf_map,
                                      const uint8_t* __restrict__ op1, float* __restrict__ E,
                                      int nodes1, int d) {
  const int m = blockIdx.x, i = blockIdx.y;
  const int op = op1[m];
  const float* src = nullptr;
  if (op == 0) src = Phi1 + ((size_t)i * nodes1 + m) * d;
  else if (op == 1 && i < 4) src = leaf_map + ((size_t)(2 * m) * 4 + i) * d;
  else if (op == 2 && i < 4) src = leaf_map + ((size_t)(2 * m + 1) * 4 + i) * d;
  float* dst = E + ((size_t)m * 16 + i) * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) dst[c] = src ? src[c] : 0.f;
}

// fake batch: walker w = 16 i + j carries E[m][i] on left children and E[m][j] on right ones
__global__ void l2_fake_kernel(const float* __restrict__ E, const int* __restrict__ expo,
                               float* __restrict__ U, int nodes1, int d) {
  const int m = blockIdx.x, wk = blockIdx.y;
  const int idx = (m & 1) ? (wk & 15) : (wk >> 4);
  const float* src = E + ((size_t)m * 16 + idx) * d;
  const int e = expo[m * 16 + idx];
  float* dst = U + ((size_t)wk * nodes1 + m) * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) dst[c] = ldexpf(src[c], -e);
}

// B2[n][k][:] dense
__global__ void l2_basis_kernel(const float* __restrict__ Phi2, const float* __restrict__ E,
                                float* __restrict__ B2, int nodes2, int d) {
  const int k = blockIdx.x, n = blockIdx.y;
  const float* src = k < 256 ? Phi2 + ((size_t)k * nodes2 + n) * d
                             : E + ((size_t)(2 * n + (k >= 272 ? 1 : 0)) * 16 + ((k - 256) & 15)) * d;
  float* dst = B2 + ((size_t)n * kL2K + k) * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) dst[c] = src[c];
}

// G2[n] = B2[n] B2[n]^T in fp32 products, chunk sums folded in double
__global__ void __launch_bounds__(256) l2_gram_kernel(const float* __restrict__ B2, float* __restrict__ G2, int d) {
  __shared__ float As[32][33], Bs[32][33];
  const int n = blockIdx.z, i0 = blockIdx.y * 32, j0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const float* base = B2 + (size_t)n * kL2K * d;
  double acc[4] = {0.0, 0.0, 0.0, 0.0};
  for (int c0 = 0; c0 < d; c0 += 32) {
    for (int r = ty; r < 32; r += 8) {
      As[r][tx] = (c0 + tx < d) ? base[(size_t)(i0 + r) * d + c0 + tx] : 0.f;
      Bs[r][tx] = (c0 + tx < d) ? base[(size_t)(j0 + r) * d + c0 + tx] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float part = 0.f;
#pragma unroll
      for (int c = 0; c < 32; ++c) part = fmaf(As[ty + 8 * k][c], Bs[tx][c], part);
      acc[k] += (double)part;
    }
    __syncthreads();
  }
  for (int k = 0; k < 4; ++k)
    G2[((size_t)n * kL2K + i0 + ty + 8 * k) * kL2K + j0 + tx] = (float)acc[k];
}

// head/tail split of G2[n] (symmetric, so it is its own transpose), rows padded with zeros
__global__ void l2_gram_split_kernel(const float* __restrict__ G2, float* __restrict__ hi,
                                     float* __restrict__ lo) {
  const int r = blockIdx.x, n = blockIdx.y;
  for (int k = threadIdx.x; k < kL2K; k += blockDim.x) {
    const float x = r < kL2K ? G2[((size_t)n * kL2K + r) * kL2K + k] : 0.f;
    const float h = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
    hi[((size_t)n * kL2GN + r) * kL2K + k] = h;
    lo[((size_t)n * kL2GN + r) * kL2K + k] = x - h;
  }
}

struct L2Args {
  int N, d, nodes1, nodes2, Bc, tiles;
  float eps;
  const float* coef1;        // [Bc, nodes1, 8, 24]
  const float* J_eff;
  const uint8_t* op1;
  const uint8_t* op2;
  float* X;                  // [nodes2, tiles * 128, 288]
  const float* Y;            // [nodes2, tiles * 128, 384] = X G2
  const float *s_in, *js_in, *ls_in;     // first-level scalar carriers
  float *s_out, *js_out, *ls_out;
};

// raw coefficient rows of (walker, second-level node); one CTA = one tile of 8 walkers
__global__ void __launch_bounds__(256) l2_coeff_kernel(L2Args a) {
  __shared__ float ch[2][8][8][16];       // child, walker, row (J0..J5, U, L), coefficient
  __shared__ float wb[8][6][16];          // sum_B W_off[A][B] right.J[B]
  __shared__ float woff[36];
  const int tile = blockIdx.x, n = blockIdx.y, tid = threadIdx.x;
  const int threeN = 3 * a.N;
  const int op = a.op2[n];
  for (int idx = tid; idx < 2 * 8 * 8 * 16; idx += 256) {
    const int i = idx & 15, r = (idx >> 4) & 7, w = (idx >> 7) & 7, c = idx >> 10;
    const int b = tile * 8 + w, m = 2 * n + c;
    const int col = l2_child_col(a.op1[m], i);
    float v = 0.f;
    if (b < a.Bc && col >= 0) v = a.coef1[(((size_t)b * a.nodes1 + m) * 8 + r) * kL1Basis + col];
    ch[c][w][r][i] = v;
  }
  if (tid < 36)
    woff[tid] = a.J_eff[(size_t)(12 * n + tid / 6) * threeN + 12 * n + 6 + tid % 6];
  __syncthreads();
  for (int idx = tid; idx < 8 * 6 * 16; idx += 256) {
    const int j = idx & 15, A = (idx >> 4) % 6, w = idx / 96;
    float acc = 0.f;
#pragma unroll
    for (int B = 0; B < 6; ++B) acc = fmaf(woff[A * 6 + B], ch[1][w][B][j], acc);
    wb[w][A][j] = acc;
  }
  __syncthreads();
  float* Xt = a.X + ((size_t)n * a.tiles + tile) * 128 * kL2K;
  // bilinear part: column c = 16 i + j
  {
    const int i = tid >> 4, j = tid & 15;
    for (int w = 0; w < 8; ++w) {
      const float aU = ch[0][w][6][i], bU = ch[1][w][6][j];
      const bool live = op == 0;
#pragma unroll
      for (int A = 0; A < 6; ++A) {
        Xt[(size_t)(12 * w + A) * kL2K + tid] = live ? ch[0][w][A][i] * bU : 0.f;
        Xt[(size_t)(12 * w + 6 + A) * kL2K + tid] = live ? aU * ch[1][w][A][j] : 0.f;
      }
      Xt[(size_t)(96 + w) * kL2K + tid] = live ? aU * bU : 0.f;
      float l = ch[0][w][7][i] * bU + aU * ch[1][w][7][j];
      float x = 0.f;
#pragma unroll
      for (int A = 0; A < 6; ++A) x = fmaf(ch[0][w][A][i], wb[w][A][j], x);
      Xt[(size_t)(104 + w) * kL2K + tid] = live ? l + 2.f * x : 0.f;
    }
    for (int r = 112; r < 128; ++r) Xt[(size_t)r * kL2K + tid] = 0.f;
  }
  // carried part: columns 256 + 16 c + i hold child c's own rows when the node carries it
  if (tid < 32) {
    const int c = tid >> 4, i = tid & 15;
    const bool mine = (op == 1 && c == 0) || (op == 2 && c == 1);
    for (int w = 0; w < 8; ++w) {
#pragma unroll
      for (int A = 0; A < 12; ++A) {
        const bool own = mine && (A / 6 == c);
        Xt[(size_t)(12 * w + A) * kL2K + 256 + tid] = own ? ch[c][w][A % 6][i] : 0.f;
      }
      Xt[(size_t)(96 + w) * kL2K + 256 + tid] = mine ? ch[c][w][6][i] : 0.f;
      Xt[(size_t)(104 + w) * kL2K + 256 + tid] = mine ? ch[c][w][7][i] : 0.f;
    }
    for (int r = 112; r < 128; ++r) Xt[(size_t)r * kL2K + 256 + tid] = 0.f;
  }
  // scalar carriers of gated nodes (merged nodes: l2_norm_kernel)
  if (op != 0 && tid < 8) {
    const int b = tile * 8 + tid;
    if (b < a.Bc) {
      const bool carry = op == 1 || op == 2;
      const int c = op == 2 ? 1 : 0, m = 2 * n + c;
      a.s_out[(size_t)b * a.nodes2 + n] = carry ? a.s_in[(size_t)b * a.nodes1 + m] : 0.f;
      a.ls_out[(size_t)b * a.nodes2 + n] = carry ? a.ls_in[(size_t)b * a.nodes1 + m] : 0.f;
      for (int A = 0; A < 12; ++A) {
        const bool keep = carry && (A / 6 == c);
        a.js_out[(size_t)b * threeN + 12 * n + A] = keep ? a.js_in[(size_t)b * threeN + 12 * n + A] : 0.f;
      }
    }
  }
}

// normalisation of a merged second-level node in coefficient space; one warp per walker
__global__ void __launch_bounds__(256) l2_norm_kernel(L2Args a) {
  __shared__ float W2[144];
  const int tile = blockIdx.x, n = blockIdx.y, tid = threadIdx.x;
  const int w = tid >> 5, lane = tid & 31;
  const int threeN = 3 * a.N;
  if (a.op2[n] != 0) return;
  if (tid < 144) W2[tid] = a.J_eff[(size_t)(12 * n + tid / 12) * threeN + 12 * n + tid % 12];
  __syncthreads();
  const int b = tile * 8 + w;
  if (b >= a.Bc) return;
  float* Xt = a.X + ((size_t)n * a.tiles + tile) * 128 * kL2K;
  const float* Yt = a.Y + ((size_t)n * a.tiles + tile) * 128 * kL2GN;
  float* Ju = Xt + (size_t)(12 * w) * kL2K;
  float* Uu = Xt + (size_t)(96 + w) * kL2K;
  float* Lu = Xt + (size_t)(104 + w) * kL2K;
  const float* Yj = Yt + (size_t)(12 * w) * kL2GN;
  const float* Yu = Yt + (size_t)(96 + w) * kL2GN;
  float oo = 0.f, oL = 0.f, gram = 0.f, aA[12];
#pragma unroll
  for (int A = 0; A < 12; ++A) aA[A] = 0.f;
  for (int c = lane; c < kL2K; c += 32) {
    const float gu = Yu[c];
    oo = fmaf(Uu[c], gu, oo);
    oL = fmaf(Lu[c], gu, oL);
    float jv[12], yv[12];
#pragma unroll
    for (int A = 0; A < 12; ++A) {
      jv[A] = Ju[(size_t)A * kL2K + c];
      yv[A] = Yj[(size_t)A * kL2GN + c];
      aA[A] = fmaf(jv[A], gu, aA[A]);
    }
#pragma unroll
    for (int A = 0; A < 12; ++A) {
      float t = 0.f;
#pragma unroll
      for (int B = 0; B < 12; ++B) t = fmaf(W2[A * 12 + B], yv[B], t);
      gram = fmaf(jv[A], t, gram);
    }
  }
  oo = warp_sum(oo); oL = warp_sum(oL); gram = warp_sum(gram);
#pragma unroll
  for (int A = 0; A < 12; ++A) aA[A] = warp_sum(aA[A]);
  const float inv_d = 1.f / (float)a.d;
  const float y = oo * inv_d + a.eps;
  const float r = rsqrtf(y);
  float dy[12], wdy[12], dywdy = 0.f;
#pragma unroll
  for (int A = 0; A < 12; ++A) dy[A] = 2.f * inv_d * aA[A];
#pragma unroll
  for (int A = 0; A < 12; ++A) {
    float acc = 0.f;
#pragma unroll
    for (int B = 0; B < 12; ++B) acc = fmaf(W2[A * 12 + B], dy[B], acc);
    wdy[A] = acc;
    dywdy = fmaf(dy[A], acc, dywdy);
  }
  const float lap_y = 2.f * inv_d * (oL + gram);
  const float y15 = r * r * r, y25 = y15 * r * r;
  const float lap_r = -0.5f * y15 * lap_y + 0.75f * y25 * dywdy;
  const float s_lap = 0.5f * (lap_y / y - dywdy / (y * y));
  if (lane == 0) {
    const size_t m0 = (size_t)b * a.nodes1 + 2 * n;
    a.s_out[(size_t)b * a.nodes2 + n] = a.s_in[m0] + a.s_in[m0 + 1] + 0.5f * logf(y);
    a.ls_out[(size_t)b * a.nodes2 + n] = a.ls_in[m0] + a.ls_in[m0 + 1] + s_lap;
  }
#pragma unroll
  for (int A = 0; A < 12; ++A)
    if (lane == A)
      a.js_out[(size_t)b * threeN + 12 * n + A] =
          a.js_in[(size_t)b * threeN + 12 * n + A] + 0.5f * dy[A] / y;
  float drA[12], wdrA[12];
#pragma unroll
  for (int A = 0; A < 12; ++A) { drA[A] = -0.5f * y15 * dy[A]; wdrA[A] = -y15 * wdy[A]; }
  for (int c = lane; c < kL2K; c += 32) {
    const float u = Uu[c];
    float l = r * Lu[c] + lap_r * u;
#pragma unroll
    for (int A = 0; A < 12; ++A) {
      const float j = Ju[(size_t)A * kL2K + c];
      l = fmaf(wdrA[A], j, l);
      Ju[(size_t)A * kL2K + c] = r * j + drA[A] * u;
    }
    Uu[c] = r * u;
    Lu[c] = l;
  }
}

// ------------------------------------------------------------------ root
// psi rows = ((row V_r) * h_r) U_r for the root's value, Jacobian rows and Laplacian;
// then log|psi| + s, atan2 and the energy assembly (energy/kernel.py:80-119).
constexpr int kRootThreads = 256;

__global__ void __launch_bounds__(kRootThreads)
root_kernel(Level L, int r_ro, const float* __restrict__ Z /* [Bc*rows][r_ro] */,
            const float* __restrict__ Ur /* [r_ro][2] */, const float* __restrict__ J_eff,
            const float* __restrict__ field, float radial_const, const float* __restrict__ s_in,
            const float* __restrict__ js_in, const float* __restrict__ ls_in,
            float* __restrict__ log_abs, float* __restrict__ phase,
            float* __restrict__ energies /* [4][Btot][2] */, float* __restrict__ grad,
            long long b_offset, long long b_total, const int* __restrict__ status) {
  extern __shared__ __align__(16) float sm[];
  const int N = L.N, threeN = 3 * N, rows = L.rows_out;
  const int b = blockIdx.x, tid = threadIdx.x;
  const long long bg = b_offset + b;
  float* Ur_s = sm;                        // [r_ro][2]
  float* vx = Ur_s + 2 * r_ro;             // [3N] d psi_x
  float* vy = vx + threeN;
  float* vs = vy + threeN;                 // [3N] d s
  double* dscr = reinterpret_cast<double*>(vs + threeN + (threeN & 1));   // [9 * 8]
  __shared__ float head[4];                // psi_x, psi_y, L psi_x, L psi_y

  for (int i = tid; i < 2 * r_ro; i += kRootThreads) Ur_s[i] = Ur[i];
  __syncthreads();
  const int nrows = L.jets ? threeN + 2 : 1;
  for (int rr = tid; rr < nrows; rr += kRootThreads) {
    const float* z = Z + ((size_t)b * rows + rr) * r_ro;
    float x = 0.f, y = 0.f;
    for (int k = 0; k < r_ro; ++k) {
      const float zz = z[k];
      x = fmaf(zz, Ur_s[2 * k], x);
      y = fmaf(zz, Ur_s[2 * k + 1], y);
    }
    if (!L.jets) { head[0] = x; head[1] = y; }
    else if (rr < threeN) { vx[rr] = x; vy[rr] = y; vs[rr] = js_in[(size_t)b * threeN + rr]; }
    else if (rr == threeN) { head[0] = x; head[1] = y; }
    else { head[2] = x; head[3] = y; }
  }
  __syncthreads();
  // a bounded device wait that ran out upstream poisons the results instead of passing
  // silently: every output of this walker becomes NaN
  const double poison = (*status != 0) ? (double)NAN : 0.0;
  const double x = head[0] + poison, y = head[1];
  const double rho = x * x + y * y;
  const double s = s_in[b];
  if (tid == 0) {
    log_abs[bg] = (float)(0.5 * log(rho) + s);
    phase[bg] = (float)atan2(y, x);
  }
  if (!L.jets) return;

  // nine J_eff-weighted / field-weighted forms of (vx, vy, vs)
  double acc[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};   // Qxx Qxy Qyy Qxs Qys Qss hx hy hs
  for (int a = tid; a < threeN; a += kRootThreads) {
    double wx = 0, wy = 0, ws = 0;
    for (int c = 0; c < threeN; ++c) {
      const double w = J_eff[(size_t)c * threeN + a];     // symmetric: column read is coalesced
      wx += w * vx[c]; wy += w * vy[c]; ws += w * vs[c];
    }
    const double ax = vx[a], ay = vy[a], as = vs[a], h = field[a];
    acc[0] += ax * wx; acc[1] += ax * wy; acc[2] += ay * wy;
    acc[3] += ax * ws; acc[4] += ay * ws; acc[5] += as * ws;
    acc[6] += h * ax; acc[7] += h * ay; acc[8] += h * as;
  }
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int i = 0; i < 9; ++i)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  if (lane == 0)
    for (int i = 0; i < 9; ++i) dscr[warp * 9 + i] = acc[i];
  __syncthreads();
  const double al = x / rho, be = y / rho;
  if (grad != nullptr)
    for (int a = tid; a < threeN; a += kRootThreads) {
      grad[((size_t)bg * threeN + a) * 2] = (float)(al * vx[a] + be * vy[a] + vs[a]);
      grad[((size_t)bg * threeN + a) * 2 + 1] = (float)(al * vy[a] - be * vx[a]);
    }
  if (tid != 0) return;
  double Q[9];
  for (int i = 0; i < 9; ++i) {
    Q[i] = 0;
    for (int w = 0; w < kRootThreads / 32; ++w) Q[i] += dscr[w * 9 + i];
  }
  const double Qxx = Q[0], Qxy = Q[1], Qyy = Q[2], Qxs = Q[3], Qys = Q[4], Qss = Q[5];
  const double Lx = head[2], Ly = head[3], ls = ls_in[b];
  const double lap_rho = 2.0 * (x * Lx + y * Ly + Qxx + Qyy);
  const double drwdr = 4.0 * (x * x * Qxx + 2.0 * x * y * Qxy + y * y * Qyy);
  const double la_lap = 0.5 * (lap_rho / rho - drwdr / (rho * rho)) + ls;
  const double ph_lap = (x * Ly - y * Lx) / rho +
                        (2.0 * x * y * (Qxx - Qyy) + 2.0 * (y * y - x * x) * Qxy) / (rho * rho);
  // g = la + i ph, la = al vx + be vy + vs, ph = al vy - be vx
  const double lala = al * al * Qxx + 2 * al * be * Qxy + be * be * Qyy + 2 * al * Qxs + 2 * be * Qys + Qss;
  const double phph = be * be * Qxx - 2 * al * be * Qxy + al * al * Qyy;
  const double laph = -al * be * Qxx + (al * al - be * be) * Qxy + al * be * Qyy - be * Qxs + al * Qys;
  const double quad_re = lala - phph, quad_im = 2.0 * laph;
  const double la_h = al * Q[6] + be * Q[7] + Q[8], ph_h = al * Q[7] - be * Q[6];
  const double f_re = -0.5 * ph_h, f_im = 0.5 * la_h;          // i/2 * sum h g
  const double t_re = la_lap + quad_re + (double)radial_const + f_re;
  const double t_im = ph_lap + quad_im + f_im;
  if (energies == nullptr) return;      // value-and-gradient callers need no energy samples
  float* e = energies;
  const size_t st = (size_t)b_total * 2;
  e[0 * st + bg * 2] = (float)t_re;            e[0 * st + bg * 2 + 1] = (float)t_im;
  e[1 * st + bg * 2] = (float)(t_re - f_re);   e[1 * st + bg * 2 + 1] = (float)(t_im - f_im);
  e[2 * st + bg * 2] = 0.f;                    e[2 * st + bg * 2 + 1] = 0.f;
  e[3 * st + bg * 2] = (float)f_re;            e[3 * st + bg * 2 + 1] = (float)f_im;
}

// ------------------------------------------------------------------ host orchestration
struct Workspace {
  float *bufA, *bufB, *Z, *leaf_map, *leaf_tmp;
  int* row_expo;                                          // FP16-split GEMMs: one exponent per row of A
  float *vt_hi, *vt_lo, *ut_hi, *ut_lo, *rt_hi, *rt_lo;   // weights transposed + split (tcgen05 path)
  int* status;                                            // device word set by a timed-out wait
  int *l1_exp, *l2_exp;                                   // binary exponents of the fake batches' rows
  float *t_packed, *t_scale, *lap_b;                      // merge_tc_kernel: packed T, group scales, A_L L_R
  float *cross_w, *cross_ws;                              // cross_tc_kernel: W_off images, node scales
  float *ta_packed, *ta_scale;                            // value-only passes: T for tapply_tc_kernel
  float* zero_frame;                                      // jets == 2: stands in for the energy frame
  float *l1_gs, *l1_g16, *l1_fake, *l1_phi, *l1_z, *l1_coef;  // first level in coefficient space
  float *l2_E, *l2_fake, *l2_phi, *l2_z, *l2_B2, *l2_bt_hi, *l2_bt_lo, *l2_G2, *l2_g_hi, *l2_g_lo;
  float *l2_X, *l2_Y;                                         // second level, per chunk
  int l2_tiles;
  float *sA, *sB, *lsA, *lsB, *jsA, *jsB, *dr, *wdr;
  float *gram, *ga, *goo, *goL, *gw;    // tcgen05 reductions of the normalisation stage
  NormOut* nout;
  size_t bytes;
};

size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

bool use_tc_gemm();
bool use_level1();
// Second tree level in coefficient space: energy/gradient passes of trees with at least two
// levels, when the tcgen05 GEMM can tile d_m; HZ_LEVEL2=generic switches it off.
bool use_level2(const hz_wavefunction* w, int jets) {
  static const bool enabled = !env_equals("HZ_LEVEL2", "generic");
  return enabled && jets && w->n_sites >= 4 && (w->d_m % 128) == 0 && use_level1() &&
         use_tc_gemm() && encode_tiled_fn() != nullptr;
}

// Lays the chunk's arrays out in `base` (may be null: size query).
Workspace carve(const hz_wavefunction* w, int jets, long long Bc, char* base) {
  Workspace ws{};
  const size_t N = w->n_sites, d = w->d_m;
  const size_t rows0 = packed_rows((int)N, (int)N, jets);
  const size_t zc = (size_t)(w->r_merge > w->r_ro ? w->r_merge : w->r_ro);
  size_t off = 0;
  auto take = [&](size_t nfloats) {
    float* p = base ? reinterpret_cast<float*>(base + off) : nullptr;
    off += align_up(nfloats * sizeof(float));
    return p;
  };
  // the status word of the device waits is the first word of every workspace
  // (hz_workspace_status reads it there)
  ws.status = reinterpret_cast<int*>(take(64));      // 256 bytes after alignment
  ws.leaf_map = take(N * 4 * d);
  ws.leaf_tmp = take(N * 4 * (size_t)w->r_leaf);
  ws.vt_hi = take(d * (size_t)w->r_merge); ws.vt_lo = take(d * (size_t)w->r_merge);
  ws.ut_hi = take(d * (size_t)w->r_merge); ws.ut_lo = take(d * (size_t)w->r_merge);
  ws.rt_hi = take(d * (size_t)w->r_ro);    ws.rt_lo = take(d * (size_t)w->r_ro);
  ws.l1_exp = reinterpret_cast<int*>(take(N * 4));
  if (jets == 2) ws.zero_frame = take(9 * N * N + 3 * N);
  if (!jets && N > 1 && use_tapply_tc()) {
    ws.ta_packed = take((size_t)(d / kDr) * 1024 * 32);
    ws.ta_scale = take(d / kDr);
  }
  if (jets && N > 1) {
    ws.t_packed = take((size_t)2 * (d / kDr) * 1024 * 32);
    ws.t_scale = take(d / kDr);
    ws.lap_b = take((size_t)Bc * (N / 2) * d);
    ws.cross_w = take((size_t)kCxMaxWRows * 32);
    ws.cross_ws = take(64);
  }
  ws.l1_gs = take(N * 16);
  ws.l1_g16 = take((N / 2 + 1) * 256);
  ws.l1_fake = take(16 * N * d);
  ws.l1_phi = take(16 * (N / 2 + 1) * d);
  ws.l1_z = take(16 * (N / 2 + 1) * (size_t)w->r_merge);
  ws.l1_coef = take((size_t)Bc * (N / 2 + 1) * 8 * kL1Basis);
  if (use_level2(w, jets)) {
    const size_t n1 = N / 2, n2 = N / 4;
    ws.l2_tiles = (int)((Bc + 7) / 8);
    ws.l2_exp = reinterpret_cast<int*>(take(n1 * 16));
    ws.l2_E = take(n1 * 16 * d);
    ws.l2_fake = take(256 * n1 * d);
    ws.l2_phi = take(256 * n2 * d);
    ws.l2_z = take(256 * n2 * (size_t)w->r_merge);
    ws.l2_B2 = take(n2 * kL2K * d);
    ws.l2_bt_hi = take(n2 * d * kL2K); ws.l2_bt_lo = take(n2 * d * kL2K);
    ws.l2_G2 = take(n2 * kL2K * kL2K);
    ws.l2_g_hi = take(n2 * kL2GN * kL2K); ws.l2_g_lo = take(n2 * kL2GN * kL2K);
    ws.l2_X = take(n2 * (size_t)ws.l2_tiles * 128 * kL2K);
    ws.l2_Y = take(n2 * (size_t)ws.l2_tiles * 128 * kL2GN);
  }
  ws.bufA = take((size_t)Bc * rows0 * d);
  ws.bufB = take((size_t)Bc * rows0 * d);
  ws.Z = take((size_t)Bc * rows0 * zc);
  ws.row_expo = reinterpret_cast<int*>(take((size_t)Bc * rows0));
  ws.sA = take((size_t)Bc * N);  ws.sB = take((size_t)Bc * N);
  ws.lsA = take((size_t)Bc * N); ws.lsB = take((size_t)Bc * N);
  ws.jsA = take((size_t)Bc * 3 * N); ws.jsB = take((size_t)Bc * 3 * N);
  ws.dr = take((size_t)Bc * 3 * N);  ws.wdr = take((size_t)Bc * 3 * N);
  ws.nout = reinterpret_cast<NormOut*>(take((size_t)Bc * N * 2));
  if (jets && N > 1) {
    ws.gram = take((size_t)Bc * ((3 * N + N + 127) / 128) * 3 * N); ws.ga = take((size_t)Bc * 3 * N);
    ws.goo = take((size_t)Bc * N); ws.goL = take((size_t)Bc * N);
    ws.gw = take((size_t)8 * 3 * N * 3 * N);                                  // one masked W per tree level
  }
  ws.bytes = off;
  return ws;
}

int check_wavefunction(const hz_wavefunction* w) {
  if (!w) return HZ_ERR_NULL_POINTER;
  const int N = w->n_sites;
  if (N <= 0 || (N & (N - 1)) || w->d_m <= 0 || w->d_o <= 0 || w->r_leaf <= 0 ||
      w->r_merge <= 0 || w->r_ro <= 0)
    return HZ_ERR_BAD_SHAPE;
  if (N > 256) return HZ_ERR_UNSUPPORTED;
  if (w->d_r != kDr || w->d_m % kDr) return HZ_ERR_UNSUPPORTED;
  if ((w->r_leaf % 4) || (w->r_merge % 4) || (w->r_ro % 4)) return HZ_ERR_UNSUPPORTED;
  if (!w->q_weight || !w->leaf_V || !w->leaf_U || !w->leaf_h || !w->readout_V ||
      !w->readout_U || !w->readout_h)
    return HZ_ERR_NULL_POINTER;
  if (N > 1 && (!w->merge_T || !w->merge_V || !w->merge_U || !w->merge_h || !w->opcodes))
    return HZ_ERR_NULL_POINTER;
  return HZ_OK;
}

// tcgen05 GEMM unless the shape is outside what it tiles or HZ_GEMM_IMPL=legacy is set.
bool use_tc_gemm() {
  static const bool enabled = !env_equals("HZ_GEMM_IMPL", "legacy");
  return enabled;
}

// f16 = true: the weights were prepared by prepare_weights_f16 (packed halves in bt_hi, their
// scale in bt_lo[0]) and the GEMM runs on the FP16 split.
int gemm_dispatch(int epi, const GemmArgs& a, const float* bt_hi, const float* bt_lo, int* status,
                  cudaStream_t stream, bool f16 = false) {
  if (use_tc_gemm() && gemm_tc_supported(a) && encode_tiled_fn() != nullptr)
    return f16 ? launch_gemm_tcf(epi, a, bt_hi, bt_lo, status, stream)
               : launch_gemm_tc(epi, a, bt_hi, bt_lo, status, stream);
  return launch_gemm(epi, a, stream);
}

// The factor GEMMs of the energy and log-psi passes run on the FP16 split when every weight
// matrix has a shape the tcgen05 path tiles (then no call falls back to the kernel that reads
// the unprepared weights, and the packed form is the only one needed).
bool walker_gemm_f16(const hz_wavefunction* w) {
  return use_tc_gemm() && use_f16_gemm() && encode_tiled_fn() != nullptr && w->d_m % 128 == 0 &&
         w->r_merge % 128 == 0 && w->r_ro % 128 == 0;
}

int prepare_weights(const hz_wavefunction* w, const Workspace& ws, cudaStream_t stream) {
  HZ_CUDA_TRY(cudaMemsetAsync(ws.status, 0, sizeof(int), stream));
  if (!use_tc_gemm()) return HZ_OK;
  const int d = w->d_m;
  if (walker_gemm_f16(w)) {
    if (w->n_sites > 1) {
      int st = prepare_weights_f16(w->merge_V, ws.vt_hi, ws.vt_lo, d, w->r_merge, true, stream);
      if (st != HZ_OK) return st;
      st = prepare_weights_f16(w->merge_U, ws.ut_hi, ws.ut_lo, w->r_merge, d, true, stream);
      if (st != HZ_OK) return st;
    }
    return prepare_weights_f16(w->readout_V, ws.rt_hi, ws.rt_lo, d, w->r_ro, true, stream);
  }
  dim3 blk(32, 8);
  if (w->n_sites > 1) {
    split_transpose_kernel<<<dim3((w->r_merge + 31) / 32, (d + 31) / 32), blk, 0, stream>>>(
        w->merge_V, ws.vt_hi, ws.vt_lo, d, w->r_merge);
    split_transpose_kernel<<<dim3((d + 31) / 32, (w->r_merge + 31) / 32), blk, 0, stream>>>(
        w->merge_U, ws.ut_hi, ws.ut_lo, w->r_merge, d);
  }
  split_transpose_kernel<<<dim3((w->r_ro + 31) / 32, (d + 31) / 32), blk, 0, stream>>>(
      w->readout_V, ws.rt_hi, ws.rt_lo, d, w->r_ro);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// First tree level in coefficient space unless HZ_LEVEL1=generic is set.
bool use_level1() {
  static const bool enabled = !env_equals("HZ_LEVEL1", "generic");
  return enabled;
}

int sm_count_of_current_device(int* out) {
  int dev = 0;
  HZ_CUDA_TRY(cudaGetDevice(&dev));
  HZ_CUDA_TRY(cudaDeviceGetAttribute(out, cudaDevAttrMultiProcessorCount, dev));
  return HZ_OK;
}

int launch_tstage(const Level& L, const hz_wavefunction* w, const float* J_eff, const float* in,
                  float* out, cudaStream_t stream) {
  int sm_count = 148;
  int st = sm_count_of_current_device(&sm_count);
  if (st != HZ_OK) return st;
  const size_t smem = kTsSmemFloats * sizeof(float);
  st = ensure_kernel_attributes(reinterpret_cast<const void*>(merge_tstage_kernel<false>), (int)smem);
  if (st != HZ_OK) return st;
  const long long tiles = ((long long)L.Bc * L.nodes + kTsPairs - 1) / kTsPairs;
  // one resident CTA per SM (T_i fills shared memory) and every CTA walks a fixed share of the
  // tiles: the grid must fit one wave, so the CTAs per group are rounded down
  long long gy = sm_count / L.G;
  if (gy > tiles) gy = tiles;
  if (gy < 1) gy = 1;
  merge_tstage_kernel<false><<<dim3(L.G, (unsigned)gy), kTsThreads, smem, stream>>>(
      L, w->merge_T, J_eff, in, out, nullptr);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// The merge of a jet pass on tcgen05 (merge_tc_kernel: tensor applications, value, Jacobian rows,
// the two plain Laplacian terms) followed, for energy passes, by the cross term
// (merge_tstage_kernel<true>). HZ_MERGE=legacy keeps the single mma.sync kernel.
bool use_merge_tc(const hz_wavefunction* w, int jets) {
  static const bool enabled = !env_equals("HZ_MERGE", "legacy");
  return enabled && jets && w->n_sites > 1 && use_tc_gemm() && encode_tiled_fn() != nullptr;
}

int launch_merge_tc(const Level& L, const hz_wavefunction* w, const float* J_eff, const Workspace& ws,
                    const float* in, float* out, cudaStream_t stream) {
  int sm_count = 148;
  int st = sm_count_of_current_device(&sm_count);
  if (st != HZ_OK) return st;
  MergeTcArgs a{};
  a.L = L; a.in = in; a.out = out;
  a.lap_b = L.jets == 1 ? ws.lap_b : nullptr;
  a.t_scale = ws.t_scale;
  a.total_pairs = (long long)L.Bc * L.nodes;
  a.tiles = (int)((a.total_pairs + kMcPairs - 1) / kMcPairs);
  a.boxr = L.m < 16 ? L.m : 16;
  a.nrb = (L.m + 15) / 16;
  a.lg_nodes = 0;
  while ((1 << a.lg_nodes) < L.nodes) ++a.lg_nodes;
  MergeTcMaps maps;
  if (!make_map(&maps.t, ws.t_packed, 2ll * L.G * 1024, 32, 32, 128) ||
      !make_map(&maps.in, in, (long long)L.Bc * L.rows_in, L.d, L.d, a.boxr))
    return HZ_ERR_CUDA;
  st = ensure_kernel_attributes(reinterpret_cast<const void*>(merge_tc_kernel), (int)kMcSmemBytes);
  if (st != HZ_OK) return st;
  const long long W = 2ll * L.G * a.tiles;
  const unsigned grid = (unsigned)(W < sm_count ? W : sm_count);
  merge_tc_kernel<<<grid, kMcThreads, kMcSmemBytes, stream>>>(maps, a, ws.status);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// levels whose cross term takes cross_tc_kernel (the others stay on merge_tstage_kernel<true>)
bool cross_on_tcgen05(const Level& L) {
  return use_cross_tc() && cross_tc_supported(L) && cross_tc_level_enabled(L.m) && L.d == L.G * kDr;
}

// the cross term of the Laplacian row, after launch_merge_tc (energy passes only)
int launch_merge_cross(const Level& L, const hz_wavefunction* w, const float* J_eff, const Workspace& ws,
                       const float* in, float* out, cudaStream_t stream) {
  if (cross_on_tcgen05(L))
    return launch_cross_tc(L, w->merge_T, J_eff, in, out, ws.lap_b, ws.cross_w, ws.cross_ws, ws.status, stream);
  int sm_count = 148;
  int st = sm_count_of_current_device(&sm_count);
  if (st != HZ_OK) return st;
  const size_t smem = kTsSmemFloats * sizeof(float);
  st = ensure_kernel_attributes(reinterpret_cast<const void*>(merge_tstage_kernel<true>), (int)smem);
  if (st != HZ_OK) return st;
  const long long tiles = ((long long)L.Bc * L.nodes + kTsPairs - 1) / kTsPairs;
  long long gy = sm_count / L.G;
  if (gy > tiles) gy = tiles;
  if (gy < 1) gy = 1;
  merge_tstage_kernel<true><<<dim3(L.G, (unsigned)gy), kTsThreads, smem, stream>>>(
      L, w->merge_T, J_eff, in, out, ws.lap_b);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// leaf map M[site][4][d] = ((q_weight V_leaf) * h_site) U_leaf, once per call
int prepare_leaf_map(const hz_wavefunction* w, const Workspace& ws, cudaStream_t stream) {
  const int N = w->n_sites, d = w->d_m;
  StageScope scope(kStLeafMap, stream, 2.0 * 4 * N * w->r_leaf * (double)(w->d_o + d), 2);
  const int total = N * 4 * w->r_leaf;
  leaf_tmp_kernel<<<(total + 255) / 256, 256, 0, stream>>>(w->q_weight, w->leaf_V, w->leaf_h,
                                                           ws.leaf_tmp, N, w->d_o, w->r_leaf);
  HZ_CUDA_TRY(cudaGetLastError());
  GemmArgs ga{};
  ga.A = ws.leaf_tmp; ga.B = w->leaf_U; ga.C = ws.leaf_map;
  ga.M = 4 * N; ga.N = d; ga.K = w->r_leaf; ga.lda = w->r_leaf; ga.ldb = d; ga.ldc = d;
  return launch_gemm(kEpiStore, ga, stream);
}

// Phi_n[4o+o'] = F_h(T(M_left[o], M_right[o'])) and its Gram matrix, once per call: the
// generic merge and factor kernels run on a fake batch of 16 value-only "walkers".
int prepare_level1(const hz_wavefunction* w, const Workspace& ws, cudaStream_t stream) {
  const int N = w->n_sites, d = w->d_m, nodes = N / 2;
  StageScope scope(kStL1Prep, stream, 16.0 * nodes * (2.0 * (d / kDr) * (32768.0 + 1024.0) + 4.0 * d * w->r_merge), 8);
  leaf_gram_kernel<<<N, 128, 0, stream>>>(ws.leaf_map, ws.l1_gs, d);
  row_exponent_kernel<<<N * 4, 128, 0, stream>>>(ws.leaf_map, ws.l1_exp, d);
  l1_fake_kernel<<<dim3(N, 16), 256, 0, stream>>>(ws.leaf_map, ws.l1_exp, ws.l1_fake, N, d);
  HZ_CUDA_TRY(cudaGetLastError());
  Level L{};
  L.N = N; L.d = d; L.G = d / kDr; L.jets = 0; L.Bc = 16; L.nodes = nodes; L.m = 3;
  L.rows_in = N; L.rows_out = nodes;
  int st = launch_tstage(L, w, nullptr, ws.l1_fake, ws.l1_phi, stream);
  if (st != HZ_OK) return st;
  fake_unscale_kernel<<<dim3(nodes, 16), 256, 0, stream>>>(ws.l1_phi, ws.l1_exp, nodes, 4, d);
  HZ_CUDA_TRY(cudaGetLastError());
  const int M = 16 * nodes;
  GemmArgs g1{};
  g1.A = ws.l1_phi; g1.B = w->merge_V; g1.C = ws.l1_z; g1.M = M; g1.N = w->r_merge; g1.K = d;
  g1.lda = d; g1.ldb = w->r_merge; g1.ldc = w->r_merge;
  g1.h = w->merge_h; g1.rows_per_walker = nodes; g1.three_n = 0; g1.rows_per_node = 6; g1.nodes = nodes;
  st = gemm_dispatch(kEpiNodeScale, g1, ws.vt_hi, ws.vt_lo, ws.status, stream, walker_gemm_f16(w));
  if (st != HZ_OK) return st;
  GemmArgs g2{};
  g2.A = ws.l1_z; g2.B = w->merge_U; g2.C = ws.l1_phi; g2.R = ws.l1_phi; g2.M = M; g2.N = d;
  g2.K = w->r_merge; g2.lda = w->r_merge; g2.ldb = d; g2.ldc = d;
  st = gemm_dispatch(kEpiResidual, g2, ws.ut_hi, ws.ut_lo, ws.status, stream, walker_gemm_f16(w));
  if (st != HZ_OK) return st;
  l1_gram_kernel<<<nodes, 256, 0, stream>>>(ws.l1_phi, ws.l1_g16, nodes, d);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// The reductions of the normalisation stage on tcgen05 (syrk_tc_kernel) for trees of at least 32
// sites, from the third level on (below that the rows of a walker fill too little of a 128-row
// block, and the mma.sync kernel with W in shared memory is faster); HZ_NORM=legacy switches it
// off.
bool use_tc_norm(const hz_wavefunction* w, int jets, int m2) {
  static const bool enabled = !env_equals("HZ_NORM", "legacy");
  // nodes with fewer Jacobian rows keep the mma.sync reduction: the tcgen05 kernel forms the whole
  // walker's Gram matrix at every level, and below 96 rows per node (third and fourth level of a
  // 64-site tree) the node-local kernel is faster (measured +2 % on the step)
  static const int min_rows = env_int("HZ_NORM_TC_MIN_ROWS", 96);
  return enabled && jets && m2 >= min_rows && w->n_sites >= 32 && use_tc_gemm() &&
         syrk_tc_supported(3 * w->n_sites, w->d_m);
}

// every level's block-diagonal W, once per call
int prepare_tc_norm(const hz_wavefunction* w, const hz_energy_frame* f, const Workspace& ws, cudaStream_t stream) {
  const int N = w->n_sites, three_n = 3 * N;
  int level_index = 0;
  for (int k = 1; k < N; k *= 2, ++level_index) {
    const int m2 = 6 * k;
    if (!use_tc_norm(w, 1, m2)) continue;
    syrk_w_mask_kernel<<<three_n, 128, 0, stream>>>(f->J_eff, three_n, m2,
                                                    ws.gw + (size_t)level_index * three_n * three_n);
  }
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// B2_n, its transposed head/tail split and its Gram matrix, once per call.
int prepare_level2(const hz_wavefunction* w, const Workspace& ws, cudaStream_t stream) {
  const int N = w->n_sites, d = w->d_m, n1 = N / 2, n2 = N / 4;
  StageScope scope(kStL2Prep, stream,
                   256.0 * n2 * (2.0 * (d / kDr) * (32768.0 + 1024.0) + 4.0 * d * w->r_merge) +
                       2.0 * n2 * kL2K * kL2K * d,
                   10 + n2);
  l2_child_basis_kernel<<<dim3(n1, 16), 256, 0, stream>>>(ws.l1_phi, ws.leaf_map, w->opcodes, ws.l2_E, n1, d);
  row_exponent_kernel<<<n1 * 16, 128, 0, stream>>>(ws.l2_E, ws.l2_exp, d);
  l2_fake_kernel<<<dim3(n1, 256), 256, 0, stream>>>(ws.l2_E, ws.l2_exp, ws.l2_fake, n1, d);
  HZ_CUDA_TRY(cudaGetLastError());
  Level L{};
  L.N = N; L.d = d; L.G = d / kDr; L.jets = 0; L.Bc = 256; L.nodes = n2; L.m = 6;
  L.rows_in = n1; L.rows_out = n2;
  int st = launch_tstage(L, w, nullptr, ws.l2_fake, ws.l2_phi, stream);
  if (st != HZ_OK) return st;
  fake_unscale_kernel<<<dim3(n2, 256), 256, 0, stream>>>(ws.l2_phi, ws.l2_exp, n2, 16, d);
  HZ_CUDA_TRY(cudaGetLastError());
  const int M = 256 * n2;
  GemmArgs g1{};
  g1.A = ws.l2_phi; g1.B = w->merge_V; g1.C = ws.l2_z; g1.M = M; g1.N = w->r_merge; g1.K = d;
  g1.lda = d; g1.ldb = w->r_merge; g1.ldc = w->r_merge;
  g1.h = w->merge_h + (size_t)n1 * w->r_merge; g1.rows_per_walker = n2; g1.three_n = 0;
  g1.rows_per_node = 12; g1.nodes = n2;
  st = gemm_dispatch(kEpiNodeScale, g1, ws.vt_hi, ws.vt_lo, ws.status, stream, walker_gemm_f16(w));
  if (st != HZ_OK) return st;
  GemmArgs g2{};
  g2.A = ws.l2_z; g2.B = w->merge_U; g2.C = ws.l2_phi; g2.R = ws.l2_phi; g2.M = M; g2.N = d;
  g2.K = w->r_merge; g2.lda = w->r_merge; g2.ldb = d; g2.ldc = d;
  st = gemm_dispatch(kEpiResidual, g2, ws.ut_hi, ws.ut_lo, ws.status, stream, walker_gemm_f16(w));
  if (st != HZ_OK) return st;
  l2_basis_kernel<<<dim3(kL2K, n2), 256, 0, stream>>>(ws.l2_phi, ws.l2_E, ws.l2_B2, n2, d);
  for (int n = 0; n < n2; ++n)
    split_transpose_kernel<<<dim3((d + 31) / 32, kL2K / 32), dim3(32, 8), 0, stream>>>(
        ws.l2_B2 + (size_t)n * kL2K * d, ws.l2_bt_hi + (size_t)n * d * kL2K,
        ws.l2_bt_lo + (size_t)n * d * kL2K, kL2K, d);
  l2_gram_kernel<<<dim3(kL2K / 32, kL2K / 32, n2), 256, 0, stream>>>(ws.l2_B2, ws.l2_G2, d);
  l2_gram_split_kernel<<<dim3(kL2GN, n2), 96, 0, stream>>>(ws.l2_G2, ws.l2_g_hi, ws.l2_g_lo);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// Second level of one chunk in coefficient space: rows of the level land in `out`.
int run_level2(const hz_wavefunction* w, const hz_energy_frame* f, long long Bc, const Workspace& ws,
               float* out, cudaStream_t stream) {
  const int N = w->n_sites, d = w->d_m, n1 = N / 2, n2 = N / 4;
  const int tiles = (int)((Bc + 7) / 8), Mpad = tiles * 128;
  L2Args a{};
  a.N = N; a.d = d; a.nodes1 = n1; a.nodes2 = n2; a.Bc = (int)Bc; a.tiles = tiles; a.eps = w->merge_eps;
  a.coef1 = ws.l1_coef; a.J_eff = f->J_eff; a.op1 = w->opcodes; a.op2 = w->opcodes + n1;
  a.X = ws.l2_X; a.Y = ws.l2_Y;
  a.s_in = ws.sA; a.js_in = ws.jsA; a.ls_in = ws.lsA;
  a.s_out = ws.sB; a.js_out = ws.jsB; a.ls_out = ws.lsB;
  {
    StageScope scope(kStL2Coeff, stream, (double)Bc * n2 * 2.0 * 21 * 256);
    l2_coeff_kernel<<<dim3(tiles, n2), 256, 0, stream>>>(a);
    HZ_CUDA_TRY(cudaGetLastError());
  }
  {
    StageScope scope(kStL2Gram, stream, 2.0 * Mpad * (double)n2 * kL2K * kL2GN, n2);
    for (int n = 0; n < n2; ++n) {
      GemmArgs g{};
      g.A = ws.l2_X + (size_t)n * Mpad * kL2K; g.C = ws.l2_Y + (size_t)n * Mpad * kL2GN;
      g.M = Mpad; g.N = kL2GN; g.K = kL2K; g.lda = kL2K; g.ldb = kL2GN; g.ldc = kL2GN;
      int st = launch_gemm_tc(kEpiStore, g, ws.l2_g_hi + (size_t)n * kL2GN * kL2K,
                              ws.l2_g_lo + (size_t)n * kL2GN * kL2K, ws.status, stream);
      if (st != HZ_OK) return st;
    }
  }
  {
    StageScope scope(kStL2Norm, stream, (double)Bc * n2 * 2.0 * kL2K * (144 + 12 + 2 + 26));
    l2_norm_kernel<<<dim3(tiles, n2), 256, 0, stream>>>(a);
    HZ_CUDA_TRY(cudaGetLastError());
  }
  StageScope scope(kStL2Expand, stream, 2.0 * Mpad * (double)n2 * kL2K * d, n2);
  for (int n = 0; n < n2; ++n) {
    GemmArgs g{};
    g.A = ws.l2_X + (size_t)n * Mpad * kL2K; g.C = out;
    g.M = Mpad; g.N = d; g.K = kL2K; g.lda = kL2K; g.ldb = d; g.ldc = d;
    g.sc_rows = packed_rows(N, n2, 1); g.sc_walkers = (int)Bc;
    g.sc_j0 = 12 * n; g.sc_u = 3 * N + n; g.sc_l = 3 * N + n2 + n;
    int st = launch_gemm_tc(kEpiScatter, g, ws.l2_bt_hi + (size_t)n * d * kL2K,
                            ws.l2_bt_lo + (size_t)n * d * kL2K, ws.status, stream);
    if (st != HZ_OK) return st;
  }
  return HZ_OK;
}

int run_chunk(const hz_wavefunction* w, const hz_energy_frame* f, int jets, const float* q,
              long long b0, long long Bc, long long Btot, float* log_abs, float* phase,
              float* energies, float* grad, const Workspace& ws, cudaStream_t stream) {
  const int N = w->n_sites, d = w->d_m, G = d / kDr;
  Level L{};
  L.N = N; L.d = d; L.G = G; L.jets = jets; L.Bc = (int)Bc;

  const bool level1 = use_level1() && N >= 2;
  const bool level2 = use_level2(w, jets);
  if (!level1) {
    L.nodes = N; L.m = 0; L.rows_in = 0; L.rows_out = packed_rows(N, N, jets);
    StageScope scope(kStLeaf, stream, (double)Bc * N * d * (jets ? 2.0 * (16 + 10 + 12) : 2.0 * 5));
    leaf_kernel<<<dim3(N, (unsigned)Bc), kLeafThreads, 0, stream>>>(
        L, q + (size_t)b0 * N * 4, ws.leaf_map, f ? f->J_eff : nullptr, ws.bufA, ws.sA, ws.jsA, ws.lsA);
    HZ_CUDA_TRY(cudaGetLastError());
  } else {
    // leaves and first level: coefficients, then the rows the second level reads
    const int nodes = N / 2;
    L.nodes = nodes; L.m = 3; L.rows_in = 0; L.rows_out = packed_rows(N, nodes, jets);
    L1Args la{};
    la.N = N; la.d = d; la.nodes = nodes; la.jets = jets; la.Bc = (int)Bc; la.eps = w->merge_eps;
    la.q = q + (size_t)b0 * N * 4; la.Gs = ws.l1_gs; la.G16 = ws.l1_g16;
    la.J_eff = f ? f->J_eff : nullptr; la.opcodes = w->opcodes; la.coef = ws.l1_coef;
    la.s_out = ws.sA; la.js_out = ws.jsA; la.ls_out = ws.lsA;
    {
      StageScope scope(kStL1Coeff, stream, (double)Bc * nodes * (jets ? 9000.0 : 1200.0));
      l1_coeff_kernel<<<(unsigned)((Bc * nodes + 127) / 128), 128, 0, stream>>>(la);
      HZ_CUDA_TRY(cudaGetLastError());
    }
    if (level2) {
      int st = run_level2(w, f, Bc, ws, ws.bufA, stream);
      if (st != HZ_OK) return st;
    } else {
      StageScope scope(kStL1Expand, stream, 2.0 * Bc * nodes * (jets ? 8.0 : 1.0) * kL1Basis * d);
      l1_expand_kernel<<<dim3((d + 255) / 256, nodes, (unsigned)((Bc + kL1WalkersPerCta - 1) / kL1WalkersPerCta)),
                         256, 0, stream>>>(L, ws.l1_coef, ws.l1_phi, ws.leaf_map, ws.bufA);
      HZ_CUDA_TRY(cudaGetLastError());
    }
  }

  float *cur = ws.bufA, *nxt = ws.bufB;
  float *s_c = ws.sA, *s_n = ws.sB, *ls_c = ws.lsA, *ls_n = ws.lsB, *js_c = ws.jsA, *js_n = ws.jsB;
  size_t h_off = level1 ? (size_t)(N / 2) * w->r_merge : 0, op_off = level1 ? N / 2 : 0;
  if (level2) {       // the second level's scalar carriers sit in the "next" set
    s_c = ws.sB; s_n = ws.sA; ls_c = ws.lsB; ls_n = ws.lsA; js_c = ws.jsB; js_n = ws.jsA;
    h_off += (size_t)(N / 4) * w->r_merge;
    op_off += N / 4;
  }
  for (int k = level2 ? 4 : (level1 ? 2 : 1); k < N; k *= 2) {
    const int nodes = N / (2 * k);
    int level_index = 0;
    while ((1 << level_index) < k) ++level_index;
    L.nodes = nodes; L.m = 3 * k;
    L.rows_in = packed_rows(N, 2 * nodes, jets);
    L.rows_out = packed_rows(N, nodes, jets);
    // merge
    {
      // per (pair, group): A_R, A_L and the cross term are 32^3 MACs each; raw and the two
      // Laplacian terms 32^2; with jets 2m rows through 32x32 maps, Y = W_off J_R and C = J_L^T Y
      const double mm = L.m;
      const double per = jets ? 2.0 * (3 * 32768.0 + 3 * 1024.0 + 2 * mm * 1024.0 + mm * mm * 32.0 + mm * 1024.0)
                              : 2.0 * (32768.0 + 1024.0);
      const double per_cross = 2.0 * (32768.0 + mm * mm * 32.0 + mm * 1024.0);
      if (use_merge_tc(w, jets)) {
        {
          StageScope scope(kStMerge, stream, (per - (jets == 1 ? per_cross : 0.0)) * (double)Bc * nodes * G);
          int st = launch_merge_tc(L, w, f ? f->J_eff : nullptr, ws, cur, nxt, stream);
          if (st != HZ_OK) return st;
        }
        if (jets == 1) {      // value-and-gradient passes need no Laplacian
          // cross_tc_kernel is preceded by the pack of the level's W images
          StageScope scope(kStMergeCross, stream, per_cross * (double)Bc * nodes * G,
                           cross_on_tcgen05(L) ? 2 : 1);
          int st = launch_merge_cross(L, w, f->J_eff, ws, cur, nxt, stream);
          if (st != HZ_OK) return st;
        }
      } else if (!jets && use_tapply_tc()) {
        // values only: raw = A_R u_L with A_R from u_R on tcgen05 (children rows 2p, 2p + 1, parent row p)
        StageScope scope(kStMerge, stream, per * (double)Bc * nodes * G);
        TapplyArgs ta{cur, cur, nxt, 2, 1, 2, 0, 1, 0, Bc * nodes, nodes, nullptr, d, ws.ta_scale, 0};
        int st = launch_tapply(0, ta, G, ws.ta_packed, ws.status, stream, 1);
        if (st != HZ_OK) return st;
      } else {
        StageScope scope(kStMerge, stream, per * (double)Bc * nodes * G);
        int st = launch_tstage(L, w, f ? f->J_eff : nullptr, cur, nxt, stream);
        if (st != HZ_OK) return st;
      }
    }
    // out = raw + ((raw V) * h) U on every packed row
    {
      const long long M = Bc * L.rows_out;
      GemmArgs g1{};
      g1.A = nxt; g1.B = w->merge_V; g1.C = ws.Z; g1.M = (int)M; g1.N = w->r_merge; g1.K = d;
      g1.lda = d; g1.ldb = w->r_merge; g1.ldc = w->r_merge;
      g1.h = w->merge_h + h_off; g1.rows_per_walker = L.rows_out; g1.three_n = jets ? 3 * N : 0;
      g1.rows_per_node = 2 * L.m; g1.nodes = nodes;
      int st;
      {
        StageScope scope(kStGemmV, stream, 2.0 * (double)M * d * w->r_merge);
        st = gemm_dispatch(kEpiNodeScale, g1, ws.vt_hi, ws.vt_lo, ws.status, stream, walker_gemm_f16(w));
      }
      if (st != HZ_OK) return st;
      GemmArgs g2{};
      g2.A = ws.Z; g2.B = w->merge_U; g2.C = nxt; g2.R = nxt; g2.M = (int)M; g2.N = d;
      g2.K = w->r_merge; g2.lda = w->r_merge; g2.ldb = d; g2.ldc = d;
      // K = r_merge is short: one pass over Z for the row exponents is cheap, and eight k-tiles
      // then share an accumulator (for the V product the pass over the 6 KB rows cost what it saved)
      g2.a_expo = ws.row_expo;
      {
        StageScope scope(kStGemmU, stream, 2.0 * (double)M * d * w->r_merge);
        st = gemm_dispatch(kEpiResidual, g2, ws.ut_hi, ws.ut_lo, ws.status, stream, walker_gemm_f16(w));
      }
      if (st != HZ_OK) return st;
    }
    // normalise + gate
    if (!jets && d <= kNvMaxD) {
      StageScope scope(kStNormReduce, stream, (double)Bc * nodes * d * 3.0);
      const long long rows_total = Bc * nodes;
      norm_values_kernel<<<(unsigned)((rows_total + 7) / 8), 256, 0, stream>>>(
          d, nodes, rows_total, w->merge_eps, w->opcodes + op_off, cur, nxt, s_c, s_n, ws.nout);
      HZ_CUDA_TRY(cudaGetLastError());
    } else {
      const int m2 = 2 * L.m, mp = pad16(m2);
      // nodes with many Jacobian rows: W J on tcgen05 (gram_tc_kernel), then the scalar part only
      // value-and-gradient passes (jets == 2) need only |out|^2 and J.out: no Gram matrix, no W
      const bool vg = jets == 2;
      const bool tc_norm = !vg && use_tc_norm(w, jets, m2);
      const bool wide = !vg && mp <= 48;
      const bool huge = jets && !tc_norm && mp > kNrMaxRowsShared;
      const int cols = (wide || tc_norm) ? kNrColsWide : (huge ? kNrColsHuge : kNrColsNarrow);
      const bool w_shared = jets && !tc_norm && !huge && !vg;
      const size_t smem_r = ((jets && !tc_norm ? (w_shared ? (size_t)mp * (mp + 4) : 0) + (size_t)mp * (cols + 8) : 0) +
                             cols + 2 * (size_t)mp + 3 * kNrWarps + 8) * sizeof(float);
      auto kernel = tc_norm ? norm_reduce_kernel<kNrColsWide, true>
                    : wide  ? norm_reduce_kernel<kNrColsWide, false>
                    : huge  ? norm_reduce_kernel<kNrColsHuge, true>
                    : vg    ? norm_reduce_kernel<kNrColsNarrow, true>
                            : norm_reduce_kernel<kNrColsNarrow, false>;
      {
        const int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(kernel), (int)smem_r);
        if (rc != HZ_OK) return rc;
      }
      {
        StageScope scope(kStNormReduce, stream,
                         (double)Bc * nodes * d * (jets ? 2.0 * (2 + m2 + (double)m2 * m2) : 2.0),
                         tc_norm ? 2 : 1);
        if (tc_norm) {
          SyrkArgs sa{};
          sa.X = nxt; sa.rows_pw = L.rows_out; sa.d = d; sa.three_n = 3 * N; sa.Bc = (int)Bc;
          sa.m2 = m2; sa.nodes = nodes; sa.blocks = (3 * N + 2 * nodes + 127) / 128;
          sa.W = ws.gw + (size_t)level_index * 9 * N * N;
          sa.part = ws.gram; sa.a = ws.ga; sa.oo = ws.goo; sa.oL = ws.goL;
          int st = launch_syrk_tc(sa, ws.status, stream);
          if (st != HZ_OK) return st;
        }
        kernel<<<dim3(nodes, (unsigned)Bc), kNrThreads, smem_r, stream>>>(
            L, w->merge_eps, f ? f->J_eff : nullptr, w->opcodes + op_off, nxt, s_c, js_c, ls_c,
            s_n, js_n, ls_n, ws.nout, ws.dr, ws.wdr, tc_norm ? ws.gram : nullptr,
            tc_norm ? ws.ga : nullptr, tc_norm ? ws.goo : nullptr, tc_norm ? ws.goL : nullptr);
        HZ_CUDA_TRY(cudaGetLastError());
      }
      StageScope scope(kStNormApply, stream, (double)Bc * nodes * d * (jets ? 2.0 * (3 + 2.0 * m2) : 1.0));
      norm_apply_kernel<<<dim3((d + kNaThreads - 1) / kNaThreads, nodes, (unsigned)Bc), kNaThreads,
                          2 * (size_t)(m2 + 1) * sizeof(float), stream>>>(
          L, w->opcodes + op_off, cur, nxt, ws.nout, ws.dr, ws.wdr);
      HZ_CUDA_TRY(cudaGetLastError());
    }
    h_off += (size_t)nodes * w->r_merge;
    op_off += nodes;
    float* tmp;
    tmp = cur; cur = nxt; nxt = tmp;
    tmp = s_c; s_c = s_n; s_n = tmp;
    tmp = ls_c; ls_c = ls_n; ls_n = tmp;
    tmp = js_c; js_c = js_n; js_n = tmp;
  }
  // root readout
  L.nodes = 1; L.rows_out = packed_rows(N, 1, jets); L.m = 3 * N / 2;
  {
    const long long M = Bc * L.rows_out;
    GemmArgs g1{};
    g1.A = cur; g1.B = w->readout_V; g1.C = ws.Z; g1.M = (int)M; g1.N = w->r_ro; g1.K = d;
    g1.lda = d; g1.ldb = w->r_ro; g1.ldc = w->r_ro;
    g1.h = w->readout_h; g1.rows_per_walker = L.rows_out; g1.three_n = jets ? 3 * N : 0;
    g1.rows_per_node = 3 * N; g1.nodes = 1;
    int st;
    {
      StageScope scope(kStRootGemm, stream, 2.0 * (double)M * d * w->r_ro);
      st = gemm_dispatch(kEpiNodeScale, g1, ws.rt_hi, ws.rt_lo, ws.status, stream, walker_gemm_f16(w));
    }
    if (st != HZ_OK) return st;
    StageScope scope(kStRoot, stream, (double)Bc * (2.0 * L.rows_out * 2 * w->r_ro + (jets ? 6.0 * 9 * N * N : 0)));
    const size_t smem = ((size_t)2 * w->r_ro + 9 * N + 2) * sizeof(float) + 9 * 8 * sizeof(double) + 16;
    st = ensure_kernel_attributes(reinterpret_cast<const void*>(root_kernel), (int)smem);
    if (st != HZ_OK) return st;
    root_kernel<<<(unsigned)Bc, kRootThreads, smem, stream>>>(
        L, w->r_ro, ws.Z, w->readout_U, f ? f->J_eff : nullptr, f ? f->one_body_field : nullptr,
        f ? f->radial_const : 0.f, s_c, js_c, ls_c, log_abs, phase, energies, grad, b0, Btot,
        ws.status);
    HZ_CUDA_TRY(cudaGetLastError());
  }
  return HZ_OK;
}

// jets: 0 values only, 1 value + Jacobian + Laplacian (energy), 2 value + Jacobian (the sampler's
// value-and-gradient). prepared: the once-per-call arrays in `workspace` (weight splits, leaf map,
// level bases, packed T) are those of an earlier call with the same wavefunction, jets and
// workspace size, and are not rebuilt.
int run(const hz_wavefunction* w, const hz_energy_frame* f, int jets, const float* q,
        long long B, float* log_abs, float* phase, float* energies, float* grad, void* workspace,
        long long workspace_bytes, void* stream, bool prepared = false) {
  int st = check_wavefunction(w);
  if (st != HZ_OK) return st;
  if (B < 0) return HZ_ERR_BAD_SHAPE;
  if (B == 0) return HZ_OK;
  if (!q || !log_abs || !phase || !workspace) return HZ_ERR_NULL_POINTER;
  if (jets == 1 && (!f || !f->J_eff || !f->one_body_field)) return HZ_ERR_NULL_POINTER;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return HZ_ERR_MISALIGNED;
  const size_t per1 = carve(w, jets, 1, nullptr).bytes;
  if ((size_t)workspace_bytes < per1) return HZ_ERR_WORKSPACE;
  // largest chunk that fits the workspace (and keeps every grid dimension below 65535)
  long long Bc = B < 60000 ? B : 60000;
  if (carve(w, jets, Bc, nullptr).bytes > (size_t)workspace_bytes) {
    long long lo = 1, hi = Bc;            // carve(lo) fits, carve(hi) does not
    while (hi - lo > 1) {
      const long long mid = lo + (hi - lo) / 2;
      if (carve(w, jets, mid, nullptr).bytes <= (size_t)workspace_bytes) lo = mid; else hi = mid;
    }
    Bc = lo;
  }
  // packed row counts must fit the GEMM's 32-bit row index
  while (Bc > 1 && Bc * packed_rows(w->n_sites, w->n_sites, jets) > 0x7fffffffLL / 2) Bc /= 2;
  Workspace ws = carve(w, jets, Bc, static_cast<char*>(workspace));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // value-and-gradient passes carry no Laplacian: where a kernel still takes an energy frame it
  // gets one of zeros (in the workspace)
  hz_energy_frame zero{};
  if (jets == 2) {
    zero.J_eff = ws.zero_frame;
    zero.one_body_field = ws.zero_frame + (size_t)9 * w->n_sites * w->n_sites;
    zero.radial_const = 0.f;
    f = &zero;
    if (!prepared)
      HZ_CUDA_TRY(cudaMemsetAsync(ws.zero_frame, 0,
                                  (size_t)(9 * w->n_sites * w->n_sites + 3 * w->n_sites) * sizeof(float), s));
  }
  if (!prepared) {
    st = prepare_weights(w, ws, s);
    if (st != HZ_OK) return st;
    st = prepare_leaf_map(w, ws, s);
    if (st != HZ_OK) return st;
    if (use_level1() && w->n_sites >= 2) {
      st = prepare_level1(w, ws, s);
      if (st != HZ_OK) return st;
    }
    if (use_level2(w, jets)) {
      st = prepare_level2(w, ws, s);
      if (st != HZ_OK) return st;
    }
    if (jets == 1 && w->n_sites > 1) {
      st = prepare_tc_norm(w, f, ws, s);
      if (st != HZ_OK) return st;
    }
    if (use_merge_tc(w, jets)) {
      merge_t_pack_kernel<<<w->d_m / kDr, 256, 0, s>>>(w->merge_T, reinterpret_cast<__half*>(ws.t_packed),
                                                      ws.t_scale);
      HZ_CUDA_TRY(cudaGetLastError());
    }
    if (!jets && w->n_sites > 1 && use_tapply_tc()) {
      st = tapply_prepare(w->merge_T, w->d_m / kDr, ws.ta_packed, ws.ta_scale, s, 1);
      if (st != HZ_OK) return st;
    }
  }
  for (long long b0 = 0; b0 < B; b0 += Bc) {
    const long long nb = (B - b0 < Bc) ? (B - b0) : Bc;
    st = run_chunk(w, f, jets, q, b0, nb, B, log_abs, phase, energies, grad, ws, s);
    if (st != HZ_OK) return st;
  }
  return HZ_OK;
}

#include "hz_vjp.cuh"

}  // namespace
}  // namespace hz

// Value and chart gradient for the sampler (hz_mcmc.cu): a reverse sweep without parameter
// gradients, or one value-and-Jacobian pass (no Laplacian rows are propagated through the merge,
// no Gram matrices are formed). prepared: see run().
namespace hz {
// HZ_MCMC_GRAD=jets keeps the forward pass with Jacobian rows; the default is one value-only
// forward sweep and one reverse sweep for d log|psi| / dq (the only gradient the sampler reads).
static bool chart_grad_by_reverse_sweep() {
  static const bool enabled = !env_equals("HZ_MCMC_GRAD", "jets");
  return enabled;
}
int chart_value_and_grad(const hz_wavefunction* w, const float* q, long long n, float* log_abs,
                         float* phase, float* grad, void* workspace, long long workspace_bytes,
                         cudaStream_t stream, bool prepared) {
  if (chart_grad_by_reverse_sweep())
    return vjp_chart_value_and_grad(w, q, n, log_abs, phase, grad, workspace, workspace_bytes, stream, prepared);
  return run(w, nullptr, 2, q, n, log_abs, phase, nullptr, grad, workspace, workspace_bytes, stream,
             prepared);
}
long long chart_workspace_bytes(const hz_wavefunction* w, long long walkers_per_chunk) {
  if (check_wavefunction(w) != HZ_OK || walkers_per_chunk <= 0) return -1;
  const size_t jets = carve(w, 2, walkers_per_chunk, nullptr).bytes;
  const size_t reverse = vjp_chart_bytes(w, walkers_per_chunk);
  return (long long)(jets > reverse ? jets : reverse);
}
}  // namespace hz

extern "C" long long hz_walker_workspace_bytes(const hz_wavefunction* w, int with_jets,
                                               long long walkers_per_chunk) {
  if (hz::check_wavefunction(w) != HZ_OK || walkers_per_chunk <= 0) return -1;
  if (with_jets < 0 || with_jets > 2) return -1;
  return (long long)hz::carve(w, with_jets, walkers_per_chunk, nullptr).bytes;
}

extern "C" int hz_logpsi_grad(const hz_wavefunction* w, const float* q, long long B, float* log_abs,
                              float* phase, float* grad, void* workspace, long long workspace_bytes,
                              void* stream) {
  if (B > 0 && !grad) return HZ_ERR_NULL_POINTER;
  return hz::run(w, nullptr, 2, q, B, log_abs, phase, nullptr, grad, workspace, workspace_bytes,
                 stream);
}

extern "C" int hz_logpsi(const hz_wavefunction* w, const float* q, long long B, float* log_abs,
                         float* phase, void* workspace, long long workspace_bytes, void* stream) {
  return hz::run(w, nullptr, 0, q, B, log_abs, phase, nullptr, nullptr, workspace,
                 workspace_bytes, stream);
}

extern "C" int hz_local_energy(const hz_wavefunction* w, const hz_energy_frame* frame,
                               const float* q, long long B, float* energies, float* log_abs,
                               float* phase, float* grad, void* workspace,
                               long long workspace_bytes, void* stream) {
  if (B > 0 && !energies) return HZ_ERR_NULL_POINTER;
  return hz::run(w, frame, 1, q, B, log_abs, phase, energies, grad, workspace, workspace_bytes,
                 stream);
}

// ------------------------------------------------------------------ log-psi without allocation
// Some hosts of this library cannot hand it device memory and must not let it allocate any:
// a plugin inside a runtime whose own pool has already claimed the GPU (a cudaMalloc from the
// plugin can fail there, and it stalls every stream of the device while it runs), or a binding
// that is given input and output buffers only and has no scratch-allocator to ask. For them
// hz_logpsi_static runs the same pipeline as hz_logpsi with its scratch in the fixed array
// below, which every GPU that loads this library holds until the process exits.
#define HZ_STATIC_SCRATCH_BYTES (32ll << 20)
static __device__ __align__(256) unsigned char g_static_scratch[HZ_STATIC_SCRATCH_BYTES];

namespace hz {
namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {};

// Device address of g_static_scratch on the current device. In host code the array's name is
// only a handle for the runtime, never an address a kernel may use; the address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_of_current_device(void** out) {
  int dev = -1;
  HZ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return HZ_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    HZ_CUDA_TRY(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
    if (ptr == nullptr) return HZ_ERR_CUDA;
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return HZ_OK;
}
}  // namespace
}  // namespace hz

extern "C" long long hz_vjp_workspace_bytes(const hz_wavefunction* w, long long walkers_per_chunk,
                                            int with_factors) {
  if (hz::check_wavefunction(w) != HZ_OK || walkers_per_chunk <= 0) return -1;
  if (with_factors < 0 || with_factors > 2) return -1;
  return (long long)hz::vjp_carve(w, walkers_per_chunk, with_factors, nullptr).bytes;
}

extern "C" int hz_logpsi_vjp(const hz_wavefunction* w, const float* q, long long B,
                             const float* cot_log_abs, const float* cot_phase,
                             const hz_wavefunction_grads* grads, const hz_kfac_factors* factors,
                             float* dq, float* log_abs, float* phase, void* workspace,
                             long long workspace_bytes, void* stream) {
  return hz::vjp_run(w, q, B, cot_log_abs, cot_phase, grads, factors, dq, log_abs, phase, workspace,
                     workspace_bytes, stream);
}

extern "C" long long hz_static_scratch_bytes(void) { return HZ_STATIC_SCRATCH_BYTES; }

extern "C" int hz_logpsi_static(const hz_wavefunction* w, const float* q, long long B,
                                float* log_abs, float* phase, void* stream) {
  int st = hz::check_wavefunction(w);
  if (st != HZ_OK) return st;
  // the stage timer creates CUDA events, which is an allocation: not on this path
  if (hz::stage_timing_on()) return HZ_ERR_UNSUPPORTED;
  // one walker's scratch is the smallest chunk the pipeline can run; beyond the array: refuse
  const long long need = (long long)hz::carve(w, 0, 1, nullptr).bytes;
  if (need > HZ_STATIC_SCRATCH_BYTES) return HZ_ERR_STATIC_SCRATCH;
  void* scratch = nullptr;
  st = hz::static_scratch_of_current_device(&scratch);
  if (st != HZ_OK) return st;
  // the array of the CURRENT device is used: inputs and outputs must live there too
  // (cudaPointerGetAttributes allocates nothing)
  if (B > 0) {
    int dev = -1;
    HZ_CUDA_TRY(cudaGetDevice(&dev));
    const void* ptrs[3] = {q, log_abs, phase};
    for (const void* p : ptrs) {
      if (p == nullptr) return HZ_ERR_NULL_POINTER;
      cudaPointerAttributes attr;
      HZ_CUDA_TRY(cudaPointerGetAttributes(&attr, p));
      if ((attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) &&
          attr.device != dev)
        return HZ_ERR_WRONG_DEVICE;
    }
  }
  return hz::run(w, nullptr, 0, q, B, log_abs, phase, nullptr, nullptr, scratch,
                 HZ_STATIC_SCRATCH_BYTES, stream);
}

// A device wait that nothing will ever satisfy, with a limit of about a millisecond: the wait
// runs out, the thread records the code in the status word and the kernel returns - the same
// bounded-wait routine, status word and reporting path as the tensor-core kernels use, exercised
// without touching any of them.
namespace hz {
namespace {
__global__ void wait_timeout_probe_kernel(int* __restrict__ status, long long limit_cycles) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const uint32_t addr = smem_u32(&bar);
    const long long t0 = clock64();
    bool done = false;
    while (!done && clock64() - t0 <= limit_cycles) {
      uint32_t ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(addr), "r"(0u)
          : "memory");
      done = ok != 0;
    }
    if (!done) atomicCAS(status, 0, kTcTimeoutLoad);
  }
}
}  // namespace
}  // namespace hz

extern "C" int hz_selftest_wait_timeout(void* workspace, long long workspace_bytes, void* stream) {
  if (!workspace) return HZ_ERR_NULL_POINTER;
  if (workspace_bytes < 256) return HZ_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return HZ_ERR_MISALIGNED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  HZ_CUDA_TRY(cudaMemsetAsync(workspace, 0, sizeof(int), s));
  hz::wait_timeout_probe_kernel<<<1, 32, 0, s>>>(static_cast<int*>(workspace), 2000000ll);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// Status word of the last call that used `workspace` (its first word): 0, or the code of the
// first device wait that ran out. Waits for `stream`.
extern "C" int hz_workspace_status(const void* workspace, void* stream) {
  if (!workspace) return HZ_ERR_NULL_POINTER;
  int word = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  HZ_CUDA_TRY(cudaMemcpyAsync(&word, workspace, sizeof(int), cudaMemcpyDeviceToHost, s));
  HZ_CUDA_TRY(cudaStreamSynchronize(s));
  return word == 0 ? HZ_OK : HZ_ERR_TIMEOUT;
}
