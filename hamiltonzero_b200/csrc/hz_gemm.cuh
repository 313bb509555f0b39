// Row-major fp32 GEMM C = epilogue(A @ B) on the tensor cores with 3xTF32 split
// products (fp32-level accuracy), used for the walker path's shared-weight linear
// maps: rows are (walker, Jacobian-row) pairs, weights are the model's factors.
//
// Tile 128 x 128 x 16, 8 warps (2 x 4), warp tile 64 x 32, cp.async double buffer.
// Requirements: K, N, lda, ldb, ldc multiples of 4 and 16-byte aligned bases.
#pragma once
#include "hz_internal.h"
#include "hz_mma.cuh"

namespace hz {

enum GemmEpilogue { kEpiStore = 0, kEpiNodeScale = 1, kEpiResidual = 2, kEpiScatter = 3 };

struct GemmArgs {
  const float* A;
  const float* B;
  float* C;
  const float* R;      // residual (kEpiResidual), may alias C
  int M, N, K;
  int lda, ldb, ldc;
  // kEpiNodeScale: C[row, col] = acc * h[node(row) * N + col] with rows packed per walker as
  // [three_n Jacobian rows | nodes value rows | nodes Laplacian rows]
  const float* h;
  int rows_per_walker, three_n, rows_per_node, nodes;
  // kEpiScatter (tcgen05 kernel only): the rows of a 128-row tile are 8 walkers x 12 Jacobian
  // rows, then 8 value rows, 8 Laplacian rows and 16 unused rows; they go to the packed jet
  // rows [sc_j0, sc_j0 + 12), sc_u and sc_l of walkers 8*tile ... of C, which holds sc_rows
  // rows per walker for sc_walkers walkers.
  int sc_rows, sc_walkers, sc_j0, sc_u, sc_l;
  // FP16-split tcgen05 kernel only: scratch for one exponent per row of A (M ints). When given,
  // every row is scaled by one power of two for the whole K, and several k-tiles share a TMEM
  // accumulator between two folds into registers; when null the scale is per (row, k-tile).
  int* a_expo;
};

constexpr int kGemmBM = 128, kGemmBN = 128, kGemmBK = 16, kGemmThreads = 256;
constexpr int kGemmLdA = kGemmBK + 4;     // 20: conflict-free A fragments
constexpr int kGemmLdB = kGemmBN + 8;     // 136: conflict-free B fragments

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, int src_bytes) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src),
               "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ int gemm_node_of_row(const GemmArgs& a, int row) {
  const int r = row % a.rows_per_walker;
  return (r < a.three_n) ? (r / a.rows_per_node) : ((r - a.three_n) % a.nodes);
}

template <int EPI>
__global__ void __launch_bounds__(kGemmThreads) gemm3_kernel(GemmArgs a) {
  __shared__ __align__(16) float As[2][kGemmBM * kGemmLdA];
  __shared__ __align__(16) float Bs[2][kGemmBK * kGemmLdB];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wm = warp >> 2, wn = warp & 3;          // 2 x 4 warps
  const int row0 = blockIdx.y * kGemmBM, col0 = blockIdx.x * kGemmBN;

  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

  auto load_tiles = [&](int stage, int k0) {
    // A tile: 128 rows x 16 floats = 512 float4, two per thread
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * kGemmThreads;
      const int r = idx >> 2, c = (idx & 3) * 4;
      const int row = row0 + r, col = k0 + c;
      const bool ok = row < a.M && col < a.K;
      const float* src = ok ? a.A + (size_t)row * a.lda + col : a.A;
      cp_async16(&As[stage][r * kGemmLdA + c], src, ok ? 16 : 0);
    }
    // B tile: 16 rows x 128 floats = 512 float4, two per thread
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * kGemmThreads;
      const int r = idx >> 5, c = (idx & 31) * 4;
      const int row = k0 + r, col = col0 + c;
      const bool ok = row < a.K && col < a.N;
      const float* src = ok ? a.B + (size_t)row * a.ldb + col : a.B;
      cp_async16(&Bs[stage][r * kGemmLdB + c], src, ok ? 16 : 0);
    }
    cp_async_commit();
  };

  const int ktiles = (a.K + kGemmBK - 1) / kGemmBK;
  load_tiles(0, 0);
  for (int kt = 0; kt < ktiles; ++kt) {
    const int stage = kt & 1;
    if (kt + 1 < ktiles) {
      load_tiles(stage ^ 1, (kt + 1) * kGemmBK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* as = As[stage];
    const float* bs = Bs[stage];
    // The tensor core's fp32 accumulation truncates; over a K of a thousand that is a
    // systematic loss of ~1e-5. Each k-tile therefore accumulates a short chain in `part`
    // and is folded into `acc` with round-to-nearest adds.
    float part[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) part[i][j][c] = 0.f;
#pragma unroll
    for (int ks = 0; ks < kGemmBK / 8; ++ks) {
      FragB fb[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = wn * 32 + j * 8 + g;
        fb[j].set(bs[(ks * 8 + t) * kGemmLdB + n], bs[(ks * 8 + t + 4) * kGemmLdB + n]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = wm * 64 + i * 16 + g;
        FragA fa;
        fa.set(as[r * kGemmLdA + ks * 8 + t], as[(r + 8) * kGemmLdA + ks * 8 + t],
               as[r * kGemmLdA + ks * 8 + t + 4], as[(r + 8) * kGemmLdA + ks * 8 + t + 4]);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma3(part[i][j], fa, fb[j]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][j][c] += part[i][j][c];
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = row0 + wm * 64 + i * 16 + g + half * 8;
      if (row >= a.M) continue;
      const float* hrow = nullptr;
      if (EPI == kEpiNodeScale) hrow = a.h + (size_t)gemm_node_of_row(a, row) * a.N;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = col0 + wn * 32 + j * 8 + 2 * t;
        if (col >= a.N) continue;      // N is even, so col + 1 < N as well
        float2 v = make_float2(acc[i][j][half * 2], acc[i][j][half * 2 + 1]);
        if (EPI == kEpiNodeScale) {
          const float2 hh = *reinterpret_cast<const float2*>(hrow + col);
          v.x *= hh.x;
          v.y *= hh.y;
        }
        if (EPI == kEpiResidual) {
          const float2 rr = *reinterpret_cast<const float2*>(a.R + (size_t)row * a.ldc + col);
          v.x += rr.x;
          v.y += rr.y;
        }
        *reinterpret_cast<float2*>(a.C + (size_t)row * a.ldc + col) = v;
      }
    }
  }
}

inline int launch_gemm(int epi, const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return HZ_OK;
  dim3 grid((a.N + kGemmBN - 1) / kGemmBN, (a.M + kGemmBM - 1) / kGemmBM);
  switch (epi) {
    case kEpiStore: gemm3_kernel<kEpiStore><<<grid, kGemmThreads, 0, stream>>>(a); break;
    case kEpiNodeScale: gemm3_kernel<kEpiNodeScale><<<grid, kGemmThreads, 0, stream>>>(a); break;
    default: gemm3_kernel<kEpiResidual><<<grid, kGemmThreads, 0, stream>>>(a); break;
  }
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

}  // namespace hz
