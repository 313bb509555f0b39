// tcgen05 kernel for the reductions of the normalisation stage: the Gram matrix of a walker's
// packed jet rows, G = X X^T with X = [3N Jacobian rows | nodes value rows | nodes Laplacian
// rows] and K = d_m channels, evaluated block by block (128 x 128 blocks on and above the
// diagonal) and reduced on the fly to
//   part[b, bj, A] = sum_{B in column block bj} W[A, B] G[A, B]   (their sum over A in node n and
//                    bj: tr(W J J^T) of the node; plain stores, so the result is deterministic)
//   a[b, A]    = G[A, value row of A's node]                 (J_A . out)
//   oo[b, n]   = G[value row n, value row n],  oL[b, n] = G[value row n, Laplacian row n].
// Both operands of a block are rows of X, K-major as they lie in HBM: TMA lands 128 rows x 32
// channels per operand in the 128-byte swizzle, four warps rewrite them in place as TF32 head +
// tail, and three UMMAs per product accumulate in TMEM; the folders add every k-tile into fp32
// registers (the tensor core's accumulation truncates) and weight the finished block with the
// level's block-diagonal W, which is walker independent and stays in L2. A block above the
// diagonal stands for its mirror image too (weight two). Persistent CTAs, warp roles, barriers
// and bounded waits are those of gemm_tcp_kernel; a diagonal block loads its rows once.
#pragma once
#include "hz_gemm_tc.cuh"

namespace hz {

struct SyrkArgs {
  const float* X;      // packed jets of the chunk: [Bc * rows_pw, d]
  const float* W;      // [three_n, three_n] fp32: J_eff masked to the level's diagonal blocks
  int rows_pw, d, three_n, Bc;
  int m2, nodes;       // Jacobian rows per node, nodes of the level
  int blocks;          // ceil((three_n + 2 nodes) / 128)
  float* part;         // [Bc, blocks, three_n]: entries with bj >= block of row A are written
  float* a;            // [Bc, three_n]
  float* oo;           // [Bc, nodes]
  float* oL;           // [Bc, nodes]
};

template <int STAGES>
__global__ void __launch_bounds__(kTcThreads, 1)
syrk_tc_kernel(const __grid_constant__ CUtensorMap xmap, SyrkArgs a, int* __restrict__ status) {
  constexpr int BN = 128;
  constexpr int kStageBytes = 4 * kTcABytes;      // A head (raw on arrival), A tail, B head, B tail
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t full_bar[STAGES], conv_bar[STAGES], empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2], tfree_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KT = a.d / kTcBK;
  const int per_walker = a.blocks * (a.blocks + 1) / 2;
  const long long total = (long long)per_walker * a.Bc;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&conv_bar[s], kTcRewriteThreads);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tfree_bar[b], 128); }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)(2 * BN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  auto stage_ptr = [&](int s) { return smem + (size_t)s * kStageBytes; };
  auto fail = [&](int code) { atomicExch(status, code); abort_s = 1; };
  // tile -> (walker, row block bi, column block bj >= bi); the blocks of a walker are neighbours
  auto decode = [&](long long tile, int& b, int& bi, int& bj) {
    b = (int)(tile / per_walker);
    int rem = (int)(tile % per_walker);
    bi = 0;
    while (rem >= a.blocks - bi) { rem -= a.blocks - bi; ++bi; }
    bj = bi + rem;
  };

  if (warp < kTcRewriteWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      if (lane == 0) {
        long long it = 0;
        bool alive = true;
        for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
          int b, bi, bj;
          decode(tile, b, bi, bj);
          for (int kt = 0; kt < KT; ++kt, ++it) {
            const int s = (int)(it % STAGES);
            if (it >= STAGES &&
                !mbar_wait_abortable(&empty_bar[s], (uint32_t)((it / STAGES) - 1) & 1, &abort_s)) {
              fail(kTcTimeoutMma);
              alive = false;
              break;
            }
            uint8_t* st = stage_ptr(s);
            mbar_expect_tx(&full_bar[s], (bi == bj ? 1 : 2) * kTcABytes);
            tma_load_2d(st, &xmap, kt * kTcBK, b * a.rows_pw + bi * kTcBM, &full_bar[s]);
            if (bi != bj)
              tma_load_2d(st + 2 * kTcABytes, &xmap, kt * kTcBK, b * a.rows_pw + bj * kTcBM, &full_bar[s]);
          }
        }
        if (abort_s != 0) {
          for (long long j = (it > STAGES ? it - STAGES : 0); j < it; ++j)
            mbar_wait(&full_bar[j % STAGES], (uint32_t)(j / STAGES) & 1);
        }
      }
    } else if (warp == kTcIssueWarp) {
      if (lane == 0) {
        // the last column block holds only the tail of the packed rows: a narrower UMMA
        const int used = a.three_n + 2 * a.nodes - (a.blocks - 1) * kTcBM;
        const int n_last = min(BN, (used + 15) & ~15);
        long long it = 0;
        bool alive = true;
        for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
          int b, bi, bj;
          decode(tile, b, bi, bj);
          const uint32_t idesc = umma_idesc_tf32(bj == a.blocks - 1 ? n_last : BN);
          for (int kt = 0; kt < KT; ++kt, ++it) {
            const int s = (int)(it % STAGES), buf = (int)(it & 1);
            if (!mbar_wait_abortable(&conv_bar[s], (uint32_t)(it / STAGES) & 1, &abort_s) ||
                (it >= 2 && !mbar_wait_abortable(&tfree_bar[buf], (uint32_t)((it >> 1) - 1) & 1, &abort_s))) {
              fail(kTcTimeoutMma);
              alive = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(stage_ptr(s));
            const uint32_t a_lo = a_hi + kTcABytes;
            const uint32_t b_hi = (bi == bj) ? a_hi : a_hi + 2 * kTcABytes;
            const uint32_t b_lo = b_hi + kTcABytes;
            const uint32_t tacc = tmem_base + (uint32_t)(buf * BN);
#pragma unroll
            for (int k8 = 0; k8 < kTcBK / 8; ++k8) {
              const uint32_t off = k8 * 32;
              const uint64_t dah = umma_desc_sw128(a_hi + off), dal = umma_desc_sw128(a_lo + off);
              const uint64_t dbh = umma_desc_sw128(b_hi + off), dbl = umma_desc_sw128(b_lo + off);
              umma_tf32(tacc, dal, dbh, idesc, k8 > 0 ? 1u : 0u);
              umma_tf32(tacc, dah, dbl, idesc, 1u);
              umma_tf32(tacc, dah, dbh, idesc, 1u);
            }
            umma_commit(&empty_bar[s]);
            umma_commit(&tfull_bar[buf]);
          }
        }
      }
    }
  } else if (warp < kTcFoldWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    // rewriters: row tiles -> head (in place) + tail
    const int rt = tid - kTcRewriteWarp0 * 32;
    long long it = 0;
    bool alive = true;
    for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
      int b, bi, bj;
      decode(tile, b, bi, bj);
      const int operands = (bi == bj) ? 1 : 2;
      for (int kt = 0; kt < KT; ++kt, ++it) {
        const int s = (int)(it % STAGES);
        if (!mbar_wait_abortable(&full_bar[s], (uint32_t)(it / STAGES) & 1, &abort_s)) {
          if (lane == 0) fail(kTcTimeoutLoad);
          alive = false;
          break;
        }
        for (int op = 0; op < operands; ++op) {
          float4* hi = reinterpret_cast<float4*>(stage_ptr(s) + op * 2 * kTcABytes);
          float4* lo = reinterpret_cast<float4*>(stage_ptr(s) + op * 2 * kTcABytes + kTcABytes);
#pragma unroll 4
          for (int i = 0; i < 1024 / kTcRewriteThreads; ++i) {
            const int idx = rt + i * kTcRewriteThreads;
            const float4 x = hi[idx];
            float4 h, l;
            h.x = __uint_as_float((__float_as_uint(x.x) + 0x1000u) & 0xFFFFE000u); l.x = x.x - h.x;
            h.y = __uint_as_float((__float_as_uint(x.y) + 0x1000u) & 0xFFFFE000u); l.y = x.y - h.y;
            h.z = __uint_as_float((__float_as_uint(x.z) + 0x1000u) & 0xFFFFE000u); l.z = x.z - h.z;
            h.w = __uint_as_float((__float_as_uint(x.w) + 0x1000u) & 0xFFFFE000u); l.w = x.w - h.w;
            hi[idx] = h;
            lo[idx] = l;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(&conv_bar[s]);
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int q = warp & 3;
    bool ok = true;
    long long it = 0;
    for (long long tile = blockIdx.x; tile < total; tile += gridDim.x) {
      int b, bi, bj;
      decode(tile, b, bi, bj);
      float acc[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      for (int kt = 0; kt < KT; ++kt, ++it) {
        if (!ok) continue;
        const int buf = (int)(it & 1);
        if (!mbar_wait_abortable(&tfull_bar[buf], (uint32_t)(it >> 1) & 1, &abort_s)) {
          if (lane == 0) fail(kTcTimeoutMma);
          ok = false;
          continue;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c0);
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
              "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
              "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
              : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
                "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
                "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
                "=r"(v[31])
              : "r"(taddr)
              : "memory");
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c0 + j] += __uint_as_float(v[j]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(&tfree_bar[buf]);
      }
      if (!ok) continue;
      // ---- epilogue: this thread's row of the block, acc[c] = G[row, bj * 128 + c]
      const int row = bi * kTcBM + q * 32 + lane;        // packed row of the walker
      const int c0 = bj * kTcBM;
      const int three_n = a.three_n, nodes = a.nodes;
      float pg = 0.f;
      if (row < three_n) {
        const int node = row / a.m2;
        // Jacobian x Jacobian entries, weighted by W (zero outside the node's block)
        const int ncols = min(BN, three_n - c0);          // Jacobian columns of this block (<= 0: none)
        const float wgt = (bi == bj) ? 1.f : 2.f;
        const float* wrow = a.W + (size_t)row * three_n + c0;
#pragma unroll
        for (int c = 0; c < BN; c += 4) {
          if (c < ncols) {                                // three_n is a multiple of 4
            const float4 w = *reinterpret_cast<const float4*>(wrow + c);
            pg = fmaf(w.x, acc[c], pg); pg = fmaf(w.y, acc[c + 1], pg);
            pg = fmaf(w.z, acc[c + 2], pg); pg = fmaf(w.w, acc[c + 3], pg);
          }
        }
        pg *= wgt;
        // J_A . out: the column of the node's value row, if it lies in this block
        const int uc = three_n + node - c0;
        if (uc >= 0 && uc < BN) {
          float v = 0.f;
#pragma unroll
          for (int c = 0; c < BN; ++c) v = (c == uc) ? acc[c] : v;
          a.a[(size_t)b * three_n + row] = v;
        }
      } else if (row < three_n + nodes) {
        // value row n: |out|^2 on its own column, out . L on the Laplacian row's column
        const int n = row - three_n;
        const int c_self = row - c0, c_lap = three_n + nodes + n - c0;
        float vs = 0.f, vl = 0.f;
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          vs = (c == c_self) ? acc[c] : vs;
          vl = (c == c_lap) ? acc[c] : vl;
        }
        if (c_self >= 0 && c_self < BN) a.oo[(size_t)b * nodes + n] = vs;
        if (c_lap >= 0 && c_lap < BN) a.oL[(size_t)b * nodes + n] = vl;
      }
      if (row < three_n) a.part[((size_t)b * a.blocks + bj) * three_n + row] = pg;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)(2 * BN))
                 : "memory");
  }
}

// The same reductions with twice the rewriting capacity and half the shared-memory operand
// traffic: the row block's head and tail live in TMEM (A operand of the UMMAs, written by one
// group of rewriter warps), the column block's in shared memory (second group); roles and the
// register budget are those of gemm_tcf_kernel (512 threads: 40 / 96 / 232 registers). The
// rewrite of two operands by four warps was the limit of syrk_tc_kernel (one warp per scheduler).
template <int STAGES, int FOLD>
__global__ void __launch_bounds__(kTfThreads, 1)
syrk_tc2_kernel(const __grid_constant__ CUtensorMap xmap, SyrkArgs a, int* __restrict__ status) {
  constexpr int BN = 128;
  // stage: rows of the row block as they arrive (their head and tail go to TMEM), head and tail
  // of the column block's rows
  constexpr int kStageBytes = 3 * kTcABytes;
  constexpr uint32_t kColALo = 2 * BN, kColAHi = kColALo + 32;     // + 64 per stage
  static_assert(2 * BN + STAGES * 64 <= 512, "TMEM columns");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t full_bar[STAGES], conv_bar[STAGES], empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2], tfree_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KT = a.d / kTcBK;
  const int per_walker = a.blocks * (a.blocks + 1) / 2;
  const long long total = (long long)per_walker * a.Bc;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&conv_bar[s], 2 * kTcRewriteThreads);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tfree_bar[b], 128); }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  auto stage_ptr = [&](int s) { return smem + (size_t)s * kStageBytes; };
  auto fail = [&](int code) { atomicExch(status, code); abort_s = 1; };
  // tile -> (walker, row block bi, column block bj >= bi); the blocks of a walker are neighbours
  auto decode = [&](long long tile, int& b, int& bi, int& bj) {
    b = (int)(tile / per_walker);
    int rem = (int)(tile % per_walker);
    bi = 0;
    while (rem >= a.blocks - bi) { rem -= a.blocks - bi; ++bi; }
    bj = bi + rem;
  };

  if (warp < kTcRewriteWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      if (lane == 0) {
        long long it = 0;
        bool alive = true;
        for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
          int b, bi, bj;
          decode(tile, b, bi, bj);
          for (int kt = 0; kt < KT; ++kt, ++it) {
            const int s = (int)(it % STAGES);
            if (it >= STAGES &&
                !mbar_wait_abortable(&empty_bar[s], (uint32_t)((it / STAGES) - 1) & 1, &abort_s)) {
              fail(kTcTimeoutMma);
              alive = false;
              break;
            }
            uint8_t* st = stage_ptr(s);
            mbar_expect_tx(&full_bar[s], (bi == bj ? 1 : 2) * kTcABytes);
            tma_load_2d(st, &xmap, kt * kTcBK, b * a.rows_pw + bi * kTcBM, &full_bar[s]);
            if (bi != bj)
              tma_load_2d(st + kTcABytes, &xmap, kt * kTcBK, b * a.rows_pw + bj * kTcBM, &full_bar[s]);
          }
        }
        if (abort_s != 0) {
          for (long long j = (it > STAGES ? it - STAGES : 0); j < it; ++j)
            mbar_wait(&full_bar[j % STAGES], (uint32_t)(j / STAGES) & 1);
        }
      }
    } else if (warp == kTcIssueWarp) {
      if (lane == 0) {
        // the last column block holds only the tail of the packed rows: a narrower UMMA
        const int used = a.three_n + 2 * a.nodes - (a.blocks - 1) * kTcBM;
        const int n_last = min(BN, (used + 15) & ~15);
        long long it = 0, gi = 0;        // running k-tile and fold-group counters
        bool alive = true;
        for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
          int b, bi, bj;
          decode(tile, b, bi, bj);
          const uint32_t idesc = umma_idesc_tf32(bj == a.blocks - 1 ? n_last : BN);
          for (int kt = 0; kt < KT; ++kt, ++it) {
            // FOLD consecutive k-tiles share one TMEM accumulator
            const bool first = (kt % FOLD) == 0, last = (kt % FOLD) == FOLD - 1 || kt == KT - 1;
            const int s = (int)(it % STAGES), buf = (int)(gi & 1);
            if (!mbar_wait_abortable(&conv_bar[s], (uint32_t)(it / STAGES) & 1, &abort_s) ||
                (first && gi >= 2 &&
                 !mbar_wait_abortable(&tfree_bar[buf], (uint32_t)((gi >> 1) - 1) & 1, &abort_s))) {
              fail(kTcTimeoutMma);
              alive = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t b_hi = smem_u32(stage_ptr(s)) + kTcABytes;
            const uint32_t b_lo = b_hi + kTcABytes;
            const uint32_t tacc = tmem_base + (uint32_t)(buf * BN);
#pragma unroll
            for (int k8 = 0; k8 < kTcBK / 8; ++k8) {
              const uint32_t off = k8 * 32;
              const uint64_t dbh = umma_desc_sw128(b_hi + off), dbl = umma_desc_sw128(b_lo + off);
              const uint32_t ta = tmem_base + (uint32_t)(s * 64 + k8 * 8);
              umma_tf32_ts(tacc, ta + kColALo, dbh, idesc, (k8 > 0 || !first) ? 1u : 0u);
              umma_tf32_ts(tacc, ta + kColAHi, dbl, idesc, 1u);
              umma_tf32_ts(tacc, ta + kColAHi, dbh, idesc, 1u);
            }
            umma_commit(&empty_bar[s]);
            if (last) {
              umma_commit(&tfull_bar[buf]);
              ++gi;
            }
          }
        }
      }
    }
  } else if (warp < kTfFoldWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    // rewriters. Group 0 (thread = row of the row block = TMEM lane): head and tail of the row go
    // to the stage's 64 TMEM columns, the A operand of the UMMAs. Group 1: head and tail of the
    // column block's rows into the stage's two B tiles (from the tile TMA delivered there, or,
    // for a block on the diagonal, from the row block's tile, which nobody writes).
    const int rgrp = (warp - kTcRewriteWarp0) >> 2;
    const int rt = (warp & 3) * 32 + lane;
    long long it = 0;
    bool alive = true;
    for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
      int b, bi, bj;
      decode(tile, b, bi, bj);
      for (int kt = 0; kt < KT; ++kt, ++it) {
        const int s = (int)(it % STAGES);
        if (!__all_sync(0xffffffffu,
                        mbar_wait_abortable(&full_bar[s], (uint32_t)(it / STAGES) & 1, &abort_s))) {
          if (lane == 0) fail(kTcTimeoutLoad);
          alive = false;
          break;
        }
        if (rgrp == 0) {
          const float4* rowp = reinterpret_cast<const float4*>(stage_ptr(s) + rt * 128);
          uint32_t tl[32], th[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 x = rowp[c ^ (rt & 7)];
            float4 h;
            h.x = __uint_as_float((__float_as_uint(x.x) + 0x1000u) & 0xFFFFE000u);
            h.y = __uint_as_float((__float_as_uint(x.y) + 0x1000u) & 0xFFFFE000u);
            h.z = __uint_as_float((__float_as_uint(x.z) + 0x1000u) & 0xFFFFE000u);
            h.w = __uint_as_float((__float_as_uint(x.w) + 0x1000u) & 0xFFFFE000u);
            th[4 * c] = __float_as_uint(h.x); th[4 * c + 1] = __float_as_uint(h.y);
            th[4 * c + 2] = __float_as_uint(h.z); th[4 * c + 3] = __float_as_uint(h.w);
            tl[4 * c] = __float_as_uint(x.x - h.x); tl[4 * c + 1] = __float_as_uint(x.y - h.y);
            tl[4 * c + 2] = __float_as_uint(x.z - h.z); tl[4 * c + 3] = __float_as_uint(x.w - h.w);
          }
          const uint32_t trow = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(s * 64);
          tmem_st32(trow + kColALo, tl);
          tmem_st32(trow + kColAHi, th);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        } else {
          const float4* src = reinterpret_cast<const float4*>(stage_ptr(s) + (bi == bj ? 0 : kTcABytes));
          float4* hi = reinterpret_cast<float4*>(stage_ptr(s) + kTcABytes);
          float4* lo = reinterpret_cast<float4*>(stage_ptr(s) + 2 * kTcABytes);
#pragma unroll 4
          for (int i = 0; i < 1024 / kTcRewriteThreads; ++i) {
            const int idx = rt + i * kTcRewriteThreads;
            const float4 x = src[idx];
            float4 h, l;
            h.x = __uint_as_float((__float_as_uint(x.x) + 0x1000u) & 0xFFFFE000u); l.x = x.x - h.x;
            h.y = __uint_as_float((__float_as_uint(x.y) + 0x1000u) & 0xFFFFE000u); l.y = x.y - h.y;
            h.z = __uint_as_float((__float_as_uint(x.z) + 0x1000u) & 0xFFFFE000u); l.z = x.z - h.z;
            h.w = __uint_as_float((__float_as_uint(x.w) + 0x1000u) & 0xFFFFE000u); l.w = x.w - h.w;
            hi[idx] = h;
            lo[idx] = l;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        mbar_arrive(&conv_bar[s]);
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int q = warp & 3;
    bool ok = true;
    long long it = 0;
    for (long long tile = blockIdx.x; tile < total; tile += gridDim.x) {
      int b, bi, bj;
      decode(tile, b, bi, bj);
      float acc[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      for (int kt = 0; kt < (KT + FOLD - 1) / FOLD; ++kt, ++it) {
        if (!ok) continue;
        const int buf = (int)(it & 1);
        if (!mbar_wait_abortable(&tfull_bar[buf], (uint32_t)(it >> 1) & 1, &abort_s)) {
          if (lane == 0) fail(kTcTimeoutMma);
          ok = false;
          continue;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c0);
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
              "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
              "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
              : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
                "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
                "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
                "=r"(v[31])
              : "r"(taddr)
              : "memory");
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c0 + j] += __uint_as_float(v[j]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(&tfree_bar[buf]);
      }
      if (!ok) continue;
      // ---- epilogue: this thread's row of the block, acc[c] = G[row, bj * 128 + c]
      const int row = bi * kTcBM + q * 32 + lane;        // packed row of the walker
      const int c0 = bj * kTcBM;
      const int three_n = a.three_n, nodes = a.nodes;
      float pg = 0.f;
      if (row < three_n) {
        const int node = row / a.m2;
        // Jacobian x Jacobian entries, weighted by W (zero outside the node's block)
        const int ncols = min(BN, three_n - c0);          // Jacobian columns of this block (<= 0: none)
        const float wgt = (bi == bj) ? 1.f : 2.f;
        const float* wrow = a.W + (size_t)row * three_n + c0;
#pragma unroll
        for (int c = 0; c < BN; c += 4) {
          if (c < ncols) {                                // three_n is a multiple of 4
            const float4 w = *reinterpret_cast<const float4*>(wrow + c);
            pg = fmaf(w.x, acc[c], pg); pg = fmaf(w.y, acc[c + 1], pg);
            pg = fmaf(w.z, acc[c + 2], pg); pg = fmaf(w.w, acc[c + 3], pg);
          }
        }
        pg *= wgt;
        // J_A . out: the column of the node's value row, if it lies in this block
        const int uc = three_n + node - c0;
        if (uc >= 0 && uc < BN) {
          float v = 0.f;
#pragma unroll
          for (int c = 0; c < BN; ++c) v = (c == uc) ? acc[c] : v;
          a.a[(size_t)b * three_n + row] = v;
        }
      } else if (row < three_n + nodes) {
        // value row n: |out|^2 on its own column, out . L on the Laplacian row's column
        const int n = row - three_n;
        const int c_self = row - c0, c_lap = three_n + nodes + n - c0;
        float vs = 0.f, vl = 0.f;
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          vs = (c == c_self) ? acc[c] : vs;
          vl = (c == c_lap) ? acc[c] : vl;
        }
        if (c_self >= 0 && c_self < BN) a.oo[(size_t)b * nodes + n] = vs;
        if (c_lap >= 0 && c_lap < BN) a.oL[(size_t)b * nodes + n] = vl;
      }
      if (row < three_n) a.part[((size_t)b * a.blocks + bj) * three_n + row] = pg;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(512u)
                 : "memory");
  }
}

// Requires the value row and the Laplacian row of a node in the same or a later block than its
// Jacobian rows (true for the packed layout) and 16-byte aligned rows of W.
inline bool syrk_tc_supported(int three_n, int d) {
  return d % kTcBK == 0 && three_n % 4 == 0 && encode_tiled_fn() != nullptr;
}

inline int launch_syrk_tc(const SyrkArgs& a, int* status, cudaStream_t stream) {
  if (a.Bc <= 0) return HZ_OK;
  CUtensorMap xmap;
  if (!make_map(&xmap, a.X, (long long)a.Bc * a.rows_pw, a.d, a.d, kTcBM)) return HZ_ERR_CUDA;
  const long long total = (long long)a.Bc * (a.blocks * (a.blocks + 1) / 2);
  const int sms = tc_sm_count();
  const unsigned grid = (unsigned)(total < sms ? total : sms);
  static const bool classic = env_equals("HZ_SYRK", "classic");     // the four-rewriter-warp kernel
  if (!classic) {
    constexpr int STAGES = 4;
    constexpr size_t smem = (size_t)STAGES * 3 * kTcABytes + 1024;
    // k-tiles per TMEM accumulator before the fold into fp32 registers (as in the factor GEMMs)
    static const int fold = env_int("HZ_SYRK_FOLD", 2);
    if (fold == 1) {
      const int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(syrk_tc2_kernel<STAGES, 1>), (int)smem);
      if (rc != HZ_OK) return rc;
      syrk_tc2_kernel<STAGES, 1><<<grid, kTfThreads, smem, stream>>>(xmap, a, status);
    } else {
      const int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(syrk_tc2_kernel<STAGES, 2>), (int)smem);
      if (rc != HZ_OK) return rc;
      syrk_tc2_kernel<STAGES, 2><<<grid, kTfThreads, smem, stream>>>(xmap, a, status);
    }
  } else {
    constexpr int STAGES = 3;
    constexpr size_t smem = (size_t)STAGES * 4 * kTcABytes + 1024;
    const int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(syrk_tc_kernel<STAGES>), (int)smem);
    if (rc != HZ_OK) return rc;
    syrk_tc_kernel<STAGES><<<grid, kTcThreads, smem, stream>>>(xmap, a, status);
  }
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

}  // namespace hz
