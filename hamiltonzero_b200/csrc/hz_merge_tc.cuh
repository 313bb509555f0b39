// Quadrilinear merge of the jet passes on tcgen05 / TMEM / TMA (sm_100a).
//
// Reference math: src/hamiltonzero/energy/custom_lap.py:1318-1389 (merge of two jets),
// src/hamiltonzero/compiled/execute.py:34-52 (value). Per (walker, node) pair and group i of
// the merge tensor T_i [32,32,32]:
//   A_R[j,k] = sum_l T[j,k,l] u_R[l]      left rows:  Jraw[A]   = A_R J_L[A],  raw = A_R u_L
//   A_L[j,l] = sum_k T[j,k,l] u_L[k]      right rows: Jraw[m+B] = A_L J_R[B]
//   Laplacian terms A_R L_L (left) and A_L L_R (right)
// (the cross term T : (J_L^T W_off J_R) is the separate kernel merge_tstage_kernel<true>).
//
// The two tensor applications are GEMMs once batched over pairs, and they feed 32x32 maps that
// differ per pair. One CTA is bound to a "role" = (group, side): it keeps the side's view of T_i
// resident in shared memory as the A operand of tcgen05.mma - 8 chunks of 128 rows, row
// r = 32 w + 4 g + t of chunk c holding output channel j = 8 w + g and surviving index
// x = 4 c + t - so that after the UMMA  D[(j,x), pair] = sum_y T[(j,x), y] u[pair, y]
// the thread (w, g, t) of a consumer warp finds in its own TMEM lane exactly the B fragment
// entries of mma.sync.m16n8k8 for output channels 8 w .. 8 w + 7: the per-pair maps never pass
// through shared memory. The Jacobian rows of the tile's 16 pairs arrive by TMA (128-byte
// swizzle, conflict-free fragment loads) in a two-stage ring and leave as 32-byte row segments.
//
// Arithmetic: the tensor applications contract weights with RMS-normalised carriers, both of
// bounded range, on a two-term FP16 split (kind::f16): a T row is [head(32) | tail * 2^11 (32)]
// with T_i scaled by a power of two per group, the carrier tile is [head | head * 2^-11] plus a
// second tile [tail], i.e. head*head + tail*head + head*tail, each product exact to about
// 3 * 2^-22. The per-pair maps act on jets of unbounded range and use the three-term TF32 split.
//
// Warp roles: warps 0-15 consumers (warpgroup = 4 pairs of the tile, warp in group = 8 output
// channels), warp 16 UMMA issuer (and loader of T at a role change), warp 17 TMA producer of the
// Jacobian ring, warp 18 loader of the tile's small vectors. Every mbarrier wait is bounded and
// watches a CTA-wide abort flag; on a timeout the CTA records a code, waits for its copies in
// flight, frees its TMEM columns and returns.
#pragma once
// (included inside namespace hz of hz_walker.cu, which includes <cuda_fp16.h> first)

constexpr int kMcPairs = 16;
constexpr int kMcConsumerWarps = 16;
constexpr int kMcThreads = (kMcConsumerWarps + 3) * 32;
constexpr int kMcJStages = 2;
constexpr int kMcChunkBytes = 128 * 128;                 // 128 rows of [32 heads | 32 tails] halves
constexpr int kMcTBytes = 8 * kMcChunkBytes;             // one role's T: 128 KB
constexpr int kMcJSlotBytes = 16 * 128;                  // 16 Jacobian rows x 32 floats of one pair
constexpr int kMcJStageBytes = kMcPairs * kMcJSlotBytes;
// per-tile operand buffer: two UMMA B tiles [16 pairs x 128 B], two plain vectors, row indices
constexpr int kMcOpsB1 = 0, kMcOpsB2 = 2048, kMcOpsVecA = 4096, kMcOpsVecB = 6144, kMcOpsInfo = 8192;
constexpr int kMcOpsBytes = 9216;
constexpr int kMcOpsBufs = 3;       // the loader runs up to two tiles ahead of the consumers
constexpr size_t kMcSmemBytes = (size_t)kMcTBytes + kMcJStages * kMcJStageBytes + kMcOpsBufs * kMcOpsBytes + 1024;
constexpr uint32_t kMcTmemCols = 256;                    // two tiles x 8 chunks x 16 pairs

#ifdef HZ_MC_PROF
#define MC_T0() long long mc_t0__ = clock64()
#define MC_ACC(slot) do { const long long mc_t1__ = clock64(); if (prof_on) atomicAdd(reinterpret_cast<unsigned long long*>(status) + (slot), (unsigned long long)(mc_t1__ - mc_t0__)); mc_t0__ = mc_t1__; } while (0)
#else
#define MC_T0() do {} while (0)
#define MC_ACC(slot) do {} while (0)
#endif

enum McStatus { kMcTimeoutOps = 11, kMcTimeoutTensor = 12, kMcTimeoutJets = 13, kMcTimeoutT = 14 };

struct MergeTcMaps {
  CUtensorMap t;       // packed T: [2 G x 1024 rows, 32 words], box 128 rows
  CUtensorMap in;      // the level's input rows [Bc x rows_in, d_m], box boxr rows x 32 floats
};

struct MergeTcArgs {
  Level L;
  const float* in;
  float* out;
  float* lap_b;              // [Bc x nodes, d_m]: A_L L_R, added by the cross kernel (nullable)
  const float* t_scale;      // [G] power of two by which T_i was divided
  long long total_pairs;
  int tiles;                 // tiles of 16 pairs
  int boxr, nrb;             // rows per Jacobian box (min(m, 16)) and row blocks per side
  int lg_nodes;              // nodes = 1 << lg_nodes
};

// kind::f16, fp32 accumulate, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld4(float (&v)[4], uint32_t taddr) {
  uint32_t r0, r1, r2, r3;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(taddr)
               : "memory");
  v[0] = __uint_as_float(r0); v[1] = __uint_as_float(r1);
  v[2] = __uint_as_float(r2); v[3] = __uint_as_float(r3);
}

// Packed T of every role, once per call. Role = 2 * group + side; side 0 (A_R) contracts the
// last index of T_i, side 1 (A_L) the middle one. Also the group's scale.
__global__ void __launch_bounds__(256)
merge_t_pack_kernel(const float* __restrict__ T, __half* __restrict__ packed, float* __restrict__ t_scale) {
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
    if (m > 0.f && isfinite(m)) frexpf(m, &e);
    expo_s = e;
    t_scale[grp] = ldexpf(1.f, e);
  }
  __syncthreads();
  const int e = expo_s;
  // one thread per (side, chunk, row): 2 * 8 * 128 = 2048 rows of 32 entries
  for (int rr = tid; rr < 2048; rr += 256) {
    const int side = rr >> 10, c = (rr >> 7) & 7, r = rr & 127;
    const int w = r >> 5, g = (r >> 2) & 7, t = r & 3;
    const int j = 8 * w + g, x = 4 * c + t;
    __half* dst = packed + ((size_t)(2 * grp + side) * 1024 + c * 128 + r) * 64;
    for (int y = 0; y < 32; ++y) {
      const float val = side == 0 ? Tg[(j * 32 + x) * 32 + y] : Tg[(j * 32 + y) * 32 + x];
      const float ts = ldexpf(val, -e);
      const __half hi = __float2half_rn(ts);
      dst[y] = hi;
      dst[32 + y] = __float2half_rn((ts - __half2float(hi)) * 2048.f);
    }
  }
}

__global__ void __launch_bounds__(kMcThreads, 1)
merge_tc_kernel(const __grid_constant__ MergeTcMaps maps, MergeTcArgs a, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* Ts = smem;
  uint8_t* Jr = smem + kMcTBytes;
  uint8_t* Ops = Jr + kMcJStages * kMcJStageBytes;
  __shared__ __align__(8) uint64_t t_full, t_done, j_full[kMcJStages], j_empty[kMcJStages];
  __shared__ __align__(8) uint64_t ops_full[kMcOpsBufs], ops_free[kMcOpsBufs], tm_full[2], tm_free[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const Level& L = a.L;
  const int m = L.m, d = L.d, nodes = L.nodes;
  // work units (role, tile) of this CTA: a contiguous range, so that it changes role at most twice
  const long long W = 2ll * L.G * a.tiles;
  const int w0 = (int)(W * blockIdx.x / gridDim.x), w1 = (int)(W * (blockIdx.x + 1) / gridDim.x);

  if (tid == 0) {
    mbar_init(&t_full, 1);
    mbar_init(&t_done, 1);
    for (int s = 0; s < kMcJStages; ++s) { mbar_init(&j_full[s], 1); mbar_init(&j_empty[s], kMcConsumerWarps); }
    for (int b = 0; b < kMcOpsBufs; ++b) {
      mbar_init(&ops_full[b], 32);
      mbar_init(&ops_free[b], kMcConsumerWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tm_full[b], 1);
      mbar_init(&tm_free[b], kMcConsumerWarps);
    }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kMcTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  auto fail = [&](int code) { atomicCAS(status, 0, code); abort_s = 1; };

  if (warp < kMcConsumerWarps) {
    // ---------------- consumers
    const int wg = warp >> 2, wq = warp & 3, g = lane >> 2, t = lane & 3;
    int it = 0, jc = 0;
    bool alive = true;
    // shared-memory offsets (floats) of this thread's A fragment entries inside a pair's slot:
    // rows g and g + 8 (same swizzle phase), columns 8 ks + t and 8 ks + 4 + t
    const int r0 = g * 32 + t, sw = g & 7;
#ifdef HZ_MC_PROF
    const bool prof_on = (warp == 5 && lane == 0);
#endif
    MC_T0();
    for (int w = w0; w < w1 && alive; ++w, ++it) {
      const int role = w / a.tiles;
      const int side = role & 1, grp = role >> 1, buf = it & 1, ob_i = it % kMcOpsBufs;
      const int col0 = grp * kDr;
      MC_ACC(1);
      if (!__all_sync(0xffffffffu,
                      mbar_wait_abortable(&ops_full[ob_i], (uint32_t)(it / kMcOpsBufs) & 1, &abort_s))) {
        if (lane == 0) fail(kMcTimeoutOps);
        break;
      }
      MC_ACC(2);
      if (!__all_sync(0xffffffffu, mbar_wait_abortable(&tm_full[buf], (uint32_t)(it >> 1) & 1, &abort_s))) {
        if (lane == 0) fail(kMcTimeoutTensor);
        break;
      }
      MC_ACC(3);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint8_t* ob = Ops + ob_i * kMcOpsBytes;
      const float* vecA = reinterpret_cast<const float*>(ob + kMcOpsVecA);
      const float* vecB = reinterpret_cast<const float*>(ob + kMcOpsVecB);
      const int* info = reinterpret_cast<const int*>(ob + kMcOpsInfo);
      // v[c][pp]: the pair's 32x32 map at (j = 8 wq + g, x = 4 c + t), pairs 4 wg + pp
      float v[8][4];
      {
        const uint32_t tbase = tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(buf * 128 + wg * 4);
#pragma unroll
        for (int c = 0; c < 8; ++c) tmem_ld4(v[c], tbase + c * 16);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const float sc = a.t_scale[grp];
#pragma unroll
        for (int c = 0; c < 8; ++c)
#pragma unroll
          for (int pp = 0; pp < 4; ++pp) v[c][pp] *= sc;
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&tm_free[buf]);
      MC_ACC(4);
      // value and Laplacian terms: contractions of the map with the pair's small vectors
#pragma unroll
      for (int pp = 0; pp < 4; ++pp) {
        const int p = wg * 4 + pp;
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          s1 = fmaf(v[c][pp], vecA[p * 32 + 4 * c + t], s1);
          s2 = fmaf(v[c][pp], vecB[p * 32 + 4 * c + t], s2);
        }
        s1 = quad_sum(s1);
        s2 = quad_sum(s2);
        if (t == 0 && info[p] >= 0) {
          const int j = 8 * wq + g;
          if (side == 0) {
            a.out[(size_t)info[32 + p] * d + col0 + j] = s1;          // raw = A_R u_L
            a.out[(size_t)info[48 + p] * d + col0 + j] = s2;          // A_R L_L
          } else if (a.lap_b != nullptr) {
            a.lap_b[(size_t)info[64 + p] * d + col0 + j] = s1;        // A_L L_R
          }
        }
      }
      MC_ACC(5);
      // Jacobian rows of this side through the maps
#pragma unroll 1
      for (int rb = 0; rb < a.nrb; ++rb, ++jc) {
        const int s = jc % kMcJStages;
        if (!__all_sync(0xffffffffu,
                        mbar_wait_abortable(&j_full[s], (uint32_t)(jc / kMcJStages) & 1, &abort_s))) {
          if (lane == 0) fail(kMcTimeoutJets);
          alive = false;
          break;
        }
        MC_ACC(6);
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
          const int p = wg * 4 + pp;
          if (info[p] < 0) continue;
          const float* Js = reinterpret_cast<const float*>(Jr + s * kMcJStageBytes + p * kMcJSlotBytes);
          float am[4] = {0.f, 0.f, 0.f, 0.f}, as[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const int c0 = r0 + (((2 * ks) ^ sw) << 2), c1 = r0 + (((2 * ks + 1) ^ sw) << 2);
            FA2 fa;
            fa.set(Js[c0], Js[c0 + 256], Js[c1], Js[c1 + 256]);
            FB2 fb;
            fb.set(v[2 * ks][pp], v[2 * ks + 1][pp]);
            mma3x(am, as, fa, fb);
          }
          const int A0 = rb * 16 + g;
          float* orow = a.out + (size_t)(info[16 + p] + side * m + A0) * d + col0 + 8 * wq + 2 * t;
          if (A0 < m) *reinterpret_cast<float2*>(orow) = make_float2(am[0] + as[0], am[1] + as[1]);
          if (A0 + 8 < m) *reinterpret_cast<float2*>(orow + 8 * d) = make_float2(am[2] + as[2], am[3] + as[3]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&j_empty[s]);
        MC_ACC(7);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ops_free[ob_i]);
    }
  } else if (warp == kMcConsumerWarps) {
    // ---------------- UMMA issuer; loads the role's T when the role changes
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(kMcPairs);
      int cur_role = -1;
      uint32_t tl_phase = 0, td_phase = 0;
      int it = 0;
#ifdef HZ_MC_PROF
      const bool prof_on = true;
#endif
      MC_T0();
      for (int w = w0; w < w1; ++w, ++it) {
        const int role = w / a.tiles, buf = it & 1;
        MC_ACC(8);
        if (role != cur_role) {
          if (cur_role >= 0) {       // every UMMA that reads the old T must have completed
            umma_commit(&t_done);
            if (!mbar_wait_abortable(&t_done, td_phase, &abort_s)) { fail(kMcTimeoutTensor); break; }
            td_phase ^= 1;
          }
          mbar_expect_tx(&t_full, kMcTBytes);
          for (int c = 0; c < 8; ++c)
            tma_load_2d(Ts + c * kMcChunkBytes, &maps.t, 0, role * 1024 + c * 128, &t_full);
          if (!mbar_wait_abortable(&t_full, tl_phase, &abort_s)) {
            fail(kMcTimeoutT);
            mbar_wait(&t_full, tl_phase);      // let the copies land before the CTA exits
            break;
          }
          tl_phase ^= 1;
          cur_role = role;
        }
        MC_ACC(9);
        const int ob_i = it % kMcOpsBufs;
        if (!mbar_wait_abortable(&ops_full[ob_i], (uint32_t)(it / kMcOpsBufs) & 1, &abort_s) ||
            (it >= 2 && !mbar_wait_abortable(&tm_free[buf], (uint32_t)((it >> 1) - 1) & 1, &abort_s))) {
          fail(kMcTimeoutOps);
          break;
        }
        MC_ACC(10);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t b1 = smem_u32(Ops + ob_i * kMcOpsBytes + kMcOpsB1);
        const uint32_t b2 = smem_u32(Ops + ob_i * kMcOpsBytes + kMcOpsB2);
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          const uint32_t at = smem_u32(Ts + c * kMcChunkBytes);
          const uint32_t tacc = tmem_base + (uint32_t)(buf * 128 + c * 16);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)      // [head | tail] x [head | head 2^-11]
            umma_f16(tacc, umma_desc_sw128(at + ks * 32), umma_desc_sw128(b1 + ks * 32), idesc, ks > 0 ? 1u : 0u);
#pragma unroll
          for (int ks = 0; ks < 2; ++ks)      // head x tail
            umma_f16(tacc, umma_desc_sw128(at + ks * 32), umma_desc_sw128(b2 + ks * 32), idesc, 1u);
        }
        umma_commit(&tm_full[buf]);
        MC_ACC(11);
      }
    }
  } else if (warp == kMcConsumerWarps + 1) {
    // ---------------- TMA producer of the Jacobian ring
    if (lane == 0) {
      int it = 0, jc = 0;
      bool alive = true;
      for (int w = w0; w < w1 && alive; ++w, ++it) {
        const int role = w / a.tiles, tile = w % a.tiles;
        const int side = role & 1, grp = role >> 1;
        const long long left = a.total_pairs - (long long)tile * kMcPairs;
        const int nvalid = left < kMcPairs ? (int)left : kMcPairs;
        for (int rb = 0; rb < a.nrb; ++rb, ++jc) {
          const int s = jc % kMcJStages;
          if (jc >= kMcJStages &&
              !mbar_wait_abortable(&j_empty[s], (uint32_t)((jc / kMcJStages) - 1) & 1, &abort_s)) {
            fail(kMcTimeoutJets);
            alive = false;
            break;
          }
          mbar_expect_tx(&j_full[s], (uint32_t)(nvalid * a.boxr * 128));
          for (int p = 0; p < nvalid; ++p) {
            const int pair = tile * kMcPairs + p;
            const int b = pair >> a.lg_nodes, n = pair & (nodes - 1);
            tma_load_2d(Jr + s * kMcJStageBytes + p * kMcJSlotBytes, &maps.in, grp * kDr,
                        b * L.rows_in + n * 2 * m + side * m + rb * 16, &j_full[s]);
          }
        }
      }
      if (abort_s != 0)      // let the copies still in flight land before the CTA exits
        for (int j = (jc > kMcJStages ? jc - kMcJStages : 0); j < jc; ++j)
          mbar_wait(&j_full[j % kMcJStages], (uint32_t)(j / kMcJStages) & 1);
    }
  } else if (warp == kMcConsumerWarps + 2) {
    // ---------------- loader of the tile's small vectors and row indices. The global loads of
    // tile it + 1 are in flight (in registers) while the loader waits for a free buffer.
    const int nodes_in = 2 * nodes;
    // vec 0: the carrier that the tensor application contracts (the other child's value);
    // vec 1, 2: plain vectors for the value and Laplacian terms
    auto fetch = [&](int w, float4 (&x)[12]) {
      const int role = w / a.tiles, tile = w % a.tiles;
      const int side = role & 1, grp = role >> 1;
#pragma unroll
      for (int q = 0; q < 12; ++q) {
        const int idx = q * 32 + lane;
        const int vec = idx >> 7, p = (idx >> 3) & 15, c4 = idx & 7;
        const long long pair = (long long)tile * kMcPairs + p;
        x[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (pair < a.total_pairs && !(side == 1 && vec == 2)) {
          const int b = (int)(pair >> a.lg_nodes), n = (int)(pair & (nodes - 1));
          size_t row;
          if (vec == 0) row = row_u(L, L.rows_in, nodes_in, b, 2 * n + (side == 0 ? 1 : 0));
          else if (side == 0) row = vec == 1 ? row_u(L, L.rows_in, nodes_in, b, 2 * n) : row_l(L, L.rows_in, nodes_in, b, 2 * n);
          else row = row_l(L, L.rows_in, nodes_in, b, 2 * n + 1);
          x[q] = __ldg(reinterpret_cast<const float4*>(a.in + row * d + grp * kDr + 4 * c4));
        }
      }
    };
    float4 x[12];
    if (w0 < w1) fetch(w0, x);
    int it = 0;
    for (int w = w0; w < w1; ++w, ++it) {
      const int tile = w % a.tiles;
      const int ob_i = it % kMcOpsBufs;
      if (it >= kMcOpsBufs &&
          !__all_sync(0xffffffffu, mbar_wait_abortable(&ops_free[ob_i], (uint32_t)((it / kMcOpsBufs) - 1) & 1,
                                                       &abort_s))) {
        if (lane == 0) fail(kMcTimeoutOps);
        break;
      }
      uint8_t* ob = Ops + ob_i * kMcOpsBytes;
#pragma unroll
      for (int q = 0; q < 12; ++q) {
        const int idx = q * 32 + lane;
        const int vec = idx >> 7, p = (idx >> 3) & 15, c4 = idx & 7;
        if (vec == 0) {
          // head, head * 2^-11 and tail of two values as packed halves (first value in the low half)
          auto pack3 = [](float x0, float x1, uint32_t& hi, uint32_t& h2, uint32_t& lo) {
            const __half2 h = __floats2half2_rn(x0, x1);
            const float2 hf = __half22float2(h);
            const __half2 sc = __floats2half2_rn(hf.x * (1.f / 2048.f), hf.y * (1.f / 2048.f));
            const __half2 l = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
            hi = *reinterpret_cast<const uint32_t*>(&h);
            h2 = *reinterpret_cast<const uint32_t*>(&sc);
            lo = *reinterpret_cast<const uint32_t*>(&l);
          };
          uint2 hi, h2, lo;
          pack3(x[q].x, x[q].y, hi.x, h2.x, lo.x);
          pack3(x[q].z, x[q].w, hi.y, h2.y, lo.y);
          // row p of a 128-byte-swizzled tile: 16-byte chunk cc sits at position cc ^ (p & 7)
          const int sub = (c4 & 1) * 8, cc = c4 >> 1;
          uint8_t* r1 = ob + kMcOpsB1 + p * 128;
          uint8_t* r2 = ob + kMcOpsB2 + p * 128;
          *reinterpret_cast<uint2*>(r1 + ((cc ^ (p & 7)) << 4) + sub) = hi;
          *reinterpret_cast<uint2*>(r1 + (((4 + cc) ^ (p & 7)) << 4) + sub) = h2;
          *reinterpret_cast<uint2*>(r2 + ((cc ^ (p & 7)) << 4) + sub) = lo;
        } else {
          float* dst = reinterpret_cast<float*>(ob + (vec == 1 ? kMcOpsVecA : kMcOpsVecB));
          *reinterpret_cast<float4*>(dst + p * 32 + 4 * c4) = x[q];
        }
      }
      if (lane < kMcPairs) {
        int* info = reinterpret_cast<int*>(ob + kMcOpsInfo);
        const long long pair = (long long)tile * kMcPairs + lane;
        const bool ok = pair < a.total_pairs;
        const int b = ok ? (int)(pair >> a.lg_nodes) : 0, n = ok ? (int)(pair & (nodes - 1)) : 0;
        info[lane] = ok ? (int)row_j(L.rows_in, b, n * 2 * m) : -1;
        info[16 + lane] = (int)row_j(L.rows_out, b, n * 2 * m);
        info[32 + lane] = (int)row_u(L, L.rows_out, nodes, b, n);
        info[48 + lane] = (int)row_l(L, L.rows_out, nodes, b, n);
        info[64 + lane] = ok ? (int)pair : 0;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(&ops_full[ob_i]);
      if (w + 1 < w1) fetch(w + 1, x);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kMcTmemCols)
                 : "memory");
  }
}
