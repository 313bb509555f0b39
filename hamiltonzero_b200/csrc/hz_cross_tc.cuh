// Cross term of the Laplacian row of a merge, 2 T_i : (J_L^T W_off J_R), on tcgen05.
// Reference math: energy/custom_lap.py:1318-1389 (the mixed second-order term of the bilinear
// merge under the frame metric W).
//
// Per (walker, node) pair and channel group i (32 channels):
//   Y[A][l]  = sum_B W_off[A][B] J_R[B][l]        A, B < m   (W_off: the node's off-diagonal block
//                                                             of the frame metric, walker independent)
//   C[k][l]  = sum_A J_L[A][k] Y[A][l]
//   cross[j] = sum_(k,l) T_i[j][k][l] C[k][l]
// Y is the tensor-core part: one UMMA group per four walkers of a node with the channels as M,
//   D[(walker q, channel l)][A] = sum_B J_R^T[(q, l)][B] W_off[A][B]      (M = 128, N = m, K = m)
// J_R^T is the TMEM operand: rewriter thread (q, l) reads its column of the walker's Jacobian
// tile (coalesced over l), scales it by one power of two and stores the FP16 head and tail into
// its TMEM lane; W_off (head/tail, scaled per node, 128-byte-swizzle image written once per launch
// by cross_pack_kernel) is the shared-memory operand for all nodes of the level. The consumer
// thread (q, l) then owns column l of Y in its TMEM lane: C[.][l] accumulates in 32 registers
// from broadcast reads of J_L (16-row boxes brought by TMA into a ring, two stages per consumer
// group), and
// T_i : C runs in fp32 from shared memory (T_i plain, [j][k][l], lane = l: conflict free) for two
// walkers at a time so that every word of T_i read feeds two FMAs; the sum over l is a
// reduce-scatter over the warp. Two consumer groups alternate over pairs of units, so that one
// group's T_i : C overlaps the other's C.
// Arithmetic: three FP16 products (tail x head, head x tail, head x head) accumulated in fp32;
// operands scaled into [2^14, 2^15) by exact powers of two, so any magnitude of the Jacobian rows
// or of the frame goes through; C and the T_i contraction are fp32.
#pragma once
// Included inside the walker translation unit's namespace, after Level and the row helpers.

struct CrossTcArgs {
  Level L;
  const float* T;          // merge_T [G][32][32][32]
  const float* in;
  float* out;
  const float* lap_b;      // A_L L_R of merge_tc_kernel, [pairs][d]
  const uint4* w_image;    // cross_pack_kernel's image, w_rows rows of 128 bytes
  const float* w_scale;    // [nodes] power of two by which the node's block was divided
  int w_rows;
  int sets;                // ceil(Bc / 4): groups of four walkers
  long long units;         // nodes * sets
};

// 4 service + 4 rewriter + 2 x 4 consumer warps. Registers: the CTA starts with 512 x 128;
// 128 x 40 + 128 x 152 + 256 x 160 = 512 x 128.
constexpr int kCxThreads = 512;
constexpr int kCxStageBytes = 4 * 16 * 128;      // J_L: four walkers x 16 rows x 32 floats
// stages of the J_L ring per consumer group. Two fit beside T_i (128 KB) and the W images (48 KB)
// at 96 rows; three and four per group at the lower heights were measured and gained nothing.
__host__ __device__ constexpr int cross_ring_per_group(int /*mp*/) { return 2; }
static_assert(128 * 40 + 128 * 152 + 256 * 160 <= 512 * 128, "register budget of the cross-term roles");
constexpr int kCxMaxRing = 8;
constexpr int kCxMaxWRows = 384;        // 48 KB of W images
constexpr int kCxScaleRing = 4;

__device__ __forceinline__ void tmem_ld16(uint32_t (&v)[16], uint32_t taddr) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
        "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
        "r"(v[7])
      : "memory");
}

// image rows of 64 halves; block (node, atom, part) holds rows A = 0..MP-1 of the K-atom
// (B = 64 atom .. 64 atom + 63), part 0 = head, 1 = tail, with the 16-byte chunks of a row
// permuted as the 128-byte swizzle of the UMMA descriptor expects (chunk c of row A at c ^ (A & 7)).
static __global__ void __launch_bounds__(256)
cross_pack_kernel(const float* __restrict__ J_eff, int threeN, int m, int MP, __half* __restrict__ image,
                  float* __restrict__ w_scale) {
  __shared__ float red[8];
  __shared__ int expo_s;
  const int node = blockIdx.x, tid = threadIdx.x;
  const float* W = J_eff + (size_t)(node * 2 * m) * threeN + node * 2 * m + m;
  float mx = 0.f;
  for (int i = tid; i < m * m; i += 256) mx = fmaxf(mx, fabsf(W[(size_t)(i / m) * threeN + (i % m)]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  if (tid == 0) {
    float v = 0.f;
    for (int i = 0; i < 8; ++i) v = fmaxf(v, red[i]);
    int e = 0;
    if (v > 0.f && isfinite(v)) { frexpf(v, &e); e -= 15; }
    expo_s = e;
    w_scale[node] = ldexpf(1.f, e);
  }
  __syncthreads();
  const int e = expo_s;
  const int natoms = (MP + 63) / 64;
  for (int idx = tid; idx < natoms * MP * 64; idx += 256) {
    const int k = idx & 63, A = (idx >> 6) % MP, atom = (idx >> 6) / MP;
    const int B = atom * 64 + k;
    const float val = (A < m && B < m) ? ldexpf(W[(size_t)A * threeN + B], -e) : 0.f;
    const __half hi = __float2half_rn(val);
    const __half lo = __float2half_rn(val - __half2float(hi));
    const int pos = (((k >> 3) ^ (A & 7)) << 3) + (k & 7);
    const size_t block = (size_t)(node * natoms + atom) * 2;
    image[((block + 0) * MP + A) * 64 + pos] = hi;
    image[((block + 1) * MP + A) * 64 + pos] = lo;
  }
}

// sum over the warp of v[jj] for eight values per lane; every lane returns the total of
// jj = lane >> 2
__device__ __forceinline__ float cross_reduce8(float (&v)[8], int lane) {
#pragma unroll
  for (int off = 16, n = 8; n > 1; off >>= 1, n >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float send = upper ? v[i] : v[i + n / 2];
      const float keep = upper ? v[i + n / 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  float r = v[0];
  r += __shfl_xor_sync(0xffffffffu, r, 2);
  r += __shfl_xor_sync(0xffffffffu, r, 1);
  return r;
}

template <int MP>
__global__ void __launch_bounds__(kCxThreads, 1)
cross_tc_kernel(const __grid_constant__ CUtensorMap jmap, CrossTcArgs a, int* __restrict__ status) {
  constexpr int S = (MP + 31) & ~31;                     // TMEM columns per buffer
  constexpr uint32_t kCols = 4 * S <= 128 ? 128u : (4 * S <= 256 ? 256u : 512u);
  constexpr int KS = MP / 16, NATOMS = (MP + 63) / 64, NCH = MP / 16, RG = cross_ring_per_group(MP);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  float* Ts = reinterpret_cast<float*>(smem);                                   // [j][k][l]
  uint8_t* Ws = smem + 131072;                                                  // W images
  uint8_t* Js = Ws + (size_t)a.w_rows * 128;                                    // J_L ring
  float* sc = reinterpret_cast<float*>(Js + 2 * RG * kCxStageBytes);            // [ring][128]
  float* wsc = sc + kCxScaleRing * 128;                                         // [nodes]
  // Every barrier has one waiter that sees each of its phases in turn (a parity wait cannot tell
  // phases two apart): tfull/tfree are per (consumer group, unit of the pair) although the two
  // groups share the two accumulators, and each group owns RG stages of the J_L ring.
  __shared__ __align__(8) uint64_t conv_bar[2], afree_bar[2], tfull_bar[4], tfree_bar[4];
  __shared__ __align__(8) uint64_t jfull_bar[kCxMaxRing], jfree_bar[kCxMaxRing];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = blockIdx.x;
  const Level& L = a.L;
  const int d = L.d, m = L.m, nodes = L.nodes, col0 = grp * 32;
  const long long gy = gridDim.y, y0 = blockIdx.y;
  const long long n_i = y0 < a.units ? (a.units - y0 + gy - 1) / gy : 0;

  {
    const uint4* Tg = reinterpret_cast<const uint4*>(a.T + (size_t)grp * 32768);
    uint4* Td = reinterpret_cast<uint4*>(Ts);
    for (int i = tid; i < 8192; i += kCxThreads) Td[i] = __ldg(Tg + i);
    uint4* Wd = reinterpret_cast<uint4*>(Ws);
    for (int i = tid; i < a.w_rows * 8; i += kCxThreads) Wd[i] = __ldg(a.w_image + i);
    if (tid < nodes) wsc[tid] = a.w_scale[tid];
  }
  if (tid == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(&conv_bar[s], 128); mbar_init(&afree_bar[s], 1); }
    for (int s = 0; s < 4; ++s) { mbar_init(&tfull_bar[s], 1); mbar_init(&tfree_bar[s], 128); }
    for (int s = 0; s < 2 * RG; ++s) { mbar_init(&jfull_bar[s], 1); mbar_init(&jfree_bar[s], 128); }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // the W images are read by the tensor core through the async proxy
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  auto fail = [&](int code) { atomicExch(status, code); abort_s = 1; };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0 && lane == 0) {
      // ---------------- producer: J_L of a unit in boxes of 16 rows x 32 channels per walker
      bool alive = true;
      long long last_use[kCxMaxRing];
      for (int w = 0; w < kCxMaxRing; ++w) last_use[w] = -1;
      for (long long i = 0; i < n_i && alive; ++i) {
        const long long u = y0 + i * gy;
        const int node = (int)(u / a.sets), b0 = (int)(u % a.sets) * 4;
        const int g = (int)((i >> 1) & 1);
        const long long lu = (i >> 2) * 2 + (i & 1);          // the group's own count of units
        for (int ch = 0; ch < NCH; ++ch) {
          const long long lidx = lu * NCH + ch;
          const int slot = g * RG + (int)(lidx % RG);
          if (lidx >= RG && !mbar_wait_abortable(&jfree_bar[slot], (uint32_t)((lidx / RG) - 1) & 1, &abort_s)) {
            fail(kTcTimeoutLoad);
            alive = false;
            break;
          }
          mbar_expect_tx(&jfull_bar[slot], kCxStageBytes);
          for (int q = 0; q < 4; ++q)
            tma_load_2d(Js + (size_t)slot * kCxStageBytes + q * 2048, &jmap, col0,
                        (b0 + q) * L.rows_in + node * 2 * m + ch * 16, &jfull_bar[slot]);
          last_use[slot] = lidx / RG;
        }
      }
      // own copies landed before the CTA may exit
      for (int w = 0; w < 2 * RG; ++w)
        if (last_use[w] >= 0 && !mbar_wait(&jfull_bar[w], (uint32_t)last_use[w] & 1)) fail(kTcTimeoutLoad);
    } else if (warp == 1 && lane == 0) {
      // ---------------- issuer: 3 KS UMMAs of N = MP per unit
      constexpr uint32_t idesc = umma_idesc_f16_n(MP);
      for (long long i = 0; i < n_i; ++i) {
        const int buf = (int)(i & 1);
        if (!mbar_wait_abortable(&conv_bar[buf], (uint32_t)(i >> 1) & 1, &abort_s)) {
          fail(kTcTimeoutMma);
          break;
        }
        // the accumulator was last read for unit i - 2, by the other consumer group
        const int g = (int)((i >> 1) & 1);
        if (i >= 2 &&
            !mbar_wait_abortable(&tfree_bar[(g ^ 1) * 2 + buf], (uint32_t)((i - 2) >> 2) & 1, &abort_s)) {
          fail(kTcTimeoutMma);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int node = (int)((y0 + i * gy) / a.sets);
        const uint32_t ta = tmem_base + (uint32_t)(buf * S);
        const uint32_t tacc = tmem_base + (uint32_t)(2 * S + buf * S);
        const uint32_t wnode = smem_u32(Ws) + (uint32_t)(node * NATOMS * 2 * MP * 128);
        // small terms first: tail x head, head x tail, then head x head
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
          umma_f16_ts(tacc, ta + MP / 2 + ks * 8,
                      umma_desc_sw128(wnode + (uint32_t)(((ks >> 2) * 2 + 0) * MP * 128 + (ks & 3) * 32)), idesc,
                      ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
          umma_f16_ts(tacc, ta + ks * 8,
                      umma_desc_sw128(wnode + (uint32_t)(((ks >> 2) * 2 + 1) * MP * 128 + (ks & 3) * 32)), idesc, 1u);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
          umma_f16_ts(tacc, ta + ks * 8,
                      umma_desc_sw128(wnode + (uint32_t)(((ks >> 2) * 2 + 0) * MP * 128 + (ks & 3) * 32)), idesc, 1u);
        umma_commit(&tfull_bar[g * 2 + buf]);
        umma_commit(&afree_bar[buf]);
      }
    }
  } else if (warp < 8) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
    // ---------------- J_R column of (walker q, channel l) -> FP16 head/tail in TMEM lane (q, l)
    const int q = warp & 3, row = q * 32 + lane;
    auto load_unit = [&](long long i, float (&x)[MP]) {
      const long long u = y0 + i * gy;
      const int node = (int)(u / a.sets), b = (int)(u % a.sets) * 4 + q;
      if (i < n_i && b < L.Bc) {
        const float* p = a.in + (row_j(L.rows_in, b, node * 2 * m) + m) * d + col0 + lane;
#pragma unroll
        for (int B = 0; B < MP; ++B) x[B] = B < m ? __ldg(p + (size_t)B * d) : 0.f;
      } else {
#pragma unroll
        for (int B = 0; B < MP; ++B) x[B] = 0.f;
      }
    };
    // scale, split and store one unit's column; false after a wait that ran out
    auto convert_store = [&](long long i, const float (&x)[MP]) -> bool {
      const int buf = (int)(i & 1);
      float mx = 0.f;
#pragma unroll
      for (int B = 0; B < MP; ++B) mx = fmaxf(mx, fabsf(x[B]));
      int e = 0;
      if (mx > 0.f && isfinite(mx)) e = max((int)((__float_as_uint(mx) >> 23) & 0xff) - 141, -126);
      const float down = __uint_as_float((uint32_t)(127 - e) << 23);
      if (i >= 2 &&
          !__all_sync(0xffffffffu, mbar_wait_abortable(&afree_bar[buf], (uint32_t)((i >> 1) - 1) & 1, &abort_s))) {
        if (lane == 0) fail(kTcTimeoutMma);
        return false;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      sc[(int)(i & (kCxScaleRing - 1)) * 128 + row] = __uint_as_float((uint32_t)(127 + e) << 23);
      const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * S);
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t hv[8], lv[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float v0 = x[16 * ks + 2 * c] * down, v1 = x[16 * ks + 2 * c + 1] * down;
          const __half2 hi = __floats2half2_rn(v0, v1);
          const float2 hf = __half22float2(hi);
          const __half2 lo = __floats2half2_rn(v0 - hf.x, v1 - hf.y);
          hv[c] = *reinterpret_cast<const uint32_t*>(&hi);
          lv[c] = *reinterpret_cast<const uint32_t*>(&lo);
        }
        tmem_st8(ta + ks * 8, hv);
        tmem_st8(ta + MP / 2 + ks * 8, lv);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&conv_bar[buf]);
      return true;
    };
    // A unit's column is short at the lower levels and the load latency is not: the loads of the
    // next D units are in flight (about 96 per thread at every height) while one is converted.
    constexpr int D = MP == 16 ? 6 : (MP == 32 ? 3 : (MP == 48 ? 1 : 0));
    if constexpr (D == 0) {
      for (long long i = 0; i < n_i; ++i) {
        float x[MP];
        load_unit(i, x);
        if (!convert_store(i, x)) break;
      }
    } else {
      float xr[D][MP];
#pragma unroll
      for (int t = 0; t < D; ++t) load_unit(t, xr[t]);
      bool alive = true;
      for (long long i0 = 0; i0 < n_i && alive; i0 += D) {
#pragma unroll
        for (int t = 0; t < D; ++t) {
          const long long i = i0 + t;
          if (!alive || i >= n_i) continue;
          float x[MP];
#pragma unroll
          for (int B = 0; B < MP; ++B) x[B] = xr[t][B];
          load_unit(i + D, xr[t]);
          alive = convert_store(i, x);
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 160;");
    // ---------------- consumers: thread = (walker q, channel l); two units per pass over T_i,
    // the two groups take the pairs of units in turn
    const int q = warp & 3, row = q * 32 + lane, group = (warp - 8) >> 2;
    const uint32_t tlane = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint8_t* Jq = Js + q * 2048;
    bool ok = true;
    for (long long i = 2 * group; i < n_i && ok; i += 4) {
      float c[2][32];
      int wb[2], wn[2];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
#pragma unroll
        for (int k = 0; k < 32; ++k) c[s][k] = 0.f;
        wb[s] = -1; wn[s] = 0;
        const long long ii = i + s;
        if (!ok || ii >= n_i) continue;
        const long long u = y0 + ii * gy;
        const int node = (int)(u / a.sets), b = (int)(u % a.sets) * 4 + q;
        const int buf = (int)(ii & 1);
        if (!mbar_wait_abortable(&tfull_bar[group * 2 + buf], (uint32_t)(ii >> 2) & 1, &abort_s)) {
          if (lane == 0) fail(kTcTimeoutMma);
          ok = false;
          continue;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float scale = sc[(int)(ii & (kCxScaleRing - 1)) * 128 + row] * wsc[node];
        const bool valid = b < L.Bc;
#pragma unroll 1
        for (int ch = 0; ch < NCH; ++ch) {
          const long long lidx = ((ii >> 2) * 2 + s) * NCH + ch;
          const int slot = group * RG + (int)(lidx % RG);
          uint32_t yv[16];
          tmem_ld16(yv, tlane + (uint32_t)(2 * S + buf * S + ch * 16));
          const bool landed = mbar_wait_abortable(&jfull_bar[slot], (uint32_t)(lidx / RG) & 1, &abort_s);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (!landed) {
            if (lane == 0) fail(kTcTimeoutLoad);
            ok = false;
            break;
          }
          if (ch == NCH - 1) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&tfree_bar[group * 2 + buf]);
          }
          if (valid) {
            const uint8_t* Jc = Jq + (size_t)slot * kCxStageBytes;
#pragma unroll
            // rows A >= m of the last box are the first rows of the same pair's J_R and meet
            // Y columns that are exactly zero (zero rows of the W image): no guard
            for (int aa = 0; aa < 16; ++aa) {
              const float yy = __uint_as_float(yv[aa]);
#pragma unroll
              for (int kk = 0; kk < 8; ++kk) {
                const float4 j4 = *reinterpret_cast<const float4*>(Jc + aa * 128 + ((kk ^ (aa & 7)) << 4));
                c[s][4 * kk] = fmaf(yy, j4.x, c[s][4 * kk]);
                c[s][4 * kk + 1] = fmaf(yy, j4.y, c[s][4 * kk + 1]);
                c[s][4 * kk + 2] = fmaf(yy, j4.z, c[s][4 * kk + 2]);
                c[s][4 * kk + 3] = fmaf(yy, j4.w, c[s][4 * kk + 3]);
              }
            }
          }
          mbar_arrive(&jfree_bar[slot]);
        }
        if (!ok) continue;
#pragma unroll
        for (int k = 0; k < 32; ++k) c[s][k] *= scale;
        if (valid) { wb[s] = b; wn[s] = node; }
      }
      if (!ok) break;
      // the row to update is fetched while T_i : C runs
      const int j = (lane & 3) * 8 + (lane >> 2);
      float* dstp[2] = {nullptr, nullptr};
      float prev[2] = {0.f, 0.f};
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (wb[s] < 0) continue;
        const long long pair = (long long)wb[s] * nodes + wn[s];
        dstp[s] = a.out + row_l(L, L.rows_out, nodes, wb[s], wn[s]) * d + col0 + j;
        prev[s] = *dstp[s] + a.lap_b[(size_t)pair * d + col0 + j];
      }
      // cross[j] = sum_l sum_k T[j][k][l] C[k][l]
      float res0 = 0.f, res1 = 0.f;
#pragma unroll 1
      for (int jb = 0; jb < 4; ++jb) {
        const float* Tj = Ts + jb * 8192 + lane;
        float r0[8], r1[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          float a0 = 0.f, a1 = 0.f;
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const float tv = Tj[(jj * 32 + k) * 32];
            a0 = fmaf(tv, c[0][k], a0);
            a1 = fmaf(tv, c[1][k], a1);
          }
          r0[jj] = a0;
          r1[jj] = a1;
        }
        const float t0 = cross_reduce8(r0, lane), t1 = cross_reduce8(r1, lane);
        if ((lane & 3) == jb) { res0 = t0; res1 = t1; }
      }
      if (dstp[0] != nullptr) *dstp[0] = prev[0] + 2.f * res0;
      if (dstp[1] != nullptr) *dstp[1] = prev[1] + 2.f * res1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kCols)
                 : "memory");
  }
}

inline int cross_tc_pad(int m) { return (m + 15) & ~15; }
// dynamic shared memory: alignment slack, T_i, W images, J_L ring, row scales, node scales
inline size_t cross_tc_smem(int mp, int w_rows) {
  return 1024 + 131072 + (size_t)w_rows * 128 + 2 * cross_ring_per_group(mp) * kCxStageBytes +
         kCxScaleRing * 128 * sizeof(float) + 64;
}

// m padded to 16, 32, 48 or 96 rows and every node's W images together within 48 KB
inline bool cross_tc_supported(const Level& L) {
  const int mp = cross_tc_pad(L.m);
  if (mp != 16 && mp != 32 && mp != 48 && mp != 96) return false;
  const int natoms = (mp + 63) / 64;
  const int w_rows = L.nodes * natoms * 2 * mp;
  return w_rows <= kCxMaxWRows && cross_tc_smem(mp, w_rows) <= 227 * 1024 - 1024 && L.nodes <= 8 && L.jets == 1;
}

template <int MP>
int launch_cross_tc_mp(const CUtensorMap& jmap, const CrossTcArgs& a, dim3 grid, size_t smem, int* status,
                       cudaStream_t stream) {
  const int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(cross_tc_kernel<MP>), (int)smem);
  if (rc != HZ_OK) return rc;
  cross_tc_kernel<MP><<<grid, kCxThreads, smem, stream>>>(jmap, a, status);
  return HZ_OK;
}

// w_image: kCxMaxWRows * 128 bytes, w_scale: 8 floats (workspace)
inline int launch_cross_tc(const Level& L, const float* T, const float* J_eff, const float* in, float* out,
                           const float* lap_b, float* w_image, float* w_scale, int* status,
                           cudaStream_t stream) {
  const int mp = cross_tc_pad(L.m), natoms = (mp + 63) / 64;
  cross_pack_kernel<<<L.nodes, 256, 0, stream>>>(J_eff, 3 * L.N, L.m, mp, reinterpret_cast<__half*>(w_image),
                                                 w_scale);
  HZ_CUDA_TRY(cudaGetLastError());
  CrossTcArgs a{};
  a.L = L; a.T = T; a.in = in; a.out = out; a.lap_b = lap_b;
  a.w_image = reinterpret_cast<const uint4*>(w_image);
  a.w_scale = w_scale;
  a.w_rows = L.nodes * natoms * 2 * mp;
  a.sets = (L.Bc + 3) / 4;
  a.units = (long long)L.nodes * a.sets;
  long long gy = tc_sm_count() / L.G;
  if (gy > (a.units + 1) / 2) gy = (a.units + 1) / 2;
  if (gy < 1) gy = 1;
  const dim3 grid(L.G, (unsigned)gy);
  CUtensorMap jmap;
  if (!make_map(&jmap, in, (long long)L.Bc * L.rows_in, L.d, L.d, 16)) return HZ_ERR_CUDA;
  const size_t smem = cross_tc_smem(mp, a.w_rows);
  int rc = HZ_OK;
  switch (mp) {
    case 16: rc = launch_cross_tc_mp<16>(jmap, a, grid, smem, status, stream); break;
    case 32: rc = launch_cross_tc_mp<32>(jmap, a, grid, smem, status, stream); break;
    case 48: rc = launch_cross_tc_mp<48>(jmap, a, grid, smem, status, stream); break;
    default: rc = launch_cross_tc_mp<96>(jmap, a, grid, smem, status, stream); break;
  }
  if (rc != HZ_OK) return rc;
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// HZ_CROSS=legacy keeps the mma.sync kernel (merge_tstage_kernel<true>).
inline bool use_cross_tc() {
  static const bool on = !env_equals("HZ_CROSS", "legacy");
  return on;
}
// HZ_CROSS_MP: bit mask of the padded child heights (16: 1, 32: 2, 48: 4, 96: 8) that take this
// kernel. Default 8: measured per level at 64 sites, 2048 walkers per pass, it is faster than the
// mma.sync kernel only at 96 rows per child (the step 381.8 -> 370.5 ms), equal at 48 and slower
// at 24 and 12, where a unit is short and the fixed work per unit (T_i : C, the barrier round
// trips) dominates.
inline bool cross_tc_level_enabled(int m) {
  static const int mask = [] {
    const char* e = std::getenv("HZ_CROSS_MP");
    return e ? std::atoi(e) : 8;
  }();
  const int mp = cross_tc_pad(m);
  const int bit = mp == 16 ? 1 : mp == 32 ? 2 : mp == 48 ? 4 : 8;
  return (mask & bit) != 0;
}

