// Fast path of the attention kernels for the shape the reference's level-edge heads and the
// benchmark use: N = 64 tokens, D = 32, square-mask convention. The whole sequence of a
// (batch, head) pair is on chip. Persistent CTAs walk over the (batch, head) pairs with a
// two-stage cp.async pipeline (the next pair's tiles land while the current pair is computed),
// tiles are XOR-swizzled so that every tensor-core fragment is one 128-bit shared-memory
// load, and the contraction / output indices are permuted so that fragments need no shuffles:
//   Q K^T : k-slots (t, t+4) of step h of a 16-wide chunk <-> d = 16c + 4t + 2h, +1
//   P V   : k-slots (t, t+4) <-> keys (2t, 2t+1); column g of n-tile n <-> d = 4g + n
// Included by hz_attn.cu inside its anonymous namespace.
#pragma once

constexpr int kFN = 64, kFD = 32;
constexpr int kFTile = kFN * kFD;            // floats per tile

// float4 index of (row, 16-byte chunk) in a swizzled [64, 32] tile. One swizzle serves both
// access patterns without bank conflicts: "row pattern" (a quarter-warp reads rows {2q, 2q+1},
// chunks 4c+t: operands contracted over d) and "column pattern" (rows 2t or 2t+1, chunks
// {2q, 2q+1}: operands contracted over tokens).
__device__ __forceinline__ int sw_c4(int r, int c) {
  return r * 8 + (c ^ ((r & 6) ^ ((r & 1) << 2)));
}
__device__ __forceinline__ int qk_c4(int r, int c) { return sw_c4(r, c); }
__device__ __forceinline__ int v_c4(int r, int c) { return sw_c4(r, c); }

// Arithmetic of the contractions (template parameter AR of the kernels):
//   kArTf32x3  three-term TF32 split, fp32-faithful (default)
//   kArTf32    one TF32 product, the arithmetic of the reference's Triton kernels (tl.dot on
//              fp32 operands); the tail words are then dead and the compiler drops them
//   kArBf16x3  two-term BF16 split, three products (tail*head + head*tail + head*head) on
//              m16n8k16: each product is exact to about 3 * 2^-16 of its magnitude, outputs stay
//              within 1e-4 of their scale, and one k16 instruction replaces two k8 steps, i.e.
//              half of the tensor-pipe time of the TF32 split
//   kArFp16x3  the same with FP16 heads and tails (11 significant bits each): a product is exact
//              to about 3 * 2^-22 of its magnitude, as close to fp32 as the TF32 split, at the
//              speed of the BF16 split; operands must stay inside the FP16 range (|x| < 65504,
//              tails below 6e-5 round to multiples of 6e-8)
constexpr int kArTf32x3 = 0, kArTf32 = 1, kArBf16x3 = 2, kArFp16x3 = 3;
__host__ __device__ constexpr bool ar_k16(int ar) { return ar == kArBf16x3 || ar == kArFp16x3; }

__device__ __forceinline__ void split2(float x, uint32_t& hi, uint32_t& lo) {
  hi = to_tf32(x);
  lo = __float_as_uint(x - __uint_as_float(hi));   // the tensor core ignores the low bits
}
// (x, y) -> packed BF16 heads and tails; x sits in the low half (the lower k index)
__device__ __forceinline__ void split_bf(float x, float y, uint32_t& hi, uint32_t& lo) {
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(y), "f"(x));
  const float xh = __uint_as_float(hi << 16), yh = __uint_as_float(hi & 0xffff0000u);
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(y - yh), "f"(x - xh));
}
// the same with FP16 halves
__device__ __forceinline__ void split_hf(float x, float y, uint32_t& hi, uint32_t& lo) {
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(y), "f"(x));
  float xh, yh;
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}"
      : "=f"(xh), "=f"(yh) : "r"(hi));
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(y - yh), "f"(x - xh));
}
template <int AR>
__device__ __forceinline__ void split_16(float x, float y, uint32_t& hi, uint32_t& lo) {
  if (AR == kArFp16x3) split_hf(x, y, hi, lo);
  else split_bf(x, y, hi, lo);
}
__device__ __forceinline__ void mma_tf32p(float (&c)[4], const uint32_t* a, const uint32_t* b) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
template <int AR>
__device__ __forceinline__ void mma_bf16p(float (&c)[4], const uint32_t* a, const uint32_t* b) {
  if (AR == kArFp16x3)
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  else
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Operands of TWO consecutive k8 steps of the TF32 fragment layout (hz_mma.cuh). In the TF32
// modes they are kept as two k8 fragments; in the BF16 mode the two steps fuse into one k16
// fragment: k index 2t, 2t+1 <-> slots t, t+4 of step 0 and 2t+8, 2t+9 <-> slots t, t+4 of
// step 1, for the A and the B operand alike, so the loads and index permutations of the
// kernels below do not depend on the arithmetic.
template <int AR>
struct PA {
  static constexpr int kW = ar_k16(AR) ? 4 : 8;
  uint32_t hi[kW], lo[kW];
  // (a0..a3) = (g,t) (g+8,t) (g,t+4) (g+8,t+4) of step 0, (c0..c3) the same of step 1
  __device__ __forceinline__ void set(float a0, float a1, float a2, float a3, float c0, float c1,
                                      float c2, float c3) {
    if constexpr (ar_k16(AR)) {
      split_16<AR>(a0, a2, hi[0], lo[0]); split_16<AR>(a1, a3, hi[1], lo[1]);
      split_16<AR>(c0, c2, hi[2], lo[2]); split_16<AR>(c1, c3, hi[3], lo[3]);
    } else {
      split2(a0, hi[0], lo[0]); split2(a1, hi[1], lo[1]);
      split2(a2, hi[2], lo[2]); split2(a3, hi[3], lo[3]);
      split2(c0, hi[4], lo[4]); split2(c1, hi[5], lo[5]);
      split2(c2, hi[6], lo[6]); split2(c3, hi[7], lo[7]);
    }
  }
};
template <int AR>
struct PB {
  static constexpr int kW = ar_k16(AR) ? 2 : 4;
  uint32_t hi[kW], lo[kW];
  // (b0, b1) = (k=t, n=g), (k=t+4, n=g) of step 0, (d0, d1) the same of step 1
  __device__ __forceinline__ void set(float b0, float b1, float d0, float d1) {
    if constexpr (ar_k16(AR)) {
      split_16<AR>(b0, b1, hi[0], lo[0]); split_16<AR>(d0, d1, hi[1], lo[1]);
    } else {
      split2(b0, hi[0], lo[0]); split2(b1, hi[1], lo[1]);
      split2(d0, hi[2], lo[2]); split2(d1, hi[3], lo[3]);
    }
  }
};
// one k8 step (TF32 modes): small terms first
template <int AR>
__device__ __forceinline__ void mma_step(float (&c)[4], const PA<AR>& a, const PB<AR>& b, int st) {
  if (AR == kArTf32x3) {
    mma_tf32p(c, a.lo + 4 * st, b.hi + 2 * st);
    mma_tf32p(c, a.hi + 4 * st, b.lo + 2 * st);
  }
  mma_tf32p(c, a.hi + 4 * st, b.hi + 2 * st);
}
template <int AR>
__device__ __forceinline__ void mma_bf3(float (&c)[4], const PA<AR>& a, const PB<AR>& b) {
  mma_bf16p<AR>(c, a.lo, b.hi);
  mma_bf16p<AR>(c, a.hi, b.lo);
  mma_bf16p<AR>(c, a.hi, b.hi);
}
// c += a b over both k8 steps
template <int AR>
__device__ __forceinline__ void mma_pair(float (&c)[4], const PA<AR>& a, const PB<AR>& b) {
  if constexpr (ar_k16(AR)) {
    mma_bf3(c, a, b);
  } else {
    mma_step(c, a, b, 0);
    mma_step(c, a, b, 1);
  }
}
// c[i] += a b[i], i < NQ (n-tiles): in the TF32 modes step 0 of all four, then step 1
template <int AR, int NQ>
__device__ __forceinline__ void mma_quad(float (&c)[NQ][4], const PA<AR>& a, const PB<AR> (&b)[NQ]) {
  if constexpr (ar_k16(AR)) {
#pragma unroll
    for (int i = 0; i < NQ; ++i) mma_bf3(c[i], a, b[i]);
  } else {
#pragma unroll
    for (int st = 0; st < 2; ++st)
#pragma unroll
      for (int i = 0; i < NQ; ++i) mma_step(c[i], a, b[i], st);
  }
}
// c1[i] += a1 b1[i] and c2[i] += a2 b2[i], interleaved per n-tile (c1 and c2 may be one array)
template <int AR, int NQ>
__device__ __forceinline__ void mma_quad2(float (&c1)[NQ][4], const PA<AR>& a1, const PB<AR> (&b1)[NQ],
                                          float (&c2)[NQ][4], const PA<AR>& a2, const PB<AR> (&b2)[NQ]) {
  if constexpr (ar_k16(AR)) {
#pragma unroll
    for (int i = 0; i < NQ; ++i) { mma_bf3(c1[i], a1, b1[i]); mma_bf3(c2[i], a2, b2[i]); }
  } else {
#pragma unroll
    for (int st = 0; st < 2; ++st)
#pragma unroll
      for (int i = 0; i < NQ; ++i) { mma_step(c1[i], a1, b1[i], st); mma_step(c2[i], a2, b2[i], st); }
  }
}

__device__ __forceinline__ void cp16(float* dst, const float* src, bool pred) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src),
               "r"(pred ? 16 : 0));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Stage one [64, 32] slice (rows of tensor `src` for (b, h)) into a swizzled tile; masked rows
// are zero-filled. VT selects the V-type swizzle.
template <bool VT, bool HAS_MASK, int NT = 128>
__device__ __forceinline__ void stage_tile(float* tile, const float* src, size_t base,
                                           size_t rowstride, const uint8_t* mrow, int dchunks = 8) {
#pragma unroll
  for (int i = 0; i < 512 / NT; ++i) {
    const int idx = threadIdx.x + i * NT;        // 512 chunks of 16 bytes
    const int r = idx >> 3, c = idx & 7;
    // rows of masked tokens and (head dimension below 32) the columns beyond it arrive as zeros
    const bool keep = (HAS_MASK ? (mrow[r] != 0) : true) && c < dchunks;
    const int dst = VT ? v_c4(r, c) : qk_c4(r, c);
    cp16(tile + dst * 4, keep ? src + base + (size_t)r * rowstride + c * 4 : src, keep);
  }
}

// ------------------------------------------------------------------ forward
// NS = 2: two-stage pipeline, four CTAs per SM; NS = 1: one stage, five CTAs per SM
template <bool HAS_E, bool HAS_MASK, int AR, int NS>
__global__ void __launch_bounds__(128, NS == 1 ? 5 : 4) attn_fwd_fast(AttnArgs a, int tiles) {
  extern __shared__ __align__(16) float sm[];
  // [stage][Q | K | V] tiles, then [stage][64] mask bytes
  uint8_t* mask_s = reinterpret_cast<uint8_t*>(sm + NS * 3 * kFTile);
  const int H = a.H;
  const int D = a.D;                 // 32, or 8 / 16: the tiles are zero-padded to 32 columns on chip
  const size_t rowstride = (size_t)H * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int lr0 = warp * 16 + g, lr1 = lr0 + 8;

  auto issue = [&](int tile, int stage) {
    const int b = tile / H, h = tile % H;
    const size_t base = ((size_t)b * kFN * H + h) * D;
    float* st = sm + stage * 3 * kFTile;
    const uint8_t* mrow = HAS_MASK ? a.mask + (size_t)b * kFN : nullptr;
    if (HAS_MASK && threadIdx.x < kFN) mask_s[stage * kFN + threadIdx.x] = mrow[threadIdx.x];
    stage_tile<false, HAS_MASK>(st, a.q, base, rowstride, mrow, D >> 2);
    stage_tile<false, HAS_MASK>(st + kFTile, a.k, base, rowstride, mrow, D >> 2);
    stage_tile<true, HAS_MASK>(st + 2 * kFTile, a.v, base, rowstride, mrow, D >> 2);
    cp_commit();
  };

  int stage = 0;
  if (NS == 2 && (int)blockIdx.x < tiles) issue(blockIdx.x, 0);
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    if (NS == 2) {
      const int next = tile + gridDim.x;
      if (next < tiles) { issue(next, stage ^ 1); cp_wait<1>(); } else { cp_wait<0>(); }
    } else {
      issue(tile, 0);
      cp_wait<0>();
    }
    __syncthreads();
    const float4* Q4 = reinterpret_cast<const float4*>(sm + stage * 3 * kFTile);
    const float4* K4 = Q4 + kFTile / 4;
    const float4* V4 = K4 + kFTile / 4;
    const uint8_t* mk = mask_s + stage * kFN;
    const int b = tile / H, h = tile % H;

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[i][c] = 0.f;
#pragma unroll
    for (int c16 = 0; c16 < 2; ++c16) {
      const float4 qa = Q4[qk_c4(lr0, 4 * c16 + t)], qb = Q4[qk_c4(lr1, 4 * c16 + t)];
      PA<AR> fq;
      fq.set(qa.x, qb.x, qa.y, qb.y, qa.z, qb.z, qa.w, qb.w);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float4 kb = K4[qk_c4(nt * 8 + g, 4 * c16 + t)];
        PB<AR> bk;
        bk.set(kb.x, kb.y, kb.z, kb.w);
        mma_pair<AR>(s[nt], fq, bk);
      }
    }
    bool rok0 = true, rok1 = true;
    if (HAS_MASK) { rok0 = mk[lr0] != 0; rok1 = mk[lr1] != 0; }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int key = nt * 8 + 2 * t;
      if (HAS_E) {
        const float2 e0 = __ldg(reinterpret_cast<const float2*>(
            a.e + (((size_t)b * kFN + lr0) * H + h) * kFN + key));
        const float2 e1 = __ldg(reinterpret_cast<const float2*>(
            a.e + (((size_t)b * kFN + lr1) * H + h) * kFN + key));
        s[nt][0] += e0.x; s[nt][1] += e0.y; s[nt][2] += e1.x; s[nt][3] += e1.y;
      }
      if (HAS_MASK) {
        const bool k0 = mk[key] != 0, k1 = mk[key + 1] != 0;
        s[nt][0] = (rok0 && k0) ? s[nt][0] : kBigNegative;
        s[nt][1] = (rok0 && k1) ? s[nt][1] : kBigNegative;
        s[nt][2] = (rok1 && k0) ? s[nt][2] : kBigNegative;
        s[nt][3] = (rok1 && k1) ? s[nt][3] : kBigNegative;
      }
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = quad_max(mx0);
    mx1 = quad_max(mx1);
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      s[nt][0] = __expf(s[nt][0] - mx0); s[nt][1] = __expf(s[nt][1] - mx0);
      s[nt][2] = __expf(s[nt][2] - mx1); s[nt][3] = __expf(s[nt][3] - mx1);
      sum0 += s[nt][0] + s[nt][1];
      sum1 += s[nt][2] + s[nt][3];
    }
    sum0 = quad_sum(sum0);
    sum1 = quad_sum(sum1);

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; kk += 2) {
      PA<AR> fp;
      fp.set(s[kk][0], s[kk][2], s[kk][1], s[kk][3], s[kk + 1][0], s[kk + 1][2], s[kk + 1][1], s[kk + 1][3]);
      const float4 v0 = V4[v_c4(kk * 8 + 2 * t, g)], v1 = V4[v_c4(kk * 8 + 2 * t + 1, g)];
      const float4 w0 = V4[v_c4(kk * 8 + 8 + 2 * t, g)], w1 = V4[v_c4(kk * 8 + 9 + 2 * t, g)];
      PB<AR> bv[4];
      bv[0].set(v0.x, v1.x, w0.x, w1.x); bv[1].set(v0.y, v1.y, w0.y, w1.y);
      bv[2].set(v0.z, v1.z, w0.z, w1.z); bv[3].set(v0.w, v1.w, w0.w, w1.w);
      mma_quad<AR>(acc, fp, bv);
    }
    const float inv0 = (HAS_MASK && !rok0) ? 0.f : 1.f / sum0;
    const float inv1 = (HAS_MASK && !rok1) ? 0.f : 1.f / sum1;
    const size_t base = ((size_t)b * kFN * H + h) * D;
    float* o0 = a.out + base + (size_t)lr0 * rowstride + 8 * t;
    float* o1 = a.out + base + (size_t)lr1 * rowstride + 8 * t;
    if (8 * t < D) {       // this lane's columns 8t .. 8t+7 exist
      *reinterpret_cast<float4*>(o0) = make_float4(acc[0][0] * inv0, acc[1][0] * inv0, acc[2][0] * inv0, acc[3][0] * inv0);
      *reinterpret_cast<float4*>(o0 + 4) = make_float4(acc[0][1] * inv0, acc[1][1] * inv0, acc[2][1] * inv0, acc[3][1] * inv0);
      *reinterpret_cast<float4*>(o1) = make_float4(acc[0][2] * inv1, acc[1][2] * inv1, acc[2][2] * inv1, acc[3][2] * inv1);
      *reinterpret_cast<float4*>(o1 + 4) = make_float4(acc[0][3] * inv1, acc[1][3] * inv1, acc[2][3] * inv1, acc[3][3] * inv1);
    }
    if (t == 0) {
      a.lse[((size_t)b * kFN + lr0) * H + h] = mx0 + logf(sum0);
      a.lse[((size_t)b * kFN + lr1) * H + h] = mx1 + logf(sum1);
    }
    __syncthreads();      // the stage is refilled by the next iteration
    if (NS == 2) stage ^= 1;
  }
}

// ------------------------------------------------------------------ tangent
// NS as in attn_bwd_fast: 2 = two-stage pipeline and two CTAs per SM, 1 = one stage and three
template <bool HAS_E, bool HAS_MASK, int AR, int NS>
__global__ void __launch_bounds__(128, NS == 1 ? 3 : 2) attn_jvp_fast(AttnArgs a, int tiles) {
  extern __shared__ __align__(16) float sm[];
  // [stage][Q | Qt | K | Kt | V | Vt], then [stage][64] mask bytes
  uint8_t* mask_s = reinterpret_cast<uint8_t*>(sm + NS * 6 * kFTile);
  const int H = a.H;
  const int D = a.D;                 // 32, or 8 / 16: the tiles are zero-padded to 32 columns on chip
  const size_t rowstride = (size_t)H * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int lr0 = warp * 16 + g, lr1 = lr0 + 8;

  auto issue = [&](int tile, int stage) {
    const int b = tile / H, h = tile % H;
    const size_t base = ((size_t)b * kFN * H + h) * D;
    float* st = sm + stage * 6 * kFTile;
    const uint8_t* mrow = HAS_MASK ? a.mask + (size_t)b * kFN : nullptr;
    if (HAS_MASK && threadIdx.x < kFN) mask_s[stage * kFN + threadIdx.x] = mrow[threadIdx.x];
    stage_tile<false, HAS_MASK>(st, a.q, base, rowstride, mrow, D >> 2);
    stage_tile<false, HAS_MASK>(st + kFTile, a.qt, base, rowstride, mrow, D >> 2);
    stage_tile<false, HAS_MASK>(st + 2 * kFTile, a.k, base, rowstride, mrow, D >> 2);
    stage_tile<false, HAS_MASK>(st + 3 * kFTile, a.kt, base, rowstride, mrow, D >> 2);
    stage_tile<true, HAS_MASK>(st + 4 * kFTile, a.v, base, rowstride, mrow, D >> 2);
    stage_tile<true, HAS_MASK>(st + 5 * kFTile, a.vt, base, rowstride, mrow, D >> 2);
    cp_commit();
  };

  int stage = 0;
  if (NS == 2 && (int)blockIdx.x < tiles) issue(blockIdx.x, 0);
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    if (NS == 2) {
      const int next = tile + gridDim.x;
      if (next < tiles) { issue(next, stage ^ 1); cp_wait<1>(); } else { cp_wait<0>(); }
    } else {
      issue(tile, 0);
      cp_wait<0>();
    }
    __syncthreads();
    const float4* Q4 = reinterpret_cast<const float4*>(sm + stage * 6 * kFTile);
    const float4* Qt4 = Q4 + kFTile / 4;
    const float4* K4 = Qt4 + kFTile / 4;
    const float4* Kt4 = K4 + kFTile / 4;
    const float4* V4 = Kt4 + kFTile / 4;
    const float4* Vt4 = V4 + kFTile / 4;
    const uint8_t* mk = mask_s + stage * kFN;
    const int b = tile / H, h = tile % H;

    float s[8][4], sd[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[i][c] = sd[i][c] = 0.f;
#pragma unroll
    for (int c16 = 0; c16 < 2; ++c16) {
      PA<AR> fq, ft;
      {
        const float4 qa = Q4[sw_c4(lr0, 4 * c16 + t)], qb = Q4[sw_c4(lr1, 4 * c16 + t)];
        fq.set(qa.x, qb.x, qa.y, qb.y, qa.z, qb.z, qa.w, qb.w);
        const float4 ta = Qt4[sw_c4(lr0, 4 * c16 + t)], tb = Qt4[sw_c4(lr1, 4 * c16 + t)];
        ft.set(ta.x, tb.x, ta.y, tb.y, ta.z, tb.z, ta.w, tb.w);
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float4 kb = K4[sw_c4(nt * 8 + g, 4 * c16 + t)];
        const float4 kd = Kt4[sw_c4(nt * 8 + g, 4 * c16 + t)];
        PB<AR> bk, bd;
        bk.set(kb.x, kb.y, kb.z, kb.w);
        bd.set(kd.x, kd.y, kd.z, kd.w);
        mma_pair<AR>(s[nt], fq, bk);
        mma_pair<AR>(sd[nt], ft, bk);
        mma_pair<AR>(sd[nt], fq, bd);
      }
    }
    bool rok0 = true, rok1 = true;
    if (HAS_MASK) { rok0 = mk[lr0] != 0; rok1 = mk[lr1] != 0; }
    const float lse0 = __ldg(a.lse_in + ((size_t)b * kFN + lr0) * H + h);
    const float lse1 = __ldg(a.lse_in + ((size_t)b * kFN + lr1) * H + h);
    float mean0 = 0.f, mean1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int key = nt * 8 + 2 * t;
      if (HAS_E) {
        const size_t o0 = (((size_t)b * kFN + lr0) * H + h) * kFN + key;
        const size_t o1 = (((size_t)b * kFN + lr1) * H + h) * kFN + key;
        if (a.e != nullptr) {
          const float2 e0 = __ldg(reinterpret_cast<const float2*>(a.e + o0));
          const float2 e1 = __ldg(reinterpret_cast<const float2*>(a.e + o1));
          s[nt][0] += e0.x; s[nt][1] += e0.y; s[nt][2] += e1.x; s[nt][3] += e1.y;
        }
        if (a.et != nullptr) {
          const float2 e0 = __ldg(reinterpret_cast<const float2*>(a.et + o0));
          const float2 e1 = __ldg(reinterpret_cast<const float2*>(a.et + o1));
          sd[nt][0] += e0.x; sd[nt][1] += e0.y; sd[nt][2] += e1.x; sd[nt][3] += e1.y;
        }
      }
      bool l0 = true, l1 = true, l2 = true, l3 = true;
      if (HAS_MASK) {
        const bool k0 = mk[key] != 0, k1 = mk[key + 1] != 0;
        l0 = rok0 && k0; l1 = rok0 && k1; l2 = rok1 && k0; l3 = rok1 && k1;
      }
      const float p0 = __expf((l0 ? s[nt][0] : kBigNegative) - lse0);
      const float p1 = __expf((l1 ? s[nt][1] : kBigNegative) - lse0);
      const float p2 = __expf((l2 ? s[nt][2] : kBigNegative) - lse1);
      const float p3 = __expf((l3 ? s[nt][3] : kBigNegative) - lse1);
      s[nt][0] = p0; s[nt][1] = p1; s[nt][2] = p2; s[nt][3] = p3;
      sd[nt][0] = l0 ? p0 * sd[nt][0] : 0.f;
      sd[nt][1] = l1 ? p1 * sd[nt][1] : 0.f;
      sd[nt][2] = l2 ? p2 * sd[nt][2] : 0.f;
      sd[nt][3] = l3 ? p3 * sd[nt][3] : 0.f;
      mean0 += sd[nt][0] + sd[nt][1];
      mean1 += sd[nt][2] + sd[nt][3];
    }
    mean0 = quad_sum(mean0);
    mean1 = quad_sum(mean1);

    float acc[4][4];       // (P*Sd) V + P Vt
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; kk += 2) {
      PA<AR> fp, fs;
      fp.set(s[kk][0], s[kk][2], s[kk][1], s[kk][3], s[kk + 1][0], s[kk + 1][2], s[kk + 1][1], s[kk + 1][3]);
      fs.set(sd[kk][0], sd[kk][2], sd[kk][1], sd[kk][3], sd[kk + 1][0], sd[kk + 1][2], sd[kk + 1][1], sd[kk + 1][3]);
      const int ra = kk * 8 + 2 * t;
      const float4 v0 = V4[sw_c4(ra, g)], v1 = V4[sw_c4(ra + 1, g)];
      const float4 v2 = V4[sw_c4(ra + 8, g)], v3 = V4[sw_c4(ra + 9, g)];
      const float4 w0 = Vt4[sw_c4(ra, g)], w1 = Vt4[sw_c4(ra + 1, g)];
      const float4 w2 = Vt4[sw_c4(ra + 8, g)], w3 = Vt4[sw_c4(ra + 9, g)];
      PB<AR> bv[4], bw[4];
      bv[0].set(v0.x, v1.x, v2.x, v3.x); bw[0].set(w0.x, w1.x, w2.x, w3.x);
      bv[1].set(v0.y, v1.y, v2.y, v3.y); bw[1].set(w0.y, w1.y, w2.y, w3.y);
      bv[2].set(v0.z, v1.z, v2.z, v3.z); bw[2].set(w0.z, w1.z, w2.z, w3.z);
      bv[3].set(v0.w, v1.w, v2.w, v3.w); bw[3].set(w0.w, w1.w, w2.w, w3.w);
      mma_quad2<AR>(acc, fs, bv, acc, fp, bw);
    }
    const size_t base = ((size_t)b * kFN * H + h) * D;
    const size_t off0 = base + (size_t)lr0 * rowstride + 8 * t;
    const size_t off1 = base + (size_t)lr1 * rowstride + 8 * t;
    const float z0 = (HAS_MASK && !rok0) ? 0.f : 1.f, z1 = (HAS_MASK && !rok1) ? 0.f : 1.f;
    if (8 * t < D) {
      const float4 oa = __ldg(reinterpret_cast<const float4*>(a.out_in + off0));
      const float4 ob = __ldg(reinterpret_cast<const float4*>(a.out_in + off0 + 4));
      *reinterpret_cast<float4*>(a.tangent + off0) =
          make_float4(z0 * (acc[0][0] - mean0 * oa.x), z0 * (acc[1][0] - mean0 * oa.y),
                      z0 * (acc[2][0] - mean0 * oa.z), z0 * (acc[3][0] - mean0 * oa.w));
      *reinterpret_cast<float4*>(a.tangent + off0 + 4) =
          make_float4(z0 * (acc[0][1] - mean0 * ob.x), z0 * (acc[1][1] - mean0 * ob.y),
                      z0 * (acc[2][1] - mean0 * ob.z), z0 * (acc[3][1] - mean0 * ob.w));
    }
    if (8 * t < D) {
      const float4 oa = __ldg(reinterpret_cast<const float4*>(a.out_in + off1));
      const float4 ob = __ldg(reinterpret_cast<const float4*>(a.out_in + off1 + 4));
      *reinterpret_cast<float4*>(a.tangent + off1) =
          make_float4(z1 * (acc[0][2] - mean1 * oa.x), z1 * (acc[1][2] - mean1 * oa.y),
                      z1 * (acc[2][2] - mean1 * oa.z), z1 * (acc[3][2] - mean1 * oa.w));
      *reinterpret_cast<float4*>(a.tangent + off1 + 4) =
          make_float4(z1 * (acc[0][3] - mean1 * ob.x), z1 * (acc[1][3] - mean1 * ob.y),
                      z1 * (acc[2][3] - mean1 * ob.z), z1 * (acc[3][3] - mean1 * ob.w));
    }
    __syncthreads();
    if (NS == 2) stage ^= 1;
  }
}

// ------------------------------------------------------------------ backward
// element (q, key) of the P / dS tiles: the key index is XORed with a multiple of 8 that
// depends on the query row, so that the transposed reads of phase 2 are conflict-free
__device__ __forceinline__ int ps_idx(int q, int key) {
  // 2-bit swizzle f(q) = (bit 1, bit 0 ^ bit 2): distinct over four consecutive rows (the stores
  // of phase 1: rows g .. g+3 of a half-warp) and over rows q, q+2, q+4, q+6 (the transposed
  // reads of phase 2: rows 2t and 2t + 1)
  return q * 64 + (key ^ (((q & 2) | ((q ^ (q >> 2)) & 1)) << 3));
}

// NS = 2: two-stage cp.async pipeline, two CTAs per SM. NS = 1: one stage and a third CTA per
// SM; the other CTAs' arithmetic covers a CTA's load instead of its own prefetch.
template <bool HAS_E, bool HAS_MASK, bool WRITE_DE, int AR, int NS>
__global__ void __launch_bounds__(128, NS == 1 ? 3 : 2) attn_bwd_fast(AttnArgs a, int tiles) {
  extern __shared__ __align__(16) float sm[];
  // [stage][Q | K | V | dO], P tile, dS tile, then [stage][64] mask bytes
  float* Ps = sm + NS * 4 * kFTile;
  float* dSs = Ps + 64 * 64;
  uint8_t* mask_s = reinterpret_cast<uint8_t*>(dSs + 64 * 64);
  const int H = a.H;
  const int D = a.D;                 // 32, or 8 / 16: the tiles are zero-padded to 32 columns on chip
  const size_t rowstride = (size_t)H * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int lr0 = warp * 16 + g, lr1 = lr0 + 8;

  auto issue = [&](int tile, int stage) {
    const int b = tile / H, h = tile % H;
    const size_t base = ((size_t)b * kFN * H + h) * D;
    float* st = sm + stage * 4 * kFTile;
    const uint8_t* mrow = HAS_MASK ? a.mask + (size_t)b * kFN : nullptr;
    if (HAS_MASK && threadIdx.x < kFN) mask_s[stage * kFN + threadIdx.x] = mrow[threadIdx.x];
    stage_tile<false, HAS_MASK>(st, a.q, base, rowstride, mrow, D >> 2);
    stage_tile<false, HAS_MASK>(st + kFTile, a.k, base, rowstride, mrow, D >> 2);
    stage_tile<false, HAS_MASK>(st + 2 * kFTile, a.v, base, rowstride, mrow, D >> 2);
    stage_tile<false, HAS_MASK>(st + 3 * kFTile, a.dout, base, rowstride, mrow, D >> 2);
    cp_commit();
  };

  int stage = 0;
  if (NS == 2 && (int)blockIdx.x < tiles) issue(blockIdx.x, 0);
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    if (NS == 2) {
      const int next = tile + gridDim.x;
      if (next < tiles) { issue(next, stage ^ 1); cp_wait<1>(); } else { cp_wait<0>(); }
    } else {
      issue(tile, 0);
      cp_wait<0>();
    }
    __syncthreads();
    const float4* Q4 = reinterpret_cast<const float4*>(sm + stage * 4 * kFTile);
    const float4* K4 = Q4 + kFTile / 4;
    const float4* V4 = K4 + kFTile / 4;
    const float4* G4 = V4 + kFTile / 4;      // dO
    const uint8_t* mk = mask_s + stage * kFN;
    const int b = tile / H, h = tile % H;
    const size_t base = ((size_t)b * kFN * H + h) * D;

    // delta_i = sum_d O_id dO_id (dO rows of masked queries are already zero in the tile)
    float del0, del1;
    {
      // columns 4t .. and 16 + 4t ..: only those below the head dimension exist in global memory
      const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
      const bool lo_ok = 4 * t < D, hi_ok = 16 + 4 * t < D;
      const float4 oa = lo_ok ? __ldg(reinterpret_cast<const float4*>(a.out_in + base + (size_t)lr0 * rowstride + 4 * t)) : zero4;
      const float4 ob = hi_ok ? __ldg(reinterpret_cast<const float4*>(a.out_in + base + (size_t)lr0 * rowstride + 16 + 4 * t)) : zero4;
      const float4 oc = lo_ok ? __ldg(reinterpret_cast<const float4*>(a.out_in + base + (size_t)lr1 * rowstride + 4 * t)) : zero4;
      const float4 od = hi_ok ? __ldg(reinterpret_cast<const float4*>(a.out_in + base + (size_t)lr1 * rowstride + 16 + 4 * t)) : zero4;
      const float4 ga = G4[sw_c4(lr0, t)], gb = G4[sw_c4(lr0, 4 + t)];
      const float4 gc = G4[sw_c4(lr1, t)], gd = G4[sw_c4(lr1, 4 + t)];
      del0 = oa.x * ga.x + oa.y * ga.y + oa.z * ga.z + oa.w * ga.w + ob.x * gb.x + ob.y * gb.y + ob.z * gb.z + ob.w * gb.w;
      del1 = oc.x * gc.x + oc.y * gc.y + oc.z * gc.z + oc.w * gc.w + od.x * gd.x + od.y * gd.y + od.z * gd.z + od.w * gd.w;
      del0 = quad_sum(del0);
      del1 = quad_sum(del1);
    }

    float s[8][4], dp[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[i][c] = dp[i][c] = 0.f;
#pragma unroll
    for (int c16 = 0; c16 < 2; ++c16) {
      PA<AR> fq, fg;
      {
        const float4 qa = Q4[sw_c4(lr0, 4 * c16 + t)], qb = Q4[sw_c4(lr1, 4 * c16 + t)];
        fq.set(qa.x, qb.x, qa.y, qb.y, qa.z, qb.z, qa.w, qb.w);
        const float4 ga = G4[sw_c4(lr0, 4 * c16 + t)], gb = G4[sw_c4(lr1, 4 * c16 + t)];
        fg.set(ga.x, gb.x, ga.y, gb.y, ga.z, gb.z, ga.w, gb.w);
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float4 kb = K4[sw_c4(nt * 8 + g, 4 * c16 + t)];
        const float4 vb = V4[sw_c4(nt * 8 + g, 4 * c16 + t)];
        PB<AR> b;
        b.set(kb.x, kb.y, kb.z, kb.w);
        mma_pair<AR>(s[nt], fq, b);
        b.set(vb.x, vb.y, vb.z, vb.w);
        mma_pair<AR>(dp[nt], fg, b);
      }
    }
    bool rok0 = true, rok1 = true;
    if (HAS_MASK) { rok0 = mk[lr0] != 0; rok1 = mk[lr1] != 0; }
    const float lse0 = __ldg(a.lse_in + ((size_t)b * kFN + lr0) * H + h);
    const float lse1 = __ldg(a.lse_in + ((size_t)b * kFN + lr1) * H + h);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int key = nt * 8 + 2 * t;
      const size_t o0 = (((size_t)b * kFN + lr0) * H + h) * kFN + key;
      const size_t o1 = (((size_t)b * kFN + lr1) * H + h) * kFN + key;
      if (HAS_E) {
        const float2 e0 = __ldg(reinterpret_cast<const float2*>(a.e + o0));
        const float2 e1 = __ldg(reinterpret_cast<const float2*>(a.e + o1));
        s[nt][0] += e0.x; s[nt][1] += e0.y; s[nt][2] += e1.x; s[nt][3] += e1.y;
      }
      bool l0 = true, l1 = true, l2 = true, l3 = true;
      if (HAS_MASK) {
        const bool k0 = mk[key] != 0, k1 = mk[key + 1] != 0;
        l0 = rok0 && k0; l1 = rok0 && k1; l2 = rok1 && k0; l3 = rok1 && k1;
      }
      const float p0 = __expf((l0 ? s[nt][0] : kBigNegative) - lse0);
      const float p1 = __expf((l1 ? s[nt][1] : kBigNegative) - lse0);
      const float p2 = __expf((l2 ? s[nt][2] : kBigNegative) - lse1);
      const float p3 = __expf((l3 ? s[nt][3] : kBigNegative) - lse1);
      s[nt][0] = p0; s[nt][1] = p1; s[nt][2] = p2; s[nt][3] = p3;
      dp[nt][0] = l0 ? (dp[nt][0] - del0) * p0 : 0.f;
      dp[nt][1] = l1 ? (dp[nt][1] - del0) * p1 : 0.f;
      dp[nt][2] = l2 ? (dp[nt][2] - del1) * p2 : 0.f;
      dp[nt][3] = l3 ? (dp[nt][3] - del1) * p3 : 0.f;
      *reinterpret_cast<float2*>(Ps + ps_idx(lr0, key)) = make_float2(p0, p1);
      *reinterpret_cast<float2*>(Ps + ps_idx(lr1, key)) = make_float2(p2, p3);
      *reinterpret_cast<float2*>(dSs + ps_idx(lr0, key)) = make_float2(dp[nt][0], dp[nt][1]);
      *reinterpret_cast<float2*>(dSs + ps_idx(lr1, key)) = make_float2(dp[nt][2], dp[nt][3]);
      if (WRITE_DE) {
        *reinterpret_cast<float2*>(a.de + o0) = make_float2(dp[nt][0], dp[nt][1]);
        *reinterpret_cast<float2*>(a.de + o1) = make_float2(dp[nt][2], dp[nt][3]);
      }
    }
    // dQ = dS K  (keys contracted with slots (2t, 2t+1); columns d = 4g + n)
    {
      float acc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 8; kk += 2) {
        PA<AR> fs;
        fs.set(dp[kk][0], dp[kk][2], dp[kk][1], dp[kk][3], dp[kk + 1][0], dp[kk + 1][2], dp[kk + 1][1], dp[kk + 1][3]);
        const int ra = kk * 8 + 2 * t;
        const float4 k0 = K4[sw_c4(ra, g)], k1 = K4[sw_c4(ra + 1, g)];
        const float4 k2 = K4[sw_c4(ra + 8, g)], k3 = K4[sw_c4(ra + 9, g)];
        PB<AR> bk[4];
        bk[0].set(k0.x, k1.x, k2.x, k3.x); bk[1].set(k0.y, k1.y, k2.y, k3.y);
        bk[2].set(k0.z, k1.z, k2.z, k3.z); bk[3].set(k0.w, k1.w, k2.w, k3.w);
        mma_quad<AR>(acc, fs, bk);
      }
      float* q0 = a.dq + base + (size_t)lr0 * rowstride + 8 * t;
      float* q1 = a.dq + base + (size_t)lr1 * rowstride + 8 * t;
      if (8 * t < D) {
        *reinterpret_cast<float4*>(q0) = make_float4(acc[0][0], acc[1][0], acc[2][0], acc[3][0]);
        *reinterpret_cast<float4*>(q0 + 4) = make_float4(acc[0][1], acc[1][1], acc[2][1], acc[3][1]);
        *reinterpret_cast<float4*>(q1) = make_float4(acc[0][2], acc[1][2], acc[2][2], acc[3][2]);
        *reinterpret_cast<float4*>(q1 + 4) = make_float4(acc[0][3], acc[1][3], acc[2][3], acc[3][3]);
      }
    }
    __syncthreads();
    // phase 2: this warp's 16 keys. dV = P^T dO, dK = dS^T Q; queries contracted with slots
    // (2t, 2t+1), columns d = 4g + n.
    {
      float av[4][4], ak[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) av[i][c] = ak[i][c] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ks += 2) {
        const int qa = ks * 8 + 2 * t, qb = qa + 1, qc = qa + 8, qd = qa + 9;
        PA<AR> fp, fs;
        fp.set(Ps[ps_idx(qa, lr0)], Ps[ps_idx(qa, lr1)], Ps[ps_idx(qb, lr0)], Ps[ps_idx(qb, lr1)],
               Ps[ps_idx(qc, lr0)], Ps[ps_idx(qc, lr1)], Ps[ps_idx(qd, lr0)], Ps[ps_idx(qd, lr1)]);
        fs.set(dSs[ps_idx(qa, lr0)], dSs[ps_idx(qa, lr1)], dSs[ps_idx(qb, lr0)], dSs[ps_idx(qb, lr1)],
               dSs[ps_idx(qc, lr0)], dSs[ps_idx(qc, lr1)], dSs[ps_idx(qd, lr0)], dSs[ps_idx(qd, lr1)]);
        const float4 g0 = G4[sw_c4(qa, g)], g1 = G4[sw_c4(qb, g)];
        const float4 g2 = G4[sw_c4(qc, g)], g3 = G4[sw_c4(qd, g)];
        const float4 x0 = Q4[sw_c4(qa, g)], x1 = Q4[sw_c4(qb, g)];
        const float4 x2 = Q4[sw_c4(qc, g)], x3 = Q4[sw_c4(qd, g)];
        PB<AR> bg[4], bq[4];
        bg[0].set(g0.x, g1.x, g2.x, g3.x); bq[0].set(x0.x, x1.x, x2.x, x3.x);
        bg[1].set(g0.y, g1.y, g2.y, g3.y); bq[1].set(x0.y, x1.y, x2.y, x3.y);
        bg[2].set(g0.z, g1.z, g2.z, g3.z); bq[2].set(x0.z, x1.z, x2.z, x3.z);
        bg[3].set(g0.w, g1.w, g2.w, g3.w); bq[3].set(x0.w, x1.w, x2.w, x3.w);
        mma_quad2<AR>(av, fp, bg, ak, fs, bq);
      }
      const size_t off0 = base + (size_t)lr0 * rowstride + 8 * t;
      const size_t off1 = base + (size_t)lr1 * rowstride + 8 * t;
      if (8 * t < D) {
      *reinterpret_cast<float4*>(a.dv + off0) = make_float4(av[0][0], av[1][0], av[2][0], av[3][0]);
      *reinterpret_cast<float4*>(a.dv + off0 + 4) = make_float4(av[0][1], av[1][1], av[2][1], av[3][1]);
      *reinterpret_cast<float4*>(a.dv + off1) = make_float4(av[0][2], av[1][2], av[2][2], av[3][2]);
      *reinterpret_cast<float4*>(a.dv + off1 + 4) = make_float4(av[0][3], av[1][3], av[2][3], av[3][3]);
      *reinterpret_cast<float4*>(a.dk + off0) = make_float4(ak[0][0], ak[1][0], ak[2][0], ak[3][0]);
      *reinterpret_cast<float4*>(a.dk + off0 + 4) = make_float4(ak[0][1], ak[1][1], ak[2][1], ak[3][1]);
      *reinterpret_cast<float4*>(a.dk + off1) = make_float4(ak[0][2], ak[1][2], ak[2][2], ak[3][2]);
      *reinterpret_cast<float4*>(a.dk + off1 + 4) = make_float4(ak[0][3], ak[1][3], ak[2][3], ak[3][3]);
      }
    }
    __syncthreads();
    if (NS == 2) stage ^= 1;
  }
}
