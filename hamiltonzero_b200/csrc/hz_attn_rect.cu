// Rectangular multi-head attention with additive bias for the large-N (sequence-parallel)
// context path, forward only, for sm_100a; and the per-channel panel product of the ring 2-FWL
// edge update.
//
// Semantics follow the reference's flash kernel
// (src/hamiltonzero/evaluation/pallas_mha.py:43-161) as its only caller drives it
// (src/hamiltonzero/evaluation/sequence_parallel.py:59-95): scores q k^T d^-1/2 + bias, masked
// keys carry a bias of -1e30, online softmax in base 2 over blocks of keys, output
// sum_k p v / sum_k p. Layouts are the reference's: q [B, Lq, H, D], k, v [B, Lk, H, D],
// bias [B, Lq, Lk, H] (heads innermost), out [B, Lq, H, D].
//
// Tiling: one CTA = 16 RW query rows x all H heads, RW warps per head with 16 rows each (the bias
// of a query row is contiguous over (key, head), so a CTA that owns every head reads its bias
// tile as whole 128-byte lines through cp.async; a CTA per head would fetch every line H
// times). RW = 2 (sixteen warps for eight heads) when the CTA then stays within 512 threads.
// Keys are visited in blocks of 32 staged in shared memory (two stages when they fit). Contractions run on
// mma.sync TF32 with the three-term split; the score accumulators feed P V as the A operand
// without shuffles by mapping the k-slots (t, t+4) to keys (2t, 2t+1). HBM-bound: the bias
// (4 H bytes per (query, key) pair) is 32/D times the K/V traffic of a CTA and is read once.
#include "hz_gemm.cuh"
#include "hz_internal.h"
#include "hz_mma.cuh"

#include <math.h>
#include <stdint.h>

namespace hz {
namespace {

constexpr int kRectRows = 16;       // query rows per warp
constexpr int kRectKeys = 32;       // keys per block
constexpr float kRectMasked = -1.0e30f;            // sequence_parallel.py:83-87
constexpr float kLog2e = 1.4426950408889634f;

struct RectArgs {
  int B, Lq, Lk, H, D;
  const float* q;
  const float* k;
  const float* v;
  const float* bias;
  const uint8_t* key_mask;       // [B, Lk] or null
  float* out;
  // keys split over gridDim.z CTAs (a rank's few query rows against many gathered keys would
  // otherwise leave most SMs idle): partial sums [z][B][Lq][H][D] and (m, l) [z][B][Lq][H][2]
  int splits, blocks_per_split;
  float* part_o;
  float* part_ml;
};

// D8 = D / 8 k-steps of the score contraction and n-tiles of the output; THREADS bounds the CTA
// (256: 255 registers per thread, 512: 128); RW = warps per head
template <int D8, int THREADS, int RW>
__global__ void __launch_bounds__(THREADS) attn_rect_fwd_kernel(RectArgs a, int stages) {
  constexpr int D = D8 * 8;
  extern __shared__ __align__(16) float smem[];
  const int H = a.H;
  const int ldkv = H * D + 4;                       // padded row of a K / V block (conflict-free fragments)
  const int kv_floats = kRectKeys * ldkv;
  const int ldb = kRectKeys * H + 4;                // padded bias row (16-way -> 4-way bank conflicts)
  const int bias_floats = RW * kRectRows * ldb;
  const int stage_floats = 2 * kv_floats + bias_floats + 8;      // + 32 key-mask bytes
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int b = blockIdx.y;
  const int h = warp / RW, rw = warp % RW;
  const int qcta = blockIdx.x * (RW * kRectRows), q0 = qcta + rw * kRectRows;
  const float* qb = a.q + (size_t)b * a.Lq * H * D;
  const float* kb = a.k + (size_t)b * a.Lk * H * D;
  const float* vb = a.v + (size_t)b * a.Lk * H * D;
  const float* bb = a.bias + (size_t)b * a.Lq * a.Lk * H;
  const uint8_t* mb = a.key_mask ? a.key_mask + (size_t)b * a.Lk : nullptr;
  const int nblocks_all = (a.Lk + kRectKeys - 1) / kRectKeys;
  const int blk_begin = blockIdx.z * a.blocks_per_split;
  const int blk_end = min(blk_begin + a.blocks_per_split, nblocks_all);

  auto stage_load = [&](int s, int blk) {
    float* Ks = smem + (size_t)s * stage_floats;
    float* Vs = Ks + kv_floats;
    float* Bs = Vs + kv_floats;
    const int key0 = blk * kRectKeys;
    const int row_chunks = H * D / 4;               // 16-byte chunks per key row
    for (int idx = threadIdx.x; idx < kRectKeys * row_chunks; idx += blockDim.x) {
      const int kr = idx / row_chunks, c = idx % row_chunks;
      const bool ok = key0 + kr < a.Lk;
      const size_t off = (size_t)(key0 + kr) * H * D + c * 4;
      cp_async16(Ks + kr * ldkv + c * 4, ok ? kb + off : kb, ok ? 16 : 0);
      cp_async16(Vs + kr * ldkv + c * 4, ok ? vb + off : vb, ok ? 16 : 0);
    }
    // bias rows: [16 query rows][32 keys x H] contiguous per query row
    const int brow_chunks = kRectKeys * H / 4;
    for (int idx = threadIdx.x; idx < RW * kRectRows * brow_chunks; idx += blockDim.x) {
      const int r = idx / brow_chunks, c = idx % brow_chunks;
      const int key = key0 + (c * 4) / H;            // H is a multiple of 4: a chunk stays inside one key
      const bool ok = (qcta + r < a.Lq) && (key < a.Lk);
      const size_t off = ((size_t)(qcta + r) * a.Lk + key0) * H + c * 4;
      cp_async16(Bs + r * ldb + c * 4, ok ? bb + off : bb, ok ? 16 : 0);
    }
    if (threadIdx.x < kRectKeys) {
      // key mask of the block as bytes behind the bias tile (1 = keep); plain store, made
      // visible by the barrier that follows the wait for this stage
      const int key = key0 + threadIdx.x;
      reinterpret_cast<uint8_t*>(Bs + bias_floats)[threadIdx.x] =
          (key < a.Lk && (mb == nullptr || mb[key])) ? 1 : 0;
    }
    cp_async_commit();
  };

  // Q fragments of this warp's head, pre-scaled by d^-1/2 log2(e)
  FragA qf[D8];
  {
    const float sc = rsqrtf((float)D) * kLog2e;
    const int r0 = q0 + g, r1 = q0 + g + 8;
#pragma unroll
    for (int ks = 0; ks < D8; ++ks) {
      const int d0 = ks * 8 + t;
      const float a0 = r0 < a.Lq ? qb[((size_t)r0 * H + h) * D + d0] * sc : 0.f;
      const float a1 = r1 < a.Lq ? qb[((size_t)r1 * H + h) * D + d0] * sc : 0.f;
      const float a2 = r0 < a.Lq ? qb[((size_t)r0 * H + h) * D + d0 + 4] * sc : 0.f;
      const float a3 = r1 < a.Lq ? qb[((size_t)r1 * H + h) * D + d0 + 4] * sc : 0.f;
      qf[ks].set(a0, a1, a2, a3);
    }
  }
  float o[D8][4];
#pragma unroll
  for (int j = 0; j < D8; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[j][c] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows g and g + 8

  stage_load(0, blk_begin);
  for (int blk = blk_begin; blk < blk_end; ++blk) {
    const int s = stages == 2 ? ((blk - blk_begin) & 1) : 0;
    if (stages == 2 && blk + 1 < blk_end) {
      stage_load(s ^ 1, blk + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* Ks = smem + (size_t)s * stage_floats;
    const float* Vs = Ks + kv_floats;
    const float* Bs = Vs + kv_floats;
    const uint8_t* keep = reinterpret_cast<const uint8_t*>(Bs + bias_floats);
    const int key0 = blk * kRectKeys;

    // scores of 16 rows x 32 keys (base-2 units)
    float sc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) sc[j][c] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D8; ++ks) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        FragB kf;
        const float* kp = Ks + (j * 8 + g) * ldkv + h * D + ks * 8 + t;
        kf.set(kp[0], kp[4]);
        mma3(sc[j], qf[ks], kf);
      }
    }
    float rmax0 = -INFINITY, rmax1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = key0 + j * 8 + 2 * t + (c & 1);
        const int row = g + (c >> 1) * 8;
        float bias = Bs[(rw * kRectRows + row) * ldb + (key - key0) * H + h];
        if (!keep[key - key0]) bias = kRectMasked;
        const float x = key < a.Lk ? sc[j][c] + bias * kLog2e : -INFINITY;
        sc[j][c] = x;
        if (c >> 1) rmax1 = fmaxf(rmax1, x); else rmax0 = fmaxf(rmax0, x);
      }
    }
    rmax0 = quad_max(rmax0);
    rmax1 = quad_max(rmax1);
    const float mn0 = fmaxf(m0, rmax0), mn1 = fmaxf(m1, rmax1);
    const float corr0 = exp2f(m0 - mn0), corr1 = exp2f(m1 - mn1);     // exp2(-inf) = 0 on the first block
    float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = exp2f(sc[j][c] - ((c >> 1) ? mn1 : mn0));     // keys beyond Lk: exp2(-inf) = 0
        sc[j][c] = p;
        if (c >> 1) ls1 += p; else ls0 += p;
      }
    }
    l0 = corr0 * l0 + quad_sum(ls0);
    l1 = corr1 * l1 + quad_sum(ls1);
    m0 = mn0; m1 = mn1;
#pragma unroll
    for (int j = 0; j < D8; ++j) {
      o[j][0] *= corr0; o[j][1] *= corr0; o[j][2] *= corr1; o[j][3] *= corr1;
    }
    // O += P V: k-slots t, t + 4 of step j stand for keys 8 j + 2 t, 8 j + 2 t + 1, which is where
    // this lane's score accumulators sit
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      FragA pf;
      pf.set(sc[j][0], sc[j][2], sc[j][1], sc[j][3]);
      const float* vp = Vs + (j * 8 + 2 * t) * ldkv + h * D + g;
#pragma unroll
      for (int n = 0; n < D8; ++n) {
        FragB vf;
        vf.set(vp[n * 8], vp[ldkv + n * 8]);
        mma3(o[n], pf, vf);
      }
    }
    __syncthreads();
    if (stages == 1 && blk + 1 < blk_end) stage_load(0, blk + 1);
  }
  const int r0 = q0 + g, r1 = q0 + g + 8;
  if (a.splits > 1) {
    // this split's unnormalised sums; rect_combine_kernel merges the splits
    const size_t zb = (size_t)blockIdx.z * a.B + b;
    float* po = a.part_o + zb * a.Lq * H * D;
    float* pml = a.part_ml + zb * a.Lq * H * 2;
#pragma unroll
    for (int n = 0; n < D8; ++n) {
      if (r0 < a.Lq)
        *reinterpret_cast<float2*>(po + ((size_t)r0 * H + h) * D + n * 8 + 2 * t) = make_float2(o[n][0], o[n][1]);
      if (r1 < a.Lq)
        *reinterpret_cast<float2*>(po + ((size_t)r1 * H + h) * D + n * 8 + 2 * t) = make_float2(o[n][2], o[n][3]);
    }
    if (t == 0) {
      if (r0 < a.Lq) *reinterpret_cast<float2*>(pml + ((size_t)r0 * H + h) * 2) = make_float2(m0, l0);
      if (r1 < a.Lq) *reinterpret_cast<float2*>(pml + ((size_t)r1 * H + h) * 2) = make_float2(m1, l1);
    }
    return;
  }
  // out = O / l
  const float i0 = 1.f / l0, i1 = 1.f / l1;
  float* ob = a.out + (size_t)b * a.Lq * H * D;
#pragma unroll
  for (int n = 0; n < D8; ++n) {
    if (r0 < a.Lq)
      *reinterpret_cast<float2*>(ob + ((size_t)r0 * H + h) * D + n * 8 + 2 * t) =
          make_float2(o[n][0] * i0, o[n][1] * i0);
    if (r1 < a.Lq)
      *reinterpret_cast<float2*>(ob + ((size_t)r1 * H + h) * D + n * 8 + 2 * t) =
          make_float2(o[n][2] * i1, o[n][3] * i1);
  }
}

// out[b, q, h, :] = sum_z o_z 2^(m_z - M) / sum_z l_z 2^(m_z - M), M = max_z m_z
__global__ void rect_combine_kernel(RectArgs a) {
  const size_t rows = (size_t)a.B * a.Lq * a.H;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;      // (row, d / 4)
  const int d4 = a.D / 4;
  if (idx >= rows * d4) return;
  const size_t row = idx / d4;
  const int c = (int)(idx % d4) * 4;
  float M = -INFINITY;
  for (int z = 0; z < a.splits; ++z) M = fmaxf(M, a.part_ml[(z * rows + row) * 2]);
  float L = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int z = 0; z < a.splits; ++z) {
    const float2 ml = *reinterpret_cast<const float2*>(a.part_ml + (z * rows + row) * 2);
    const float w = exp2f(ml.x - M);
    L = fmaf(ml.y, w, L);
    const float4 o = *reinterpret_cast<const float4*>(a.part_o + (z * rows + row) * a.D + c);
    acc.x = fmaf(o.x, w, acc.x); acc.y = fmaf(o.y, w, acc.y);
    acc.z = fmaf(o.z, w, acc.z); acc.w = fmaf(o.w, w, acc.w);
  }
  const float inv = 1.f / L;
  *reinterpret_cast<float4*>(a.out + row * a.D + c) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

// key splits that give about four CTAs per SM; 1 when the rows alone do
inline int rect_splits(int B, int Lq, int Lk) {
  const long long row_ctas = (long long)((Lq + 2 * kRectRows - 1) / (2 * kRectRows)) * B;
  const int nblocks = (Lk + kRectKeys - 1) / kRectKeys;
  long long s = (4 * 148 + row_ctas - 1) / row_ctas;        // about four waves: a short tail
  if (s > nblocks / 4) s = nblocks / 4;          // at least four key blocks per split
  return s < 1 ? 1 : (int)s;
}

template <int D8, int THREADS, int RW>
int launch_rect_t(const RectArgs& a, cudaStream_t stream) {
  const int ldkv = a.H * (D8 * 8) + 4;
  const size_t stage = (size_t)(2 * kRectKeys * ldkv + RW * kRectRows * (kRectKeys * a.H + 4) + 8) * sizeof(float);
  const int stages = 2 * stage <= 220 * 1024 ? 2 : 1;
  const size_t smem = stages * stage;
  if (smem > 227 * 1024) return HZ_ERR_UNSUPPORTED;
  const int rc = ensure_kernel_attributes(
      reinterpret_cast<const void*>(attn_rect_fwd_kernel<D8, THREADS, RW>), (int)smem);
  if (rc != HZ_OK) return rc;
  dim3 grid((a.Lq + RW * kRectRows - 1) / (RW * kRectRows), a.B, a.splits);
  attn_rect_fwd_kernel<D8, THREADS, RW><<<grid, 32 * RW * a.H, smem, stream>>>(a, stages);
  if (a.splits > 1) {
    const size_t items = (size_t)a.B * a.Lq * a.H * (a.D / 4);
    rect_combine_kernel<<<(unsigned)((items + 255) / 256), 256, 0, stream>>>(a);
  }
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

template <int D8>
int launch_rect(const RectArgs& a, cudaStream_t stream) {
  // two warps per head (32 rows per CTA share a K/V block) while registers allow: D <= 32
  if (a.H <= 8 && D8 <= 4) return launch_rect_t<D8, 512, 2>(a, stream);
  return a.H <= 8 ? launch_rect_t<D8, 256, 1>(a, stream) : launch_rect_t<D8, 512, 1>(a, stream);
}

// out[i, j, c] (+)= sum_k a[i, k0 + k, c] b[k, j, c]: the contribution of one ring panel to the
// 2-FWL edge update (sequence_parallel.py:148-153). a [rows, lda_cols, C], b [panel, cols, C],
// out [rows, cols, C]; channels innermost, so a warp's 32 lanes read consecutive channels.
__global__ void __launch_bounds__(256)
fwl2_panel_kernel(const float* __restrict__ A, const float* __restrict__ Bp, float* __restrict__ out,
                  int rows, int a_cols, int k0, int panel, int cols, int C, int accumulate) {
  const int i = blockIdx.y;
  const long long jc = (long long)blockIdx.x * blockDim.x + threadIdx.x;     // (j, c) flattened
  if (jc >= (long long)cols * C) return;
  const int c = (int)(jc % C);
  const float* ap = A + ((size_t)i * a_cols + k0) * C + c;
  const float* bp = Bp + jc;
  float acc = 0.f;
#pragma unroll 4
  for (int k = 0; k < panel; ++k) acc = fmaf(ap[(size_t)k * C], bp[(size_t)k * cols * C], acc);
  float* o = out + (size_t)i * cols * C + jc;
  *o = accumulate ? *o + acc : acc;
}

}  // namespace
}  // namespace hz

extern "C" long long hz_mha_rect_workspace_bytes(int B, int Lq, int Lk, int H, int D) {
  if (B <= 0 || Lq <= 0 || Lk <= 0 || H <= 0 || D <= 0) return -1;
  const int splits = hz::rect_splits(B, Lq, Lk);
  return splits > 1 ? (long long)splits * B * Lq * H * (D + 2) * (long long)sizeof(float) : 0;
}

extern "C" int hz_mha_rect_fwd(int B, int Lq, int Lk, int H, int D, const float* q, const float* k,
                               const float* v, const float* bias, const uint8_t* key_mask, float* out,
                               void* workspace, long long workspace_bytes, void* stream) {
  using namespace hz;
  if (!q || !k || !v || !bias || !out) return HZ_ERR_NULL_POINTER;
  if (B <= 0 || Lq <= 0 || Lk <= 0 || H <= 0 || D <= 0) return HZ_ERR_BAD_SHAPE;
  if (H % 4 != 0 || H > 16 || (D != 8 && D != 16 && D != 32 && D != 64)) return HZ_ERR_UNSUPPORTED;
  RectArgs a{B, Lq, Lk, H, D, q, k, v, bias, key_mask, out, 1, (Lk + kRectKeys - 1) / kRectKeys, nullptr, nullptr};
  // without (enough) workspace the keys are not split: same result, fewer CTAs
  const int splits = rect_splits(B, Lq, Lk);
  if (splits > 1 && workspace != nullptr &&
      workspace_bytes >= (long long)splits * B * Lq * H * (D + 2) * (long long)sizeof(float)) {
    const int nblocks = (Lk + kRectKeys - 1) / kRectKeys;
    a.blocks_per_split = (nblocks + splits - 1) / splits;
    a.splits = (nblocks + a.blocks_per_split - 1) / a.blocks_per_split;
    a.part_o = static_cast<float*>(workspace);
    a.part_ml = a.part_o + (size_t)splits * B * Lq * H * D;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (D) {
    case 8: return launch_rect<1>(a, s);
    case 16: return launch_rect<2>(a, s);
    case 32: return launch_rect<4>(a, s);
    default: return launch_rect<8>(a, s);
  }
}

extern "C" int hz_fwl2_panel(const float* a, const float* b_panel, float* out, int rows, int a_cols,
                             int k0, int panel, int cols, int channels, int accumulate, void* stream) {
  using namespace hz;
  if (!a || !b_panel || !out) return HZ_ERR_NULL_POINTER;
  if (rows <= 0 || panel <= 0 || cols <= 0 || channels <= 0 || k0 < 0 || k0 + panel > a_cols)
    return HZ_ERR_BAD_SHAPE;
  const long long jc = (long long)cols * channels;
  dim3 grid((unsigned)((jc + 255) / 256), rows);
  fwl2_panel_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a, b_panel, out, rows, a_cols, k0,
                                                                        panel, cols, channels, accumulate);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}
