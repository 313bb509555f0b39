// Reverse pass of the compiled binary-merge-tree executor: the vector-Jacobian product of
// (log|psi|, phase) with respect to every parameter array and to the walkers' quaternions.
//
// Reference semantics: the executor of src/hamiltonzero/compiled/execute.py:79-118 in its
// tagged form (CompiledFinetuneWaveFunction.call_tagged, compiled/model.py:179-310), driven by
// the loss of src/hamiltonzero/optim/production.py:168-228, whose parameter tangent is
// sum_w (c_re[w] d log|psi_w| + c_im[w] d phase_w) with per-walker weights c.
//
// One chunk of walkers runs the value-only forward pass level by level and keeps, for every
// merge level, raw = T(u_L, u_R), vx = raw V, mixed = vx * h and the normalised, gated output
// (all levels in one level-major row range, so that the weight gradients of the shared factors
// are ONE transposed GEMM per chunk over all levels' rows). The backward pass walks the levels
// from the root: normalisation and gate (norm_bwd_kernel), the factor map (two GEMMs on the
// tcgen05 path and the h gradient), the quadrilinear merge (merge_bwd_kernel: the same two
// tensor applications as the forward pass, then mat-vecs for the children's cotangents and
// the rank-one updates of dT in registers), the leaves and the leaf map.
//
// Included by hz_walker.cu inside namespace hz { namespace {.
#pragma once

// ------------------------------------------------------------------ small element-wise kernels
__global__ void vjp_scale_kernel(const float* __restrict__ VX, const float* __restrict__ h,
                                 float* __restrict__ MIX, long long total, int nodes, int r) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long row = idx / r;
  const int j = (int)(idx % r), node = (int)(row % nodes);
  MIX[idx] = VX[idx] * h[(size_t)node * r + j];
}

__global__ void vjp_split_kernel(const float* __restrict__ x, float* __restrict__ hi,
                                 float* __restrict__ lo, long long n) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const float v = x[idx];
  const float h = __uint_as_float((__float_as_uint(v) + 0x1000u) & 0xFFFFE000u);
  hi[idx] = h;
  lo[idx] = v - h;
}

// out [cols, rows] = in [rows, cols]^T
__global__ void vjp_transpose_kernel(const float* __restrict__ in, float* __restrict__ out, int rows,
                                     int cols) {
  __shared__ float tile[32][33];
  const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y)
    tile[i][threadIdx.x] = (r0 + i < rows && c0 + threadIdx.x < cols)
                               ? in[(size_t)(r0 + i) * cols + c0 + threadIdx.x] : 0.f;
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y)
    if (c0 + i < cols && r0 + threadIdx.x < rows)
      out[(size_t)(c0 + i) * rows + r0 + threadIdx.x] = tile[threadIdx.x][i];
}

// ------------------------------------------------------------------ C += A^T B
// A [K, M], B [K, N] row-major (K = rows of the walker batch, large), C [M, N] accumulated. The
// contraction is split over K; every split stores its 128 x 128 tile into its own slot of a
// scratch buffer and a second kernel adds the slots to C in split order, so the result does not
// depend on the order in which CTAs finish (bitwise reproducible). mma.sync TF32 with the
// three-term split; the K chunk of 16 is a chain of six MMAs per accumulator, folded into fp32
// registers with round-to-nearest adds.
constexpr int kTnBM = 128, kTnBN = 128, kTnBK = 16, kTnLd = 136, kTnThreads = 256;

struct TnArgs {
  const float* A;
  const float* B;
  float* C;
  long long K;
  int M, N, lda, ldb, ldc;
  int k_per_split;
  int upper_only;      // C symmetric (A == B): skip the tiles strictly below the diagonal
  float* P;            // [splits][tiles_y][tiles_x][128 x 128] partial tiles; null: one split, C += directly
};

struct TnScratch {
  float* p;
  size_t floats;
};

__global__ void __launch_bounds__(kTnThreads) gemm_tn_kernel(TnArgs a) {
  __shared__ __align__(16) float As[2][kTnBK][kTnLd];
  __shared__ __align__(16) float Bs[2][kTnBK][kTnLd];
  const int m0 = blockIdx.y * kTnBM, n0 = blockIdx.x * kTnBN;
  if (a.upper_only && n0 + kTnBN <= m0) return;
  const long long k_begin = (long long)blockIdx.z * a.k_per_split;
  long long k_end = k_begin + a.k_per_split;
  if (k_end > a.K) k_end = a.K;
  if (k_begin >= k_end) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;

  auto stage = [&](int buf, long long k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * kTnThreads;        // 512 chunks of 16 bytes per operand
      const int kr = idx >> 5, c4 = (idx & 31) * 4;
      const long long k = k0 + kr;
      const bool ka = k < k_end;
      const bool oka = ka && (m0 + c4 < a.M), okb = ka && (n0 + c4 < a.N);
      cp_async16(&As[buf][kr][c4], oka ? a.A + (size_t)k * a.lda + m0 + c4 : a.A, oka ? 16 : 0);
      cp_async16(&Bs[buf][kr][c4], okb ? a.B + (size_t)k * a.ldb + n0 + c4 : a.B, okb ? 16 : 0);
    }
    cp_async_commit();
  };

  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

  const long long chunks = (k_end - k_begin + kTnBK - 1) / kTnBK;
  stage(0, k_begin);
  for (long long ch = 0; ch < chunks; ++ch) {
    const int buf = (int)(ch & 1);
    if (ch + 1 < chunks) {
      stage(buf ^ 1, k_begin + (ch + 1) * kTnBK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float part[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) part[i][j][c] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      FB2 fb[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        fb[j].set(Bs[buf][ks * 8 + t][wn + j * 8 + g], Bs[buf][ks * 8 + t + 4][wn + j * 8 + g]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        FA2 fa;
        const int mm = wm + i * 16 + g;
        fa.set(As[buf][ks * 8 + t][mm], As[buf][ks * 8 + t][mm + 8], As[buf][ks * 8 + t + 4][mm],
               As[buf][ks * 8 + t + 4][mm + 8]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mma_tf32(part[i][j], fa.lo, fb[j].hi);
          mma_tf32(part[i][j], fa.hi, fb[j].lo);
          mma_tf32(part[i][j], fa.hi, fb[j].hi);
        }
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
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = m0 + wm + i * 16 + g, col = n0 + wn + j * 8 + 2 * t;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int rr = row + (c >> 1) * 8, cc = col + (c & 1);
        if (a.P != nullptr) {
          const size_t tile = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
          a.P[tile * (kTnBM * kTnBN) + (size_t)(rr - m0) * kTnBN + (cc - n0)] = acc[i][j][c];
        } else if (rr < a.M && cc < a.N) {
          a.C[(size_t)rr * a.ldc + cc] += acc[i][j][c];
        }
      }
    }
}

// C += the splits' partial tiles, added in split order
__global__ void __launch_bounds__(256) gemm_tn_reduce_kernel(TnArgs a, int splits) {
  const int m0 = blockIdx.y * kTnBM, n0 = blockIdx.x * kTnBN;
  if (a.upper_only && n0 + kTnBN <= m0) return;
  const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
  const size_t per_split = (size_t)gridDim.y * gridDim.x * (kTnBM * kTnBN);
  // 16 CTAs per tile (blockIdx.z), one float4 per thread: a product with few tiles has many
  // splits, and its sums must not fall to a single CTA
  {
    const int e = (blockIdx.z * 256 + threadIdx.x) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int z = 0; z < splits; ++z) {
      const float4 p = *reinterpret_cast<const float4*>(a.P + z * per_split + tile * (kTnBM * kTnBN) + e);
      v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
    }
    const int rr = m0 + e / kTnBN, cc = n0 + e % kTnBN;
    if (rr >= a.M) return;
    float* c = a.C + (size_t)rr * a.ldc + cc;
    if (cc < a.N) c[0] += v.x;
    if (cc + 1 < a.N) c[1] += v.y;
    if (cc + 2 < a.N) c[2] += v.z;
    if (cc + 3 < a.N) c[3] += v.w;
  }
}

int launch_gemm_tn(const float* A, const float* B, float* C, long long K, int M, int N, int lda,
                   int ldb, int ldc, bool upper_only, const TnScratch& scratch, cudaStream_t stream) {
  if (K <= 0 || M <= 0 || N <= 0) return HZ_OK;
  TnArgs a{};
  a.A = A; a.B = B; a.C = C; a.K = K; a.M = M; a.N = N; a.lda = lda; a.ldb = ldb; a.ldc = ldc;
  a.upper_only = upper_only ? 1 : 0;
  const int tiles = ((M + kTnBM - 1) / kTnBM) * ((N + kTnBN - 1) / kTnBN);
  long long splits = (4 * 148 + tiles - 1) / tiles;
  const long long max_splits = (K + 4 * kTnBK - 1) / (4 * kTnBK);
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  long long per = (K + splits - 1) / splits;
  per = (per + kTnBK - 1) / kTnBK * kTnBK;
  splits = (K + per - 1) / per;
  // as many splits as the scratch buffer has tile slots for
  const long long fit = scratch.p ? (long long)(scratch.floats / ((size_t)tiles * kTnBM * kTnBN)) : 1;
  if (splits > fit) {
    splits = fit < 1 ? 1 : fit;
    per = (K + splits - 1) / splits;
    per = (per + kTnBK - 1) / kTnBK * kTnBK;
    splits = (K + per - 1) / per;
  }
  a.k_per_split = (int)per;
  a.P = splits > 1 ? scratch.p : nullptr;
  dim3 grid((N + kTnBN - 1) / kTnBN, (M + kTnBM - 1) / kTnBM, (unsigned)splits);
  gemm_tn_kernel<<<grid, kTnThreads, 0, stream>>>(a);
  if (splits > 1)
    gemm_tn_reduce_kernel<<<dim3(grid.x, grid.y, kTnBM * kTnBN / 1024), 256, 0, stream>>>(a, (int)splits);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// ------------------------------------------------------------------ root
// psi = ((u V_r) * h_r) U_r; log|psi| = log|psi|/2 + s, phase = atan2 (compiled/model.py:175-178).
// One CTA per walker: outputs (optional), d psi, and dvr = (dpsi U_r^T) * h_r.
__global__ void __launch_bounds__(128)
vjp_root_kernel(int r_ro, const float* __restrict__ VR, const float* __restrict__ h_r,
                const float* __restrict__ U_r, const float* __restrict__ s_root,
                const float* __restrict__ cot_abs, const float* __restrict__ cot_phase,
                float* __restrict__ dVR, float* __restrict__ dpsi_out, float* __restrict__ dS_root,
                float* __restrict__ log_abs, float* __restrict__ phase) {
  __shared__ float scratch[2 * 4];
  const int b = blockIdx.x;
  float red[2] = {0.f, 0.f};
  for (int j = threadIdx.x; j < r_ro; j += 128) {
    const float mix = VR[(size_t)b * r_ro + j] * h_r[j];
    red[0] = fmaf(mix, U_r[2 * j], red[0]);
    red[1] = fmaf(mix, U_r[2 * j + 1], red[1]);
  }
  block_sum<2, 128>(red, scratch);
  const float re = red[0], im = red[1];
  const float n2 = re * re + im * im;
  const float ca = cot_abs[b], cp = cot_phase[b];
  const float dre = (ca * re - cp * im) / n2, dim_ = (ca * im + cp * re) / n2;
  for (int j = threadIdx.x; j < r_ro; j += 128)
    dVR[(size_t)b * r_ro + j] = (dre * U_r[2 * j] + dim_ * U_r[2 * j + 1]) * h_r[j];
  if (threadIdx.x == 0) {
    dpsi_out[2 * b] = dre;
    dpsi_out[2 * b + 1] = dim_;
    dS_root[b] = ca;
    if (log_abs) log_abs[b] = 0.5f * logf(n2) + s_root[b];
    if (phase) phase[b] = atan2f(im, re);
  }
}

// dU_r[j][c] += sum_b (vr*h)[b,j] dpsi[b,c]; dh_r[j] += sum_b vr[b,j] (dpsi U_r^T)[b,j]
__global__ void vjp_root_param_kernel(int r_ro, int Bc, const float* __restrict__ VR,
                                      const float* __restrict__ h_r, const float* __restrict__ U_r,
                                      const float* __restrict__ dpsi, float* __restrict__ dU_r,
                                      float* __restrict__ dh_r, float* __restrict__ diag /* nullable */) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= r_ro) return;
  const float h = h_r[j], u0 = U_r[2 * j], u1 = U_r[2 * j + 1];
  float a0 = 0.f, a1 = 0.f, ah = 0.f, a2 = 0.f;
  for (int b = 0; b < Bc; ++b) {
    const float vr = VR[(size_t)b * r_ro + j], d0 = dpsi[2 * b], d1 = dpsi[2 * b + 1];
    a0 = fmaf(vr * h, d0, a0);
    a1 = fmaf(vr * h, d1, a1);
    const float gb = vr * (d0 * u0 + d1 * u1);
    ah += gb;
    a2 = fmaf(gb, gb, a2);
  }
  dU_r[2 * j] += a0;
  dU_r[2 * j + 1] += a1;
  dh_r[j] += ah;
  if (diag) diag[j] += a2;
}

// ------------------------------------------------------------------ normalisation and gate, backward
// In place on dX: cotangent of the gated output -> cotangent of out (zero for gated nodes, whose
// cotangent goes straight to the carried child). u = out / sigma, s = s_L + s_R + log sigma:
//   d out = r (d u + u (d s - u . d u) / d).
__global__ void __launch_bounds__(256)
vjp_norm_bwd_kernel(int d, int nodes, const uint8_t* __restrict__ opcodes,
                    const float* __restrict__ U, const NormOut* __restrict__ nout,
                    float* __restrict__ dX, const float* __restrict__ dS,
                    float* __restrict__ dU_child, float* __restrict__ dS_child,
                    float* __restrict__ RAW, float* __restrict__ MIX, int r, long long rows_total) {
  // one warp per (walker, node) row
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows_total) return;
  const int lane = threadIdx.x & 31, n = (int)(row % nodes), d4 = d >> 2;
  const uint8_t op = opcodes[n];
  float4* dx = reinterpret_cast<float4*>(dX + (size_t)row * d);
  const float ds = dS[row];
  const size_t left = 2 * (size_t)row, right = left + 1;
  if (op == 0) {
    const float4* u = reinterpret_cast<const float4*>(U + (size_t)row * d);
    float dot = 0.f;
    for (int c = lane; c < d4; c += 32) {
      const float4 a = u[c], g = dx[c];
      dot += a.x * g.x + a.y * g.y + a.z * g.z + a.w * g.w;
    }
    dot = warp_sum(dot);
    const float rr = nout[row].r;
    const float coef = (ds - dot) / (float)d;
    for (int c = lane; c < d4; c += 32) {
      const float4 a = u[c], g = dx[c];
      dx[c] = make_float4(rr * (g.x + coef * a.x), rr * (g.y + coef * a.y), rr * (g.z + coef * a.z),
                          rr * (g.w + coef * a.w));
    }
    if (lane == 0) { dS_child[left] = ds; dS_child[right] = ds; }
    return;
  }
  const bool cl = op == 1, cr = op == 2;
  float4* dl = reinterpret_cast<float4*>(dU_child + left * d);
  float4* dr = reinterpret_cast<float4*>(dU_child + right * d);
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4* raw = reinterpret_cast<float4*>(RAW + (size_t)row * d);
  for (int c = lane; c < d4; c += 32) {
    const float4 v = dx[c];
    dl[c] = cl ? v : z4;
    dr[c] = cr ? v : z4;
    dx[c] = z4;
    // the saved inputs of the factor map are dead for a gated node; zeroing them applies the
    // structural mask to the input-side second moments
    raw[c] = z4;
  }
  for (int j = lane; j < r; j += 32) MIX[(size_t)row * r + j] = 0.f;
  if (lane == 0) { dS_child[left] = cl ? ds : 0.f; dS_child[right] = cr ? ds : 0.f; }
}

// dVX = dMIX * h in place; dh[n][j] += sum_b VX[b,n,j] dMIX[b,n,j]. The walkers are cut into
// gridDim.y slices, each CTA (node n, slice s) writes its two partial sums to
// part[s][0 / 1][n][j] and vjp_hscale_reduce_kernel adds the slices in order: no atomics, the
// result does not depend on the schedule.
__global__ void __launch_bounds__(256)
vjp_hscale_bwd_kernel(int r, int nodes, int Bc, const float* __restrict__ h,
                      const float* __restrict__ VX, float* __restrict__ dMIX, float* __restrict__ part) {
  const int n = blockIdx.x, s = blockIdx.y, S = gridDim.y;
  const int b0 = (int)((long long)Bc * s / S), b1 = (int)((long long)Bc * (s + 1) / S);
  for (int j = threadIdx.x; j < r; j += blockDim.x) {
    const float hh = h[(size_t)n * r + j];
    float acc = 0.f, acc2 = 0.f;
#pragma unroll 4
    for (int b = b0; b < b1; ++b) {
      const size_t idx = ((size_t)b * nodes + n) * r + j;
      const float dm = dMIX[idx];
      const float gbn = VX[idx] * dm;
      acc += gbn;
      acc2 = fmaf(gbn, gbn, acc2);
      dMIX[idx] = dm * hh;
    }
    part[((size_t)(2 * s) * nodes + n) * r + j] = acc;
    part[((size_t)(2 * s + 1) * nodes + n) * r + j] = acc2;
  }
}

__global__ void vjp_hscale_reduce_kernel(int total, int S, const float* __restrict__ part,
                                         float* __restrict__ dh /* nullable */,
                                         float* __restrict__ diag /* nullable: += sum_b (vx dmix)^2 */) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  float a = 0.f, a2 = 0.f;
  for (int s = 0; s < S; ++s) {
    a += part[(size_t)(2 * s) * total + idx];
    a2 += part[(size_t)(2 * s + 1) * total + idx];
  }
  if (dh) dh[idx] += a;
  if (diag) diag[idx] += a2;
}

int launch_hscale_bwd(int r, int nodes, int Bc, const float* h, const float* VX, float* dMIX, float* dh,
                      float* diag, const TnScratch& scratch, cudaStream_t stream) {
  const size_t per_slice = 2 * (size_t)nodes * r;
  long long S = (long long)(scratch.floats / per_slice);
  // enough CTAs for two waves of the SMs, at least 8 walkers per slice
  const long long want = (2 * 148 + nodes - 1) / nodes;
  if (S > want) S = want;
  if (S > (Bc + 7) / 8) S = (Bc + 7) / 8;
  if (S < 1) return HZ_ERR_WORKSPACE;
  vjp_hscale_bwd_kernel<<<dim3(nodes, (unsigned)S), 256, 0, stream>>>(r, nodes, Bc, h, VX, dMIX, scratch.p);
  HZ_CUDA_TRY(cudaGetLastError());
  const int total = nodes * r;
  vjp_hscale_reduce_kernel<<<(total + 255) / 256, 256, 0, stream>>>(total, (int)S, scratch.p, dh, diag);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// ------------------------------------------------------------------ quadrilinear merge, backward
// raw[j] = sum_kl T[j,k,l] uL[k] uR[l]  =>  duL[k] = sum_j A_R[j,k] draw[j],
// duR[l] = sum_j A_L[j,l] draw[j], dT[j,k,l] += draw[j] uL[k] uR[l]. Same CTA layout as the
// forward kernel (one group per CTA, T_i in shared memory, tiles of 16 pairs). Each thread keeps
// 64 entries of dT_i in registers over all its tiles (j = tid / 16, k in {2 (tid % 16), +1}, all
// l) and adds them to its CTA's private slice of `dT_part` at the end: no atomics, and the sum
// over slices is taken once per call.
template <bool kWithDT>      // false: carrier cotangents only (no tensor gradient)
__global__ void __launch_bounds__(kTsThreads, 1)
merge_bwd_kernel(Level L, const float* __restrict__ T, const uint8_t* __restrict__ opcodes,
                 const float* __restrict__ Uin, const float* __restrict__ dRaw,
                 float* __restrict__ dUin, float* __restrict__ dT_part, int with_du) {
  // with_du == 0: only the tensor gradient (the carrier cotangents come from tapply_tc_kernel)
  extern __shared__ __align__(16) float sm[];
  float* Ts = sm;
  float* AX = Ts + 32768;
  float* vec = AX + kTsPairs * 1024;            // uL, uR, draw : [3][16][36]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int grp = blockIdx.x;
  const int d = L.d, nodes = L.nodes, nodes_in = 2 * L.nodes;
  const int col0 = grp * kDr;
  if (with_du) {
    const float* Tg = T + (size_t)grp * 32768;
    for (int idx = tid * 4; idx < 32768; idx += kTsThreads * 4) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(Tg + idx));
      const int l = idx & 31, k = (idx >> 5) & 31, j = idx >> 10;
      *reinterpret_cast<float4*>(Ts + t_idx(j, k, l)) = v;
    }
  }
  float acc[2][32];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int l = 0; l < 32; ++l) acc[i][l] = 0.f;
  const int tj = tid >> 4, tk = (tid & 15) * 2;

  const long long total_pairs = (long long)L.Bc * nodes;
  const long long tiles = (total_pairs + kTsPairs - 1) / kTsPairs;
  const float* uL = vec;
  const float* uR = vec + kTsPairs * kTsVecLd;
  const float* dW = vec + 2 * kTsPairs * kTsVecLd;
  // the three vectors of a tile's pairs (u_L, u_R, d raw; one element of each per thread) are
  // fetched one tile ahead into registers, so that their global-memory latency runs under the
  // previous tile's arithmetic
  static_assert(kTsThreads == kTsPairs * 32, "one thread per (pair, channel)");
  const int fc = tid & 31, fp = tid >> 5;
  float nxt[3];
  auto fetch = [&](long long tile) {
    const long long pair = tile * kTsPairs + fp;
    nxt[0] = nxt[1] = nxt[2] = 0.f;
    if (tile < tiles && pair < total_pairs) {
      const int b = (int)(pair / nodes), n = (int)(pair % nodes);
      if (opcodes[n] == 0) {
        nxt[0] = Uin[((size_t)b * nodes_in + 2 * n) * d + col0 + fc];
        nxt[1] = Uin[((size_t)b * nodes_in + 2 * n + 1) * d + col0 + fc];
        nxt[2] = dRaw[((size_t)b * nodes + n) * d + col0 + fc];
      }
    }
  };
  fetch(blockIdx.y);
  for (long long tile = blockIdx.y; tile < tiles; tile += gridDim.y) {
    __syncthreads();
#pragma unroll
    for (int which = 0; which < 3; ++which) vec[(which * kTsPairs + fp) * kTsVecLd + fc] = nxt[which];
    __syncthreads();
    fetch(tile + gridDim.y);
    // dT: rank-one updates on the CUDA cores (exact fp32)
    for (int p = 0; kWithDT && p < kTsPairs; ++p) {
      const float w = dW[p * kTsVecLd + tj];
      const float c0 = w * uL[p * kTsVecLd + tk], c1 = w * uL[p * kTsVecLd + tk + 1];
#pragma unroll
      for (int l4 = 0; l4 < 8; ++l4) {
        const float4 r4 = *reinterpret_cast<const float4*>(uR + p * kTsVecLd + l4 * 4);
        acc[0][l4 * 4 + 0] = fmaf(c0, r4.x, acc[0][l4 * 4 + 0]);
        acc[0][l4 * 4 + 1] = fmaf(c0, r4.y, acc[0][l4 * 4 + 1]);
        acc[0][l4 * 4 + 2] = fmaf(c0, r4.z, acc[0][l4 * 4 + 2]);
        acc[0][l4 * 4 + 3] = fmaf(c0, r4.w, acc[0][l4 * 4 + 3]);
        acc[1][l4 * 4 + 0] = fmaf(c1, r4.x, acc[1][l4 * 4 + 0]);
        acc[1][l4 * 4 + 1] = fmaf(c1, r4.y, acc[1][l4 * 4 + 1]);
        acc[1][l4 * 4 + 2] = fmaf(c1, r4.z, acc[1][l4 * 4 + 2]);
        acc[1][l4 * 4 + 3] = fmaf(c1, r4.w, acc[1][l4 * 4 + 3]);
      }
    }
    if (!with_du) continue;
    // duL = A_R^T draw
    ts_t_apply(Ts, AX, uR, true, warp, g, t);
    __syncthreads();
    {
      const int p = tid >> 5, k = tid & 31;
      const long long pair = tile * kTsPairs + p;
      float s = 0.f;
#pragma unroll 8
      for (int j = 0; j < 32; ++j) s = fmaf(AX[ax_idx(p, j, k)], dW[p * kTsVecLd + j], s);
      if (pair < total_pairs) {
        const int b = (int)(pair / nodes), n = (int)(pair % nodes);
        if (opcodes[n] == 0) dUin[((size_t)b * nodes_in + 2 * n) * d + col0 + k] = s;
      }
    }
    __syncthreads();
    // duR = A_L^T draw
    ts_t_apply(Ts, AX, uL, false, warp, g, t);
    __syncthreads();
    {
      const int p = tid >> 5, l = tid & 31;
      const long long pair = tile * kTsPairs + p;
      float s = 0.f;
#pragma unroll 8
      for (int j = 0; j < 32; ++j) s = fmaf(AX[ax_idx(p, j, l)], dW[p * kTsVecLd + j], s);
      if (pair < total_pairs) {
        const int b = (int)(pair / nodes), n = (int)(pair % nodes);
        if (opcodes[n] == 0) dUin[((size_t)b * nodes_in + 2 * n + 1) * d + col0 + l] = s;
      }
    }
  }
  if (!kWithDT) return;
  float* part = dT_part + ((size_t)blockIdx.y * gridDim.x + grp) * 32768 + ((size_t)tj * 32 + tk) * 32;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int l4 = 0; l4 < 8; ++l4) {
      float4* dst = reinterpret_cast<float4*>(part + i * 32 + l4 * 4);
      float4 v = *dst;
      v.x += acc[i][l4 * 4]; v.y += acc[i][l4 * 4 + 1]; v.z += acc[i][l4 * 4 + 2]; v.w += acc[i][l4 * 4 + 3];
      *dst = v;
    }
}

// dT[grp][:] = sum over slices
__global__ void vjp_reduce_slices_kernel(const float* __restrict__ part, float* __restrict__ out,
                                         long long n, int slices) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  float s = 0.f;
  for (int k = 0; k < slices; ++k) s += part[(size_t)k * n + idx];
  out[idx] = s;
}

// ------------------------------------------------------------------ leaves, backward
// u = u_raw / rms, s = log rms, u_raw = q . M_site. One CTA per (site, walker): the cotangent of
// u_raw is r (du + u (ds - u.du)/d); dq[o] = M_site[o] . du_raw; the per-walker scalars r and
// (ds - u.du)/d are kept for the leaf-map gradient.
__global__ void __launch_bounds__(kLeafThreads)
vjp_leaf_bwd_kernel(int N, int d, const float* __restrict__ leaf_map, const float* __restrict__ U0,
                    const float* __restrict__ S0, float* __restrict__ dU0 /* in: du, out: du_raw */,
                    const float* __restrict__ dS0, float* __restrict__ dq /* nullable */,
                    const uint8_t* __restrict__ skip_merged /* nullable: first-level opcodes; the leaves of
                                                               merged parents are handled in coefficient space */) {
  __shared__ float scratch[5 * kLeafThreads / 32];
  const int n = blockIdx.x, b = blockIdx.y;
  if (skip_merged != nullptr && skip_merged[n >> 1] == 0) return;
  const size_t row = (size_t)b * N + n;
  const float* u = U0 + row * d;
  float* du = dU0 + row * d;
  const float* M = leaf_map + (size_t)n * 4 * d;
  float red[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
  for (int c = threadIdx.x; c < d; c += kLeafThreads) red[0] = fmaf(u[c], du[c], red[0]);
  block_sum<5, kLeafThreads>(red, scratch);
  const float r = expf(-S0[row]);
  const float coef = (dS0[row] - red[0]) / (float)d;
  float acc[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
  for (int c = threadIdx.x; c < d; c += kLeafThreads) {
    const float v = r * (du[c] + coef * u[c]);
    du[c] = v;
    acc[0] = fmaf(M[c], v, acc[0]);
    acc[1] = fmaf(M[d + c], v, acc[1]);
    acc[2] = fmaf(M[2 * d + c], v, acc[2]);
    acc[3] = fmaf(M[3 * d + c], v, acc[3]);
  }
  if (!dq) return;
  block_sum<5, kLeafThreads>(acc, scratch);
  if (threadIdx.x < 4) dq[row * 4 + threadIdx.x] = acc[threadIdx.x];
}

// dM[n][o][c] += sum_b q[b,n,o] du_raw[b,n,c]
__global__ void __launch_bounds__(256)
vjp_leaf_map_grad_kernel(int N, int d, int Bc, const float* __restrict__ q,
                         const float* __restrict__ dUraw, float* __restrict__ dM) {
  const int n = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
  if (c >= d) return;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int b = 0; b < Bc; ++b) {
    const size_t row = (size_t)b * N + n;
    const float v = dUraw[row * d + c];
    const float4 qq = *reinterpret_cast<const float4*>(q + row * 4);
    acc[0] = fmaf(qq.x, v, acc[0]); acc[1] = fmaf(qq.y, v, acc[1]);
    acc[2] = fmaf(qq.z, v, acc[2]); acc[3] = fmaf(qq.w, v, acc[3]);
  }
#pragma unroll
  for (int o = 0; o < 4; ++o) dM[((size_t)n * 4 + o) * d + c] += acc[o];
}

// Chain from dM to the leaf parameters (once per call; sizes 4N x r_leaf x d):
//   M = tmp U_l, tmp[n,o][j] = WqV[o][j] h[n][j], WqV = Wq V_l.
// dtmp[row][j] = sum_c dM[row][c] U_l[j][c]: one warp per output.
__global__ void vjp_leaf_dtmp_kernel(int rows, int r, int d, const float* __restrict__ dM,
                                     const float* __restrict__ U_l, float* __restrict__ dtmp) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)rows * r) return;
  const int row = (int)(w / r), j = (int)(w % r);
  float acc = 0.f;
  for (int c = lane; c < d; c += 32) acc = fmaf(dM[(size_t)row * d + c], U_l[(size_t)j * d + c], acc);
  acc = warp_sum(acc);
  if (lane == 0) dtmp[(size_t)row * r + j] = acc;
}

// dh[n][j] = sum_o WqV[o][j] dtmp[n,o][j]; dWqV[o][j] = sum_n dtmp[n,o][j] h[n][j]
__global__ void vjp_leaf_h_kernel(int N, int d_o, int r, const float* __restrict__ Wq,
                                  const float* __restrict__ V, const float* __restrict__ h,
                                  const float* __restrict__ dtmp, float* __restrict__ dh,
                                  float* __restrict__ dWqV) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= r) return;
  float wqv[4];
  for (int o = 0; o < 4; ++o) {
    float a = 0.f;
    for (int k = 0; k < d_o; ++k) a = fmaf(Wq[o * d_o + k], V[(size_t)k * r + j], a);
    wqv[o] = a;
  }
  float dw[4] = {0.f, 0.f, 0.f, 0.f};
  for (int n = 0; n < N; ++n) {
    float a = 0.f;
    const float hh = h[(size_t)n * r + j];
    for (int o = 0; o < 4; ++o) {
      const float dt = dtmp[((size_t)n * 4 + o) * r + j];
      a = fmaf(wqv[o], dt, a);
      dw[o] = fmaf(dt, hh, dw[o]);
    }
    dh[(size_t)n * r + j] = a;
  }
  for (int o = 0; o < 4; ++o) dWqV[(size_t)o * r + j] = dw[o];
}

// dWq[o][k] = sum_j dWqV[o][j] V[k][j]; dV[k][j] = sum_o Wq[o][k] dWqV[o][j]
__global__ void vjp_leaf_qv_kernel(int d_o, int r, const float* __restrict__ Wq,
                                   const float* __restrict__ V, const float* __restrict__ dWqV,
                                   float* __restrict__ dWq, float* __restrict__ dV) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < 4 * d_o) {
    const int o = idx / d_o, k = idx % d_o;
    float a = 0.f;
    for (int j = 0; j < r; ++j) a = fmaf(dWqV[(size_t)o * r + j], V[(size_t)k * r + j], a);
    dWq[idx] = a;
  }
  if (idx < d_o * r) {
    const int k = idx / r, j = idx % r;
    float a = 0.f;
    for (int o = 0; o < 4; ++o) a = fmaf(Wq[o * d_o + k], dWqV[(size_t)o * r + j], a);
    dV[idx] = a;
  }
}

// ------------------------------------------------------------------ quadrilinear tag: two-Kronecker marginals
// The curvature block of the merge tensor (src/hamiltonzero/optim/spin_blocks.py:443-560)
// approximates the Fisher block of T [G, d_r, d_r, d_r] by sigma_left (x) sigma_right over the
// balanced axis split (i, j | k, l). With dy = d raw, a = u_left, b = u_right of one (walker, node)
// sample, viewed [G, d_r], and keep = 1 on MERGE nodes (the tag's structural mask):
//   sigma_left [(i,j),(I,J)] = sum_n keep (a_i . a_I)(b_i . b_I) dy[i,j] dy[I,J]
//   sigma_right[(k,l),(K,L)] = sum_n keep sum_i |dy_i|^2 a[i,k] a[i,K] b[i,l] b[i,L]
//   trace                    = sum_n keep sum_i |dy_i|^2 |a_i|^2 |b_i|^2,   count = sum_n keep
// (_two_kron_marginal_from_merge, _merge_gradient_trace, spin_blocks.py:140-171). Both marginals
// are accumulated as transposed GEMMs over rows that are generated a sub-chunk at a time.

// rows (sample n, group i) of X: sqrt(keep |dy_i|^2) * (a_i (x) b_i)        [S * G, d_r * d_r]
__global__ void __launch_bounds__(256)
vjp_mg_right_rows_kernel(int d, int G, int nodes, const uint8_t* __restrict__ opcodes,
                         const float* __restrict__ Uc, const float* __restrict__ dRAW, long long s0,
                         float* __restrict__ X) {
  __shared__ float a_s[32], b_s[32], w_s;
  const long long row = blockIdx.x;
  const long long n = s0 + row / G;
  const int i = (int)(row % G), node = (int)(n % nodes);
  const long long b = n / nodes;
  const int tid = threadIdx.x;
  if (tid < 32) {
    a_s[tid] = Uc[((size_t)b * 2 * nodes + 2 * node) * d + i * 32 + tid];
    b_s[tid] = Uc[((size_t)b * 2 * nodes + 2 * node + 1) * d + i * 32 + tid];
    const float y = dRAW[(size_t)n * d + i * 32 + tid];
    const float w = warp_sum(y * y);
    if (tid == 0) w_s = opcodes[node] == 0 ? sqrtf(w) : 0.f;
  }
  __syncthreads();
  const int k = tid >> 3, l0 = (tid & 7) * 4;
  const float ak = a_s[k] * w_s;
  *reinterpret_cast<float4*>(X + (size_t)row * 1024 + k * 32 + l0) =
      make_float4(ak * b_s[l0], ak * b_s[l0 + 1], ak * b_s[l0 + 2], ak * b_s[l0 + 3]);
}

// rows (sample n) of Z_I: keep (a_i . a_I)(b_i . b_I) dy[i, j]                 [S, d]
__global__ void __launch_bounds__(256)
vjp_mg_left_rows_kernel(int d, int G, int nodes, int I, const uint8_t* __restrict__ opcodes,
                        const float* __restrict__ Uc, const float* __restrict__ dRAW, long long s0,
                        float* __restrict__ Z) {
  extern __shared__ float m_s[];          // [G]
  const long long n = s0 + blockIdx.x;
  const int node = (int)(n % nodes);
  const long long b = n / nodes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float* ua = Uc + ((size_t)b * 2 * nodes + 2 * node) * d;
  const float* ub = ua + d;
  const float keep = opcodes[node] == 0 ? 1.f : 0.f;
  const float aI = ua[I * 32 + lane], bI = ub[I * 32 + lane];
  for (int i = warp; i < G; i += 8) {
    const float da = warp_sum(ua[i * 32 + lane] * aI), db = warp_sum(ub[i * 32 + lane] * bI);
    if (lane == 0) m_s[i] = keep * da * db;
  }
  __syncthreads();
  for (int c = tid; c < d; c += 256) Z[(size_t)blockIdx.x * d + c] = m_s[c >> 5] * dRAW[(size_t)n * d + c];
}

// stats[0] += trace, stats[1] += count, in a fixed order (one CTA)
__global__ void __launch_bounds__(1024)
vjp_mg_stats_kernel(int d, int G, int nodes, long long M, const uint8_t* __restrict__ opcodes,
                    const float* __restrict__ Uc, const float* __restrict__ dRAW, float* __restrict__ stats) {
  __shared__ double part[2][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  double tr = 0.0, cnt = 0.0;
  for (long long item = warp; item < M * G; item += 32) {
    const long long n = item / G;
    const int i = (int)(item % G), node = (int)(n % nodes);
    if (opcodes[node] != 0) continue;
    const long long b = n / nodes;
    const float a = Uc[((size_t)b * 2 * nodes + 2 * node) * d + i * 32 + lane];
    const float bb = Uc[((size_t)b * 2 * nodes + 2 * node + 1) * d + i * 32 + lane];
    const float y = dRAW[(size_t)n * d + i * 32 + lane];
    const float w = warp_sum(y * y), na = warp_sum(a * a), nb = warp_sum(bb * bb);
    tr += (double)w * (double)na * (double)nb;
    if (i == 0) cnt += 1.0;
  }
  if (lane == 0) { part[0][warp] = tr; part[1][warp] = cnt; }
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0, c = 0.0;
    for (int w = 0; w < 32; ++w) { t += part[0][w]; c += part[1][w]; }
    stats[0] += (float)t;
    stats[1] += (float)c;
  }
}

// A bounded device wait that ran out upstream leaves tiles unwritten. Like root_kernel on the
// forward path, the reverse pass then poisons what it returns: dq, log_abs and phase entirely,
// and the first element of every gradient and factor array.
struct VjpPoison {
  float* full[3];
  long long n_full[3];
  float* first[32];
  int n_first;
};
__global__ void vjp_poison_kernel(const int* __restrict__ status, VjpPoison p) {
  if (*status == 0) return;
  const float bad = __int_as_float(0x7fc00000);
  for (int a = 0; a < 3; ++a)
    if (p.full[a])
      for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.n_full[a];
           i += (long long)gridDim.x * blockDim.x)
        p.full[a][i] = bad;
  if (blockIdx.x == 0 && threadIdx.x < p.n_first) p.first[threadIdx.x][0] = bad;
}

// ------------------------------------------------------------------ host side
// HZ_VJP_L1=merge runs the first level of the reverse pass's forward sweep through the merge
// kernel like the other levels (A/B timing and debugging).
inline bool vjp_l1_coefficient_space() {
  static const bool enabled = !env_equals("HZ_VJP_L1", "merge");
  return enabled;
}

// the first level's backward in coefficient space as well (HZ_VJP_L1=forward keeps the merge
// backward kernel there); never with factor statistics, whose leaf moments need every du
inline bool vjp_l1_backward_coefficient_space() {
  static const bool enabled = vjp_l1_coefficient_space() && !env_equals("HZ_VJP_L1", "forward");
  return enabled;
}

struct VjpWorkspace {
  // once per call
  float *leaf_map, *leaf_tmp;
  float *vt_hi, *vt_lo, *ut_hi, *ut_lo, *rt_hi, *rt_lo;      // forward: weights transposed + split
  float *v_hi, *v_lo, *u_hi, *u_lo, *r_hi, *r_lo;            // backward: weights as stored, split
  float *Vt, *Ut, *Rt;                                       // backward, mma.sync path: transposes
  int* status;
  float *dM, *dtmp, *dWqV, *dT_part;
  float *l1_gs, *l1_fake, *l1_phi;   // first level in coefficient space: leaf Gram matrices, fake batch, basis
  int* l1_exp;
  float *l1_dphi, *l1_k, *l1_dfake;  // its backward: basis cotangent, per-site 4x4 sums, fake batch cotangent
  float *tp_packed[3], *tp_scale[3]; // the three arrangements of T for tprod_tc_kernel (FP16 head/tail, row scales)
  float *ta_packed, *ta_scale;       // the two views of T for tapply_tc_kernel and the group scales
  float* l1_D;                       // per chunk: <d raw, Phi> of every (walker, node)
  // per chunk
  float *U0, *S0, *dU0, *dS0;
  float *ZL, *VZL, *MIXL, *dMIXL, *dZL, *MIXR;               // factor statistics only
  float *lu_hi, *lu_lo, *LUt, *LVt;
  float* mg_buf;                 // generated rows of the two-Kronecker marginals (with_factors == 2)
  TnScratch tn;                  // partial tiles of the split A^T B products
  size_t mg_floats;
  float *RAW, *OUT, *VX, *MIX, *S, *dX, *dMIX, *dS, *dRAW;
  NormOut* nout;
  float *VR, *dVR, *dpsi;
  size_t bytes;
  int slices;
};

constexpr int kVjpSlices = 3;       // CTAs per group in merge_bwd_kernel (grid.y): 48 groups x 3 = one wave on 148 SMs

VjpWorkspace vjp_carve(const hz_wavefunction* w, long long Bc, int with_factors, char* base) {
  VjpWorkspace ws{};
  const size_t N = w->n_sites, d = w->d_m, r = w->r_merge, rl = w->r_leaf, rr = w->r_ro;
  const size_t G = d / kDr;
  size_t off = 0;
  auto take = [&](size_t nfloats) {
    float* p = base ? reinterpret_cast<float*>(base + off) : nullptr;
    off += align_up(nfloats * sizeof(float));
    return p;
  };
  ws.slices = kVjpSlices;
  ws.status = reinterpret_cast<int*>(take(64));        // first word of the workspace
  ws.leaf_map = take(N * 4 * d);
  ws.leaf_tmp = take(N * 4 * rl);
  ws.vt_hi = take(d * r); ws.vt_lo = take(d * r); ws.ut_hi = take(d * r); ws.ut_lo = take(d * r);
  ws.rt_hi = take(d * rr); ws.rt_lo = take(d * rr);
  ws.v_hi = take(d * r); ws.v_lo = take(d * r); ws.u_hi = take(d * r); ws.u_lo = take(d * r);
  ws.r_hi = take(d * rr); ws.r_lo = take(d * rr);
  ws.Vt = take(d * r); ws.Ut = take(d * r); ws.Rt = take(d * rr);
  ws.dM = take(N * 4 * d);
  ws.dtmp = take(N * 4 * rl);
  ws.dWqV = take(4 * rl);
  ws.dT_part = take((size_t)kVjpSlices * G * 32768);
  if (N > 1) {
    ws.l1_gs = take(N * 16);
    ws.l1_exp = reinterpret_cast<int*>(take(N * 4));
    ws.l1_fake = take(16 * N * d);
    ws.l1_phi = take(16 * (N / 2) * d);
    ws.l1_dphi = take(16 * (N / 2) * d);
    ws.l1_k = take(N * 16);
    ws.l1_dfake = take(16 * N * d);
    ws.l1_D = take((size_t)Bc * (N / 2) * 16);
    for (int i = 0; i < 3; ++i) {
      ws.tp_packed[i] = take(G * 32768);
      ws.tp_scale[i] = take(2 * G * 32);
    }
    ws.ta_packed = take(G * 65536);
    ws.ta_scale = take(G);
  }
  const size_t rows = (size_t)Bc * (N > 1 ? N - 1 : 1);     // all merge levels, level-major
  ws.U0 = take((size_t)Bc * N * d); ws.dU0 = take((size_t)Bc * N * d);
  ws.S0 = take((size_t)Bc * N); ws.dS0 = take((size_t)Bc * N);
  ws.RAW = take(rows * d); ws.OUT = take(rows * d); ws.dX = take(rows * d);
  ws.VX = take(rows * r); ws.MIX = take(rows * r); ws.dMIX = take(rows * r);
  ws.S = take(rows); ws.dS = take(rows);
  ws.nout = reinterpret_cast<NormOut*>(take(rows * 2));
  ws.dRAW = take((size_t)Bc * (N / 2 + 1) * d);
  ws.VR = take((size_t)Bc * rr); ws.dVR = take((size_t)Bc * rr); ws.dpsi = take((size_t)Bc * 2);
  if (with_factors) {
    const size_t d_o = w->d_o;
    ws.ZL = take((size_t)Bc * N * d_o); ws.dZL = take((size_t)Bc * N * d_o);
    ws.VZL = take((size_t)Bc * N * rl); ws.MIXL = take((size_t)Bc * N * rl);
    ws.dMIXL = take((size_t)Bc * N * rl);
    ws.MIXR = take((size_t)Bc * rr);
    ws.lu_hi = take(rl * d); ws.lu_lo = take(rl * d); ws.LUt = take(rl * d); ws.LVt = take(rl * d_o);
  }
  if (with_factors == 2 && N > 1) {
    // at most 128 MB, at least one sample's rows of either kind
    const size_t one = G * 1024 > d ? G * 1024 : d;
    const size_t all = (size_t)Bc * (N / 2) * one;
    ws.mg_floats = all < ((size_t)32 << 20) ? all : ((size_t)32 << 20);
    if (ws.mg_floats < one) ws.mg_floats = one;
    ws.mg_buf = take(ws.mg_floats);
  }
  // partial tiles of the split A^T B products: room for every shape used here at its full
  // split count (about 4 x 148 CTAs per product)
  {
    size_t widest = d > 1024 ? d : 1024;
    const size_t tiles = ((widest + kTnBM - 1) / kTnBM) * ((widest + kTnBN - 1) / kTnBN);
    ws.tn.floats = (4 * 148 + tiles) * (size_t)(kTnBM * kTnBN);
    ws.tn.p = take(ws.tn.floats);
  }
  ws.bytes = off;
  return ws;
}

int vjp_prepare(const hz_wavefunction* w, const VjpWorkspace& ws, bool with_factors, cudaStream_t stream) {
  HZ_CUDA_TRY(cudaMemsetAsync(ws.status, 0, sizeof(int), stream));
  const int N = w->n_sites, d = w->d_m, r = w->r_merge, rr = w->r_ro;
  dim3 blk(32, 8);
  auto split = [&](const float* x, float* hi, float* lo, long long n) {
    vjp_split_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, hi, lo, n);
  };
  if (N > 1 && use_tapply_tc()) {
    const int rc = tapply_prepare(w->merge_T, d / kDr, ws.ta_packed, ws.ta_scale, stream);
    if (rc != HZ_OK) return rc;
  } else if (N > 1 && use_tprod_tc()) {
    // ws.dT_part serves as scratch for the permuted copies; it is zeroed again below
    for (int arr = 0; arr < 3; ++arr) {
      const int rc = tprod_prepare(w->merge_T, d / kDr, arr, ws.dT_part, ws.tp_packed[arr], ws.tp_scale[arr], stream);
      if (rc != HZ_OK) return rc;
    }
    HZ_CUDA_TRY(cudaMemsetAsync(ws.dT_part, 0, (size_t)kVjpSlices * (d / kDr) * 32768 * sizeof(float), stream));
  }
  // the factor maps and their transposes on the FP16-split GEMM where every shape tiles (as in the
  // energy path), else on the three-term TF32 split
  const bool f16 = walker_gemm_f16(w);
  if (f16) {
    int rc = HZ_OK;
    if (N > 1) {
      rc = prepare_weights_f16(w->merge_V, ws.vt_hi, ws.vt_lo, d, r, true, stream);
      if (rc == HZ_OK) rc = prepare_weights_f16(w->merge_U, ws.ut_hi, ws.ut_lo, r, d, true, stream);
      // backward: dMIX = dX U^T and dRAW = dMIX V^T take the stored matrices as [N, K]
      if (rc == HZ_OK) rc = prepare_weights_f16(w->merge_U, ws.u_hi, ws.u_lo, d, r, false, stream);
      if (rc == HZ_OK) rc = prepare_weights_f16(w->merge_V, ws.v_hi, ws.v_lo, r, d, false, stream);
    }
    if (rc == HZ_OK) rc = prepare_weights_f16(w->readout_V, ws.rt_hi, ws.rt_lo, d, rr, true, stream);
    if (rc == HZ_OK) rc = prepare_weights_f16(w->readout_V, ws.r_hi, ws.r_lo, rr, d, false, stream);
    if (rc != HZ_OK) return rc;
  }
  if (N > 1 && !f16) {
    split_transpose_kernel<<<dim3((r + 31) / 32, (d + 31) / 32), blk, 0, stream>>>(w->merge_V, ws.vt_hi, ws.vt_lo, d, r);
    split_transpose_kernel<<<dim3((d + 31) / 32, (r + 31) / 32), blk, 0, stream>>>(w->merge_U, ws.ut_hi, ws.ut_lo, r, d);
    split(w->merge_V, ws.v_hi, ws.v_lo, (long long)d * r);
    split(w->merge_U, ws.u_hi, ws.u_lo, (long long)d * r);
  }
  if (N > 1) {
    vjp_transpose_kernel<<<dim3((r + 31) / 32, (d + 31) / 32), blk, 0, stream>>>(w->merge_V, ws.Vt, d, r);
    vjp_transpose_kernel<<<dim3((d + 31) / 32, (r + 31) / 32), blk, 0, stream>>>(w->merge_U, ws.Ut, r, d);
  }
  if (!f16) {
    split_transpose_kernel<<<dim3((rr + 31) / 32, (d + 31) / 32), blk, 0, stream>>>(w->readout_V, ws.rt_hi, ws.rt_lo, d, rr);
    split(w->readout_V, ws.r_hi, ws.r_lo, (long long)d * rr);
  }
  vjp_transpose_kernel<<<dim3((rr + 31) / 32, (d + 31) / 32), blk, 0, stream>>>(w->readout_V, ws.Rt, d, rr);
  if (with_factors) {
    const int rl = w->r_leaf, d_o = w->d_o;
    split(w->leaf_U, ws.lu_hi, ws.lu_lo, (long long)rl * d);
    vjp_transpose_kernel<<<dim3((d + 31) / 32, (rl + 31) / 32), blk, 0, stream>>>(w->leaf_U, ws.LUt, rl, d);
    vjp_transpose_kernel<<<dim3((rl + 31) / 32, (d_o + 31) / 32), blk, 0, stream>>>(w->leaf_V, ws.LVt, d_o, rl);
  }
  HZ_CUDA_TRY(cudaGetLastError());
  // leaf map (as prepare_leaf_map)
  const int total = N * 4 * w->r_leaf;
  leaf_tmp_kernel<<<(total + 255) / 256, 256, 0, stream>>>(w->q_weight, w->leaf_V, w->leaf_h, ws.leaf_tmp, N,
                                                           w->d_o, w->r_leaf);
  HZ_CUDA_TRY(cudaGetLastError());
  GemmArgs ga{};
  ga.A = ws.leaf_tmp; ga.B = w->leaf_U; ga.C = ws.leaf_map;
  ga.M = 4 * N; ga.N = d; ga.K = w->r_leaf; ga.lda = w->r_leaf; ga.ldb = d; ga.ldc = d;
  int st = launch_gemm(kEpiStore, ga, stream);
  if (st != HZ_OK || N == 1 || !vjp_l1_coefficient_space()) return st;
  // basis of the first level's raw rows, Phi_n[4o + o'] = T(M_left[o], M_right[o']), on a fake
  // batch of 16 walkers with every row scaled into the merge kernel's operand range
  leaf_gram_kernel<<<N, 128, 0, stream>>>(ws.leaf_map, ws.l1_gs, d);
  row_exponent_kernel<<<N * 4, 128, 0, stream>>>(ws.leaf_map, ws.l1_exp, d);
  l1_fake_kernel<<<dim3(N, 16), 256, 0, stream>>>(ws.leaf_map, ws.l1_exp, ws.l1_fake, N, d);
  HZ_CUDA_TRY(cudaGetLastError());
  Level L{};
  L.N = N; L.d = d; L.G = d / kDr; L.jets = 0; L.Bc = 16; L.nodes = N / 2; L.m = 3;
  L.rows_in = N; L.rows_out = N / 2;
  st = launch_tstage(L, w, nullptr, ws.l1_fake, ws.l1_phi, stream);
  if (st != HZ_OK) return st;
  fake_unscale_kernel<<<dim3(N / 2, 16), 256, 0, stream>>>(ws.l1_phi, ws.l1_exp, N / 2, 4, d);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// raw rows of the first level from the basis: a normalised leaf carrier is r (q . M_site) with
// r = (q G q / d + eps)^-1/2 (G the site's 4x4 Gram matrix of M_site), so
// raw[w, n] = r_L r_R sum_(o,o') q_L[o] q_R[o'] Phi_n[4o + o']. One CTA per (column block, node,
// group of walkers) keeps its 16 basis values per column in registers.
constexpr int kVjpL1Walkers = 16;
__global__ void __launch_bounds__(256)
vjp_l1_expand_kernel(int N, int d, int Bc, const float* __restrict__ q, const float* __restrict__ Gs,
                     const float* __restrict__ Phi, float* __restrict__ RAW) {
  __shared__ float coef[kVjpL1Walkers][16];
  const int n = blockIdx.y, nodes = N / 2, c = blockIdx.x * 256 + threadIdx.x;
  const int b0 = blockIdx.z * kVjpL1Walkers;
  if (threadIdx.x < kVjpL1Walkers * 2) {
    // thread (walker, side): the scaled quaternion r q of that leaf
    const int wk = threadIdx.x >> 1, side = threadIdx.x & 1, b = b0 + wk;
    float c4[4] = {0.f, 0.f, 0.f, 0.f};
    if (b < Bc) {
      const int site = 2 * n + side;
      const float4 qq = *reinterpret_cast<const float4*>(q + ((size_t)b * N + site) * 4);
      const float qv[4] = {qq.x, qq.y, qq.z, qq.w};
      const float* G = Gs + site * 16;
      float y = 0.f;
#pragma unroll
      for (int o = 0; o < 4; ++o)
#pragma unroll
        for (int p = 0; p < 4; ++p) y = fmaf(qv[o] * qv[p], G[o * 4 + p], y);
      const float r = rsqrtf(y / (float)d + kLeafEps);
#pragma unroll
      for (int o = 0; o < 4; ++o) c4[o] = r * qv[o];
    }
    // left leaf fills coef[wk][4o + o'] = cL[o] (to be multiplied by cR[o'] below)
    const float other0 = __shfl_xor_sync(0xffffffffu, c4[0], 1), other1 = __shfl_xor_sync(0xffffffffu, c4[1], 1);
    const float other2 = __shfl_xor_sync(0xffffffffu, c4[2], 1), other3 = __shfl_xor_sync(0xffffffffu, c4[3], 1);
    if (side == 0) {
      const float cr[4] = {other0, other1, other2, other3};
#pragma unroll
      for (int o = 0; o < 4; ++o)
#pragma unroll
        for (int p = 0; p < 4; ++p) coef[wk][o * 4 + p] = c4[o] * cr[p];
    }
  }
  __syncthreads();
  if (c >= d) return;
  float phi[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) phi[i] = Phi[((size_t)i * nodes + n) * d + c];
  for (int wk = 0; wk < kVjpL1Walkers && b0 + wk < Bc; ++wk) {
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc = fmaf(coef[wk][i], phi[i], acc);
    RAW[((size_t)(b0 + wk) * nodes + n) * d + c] = acc;
  }
}


// ------------------------------------------------------------------ first level, backward in coefficient space
// With raw[w, n] = sum_(o,o') cL[o] cR[o'] Phi_n[4o + o'] (c = r q the scaled quaternion of a
// leaf, u = c . M_site its carrier), the cotangent d raw of a merged first-level node reaches
// its two leaves only through D[o, o'] = <d raw, Phi_n[4o + o']>:
//   <M[o], du_L> = sum_o' D[o, o'] cR[o'],  <u_L, du_L> = <u_R, du_R> = E = sum cL[o] cR[o'] D[o, o'],
// so the leaf backward (dv = r (du - E u / d), dq = M dv, dM += q (x) dv) needs no per-walker
// tensor application:
//   dq_L[o] += r_L (sum_o' D[o, o'] cR[o'] - (E / d) (G_L c_L)[o])        (G = M M^T, 4 x 4)
//   dM_L    += K_L M_L with K_L = -sum_w (E / d) c_L (x) c_L, and the d raw (x) u_R part through
//   dPhi_n[4o + o'] = sum_w cL[o] cR[o'] d raw, which the merge backward takes through the same
//   fake batch that built Phi (it also gives this level's share of dT).
// The leaf's scale cotangent dS0 enters the same way (-E becomes dS0 - E). The leaves of carried
// (gated) parents stay with vjp_leaf_bwd_kernel, which skips the leaves of merged parents. Not
// used when factor statistics are asked for: their leaf output moment needs every walker's du.
constexpr int kVjpL1Slices = 8;

// D[b, n, 0..16): four walkers per warp share the basis loads
__global__ void __launch_bounds__(256)
vjp_l1_dots_kernel(int nodes, int d, int Bc, const uint8_t* __restrict__ opcodes, const float* __restrict__ dRAW,
                   const float* __restrict__ Phi, float* __restrict__ D) {
  const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b0 = (blockIdx.y * 8 + warp) * 4;
  if (b0 >= Bc) return;
  float acc[4][16];
#pragma unroll
  for (int w = 0; w < 4; ++w)
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[w][i] = 0.f;
  if (opcodes[n] == 0) {
    const float* rows[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const int b = b0 + w < Bc ? b0 + w : Bc - 1;
      rows[w] = dRAW + ((size_t)b * nodes + n) * d;
    }
    for (int c = lane; c < d; c += 32) {
      float x[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) x[w] = rows[w][c];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float phi = Phi[((size_t)i * nodes + n) * d + c];
#pragma unroll
        for (int w = 0; w < 4; ++w) acc[w][i] = fmaf(x[w], phi, acc[w][i]);
      }
    }
#pragma unroll
    for (int w = 0; w < 4; ++w)
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[w][i] = warp_sum(acc[w][i]);
  }
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    float out = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) out = lane == i ? acc[w][i] : out;
    if (lane < 16 && b0 + w < Bc) D[((size_t)(b0 + w) * nodes + n) * 16 + lane] = out;
  }
}

// scaled quaternion c = r q of leaf `site` of walker b
__device__ __forceinline__ void vjp_l1_leaf_coef(const float* __restrict__ q, const float* __restrict__ Gs, int N,
                                                 int d, int b, int site, float (&c4)[4], float& r) {
  const float4 qq = *reinterpret_cast<const float4*>(q + ((size_t)b * N + site) * 4);
  const float qv[4] = {qq.x, qq.y, qq.z, qq.w};
  const float* G = Gs + site * 16;
  float y = 0.f;
#pragma unroll
  for (int o = 0; o < 4; ++o)
#pragma unroll
    for (int p = 0; p < 4; ++p) y = fmaf(qv[o] * qv[p], G[o * 4 + p], y);
  r = rsqrtf(y / (float)d + kLeafEps);
#pragma unroll
  for (int o = 0; o < 4; ++o) c4[o] = r * qv[o];
}

// part[s][i][n][c] = sum over the walkers of slice s of cL[o] cR[o'] d raw[w, n, c]
__global__ void __launch_bounds__(256)
vjp_l1_dphi_kernel(int N, int d, int Bc, const uint8_t* __restrict__ opcodes, const float* __restrict__ q,
                   const float* __restrict__ Gs, const float* __restrict__ dRAW, float* __restrict__ part) {
  __shared__ float coef[256][16];
  const int n = blockIdx.y, nodes = N / 2, c = blockIdx.x * 256 + threadIdx.x;
  const int s = blockIdx.z, S = gridDim.z;
  const int bs = (int)((long long)Bc * s / S), be = (int)((long long)Bc * (s + 1) / S);
  const bool merged = opcodes[n] == 0;
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  for (int t0 = bs; t0 < be && merged; t0 += 256) {
    const int cnt = be - t0 < 256 ? be - t0 : 256;
    __syncthreads();
    if ((int)threadIdx.x < cnt) {
      float cl[4], cr[4], rl_, rr_;
      vjp_l1_leaf_coef(q, Gs, N, d, t0 + threadIdx.x, 2 * n, cl, rl_);
      vjp_l1_leaf_coef(q, Gs, N, d, t0 + threadIdx.x, 2 * n + 1, cr, rr_);
#pragma unroll
      for (int o = 0; o < 4; ++o)
#pragma unroll
        for (int p = 0; p < 4; ++p) coef[threadIdx.x][o * 4 + p] = cl[o] * cr[p];
    }
    __syncthreads();
    if (c < d) {
      for (int wk = 0; wk < cnt; ++wk) {
        const float x = dRAW[((size_t)(t0 + wk) * nodes + n) * d + c];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = fmaf(coef[wk][i], x, acc[i]);
      }
    }
  }
  if (c < d)
#pragma unroll
    for (int i = 0; i < 16; ++i) part[(((size_t)s * 16 + i) * nodes + n) * d + c] = acc[i];
}

// dst[idx] += sum_s part[s][idx], slices in order
__global__ void vjp_l1_reduce_kernel(long long total, int S, const float* __restrict__ part, float* __restrict__ dst) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  float a = 0.f;
  for (int s = 0; s < S; ++s) a += part[(size_t)s * total + idx];
  dst[idx] += a;
}

// the leaves of merged first-level nodes: dq += ..., Kpart[s][site][16] = -sum_w (E / d) c (x) c
__global__ void __launch_bounds__(256)
vjp_l1_leaf_kernel(int N, int d, int Bc, const uint8_t* __restrict__ opcodes, const float* __restrict__ q,
                   const float* __restrict__ Gs, const float* __restrict__ D, const float* __restrict__ dS0,
                   float* __restrict__ dq /* nullable; written, not added to */, float* __restrict__ Kpart) {
  __shared__ float scratch[32 * 8];
  const int n = blockIdx.x, s = blockIdx.y, S = gridDim.y, nodes = N / 2;
  const int bs = (int)((long long)Bc * s / S), be = (int)((long long)Bc * (s + 1) / S);
  float k[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) k[i] = 0.f;
  if (opcodes[n] == 0) {
    for (int b = bs + threadIdx.x; b < be; b += 256) {
      float c2[2][4], r2[2];
      vjp_l1_leaf_coef(q, Gs, N, d, b, 2 * n, c2[0], r2[0]);
      vjp_l1_leaf_coef(q, Gs, N, d, b, 2 * n + 1, c2[1], r2[1]);
      float Dv[16];
      const float4* Dp = reinterpret_cast<const float4*>(D + ((size_t)b * nodes + n) * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 v = Dp[i];
        Dv[4 * i] = v.x; Dv[4 * i + 1] = v.y; Dv[4 * i + 2] = v.z; Dv[4 * i + 3] = v.w;
      }
      float dc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, E = 0.f;
#pragma unroll
      for (int o = 0; o < 4; ++o)
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          dc[0][o] = fmaf(Dv[o * 4 + p], c2[1][p], dc[0][o]);
          dc[1][p] = fmaf(Dv[o * 4 + p], c2[0][o], dc[1][p]);
          E = fmaf(c2[0][o] * c2[1][p], Dv[o * 4 + p], E);
        }
#pragma unroll
      for (int side = 0; side < 2; ++side) {
        const int site = 2 * n + side;
        // the leaf's scale cotangent enters like -E: dv = r (du + (dS0 - <u, du>) u / d)
        const float coef = (dS0[(size_t)b * N + site] - E) / (float)d;
        const float* G = Gs + site * 16;
        float g4[4];
#pragma unroll
        for (int o = 0; o < 4; ++o) {
          float gc = 0.f;
#pragma unroll
          for (int p = 0; p < 4; ++p) gc = fmaf(G[o * 4 + p], c2[side][p], gc);
          g4[o] = r2[side] * (dc[side][o] + coef * gc);
#pragma unroll
          for (int p = 0; p < 4; ++p) k[side * 16 + o * 4 + p] = fmaf(coef * c2[side][o], c2[side][p], k[side * 16 + o * 4 + p]);
        }
        if (dq) *reinterpret_cast<float4*>(dq + ((size_t)b * N + site) * 4) = make_float4(g4[0], g4[1], g4[2], g4[3]);
      }
    }
  }
  block_sum<32, 256>(k, scratch);
  if (threadIdx.x == 0) {
    float* dst = Kpart + ((size_t)s * N + 2 * n) * 16;
#pragma unroll
    for (int i = 0; i < 32; ++i) dst[i] = k[i];
  }
}

// dM[site][o] += 2^-e[site, o] sum over the fake walkers whose leaf `site` is M_site[o] of their
// carrier cotangent, + sum_o' K[site][o][o'] M[site][o']
__global__ void __launch_bounds__(256)
vjp_l1_fold_kernel(int N, int d, const float* __restrict__ dfake, const int* __restrict__ expo,
                   const float* __restrict__ K, const float* __restrict__ M, float* __restrict__ dM) {
  const int site = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
  if (c >= d) return;
  float m[4];
#pragma unroll
  for (int o = 0; o < 4; ++o) m[o] = M[((size_t)site * 4 + o) * d + c];
#pragma unroll
  for (int o = 0; o < 4; ++o) {
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int wk = (site & 1) ? (j * 4 + o) : (o * 4 + j);
      a += dfake[((size_t)wk * N + site) * d + c];
    }
    a = ldexpf(a, -expo[site * 4 + o]);
#pragma unroll
    for (int p = 0; p < 4; ++p) a = fmaf(K[site * 16 + o * 4 + p], m[p], a);
    dM[((size_t)site * 4 + o) * d + c] += a;
  }
}

// slices of the per-chunk reductions that fit the scratch of the transposed GEMMs
inline int vjp_l1_slices(const hz_wavefunction* w, const TnScratch& scratch) {
  const size_t per = (size_t)16 * (w->n_sites / 2) * w->d_m;
  const size_t fit = scratch.floats / per;
  return (int)(fit < (size_t)kVjpL1Slices ? fit : (size_t)kVjpL1Slices);
}

// per chunk, in place of merge_bwd_kernel at the first level (dRAW = ws.dRAW of that level)
int vjp_l1_backward_chunk(const hz_wavefunction* w, const float* qc, long long Bc, const float* dRAW,
                          const float* dS0, float* dq, const TnScratch& scratch, float* D, const float* Gs,
                          const float* Phi, float* dphi, float* Ksum, cudaStream_t stream) {
  const int N = w->n_sites, d = w->d_m, nodes = N / 2;
  const int S = vjp_l1_slices(w, scratch);
  if (S < 1) return HZ_ERR_WORKSPACE;
  vjp_l1_dots_kernel<<<dim3(nodes, (unsigned)((Bc + 31) / 32)), 256, 0, stream>>>(nodes, d, (int)Bc, w->opcodes, dRAW,
                                                                                  Phi, D);
  vjp_l1_leaf_kernel<<<dim3(nodes, S), 256, 0, stream>>>(N, d, (int)Bc, w->opcodes, qc, Gs, D, dS0, dq, scratch.p);
  HZ_CUDA_TRY(cudaGetLastError());
  if (!dphi) {      // carrier cotangents only: no parameter gradients
    HZ_CUDA_TRY(cudaGetLastError());
    return HZ_OK;
  }
  vjp_l1_reduce_kernel<<<(N * 16 + 255) / 256, 256, 0, stream>>>((long long)N * 16, S, scratch.p, Ksum);
  vjp_l1_dphi_kernel<<<dim3((d + 255) / 256, nodes, S), 256, 0, stream>>>(N, d, (int)Bc, w->opcodes, qc, Gs, dRAW,
                                                                          scratch.p);
  HZ_CUDA_TRY(cudaGetLastError());
  const long long total = (long long)16 * nodes * d;
  vjp_l1_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(total, S, scratch.p, dphi);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// log of the leaf carriers' RMS from the sites' Gram matrices: s = log sqrt(q G q / d + eps)
__global__ void vjp_leaf_s0_kernel(int N, int d, long long leaves, const float* __restrict__ q,
                                   const float* __restrict__ Gs, float* __restrict__ S0) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // (walker, site)
  if (idx >= leaves) return;
  const int site = (int)(idx % N);
  const float4 qq = *reinterpret_cast<const float4*>(q + idx * 4);
  const float qv[4] = {qq.x, qq.y, qq.z, qq.w};
  const float* G = Gs + site * 16;
  float y = 0.f;
#pragma unroll
  for (int o = 0; o < 4; ++o)
#pragma unroll
    for (int p = 0; p < 4; ++p) y = fmaf(qv[o] * qv[p], G[o * 4 + p], y);
  S0[idx] = 0.5f * logf(y / (float)d + kLeafEps);
}

struct VjpOut {
  const hz_wavefunction_grads* g;
  const hz_kfac_factors* f;
  float* dq;
  float* log_abs;
  float* phase;
};

// ------------------------------------------------------------------ KFAC factor statistics
// Second moments of the inputs x and output cotangents dy of every tagged dense layer of
// call_tagged (compiled/model.py:179-310), summed over the walkers (and, for the factors
// shared by all merge levels, over levels and nodes) under the tags' structural masks - the
// sums that StructuralRepeatedDenseKroneckerFactored.update_curvature_matrix_estimate
// (src/hamiltonzero/optim/blocks.py:1122-1204) divides by its batch sizes - and the squared
// per-walker gradients of the scale tags (blocks.py:1288-1415). Output-side moments need no
// mask: the cotangent of a gated node or a padded leaf is exactly zero.

// per (walker, site): z = q Wq, vz = z V_l, mixed = vz * h_site, all zero for padded leaves
__global__ void __launch_bounds__(128)
vjp_leaf_acts_kernel(int N, int d_o, int rl, const float* __restrict__ q, const float* __restrict__ Wq,
                     const float* __restrict__ V, const float* __restrict__ h,
                     const uint8_t* __restrict__ mask, float* __restrict__ ZL, float* __restrict__ VZL,
                     float* __restrict__ MIXL) {
  const int n = blockIdx.x, b = blockIdx.y;
  const size_t row = (size_t)b * N + n;
  const float keep = (mask == nullptr || mask[n]) ? 1.f : 0.f;
  const float4 qq = *reinterpret_cast<const float4*>(q + row * 4);
  __shared__ float z[256];
  for (int k = threadIdx.x; k < d_o; k += 128) {
    const float v = qq.x * Wq[k] + qq.y * Wq[d_o + k] + qq.z * Wq[2 * d_o + k] + qq.w * Wq[3 * d_o + k];
    if (k < 256) z[k] = v;
    ZL[row * d_o + k] = keep * v;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < rl; j += 128) {
    float vz = 0.f;
    for (int k = 0; k < d_o; ++k) vz = fmaf(z[k], V[(size_t)k * rl + j], vz);
    VZL[row * rl + j] = keep * vz;
    MIXL[row * rl + j] = keep * vz * h[(size_t)n * rl + j];
  }
}

// C [M, M] += sum_rows keep(row) x x^T for M <= 4 (one CTA)
__global__ void __launch_bounds__(256)
vjp_small_gram_kernel(const float* __restrict__ X, long long rows, int M, const uint8_t* __restrict__ mask,
                      int period, float* __restrict__ C) {
  __shared__ float part_s[8][16];
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  for (long long row = threadIdx.x; row < rows; row += 256) {
    if (mask != nullptr && !mask[row % period]) continue;
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < M; ++i) x[i] = X[row * M + i];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i * 4 + j] = fmaf(x[i], x[j], acc[i * 4 + j]);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float v = warp_sum(acc[i]);
    if ((threadIdx.x & 31) == 0) part_s[threadIdx.x >> 5][i] = v;
  }
  __syncthreads();
  if (threadIdx.x < 16) {
    const int i = threadIdx.x >> 2, j = threadIdx.x & 3;
    float v = 0.f;
    for (int w = 0; w < 8; ++w) v += part_s[w][threadIdx.x];      // warp order: reproducible
    if (i < M && j < M) C[i * M + j] += v;
  }
}

// lower triangle <- upper triangle
__global__ void vjp_symmetrize_kernel(float* __restrict__ C, int M) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)M * M) return;
  const int i = (int)(idx / M), j = (int)(idx % M);
  if (i > j) C[idx] = C[(size_t)j * M + i];
}

int vjp_factor_statistics(const hz_wavefunction* w, const float* qc, long long Bc, const float* u_root,
                          long long rows_all, const VjpOut& o, const VjpWorkspace& ws, cudaStream_t stream) {
  const hz_kfac_factors* f = o.f;
  const int N = w->n_sites, d = w->d_m, r = w->r_merge, rl = w->r_leaf, rr = w->r_ro, d_o = w->d_o;
  int st = HZ_OK;
  auto gram = [&](const float* X, long long rows, int M, float* C) {
    if (C == nullptr || st != HZ_OK) return;
    st = launch_gemm_tn(X, X, C, rows, M, M, M, M, M, true, ws.tn, stream);
  };
  if (N > 1) {
    gram(ws.RAW, rows_all, d, f->merge_V_in);
    gram(ws.dMIX, rows_all, r, f->merge_V_out);
    gram(ws.MIX, rows_all, r, f->merge_U_in);
    gram(ws.dX, rows_all, d, f->merge_U_out);
  }
  gram(u_root, Bc, d, f->readout_V_in);
  gram(ws.dVR, Bc, rr, f->readout_V_out);
  if (f->readout_U_in) {
    vjp_scale_kernel<<<(unsigned)((Bc * rr + 255) / 256), 256, 0, stream>>>(ws.VR, w->readout_h, ws.MIXR, Bc * rr, 1, rr);
    gram(ws.MIXR, Bc, rr, f->readout_U_in);
  }
  if (f->readout_U_out)
    vjp_small_gram_kernel<<<1, 256, 0, stream>>>(ws.dpsi, Bc, 2, nullptr, 1, f->readout_U_out);
  if (st != HZ_OK) return st;
  // leaves
  const long long rows0 = Bc * N;
  vjp_leaf_acts_kernel<<<dim3(N, (unsigned)Bc), 128, 0, stream>>>(N, d_o, rl, qc, w->q_weight, w->leaf_V, w->leaf_h,
                                                                 f->leaf_mask, ws.ZL, ws.VZL, ws.MIXL);
  HZ_CUDA_TRY(cudaGetLastError());
  {
    GemmArgs g{};
    g.A = ws.dU0; g.B = ws.LUt; g.C = ws.dMIXL; g.M = (int)rows0; g.N = rl; g.K = d;
    g.lda = d; g.ldb = rl; g.ldc = rl;
    st = gemm_dispatch(kEpiStore, g, ws.lu_hi, ws.lu_lo, ws.status, stream);
    if (st != HZ_OK) return st;
  }
  st = launch_hscale_bwd(rl, N, (int)Bc, w->leaf_h, ws.VZL, ws.dMIXL, nullptr, f->leaf_h_diag, ws.tn, stream);
  if (st != HZ_OK) return st;
  {
    GemmArgs g{};
    g.A = ws.dMIXL; g.B = ws.LVt; g.C = ws.dZL; g.M = (int)rows0; g.N = d_o; g.K = rl;
    g.lda = rl; g.ldb = d_o; g.ldc = d_o;
    st = launch_gemm(kEpiStore, g, stream);
    if (st != HZ_OK) return st;
  }
  gram(ws.MIXL, rows0, rl, f->leaf_U_in);
  gram(ws.dU0, rows0, d, f->leaf_U_out);
  gram(ws.ZL, rows0, d_o, f->leaf_V_in);
  gram(ws.dMIXL, rows0, rl, f->leaf_V_out);
  gram(ws.dZL, rows0, d_o, f->q_out);
  if (f->q_in)
    vjp_small_gram_kernel<<<1, 256, 0, stream>>>(qc, rows0, 4, f->leaf_mask, N, f->q_in);
  HZ_CUDA_TRY(cudaGetLastError());
  return st;
}


int vjp_chunk(const hz_wavefunction* w, const float* q, const float* cot_abs, const float* cot_phase,
              long long b0, long long Bc, const VjpOut& o, const VjpWorkspace& ws, cudaStream_t stream) {
  const int N = w->n_sites, d = w->d_m, G = d / kDr, r = w->r_merge, rr = w->r_ro;
  const float* qc = q + (size_t)b0 * N * 4;
  Level L{};
  L.N = N; L.d = d; L.G = G; L.jets = 0; L.Bc = (int)Bc;
  // ---------------- forward, values only, everything kept
  L.nodes = N; L.m = 0; L.rows_in = 0; L.rows_out = N;
  // with the first level in coefficient space in both directions nothing reads the carriers of the
  // leaves of merged parents: only their log scale is needed, and it comes from the Gram matrices
  const bool l1_all = N > 1 && !o.f && vjp_l1_backward_coefficient_space() && vjp_l1_slices(w, ws.tn) >= 1;
  if (l1_all) {
    const long long leaves = Bc * N;
    vjp_leaf_s0_kernel<<<(unsigned)((leaves + 255) / 256), 256, 0, stream>>>(N, d, leaves, qc, ws.l1_gs, ws.S0);
  }
  leaf_kernel<<<dim3(N, (unsigned)Bc), kLeafThreads, 0, stream>>>(L, qc, ws.leaf_map, nullptr, ws.U0, ws.S0,
                                                                 nullptr, nullptr, l1_all ? w->opcodes : nullptr);
  HZ_CUDA_TRY(cudaGetLastError());
  const float* prev_u = ws.U0;
  const float* prev_s = ws.S0;
  size_t row_off = 0, h_off = 0, op_off = 0;
  int levels = 0;
  size_t lvl_row[16], lvl_h[16], lvl_op[16];
  for (int nodes = N / 2; nodes >= 1; nodes /= 2, ++levels) {
    lvl_row[levels] = row_off; lvl_h[levels] = h_off; lvl_op[levels] = op_off;
    L.nodes = nodes; L.m = 3; L.rows_in = 2 * nodes; L.rows_out = nodes;
    const long long M = Bc * nodes;
    float* RAW = ws.RAW + row_off * d;
    float* OUT = ws.OUT + row_off * d;
    float* VX = ws.VX + row_off * r;
    float* MIX = ws.MIX + row_off * r;
    int st = HZ_OK;
    if (levels == 0 && vjp_l1_coefficient_space()) {
      vjp_l1_expand_kernel<<<dim3((d + 255) / 256, nodes, (unsigned)((Bc + kVjpL1Walkers - 1) / kVjpL1Walkers)),
                             256, 0, stream>>>(N, d, (int)Bc, qc, ws.l1_gs, ws.l1_phi, RAW);
      HZ_CUDA_TRY(cudaGetLastError());
    } else if (use_tapply_tc()) {
      // raw = A_R u_L, A_R from u_R: children rows 2p, 2p + 1 of the level below, parent row p
      TapplyArgs ta{prev_u, prev_u, RAW, 2, 1, 2, 0, 1, 0, M, nodes, nullptr, d, ws.ta_scale, 0};
      st = launch_tapply(0, ta, G, ws.ta_packed, ws.status, stream);
    } else if (use_tprod_tc()) {
      // raw = T(u_L, u_R): children rows 2p, 2p + 1 of the level below, parent row p
      TprodArgs ta{prev_u, prev_u, RAW, 2, 0, 2, 1, 1, 0, M, nodes, nullptr, d, ws.tp_scale[0]};
      st = launch_tprod(ta, G, ws.tp_packed[0], ws.status, stream);
    } else {
      st = launch_tstage(L, w, nullptr, prev_u, RAW, stream);
    }
    if (st != HZ_OK) return st;
    GemmArgs g1{};
    g1.A = RAW; g1.B = w->merge_V; g1.C = VX; g1.M = (int)M; g1.N = r; g1.K = d;
    g1.lda = d; g1.ldb = r; g1.ldc = r;
    st = gemm_dispatch(kEpiStore, g1, ws.vt_hi, ws.vt_lo, ws.status, stream, walker_gemm_f16(w));
    if (st != HZ_OK) return st;
    vjp_scale_kernel<<<(unsigned)((M * r + 255) / 256), 256, 0, stream>>>(VX, w->merge_h + h_off, MIX, M * r,
                                                                          nodes, r);
    HZ_CUDA_TRY(cudaMemcpyAsync(OUT, RAW, (size_t)M * d * sizeof(float), cudaMemcpyDeviceToDevice, stream));
    GemmArgs g2{};
    g2.A = MIX; g2.B = w->merge_U; g2.C = OUT; g2.R = OUT; g2.M = (int)M; g2.N = d; g2.K = r;
    g2.lda = r; g2.ldb = d; g2.ldc = d;
    st = gemm_dispatch(kEpiResidual, g2, ws.ut_hi, ws.ut_lo, ws.status, stream, walker_gemm_f16(w));
    if (st != HZ_OK) return st;
    if (d <= kNvMaxD) {
      norm_values_kernel<<<(unsigned)((M + 7) / 8), 256, 0, stream>>>(
          d, nodes, M, w->merge_eps, w->opcodes + op_off, prev_u, OUT, prev_s, ws.S + row_off, ws.nout + row_off);
    } else {
      const size_t smem_r = ((size_t)kNrColsWide + 2 * 16 + 3 * kNrWarps + 8) * sizeof(float);
      norm_reduce_kernel<kNrColsWide, false><<<dim3(nodes, (unsigned)Bc), kNrThreads, smem_r, stream>>>(
          L, w->merge_eps, nullptr, w->opcodes + op_off, OUT, prev_s, nullptr, nullptr, ws.S + row_off,
          nullptr, nullptr, ws.nout + row_off, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
      norm_apply_kernel<<<dim3((d + kNaThreads - 1) / kNaThreads, nodes, (unsigned)Bc), kNaThreads,
                          2 * (size_t)(2 * L.m + 1) * sizeof(float), stream>>>(
          L, w->opcodes + op_off, prev_u, OUT, ws.nout + row_off, nullptr, nullptr);
    }
    HZ_CUDA_TRY(cudaGetLastError());
    prev_u = OUT; prev_s = ws.S + row_off;
    row_off += (size_t)M; h_off += (size_t)nodes * r; op_off += nodes;
  }
  // root readout
  {
    GemmArgs g1{};
    g1.A = prev_u; g1.B = w->readout_V; g1.C = ws.VR; g1.M = (int)Bc; g1.N = rr; g1.K = d;
    g1.lda = d; g1.ldb = rr; g1.ldc = rr;
    int st = gemm_dispatch(kEpiStore, g1, ws.rt_hi, ws.rt_lo, ws.status, stream, walker_gemm_f16(w));
    if (st != HZ_OK) return st;
  }
  // ---------------- backward
  const bool l1_bwd = levels > 0 && !o.f && vjp_l1_backward_coefficient_space() && vjp_l1_slices(w, ws.tn) >= 1;
  float* dX_top = levels ? ws.dX + lvl_row[levels - 1] * d : ws.dU0;
  float* dS_top = levels ? ws.dS + lvl_row[levels - 1] : ws.dS0;
  vjp_root_kernel<<<(unsigned)Bc, 128, 0, stream>>>(rr, ws.VR, w->readout_h, w->readout_U, prev_s,
                                                    cot_abs + b0, cot_phase + b0, ws.dVR, ws.dpsi, dS_top,
                                                    o.log_abs ? o.log_abs + b0 : nullptr,
                                                    o.phase ? o.phase + b0 : nullptr);
  if (o.g)
    vjp_root_param_kernel<<<(rr + 127) / 128, 128, 0, stream>>>(rr, (int)Bc, ws.VR, w->readout_h, w->readout_U,
                                                              ws.dpsi, o.g->readout_U, o.g->readout_h,
                                                              o.f ? o.f->readout_h_diag : nullptr);
  HZ_CUDA_TRY(cudaGetLastError());
  {
    GemmArgs g{};
    g.A = ws.dVR; g.B = ws.Rt; g.C = dX_top; g.M = (int)Bc; g.N = d; g.K = rr;
    g.lda = rr; g.ldb = d; g.ldc = d;
    int st = gemm_dispatch(kEpiStore, g, ws.r_hi, ws.r_lo, ws.status, stream, walker_gemm_f16(w));
    if (st != HZ_OK) return st;
    if (o.g) st = launch_gemm_tn(prev_u, ws.dVR, o.g->readout_V, Bc, d, rr, d, rr, rr, false, ws.tn, stream);
    if (st != HZ_OK) return st;
  }
  for (int lv = levels - 1; lv >= 0; --lv) {
    const int nodes = N >> (lv + 1);
    const long long M = Bc * nodes;
    L.nodes = nodes; L.m = 3; L.rows_in = 2 * nodes; L.rows_out = nodes;
    const size_t ro = lvl_row[lv];
    float* dX = ws.dX + ro * d;
    float* dUc = lv ? ws.dX + lvl_row[lv - 1] * d : ws.dU0;
    float* dSc = lv ? ws.dS + lvl_row[lv - 1] : ws.dS0;
    const float* Uc = lv ? ws.OUT + lvl_row[lv - 1] * d : ws.U0;
    // leaves of merged parents get no carrier cotangent on this path; only the leaf-map gradient
    // kernel still reads their rows
    if (lv == 0 && l1_bwd && o.g)
      HZ_CUDA_TRY(cudaMemsetAsync(ws.dU0, 0, (size_t)Bc * N * d * sizeof(float), stream));
    vjp_norm_bwd_kernel<<<(unsigned)((M + 7) / 8), 256, 0, stream>>>(
        d, nodes, w->opcodes + lvl_op[lv], ws.OUT + ro * d, ws.nout + ro, dX, ws.dS + ro, dUc, dSc,
        ws.RAW + ro * d, ws.MIX + ro * r, r, M);
    HZ_CUDA_TRY(cudaGetLastError());
    GemmArgs g1{};
    g1.A = dX; g1.B = ws.Ut; g1.C = ws.dMIX + ro * r; g1.M = (int)M; g1.N = r; g1.K = d;
    g1.lda = d; g1.ldb = r; g1.ldc = r;
    int st = gemm_dispatch(kEpiStore, g1, ws.u_hi, ws.u_lo, ws.status, stream, walker_gemm_f16(w));
    if (st != HZ_OK) return st;
    st = launch_hscale_bwd(r, nodes, (int)Bc, w->merge_h + lvl_h[lv], ws.VX + ro * r, ws.dMIX + ro * r,
                           o.g ? o.g->merge_h + lvl_h[lv] : nullptr,
                           (o.f && o.f->merge_h_diag) ? o.f->merge_h_diag + lvl_h[lv] : nullptr, ws.tn, stream);
    if (st != HZ_OK) return st;
    GemmArgs g2{};
    g2.A = ws.dMIX + ro * r; g2.B = ws.Vt; g2.C = ws.dRAW; g2.R = dX; g2.M = (int)M; g2.N = d; g2.K = r;
    g2.lda = r; g2.ldb = d; g2.ldc = d;
    st = gemm_dispatch(kEpiResidual, g2, ws.v_hi, ws.v_lo, ws.status, stream, walker_gemm_f16(w));
    if (st != HZ_OK) return st;
    if (o.f && ws.mg_buf && (o.f->merge_T_left || o.f->merge_T_right)) {
      const uint8_t* ops = w->opcodes + lvl_op[lv];
      if (o.f->merge_T_right) {
        const long long per = (long long)(ws.mg_floats / ((size_t)G * 1024));       // samples per sub-chunk
        for (long long s0 = 0; s0 < M; s0 += per) {
          const long long S = M - s0 < per ? M - s0 : per;
          vjp_mg_right_rows_kernel<<<(unsigned)(S * G), 256, 0, stream>>>(d, G, nodes, ops, Uc, ws.dRAW, s0, ws.mg_buf);
          HZ_CUDA_TRY(cudaGetLastError());
          st = launch_gemm_tn(ws.mg_buf, ws.mg_buf, o.f->merge_T_right, S * G, 1024, 1024, 1024, 1024, 1024, true, ws.tn, stream);
          if (st != HZ_OK) return st;
        }
      }
      if (o.f->merge_T_left) {
        const long long per = (long long)(ws.mg_floats / (size_t)d);
        for (long long s0 = 0; s0 < M; s0 += per) {
          const long long S = M - s0 < per ? M - s0 : per;
          for (int I = 0; I < G; ++I) {
            vjp_mg_left_rows_kernel<<<(unsigned)S, 256, G * sizeof(float), stream>>>(d, G, nodes, I, ops, Uc, ws.dRAW,
                                                                                    s0, ws.mg_buf);
            HZ_CUDA_TRY(cudaGetLastError());
            st = launch_gemm_tn(ws.mg_buf, ws.dRAW + (size_t)s0 * d + I * 32, o.f->merge_T_left + I * 32, S, d, 32, d,
                                d, d, false, ws.tn, stream);
            if (st != HZ_OK) return st;
          }
        }
      }
      if (o.f->merge_T_stats) {
        vjp_mg_stats_kernel<<<1, 1024, 0, stream>>>(d, G, nodes, M, ops, Uc, ws.dRAW, o.f->merge_T_stats);
        HZ_CUDA_TRY(cudaGetLastError());
      }
    }
    if (lv == 0 && l1_bwd) continue;       // vjp_l1_backward_chunk below, after the leaf kernels
    const size_t smem = kTsSmemFloats * sizeof(float);
    if (o.g) {
      int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(merge_bwd_kernel<true>), (int)smem);
      if (rc != HZ_OK) return rc;
      const int with_du = use_tapply_tc() ? 0 : 1;
      merge_bwd_kernel<true><<<dim3(G, kVjpSlices), kTsThreads, smem, stream>>>(
          L, w->merge_T, w->opcodes + lvl_op[lv], Uc, ws.dRAW, dUc, ws.dT_part, with_du);
      if (!with_du) {
        const uint8_t* ops = w->opcodes + lvl_op[lv];
        TapplyArgs tl{Uc, ws.dRAW, dUc, 2, 1, 1, 0, 2, 0, M, nodes, ops, d, ws.ta_scale, 0};
        rc = launch_tapply(1, tl, G, ws.ta_packed, ws.status, stream);
        if (rc != HZ_OK) return rc;
        TapplyArgs tr{Uc, ws.dRAW, dUc, 2, 0, 1, 0, 2, 1, M, nodes, ops, d, ws.ta_scale, G * 1024};
        rc = launch_tapply(1, tr, G, ws.ta_packed, ws.status, stream);
        if (rc != HZ_OK) return rc;
      }
    } else if (use_tapply_tc()) {
      // du_L = A_R^T d raw (A_R from u_R), du_R = A_L^T d raw (A_L from u_L), merged nodes only
      const uint8_t* ops = w->opcodes + lvl_op[lv];
      TapplyArgs tl{Uc, ws.dRAW, dUc, 2, 1, 1, 0, 2, 0, M, nodes, ops, d, ws.ta_scale, 0};
      int rc = launch_tapply(1, tl, G, ws.ta_packed, ws.status, stream);
      if (rc != HZ_OK) return rc;
      TapplyArgs tr{Uc, ws.dRAW, dUc, 2, 0, 1, 0, 2, 1, M, nodes, ops, d, ws.ta_scale, G * 1024};
      rc = launch_tapply(1, tr, G, ws.ta_packed, ws.status, stream);
      if (rc != HZ_OK) return rc;
    } else if (use_tprod_tc()) {
      // du_L = T(d raw, ., u_R), du_R = T(d raw, u_L, .), written for merged nodes only
      const uint8_t* ops = w->opcodes + lvl_op[lv];
      TprodArgs tl{ws.dRAW, Uc, dUc, 1, 0, 2, 1, 2, 0, M, nodes, ops, d, ws.tp_scale[1]};
      int rc = launch_tprod(tl, G, ws.tp_packed[1], ws.status, stream);
      if (rc != HZ_OK) return rc;
      TprodArgs tr{ws.dRAW, Uc, dUc, 1, 0, 2, 0, 2, 1, M, nodes, ops, d, ws.tp_scale[2]};
      rc = launch_tprod(tr, G, ws.tp_packed[2], ws.status, stream);
      if (rc != HZ_OK) return rc;
    } else {
      const int rc = ensure_kernel_attributes(reinterpret_cast<const void*>(merge_bwd_kernel<false>), (int)smem);
      if (rc != HZ_OK) return rc;
      merge_bwd_kernel<false><<<dim3(G, kVjpSlices), kTsThreads, smem, stream>>>(
          L, w->merge_T, w->opcodes + lvl_op[lv], Uc, ws.dRAW, dUc, nullptr, 1);
    }
    HZ_CUDA_TRY(cudaGetLastError());
  }
  // weight gradients of the shared factors: one transposed GEMM over all levels' rows
  if (levels && o.g) {
    int st = launch_gemm_tn(ws.MIX, ws.dX, o.g->merge_U, (long long)row_off, r, d, r, d, d, false, ws.tn, stream);
    if (st != HZ_OK) return st;
    st = launch_gemm_tn(ws.RAW, ws.dMIX, o.g->merge_V, (long long)row_off, d, r, d, r, r, false, ws.tn, stream);
    if (st != HZ_OK) return st;
  }
  // leaves
  vjp_leaf_bwd_kernel<<<dim3(N, (unsigned)Bc), kLeafThreads, 0, stream>>>(
      N, d, ws.leaf_map, ws.U0, ws.S0, ws.dU0, ws.dS0, o.dq ? o.dq + (size_t)b0 * N * 4 : nullptr,
      l1_bwd ? w->opcodes : nullptr);
  if (o.g) vjp_leaf_map_grad_kernel<<<dim3(N, (d + 255) / 256), 256, 0, stream>>>(N, d, (int)Bc, qc, ws.dU0, ws.dM);
  HZ_CUDA_TRY(cudaGetLastError());
  if (l1_bwd) {
    // ws.dRAW still holds the first level's cotangent: that level was the last of the loop
    const int st = vjp_l1_backward_chunk(w, qc, Bc, ws.dRAW, ws.dS0, o.dq ? o.dq + (size_t)b0 * N * 4 : nullptr, ws.tn,
                                         ws.l1_D, ws.l1_gs, ws.l1_phi, o.g ? ws.l1_dphi : nullptr,
                                         o.g ? ws.l1_k : nullptr, stream);
    if (st != HZ_OK) return st;
  }
  if (o.f) return vjp_factor_statistics(w, qc, Bc, prev_u, (long long)row_off, o, ws, stream);
  return HZ_OK;
}

int vjp_run(const hz_wavefunction* w, const float* q, long long B, const float* cot_abs,
            const float* cot_phase, const hz_wavefunction_grads* g, const hz_kfac_factors* f, float* dq,
            float* log_abs, float* phase, void* workspace, long long workspace_bytes, void* stream) {
  int st = check_wavefunction(w);
  if (st != HZ_OK) return st;
  if (B < 0) return HZ_ERR_BAD_SHAPE;
  if (!g || !g->q_weight || !g->leaf_V || !g->leaf_U || !g->leaf_h || !g->readout_V || !g->readout_U ||
      !g->readout_h)
    return HZ_ERR_NULL_POINTER;
  const int N = w->n_sites, d = w->d_m, r = w->r_merge, rl = w->r_leaf, rr = w->r_ro;
  if (N > 1 && (!g->merge_T || !g->merge_V || !g->merge_U || !g->merge_h)) return HZ_ERR_NULL_POINTER;
  if (!workspace) return HZ_ERR_NULL_POINTER;
  if (B > 0 && (!q || !cot_abs || !cot_phase)) return HZ_ERR_NULL_POINTER;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return HZ_ERR_MISALIGNED;
  const int wf = f ? ((f->merge_T_left || f->merge_T_right) ? 2 : 1) : 0;
  if ((size_t)workspace_bytes < vjp_carve(w, 1, wf, nullptr).bytes) return HZ_ERR_WORKSPACE;
  long long Bc = B < 60000 ? (B > 0 ? B : 1) : 60000;
  if (vjp_carve(w, Bc, wf, nullptr).bytes > (size_t)workspace_bytes) {
    long long lo = 1, hi = Bc;
    while (hi - lo > 1) {
      const long long mid = lo + (hi - lo) / 2;
      if (vjp_carve(w, mid, wf, nullptr).bytes <= (size_t)workspace_bytes) lo = mid; else hi = mid;
    }
    Bc = lo;
  }
  while (Bc > 1 && Bc * (long long)N > 0x7fffffffLL / 4) Bc /= 2;
  VjpWorkspace ws = vjp_carve(w, Bc, wf, static_cast<char*>(workspace));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // gradients are overwritten: zero, accumulate over chunks
  auto zero = [&](float* p, size_t n) { return cudaMemsetAsync(p, 0, n * sizeof(float), s); };
  HZ_CUDA_TRY(zero(g->readout_V, (size_t)d * rr));
  HZ_CUDA_TRY(zero(g->readout_U, (size_t)rr * 2));
  HZ_CUDA_TRY(zero(g->readout_h, rr));
  HZ_CUDA_TRY(zero(g->leaf_U, (size_t)rl * d));
  HZ_CUDA_TRY(zero(ws.dM, (size_t)N * 4 * d));
  if (g->merge_V) HZ_CUDA_TRY(zero(g->merge_V, (size_t)d * r));
  if (g->merge_U) HZ_CUDA_TRY(zero(g->merge_U, (size_t)r * d));
  if (g->merge_T) HZ_CUDA_TRY(zero(g->merge_T, (size_t)(d / kDr) * 32768));
  if (N > 1) {
    HZ_CUDA_TRY(zero(g->merge_h, (size_t)(N - 1) * r));
    HZ_CUDA_TRY(zero(ws.dT_part, (size_t)kVjpSlices * (d / kDr) * 32768));
    HZ_CUDA_TRY(zero(ws.l1_dphi, (size_t)16 * (N / 2) * d));
    HZ_CUDA_TRY(zero(ws.l1_k, (size_t)N * 16));
  }
  st = vjp_prepare(w, ws, f != nullptr, s);
  if (st != HZ_OK) return st;
  struct Sq { float* p; int m; };
  const Sq squares[] = {{f ? f->q_in : nullptr, 4}, {f ? f->q_out : nullptr, w->d_o},
                        {f ? f->leaf_V_in : nullptr, w->d_o}, {f ? f->leaf_V_out : nullptr, rl},
                        {f ? f->leaf_U_in : nullptr, rl}, {f ? f->leaf_U_out : nullptr, d},
                        {f ? f->merge_V_in : nullptr, d}, {f ? f->merge_V_out : nullptr, r},
                        {f ? f->merge_U_in : nullptr, r}, {f ? f->merge_U_out : nullptr, d},
                        {f ? f->readout_V_in : nullptr, d}, {f ? f->readout_V_out : nullptr, rr},
                        {f ? f->readout_U_in : nullptr, rr}, {f ? f->readout_U_out : nullptr, 2},
                        {f && N > 1 ? f->merge_T_left : nullptr, d}, {f && N > 1 ? f->merge_T_right : nullptr, 1024}};
  if (f) {
    for (const Sq& sq : squares)
      if (sq.p) HZ_CUDA_TRY(zero(sq.p, (size_t)sq.m * sq.m));
    if (f->leaf_h_diag) HZ_CUDA_TRY(zero(f->leaf_h_diag, (size_t)N * rl));
    if (f->merge_h_diag && N > 1) HZ_CUDA_TRY(zero(f->merge_h_diag, (size_t)(N - 1) * r));
    if (f->readout_h_diag) HZ_CUDA_TRY(zero(f->readout_h_diag, rr));
    if (f->merge_T_stats) HZ_CUDA_TRY(zero(f->merge_T_stats, 2));
  }
  VjpOut o{g, f, dq, log_abs, phase};
  for (long long b0 = 0; b0 < B; b0 += Bc) {
    const long long nb = (B - b0 < Bc) ? (B - b0) : Bc;
    st = vjp_chunk(w, q, cot_abs, cot_phase, b0, nb, o, ws, s);
    if (st != HZ_OK) return st;
  }
  if (N > 1 && !f && B > 0 && vjp_l1_backward_coefficient_space() && vjp_l1_slices(w, ws.tn) >= 1) {
    // the basis cotangent through the fake batch that built the basis: its share of dT, and the
    // leaf-map cotangent of the d raw (x) u part; rows carry the fake batch's power-of-two scaling
    const int nodes = N / 2;
    fake_unscale_kernel<<<dim3(nodes, 16), 256, 0, s>>>(ws.l1_dphi, ws.l1_exp, nodes, 4, d);
    HZ_CUDA_TRY(zero(ws.l1_dfake, (size_t)16 * N * d));
    Level L{};
    L.N = N; L.d = d; L.G = d / kDr; L.jets = 0; L.Bc = 16; L.nodes = nodes; L.m = 3;
    L.rows_in = N; L.rows_out = nodes;
    const size_t smem = kTsSmemFloats * sizeof(float);
    st = ensure_kernel_attributes(reinterpret_cast<const void*>(merge_bwd_kernel<true>), (int)smem);
    if (st != HZ_OK) return st;
    merge_bwd_kernel<true><<<dim3(d / kDr, kVjpSlices), kTsThreads, smem, s>>>(L, w->merge_T, w->opcodes, ws.l1_fake,
                                                                               ws.l1_dphi, ws.l1_dfake, ws.dT_part, 1);
    vjp_l1_fold_kernel<<<dim3(N, (d + 255) / 256), 256, 0, s>>>(N, d, ws.l1_dfake, ws.l1_exp, ws.l1_k, ws.leaf_map,
                                                               ws.dM);
    HZ_CUDA_TRY(cudaGetLastError());
  }
  if (N > 1) {
    const long long n = (long long)(d / kDr) * 32768;
    vjp_reduce_slices_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(ws.dT_part, g->merge_T, n, kVjpSlices);
  }
  // leaf parameters from dM
  st = launch_gemm_tn(ws.leaf_tmp, ws.dM, g->leaf_U, 4 * N, rl, d, rl, d, d, false, ws.tn, s);
  if (st != HZ_OK) return st;
  {
    const long long warps = (long long)4 * N * rl;
    vjp_leaf_dtmp_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, s>>>(4 * N, rl, d, ws.dM, w->leaf_U, ws.dtmp);
    vjp_leaf_h_kernel<<<(rl + 127) / 128, 128, 0, s>>>(N, w->d_o, rl, w->q_weight, w->leaf_V, w->leaf_h, ws.dtmp,
                                                      g->leaf_h, ws.dWqV);
    const int tot = (w->d_o * rl > 4 * w->d_o) ? w->d_o * rl : 4 * w->d_o;
    vjp_leaf_qv_kernel<<<(tot + 127) / 128, 128, 0, s>>>(w->d_o, rl, w->q_weight, w->leaf_V, ws.dWqV, g->q_weight,
                                                        g->leaf_V);
  }
  if (f)
    for (const Sq& sq : squares)
      if (sq.p && sq.m > 4) {
        const long long n = (long long)sq.m * sq.m;
        vjp_symmetrize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(sq.p, sq.m);
      }
  {
    VjpPoison p{};
    p.full[0] = dq; p.n_full[0] = B * (long long)N * 4;
    p.full[1] = log_abs; p.n_full[1] = B;
    p.full[2] = phase; p.n_full[2] = B;
    float* firsts[] = {g->q_weight, g->leaf_V, g->leaf_U, g->leaf_h, g->merge_T, g->merge_V,
                       g->merge_U, g->merge_h, g->readout_V, g->readout_U, g->readout_h};
    for (float* x : firsts)
      if (x) p.first[p.n_first++] = x;
    if (f) {
      for (const Sq& sq : squares)
        if (sq.p) p.first[p.n_first++] = sq.p;
      if (f->leaf_h_diag) p.first[p.n_first++] = f->leaf_h_diag;
      if (f->merge_h_diag && N > 1) p.first[p.n_first++] = f->merge_h_diag;
      if (f->readout_h_diag) p.first[p.n_first++] = f->readout_h_diag;
    }
    vjp_poison_kernel<<<64, 256, 0, s>>>(ws.status, p);
  }
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// ------------------------------------------------------------------ value and chart gradient by one reverse sweep
// The sampler needs log|psi| and its gradient in the 3N chart coordinates only
// (src/hamiltonzero/mcmc/langevin.py:25-40): one value-only forward sweep and the backward sweep
// for the cotangent (1, 0) without any parameter gradient give dq [4 per site], which is
// projected on the chart rows d q / d z of the leaf kernel. grad [n][3N][2]: column 0 =
// d log|psi| / dz; column 1 (the phase gradient, which this single sweep does not produce) = 0.
__global__ void vjp_fill_kernel(float* __restrict__ p, float v, long long n) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < n) p[idx] = v;
}

__global__ void vjp_chart_project_kernel(long long sites, const float* __restrict__ q, const float* __restrict__ dq,
                                         float* __restrict__ grad) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // (walker, site)
  if (idx >= sites) return;
  const float4 qq = *reinterpret_cast<const float4*>(q + idx * 4);
  const float4 g = *reinterpret_cast<const float4*>(dq + idx * 4);
  const float q0 = qq.x, q1 = qq.y, q2 = qq.z, q3 = qq.w;
  // rows x, y, z of d(chart)/dz at z = 0, as in leaf_kernel
  const float rows[3][4] = {{-q3, q2, -q1, q0}, {-q2, -q3, q0, q1}, {-q1, q0, q3, -q2}};
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    const float v = rows[a][0] * g.x + rows[a][1] * g.y + rows[a][2] * g.z + rows[a][3] * g.w;
    *reinterpret_cast<float2*>(grad + (idx * 3 + a) * 2) = make_float2(v, 0.f);
  }
}

size_t vjp_chart_bytes(const hz_wavefunction* w, long long Bc) {
  return vjp_carve(w, Bc, 0, nullptr).bytes + 2 * align_up((size_t)Bc * sizeof(float)) +
         align_up((size_t)Bc * w->n_sites * 4 * sizeof(float));
}

int vjp_chart_value_and_grad(const hz_wavefunction* w, const float* q, long long n, float* log_abs, float* phase,
                             float* grad, void* workspace, long long workspace_bytes, cudaStream_t s,
                             bool prepared) {
  int st = check_wavefunction(w);
  if (st != HZ_OK) return st;
  if (n < 0) return HZ_ERR_BAD_SHAPE;
  if (!workspace || (n > 0 && (!q || !log_abs || !grad))) return HZ_ERR_NULL_POINTER;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return HZ_ERR_MISALIGNED;
  const int N = w->n_sites;
  if ((size_t)workspace_bytes < vjp_chart_bytes(w, 1)) return HZ_ERR_WORKSPACE;
  long long Bc = n < 60000 ? (n > 0 ? n : 1) : 60000;
  if (vjp_chart_bytes(w, Bc) > (size_t)workspace_bytes) {
    long long lo = 1, hi = Bc;
    while (hi - lo > 1) {
      const long long mid = lo + (hi - lo) / 2;
      if (vjp_chart_bytes(w, mid) <= (size_t)workspace_bytes) lo = mid; else hi = mid;
    }
    Bc = lo;
  }
  while (Bc > 1 && Bc * (long long)N > 0x7fffffffLL / 4) Bc /= 2;
  char* base = static_cast<char*>(workspace);
  VjpWorkspace ws = vjp_carve(w, Bc, 0, base);
  float* cot_abs = reinterpret_cast<float*>(base + ws.bytes);
  float* cot_phase = reinterpret_cast<float*>(base + ws.bytes + align_up((size_t)Bc * sizeof(float)));
  float* dq = reinterpret_cast<float*>(base + ws.bytes + 2 * align_up((size_t)Bc * sizeof(float)));
  if (!prepared) {
    st = vjp_prepare(w, ws, false, s);
    if (st != HZ_OK) return st;
    vjp_fill_kernel<<<(unsigned)((Bc + 255) / 256), 256, 0, s>>>(cot_abs, 1.f, Bc);
    HZ_CUDA_TRY(cudaMemsetAsync(cot_phase, 0, (size_t)Bc * sizeof(float), s));
  }
  for (long long b0 = 0; b0 < n; b0 += Bc) {
    const long long nb = (n - b0 < Bc) ? (n - b0) : Bc;
    VjpOut o{nullptr, nullptr, dq, log_abs + b0, phase ? phase + b0 : nullptr};
    st = vjp_chunk(w, q + (size_t)b0 * N * 4, cot_abs, cot_phase, 0, nb, o, ws, s);
    if (st != HZ_OK) return st;
    const long long sites = nb * N;
    vjp_chart_project_kernel<<<(unsigned)((sites + 255) / 256), 256, 0, s>>>(sites, q + (size_t)b0 * N * 4, dq,
                                                                            grad + (size_t)b0 * 3 * N * 2);
    HZ_CUDA_TRY(cudaGetLastError());
  }
  {
    // a device wait that ran out anywhere in the sweeps: the results become NaN besides the status word
    VjpPoison p{};
    p.full[0] = log_abs; p.n_full[0] = n;
    p.full[1] = phase; p.n_full[1] = n;
    p.full[2] = grad; p.n_full[2] = n * (long long)N * 6;
    vjp_poison_kernel<<<64, 256, 0, s>>>(ws.status, p);
    HZ_CUDA_TRY(cudaGetLastError());
  }
  return HZ_OK;
}
