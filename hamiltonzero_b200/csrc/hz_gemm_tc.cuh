// tcgen05 / TMEM / TMA version of the walker path's shared-weight GEMM for sm_100a:
//   C[M,N] = epilogue(A[M,K] @ B[K,N]),  fp32 in HBM, fp32-level accuracy.
//
// The fifth-generation tensor cores take TF32 operands, so every fp32 operand is used as
// head + tail (head = value rounded to 11 significant bits, tail = value - head) and a
// product is three UMMAs: head*tail + tail*head + head*head, accumulated in TMEM.
//   * B (the model's weights) is given transposed, [N,K] with K contiguous, already split
//     into a head and a tail matrix (prepared once per call by split_transpose_kernel).
//   * A (jet rows) arrives as raw fp32: TMA lands a 128 x 32 tile in shared memory with the
//     128-byte swizzle, the CTA rewrites it in place as the head and writes the tail beside
//     it (element-wise, so the swizzled layout is untouched).
// One warp-specialised CTA owns one 128 x BN output tile: a TMA producer, four warps that
// rewrite the A tile, a UMMA issuer and four warps that read TMEM back (roles and barriers
// are listed above the kernel).
// The tensor core's fp32 accumulation truncates (measured: -9e-6 relative over K = 1536),
// so TMEM never holds more than one k-tile (12 UMMAs): two TMEM accumulators alternate, and
// while the UMMAs of k-tile t fill one, the threads fold the other (k-tile t-1) into fp32
// registers with round-to-nearest adds.
// Every mbarrier wait is bounded; on a timeout the role records an error code and raises a
// CTA-wide abort flag, the producer waits (bounded) for its outstanding copies, and the CTA
// frees its TMEM columns and returns.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#include "hz_gemm.cuh"

namespace hz {

constexpr int kTcBM = 128, kTcBK = 32;
constexpr int kTcABytes = kTcBM * kTcBK * 4;                    // 16 KB
constexpr long long kTcWaitCycles = 4000000000ll;               // ~2 s at 1.9 GHz

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
// Bounded wait for the phase with the given parity to complete.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  const long long t0 = clock64();
  for (;;) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (clock64() - t0 > kTcWaitCycles) return false;
  }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y),
      "r"(smem_u32(bar))
      : "memory");
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);       // start address
  d |= (uint64_t)1 << 16;                            // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
  return d;
}

// kind::tf32, fp32 accumulate, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 columns of TMEM -> one column per register (asynchronous: tcgen05.wait::ld)
__device__ __forceinline__ void tmem_ld32(uint32_t (&v)[32], uint32_t taddr) {
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
}

// A operand in TMEM (lane = row, one column per K element), B from shared memory
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
        "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
        "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
        "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]),
        "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}

struct TcMaps {
  CUtensorMap a, bhi, blo, c;      // c: output, boxes of 128 rows x 32 columns
  CUtensorMap c2;                  // kEpiScatter: c = [8 walkers, 12 rows, 32], c2 = [8, 1, 32]
};

enum TcStatus { kTcOk = 0, kTcTimeoutLoad = 1, kTcTimeoutMma = 2 };

// Warp roles of one CTA (three warpgroups, one 128 x BN output tile):
//   warp 0      producer: TMA loads of A (raw fp32), B head, B tail into a ring of stages
//   warp 1      issuer: 12 UMMAs per k-tile into one of two TMEM accumulators
//   warps 4-7   rewriters: A tile -> head (in place) + tail, element-wise
//   warps 8-11  folders: tcgen05.ld the finished accumulator, add into fp32 registers
//               (round-to-nearest), then the epilogue
// The folders hold the 128 x BN tile in registers, so the register file is re-partitioned
// per warpgroup with setmaxnreg (producer/issuer and rewriters give registers back).
// mbarriers: full[s] (TMA -> rewriters), conv[s] (rewriters -> issuer), empty[s] (UMMAs done
// with stage s -> producer), tfull[b] (UMMAs of a k-tile done -> folders), tfree[b]
// (folders -> issuer). Every wait is bounded and also watches a CTA-wide abort flag.
constexpr int kTcThreads = 384;
constexpr int kTcFold = 1;            // k-tiles accumulated in TMEM between two folds
constexpr int kTcIssueWarp = 1, kTcRewriteWarp0 = 4, kTcRewriteThreads = 128, kTcFoldWarp0 = 8;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait that gives up early when another role of the CTA has already failed.
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity,
                                                    volatile int* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  const long long t0 = clock64();
  for (int spin = 0;; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spin & 63) == 63) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > kTcWaitCycles) return false;
    }
  }
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ TcMaps maps, GemmArgs a, int* __restrict__ status) {
  constexpr int kBBytes = BN * kTcBK * 4;
  constexpr int kStageBytes = 2 * kTcABytes + 2 * kBBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t full_bar[STAGES], conv_bar[STAGES], empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2], tfree_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = blockIdx.y * kTcBM, col0 = blockIdx.x * BN;
  const int KT = a.K / kTcBK;

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

  // ---------------- issuer
  auto issue_role = [&]() {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(BN);
      for (int kt = 0; kt < KT; ++kt) {
        // kTcFold consecutive k-tiles share one TMEM accumulator (a chain of 12*kTcFold UMMAs)
        const int s = kt % STAGES, grp = kt / kTcFold, buf = grp & 1;
        const bool first = (kt % kTcFold) == 0, last = (kt % kTcFold) == kTcFold - 1 || kt == KT - 1;
        if (!mbar_wait_abortable(&conv_bar[s], (kt / STAGES) & 1, &abort_s) ||
            (first && grp >= 2 &&
             !mbar_wait_abortable(&tfree_bar[buf], ((grp >> 1) - 1) & 1, &abort_s))) {
          fail(kTcTimeoutMma);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_hi = smem_u32(stage_ptr(s));
        const uint32_t a_lo = a_hi + kTcABytes;
        const uint32_t b_hi = a_hi + 2 * kTcABytes;
        const uint32_t b_lo = b_hi + kBBytes;
        const uint32_t tacc = tmem_base + (uint32_t)(buf * BN);
#pragma unroll
        for (int k8 = 0; k8 < kTcBK / 8; ++k8) {
          const uint32_t off = k8 * 32;     // 8 TF32 = 32 bytes along K inside the swizzled row
          const uint64_t dah = umma_desc_sw128(a_hi + off), dal = umma_desc_sw128(a_lo + off);
          const uint64_t dbh = umma_desc_sw128(b_hi + off), dbl = umma_desc_sw128(b_lo + off);
          umma_tf32(tacc, dal, dbh, idesc, (k8 > 0 || !first) ? 1u : 0u);
          umma_tf32(tacc, dah, dbl, idesc, 1u);
          umma_tf32(tacc, dah, dbh, idesc, 1u);
        }
        umma_commit(&empty_bar[s]);      // the stage may be refilled
        if (last) umma_commit(&tfull_bar[buf]);    // the accumulator may be folded
      }
    }
  };

  if (warp < kTcRewriteWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
    // ---------------- producer
    if (lane == 0) {
      int issued = 0;
      for (int kt = 0; kt < KT; ++kt) {
        const int s = kt % STAGES;
        if (kt >= STAGES &&
            !mbar_wait_abortable(&empty_bar[s], ((kt / STAGES) - 1) & 1, &abort_s)) {
          fail(kTcTimeoutMma);
          break;
        }
        uint8_t* st = stage_ptr(s);
        mbar_expect_tx(&full_bar[s], kTcABytes + 2 * kBBytes);
        tma_load_2d(st, &maps.a, kt * kTcBK, row0, &full_bar[s]);
        tma_load_2d(st + 2 * kTcABytes, &maps.bhi, kt * kTcBK, col0, &full_bar[s]);
        tma_load_2d(st + 2 * kTcABytes + kBBytes, &maps.blo, kt * kTcBK, col0, &full_bar[s]);
        issued = kt + 1;
      }
      if (abort_s != 0) {
        // something ran out: let the copies still in flight land before the CTA exits
        for (int kt = max(0, issued - STAGES); kt < issued; ++kt)
          mbar_wait(&full_bar[kt % STAGES], (kt / STAGES) & 1);
      }
    }
    } else if (warp == kTcIssueWarp) {
      issue_role();
    }
  } else if (warp < kTcFoldWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    // ---------------- rewriters: A -> head (in place) + tail
    const int rt = tid - kTcRewriteWarp0 * 32;          // 0..127
    for (int kt = 0; kt < KT; ++kt) {
      const int s = kt % STAGES;
      if (!mbar_wait_abortable(&full_bar[s], (kt / STAGES) & 1, &abort_s)) {
        if (lane == 0) fail(kTcTimeoutLoad);
        break;
      }
      float4* hi = reinterpret_cast<float4*>(stage_ptr(s));
      float4* lo = reinterpret_cast<float4*>(stage_ptr(s) + kTcABytes);
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
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(&conv_bar[s]);
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ---------------- folders + epilogue
    const int q = warp & 3;                               // TMEM lane quadrant of this warp
    float acc[BN];
#pragma unroll
    for (int j = 0; j < BN; ++j) acc[j] = 0.f;
    bool ok = true;
    const int groups = (KT + kTcFold - 1) / kTcFold;
    for (int grp = 0; grp < groups; ++grp) {
      const int buf = grp & 1;
      if (!mbar_wait_abortable(&tfull_bar[buf], (grp >> 1) & 1, &abort_s)) {
        if (lane == 0) fail(kTcTimeoutMma);
        ok = false;
        break;
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
    // Epilogue: the tile leaves through shared memory and TMA. The stage ring is idle by now
    // (every UMMA has completed), so four 128 x 32 sub-tiles are written there in the 128-byte
    // swizzle and one thread issues four bulk tensor stores - or, for the residual form
    // out = R + A B with R already in C, four bulk tensor reduce-adds, which spare the SM the
    // read of R altogether. Rows beyond M are clipped by the tensor map.
    const bool tma_out = (EPI != kEpiResidual) || (a.R == a.C);
    if (ok && tma_out) {
      const int rloc = q * 32 + lane;
      const int row = row0 + rloc;
      const float* hrow = nullptr;
      if (EPI == kEpiNodeScale && row < a.M) hrow = a.h + (size_t)gemm_node_of_row(a, row) * a.N + col0;
      float* tile = reinterpret_cast<float*>(smem);
#pragma unroll
      for (int cb = 0; cb < BN / 32; ++cb) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int j = cb * 32 + c * 4;
          float4 o = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
          if (EPI == kEpiNodeScale && hrow != nullptr) {
            const float4 hh = *reinterpret_cast<const float4*>(hrow + j);
            o.x *= hh.x; o.y *= hh.y; o.z *= hh.z; o.w *= hh.w;
          }
          *reinterpret_cast<float4*>(tile + cb * 4096 + rloc * 32 + ((c ^ (rloc & 7)) << 2)) = o;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");      // the four folder warps only
    if (ok && tma_out && abort_s == 0 && warp == kTcFoldWarp0 && lane == 0) {
#pragma unroll
      for (int cb = 0; cb < BN / 32; ++cb) {
        const uint32_t src = smem_u32(smem) + cb * 16384;
        if (EPI == kEpiScatter) {
          const int wk0 = blockIdx.y * 8;
          asm volatile(
              "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
              ::"l"(reinterpret_cast<uint64_t>(&maps.c)), "r"(col0 + cb * 32), "r"(a.sc_j0), "r"(wk0),
                "r"(src)
              : "memory");
          asm volatile(
              "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
              ::"l"(reinterpret_cast<uint64_t>(&maps.c2)), "r"(col0 + cb * 32), "r"(a.sc_u), "r"(wk0),
                "r"(src + 96 * 128)
              : "memory");
          asm volatile(
              "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
              ::"l"(reinterpret_cast<uint64_t>(&maps.c2)), "r"(col0 + cb * 32), "r"(a.sc_l), "r"(wk0),
                "r"(src + 104 * 128)
              : "memory");
        } else if (EPI == kEpiResidual)
          asm volatile(
              "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
              ::"l"(reinterpret_cast<uint64_t>(&maps.c)), "r"(col0 + cb * 32), "r"(row0), "r"(src)
              : "memory");
        else
          asm volatile(
              "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
              ::"l"(reinterpret_cast<uint64_t>(&maps.c)), "r"(col0 + cb * 32), "r"(row0), "r"(src)
              : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    if (ok && !tma_out) {
      const int row = row0 + q * 32 + lane;
      if (row < a.M) {
        float* crow = a.C + (size_t)row * a.ldc + col0;
#pragma unroll
        for (int j = 0; j < BN; j += 4) {
          const float4 rr = *reinterpret_cast<const float4*>(a.R + (size_t)row * a.ldc + col0 + j);
          *reinterpret_cast<float4*>(crow + j) =
              make_float4(acc[j] + rr.x, acc[j + 1] + rr.y, acc[j + 2] + rr.z, acc[j + 3] + rr.w);
        }
      }
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

// Persistent form of the kernel above: one CTA per SM walks over the output tiles (tiles that
// share their A rows are neighbours), so that the prologue (barriers, TMEM allocation) is paid
// once and the epilogue of a tile overlaps the main loop of the next one. The barrier phases
// simply continue across tiles (one running k-tile counter per role). The epilogue has its own
// 32 KB buffer (two 128 x 32 sub-tiles at a time), because the stage ring is already being
// refilled for the next tile. A folder warp whose wait ran out keeps walking the loops without
// waiting or storing, so that the named barrier of the epilogue is always reached by all four.
constexpr int kTcEpiBytes = 2 * kTcBM * 32 * 4;
// TMEM allocations are powers of two of at least 32 columns
__host__ __device__ constexpr uint32_t tc_tmem_cols(int need) {
  uint32_t c = 32;
  while ((int)c < need) c *= 2;
  return c;
}

template <int BN, int STAGES, int EPI, int ATM, int FOLD>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tcp_kernel(const __grid_constant__ TcMaps maps, GemmArgs a, int* __restrict__ status) {
  constexpr int kBBytes = BN * kTcBK * 4;
  // ATM 1: the tail of A lives in TMEM (32 columns per stage, written by the rewriters with
  // tcgen05.st and read by the UMMA as its A operand), so a stage is 16 KB smaller and the ring
  // is one stage deeper in the same shared memory. ATM 2: head and tail both live in TMEM (64
  // columns per stage); the UMMAs then read only B from shared memory, whose bandwidth (operand
  // reads + TMA writes + the rewrite pass) is what bounds this kernel.
  constexpr int kAPart = (ATM ? 1 : 2) * kTcABytes;
  constexpr int kStageBytes = kAPart + 2 * kBBytes;
  constexpr int kAColsPerStage = ATM == 2 ? 64 : (ATM == 1 ? 32 : 0);
  constexpr uint32_t kTmemCols = tc_tmem_cols(2 * BN + STAGES * kAColsPerStage);
  constexpr uint32_t kColALo = 2 * BN;            // tail of stage s at kColALo + s * kAColsPerStage
  constexpr uint32_t kColAHi = kColALo + 32;      // ATM 2: head right after the stage's tail
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi = smem + (size_t)STAGES * kStageBytes;
  __shared__ __align__(8) uint64_t full_bar[STAGES], conv_bar[STAGES], empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2], tfree_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KT = a.K / kTcBK;
  const int tiles_n = a.N / BN;
  const int tiles_m = (a.M + kTcBM - 1) / kTcBM;
  const long long total = (long long)tiles_m * tiles_n;

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
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  auto stage_ptr = [&](int s) { return smem + (size_t)s * kStageBytes; };
  auto fail = [&](int code) { atomicExch(status, code); abort_s = 1; };

  if (warp < kTcRewriteWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      // ---------------- producer
      if (lane == 0) {
        long long it = 0;
        bool alive = true;
        for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
          const int row0 = (int)(tile / tiles_n) * kTcBM, col0 = (int)(tile % tiles_n) * BN;
          for (int kt = 0; kt < KT; ++kt, ++it) {
            const int s = (int)(it % STAGES);
            if (it >= STAGES &&
                !mbar_wait_abortable(&empty_bar[s], (uint32_t)((it / STAGES) - 1) & 1, &abort_s)) {
              fail(kTcTimeoutMma);
              alive = false;
              break;
            }
            uint8_t* st = stage_ptr(s);
            mbar_expect_tx(&full_bar[s], kTcABytes + 2 * kBBytes);
            tma_load_2d(st, &maps.a, kt * kTcBK, row0, &full_bar[s]);
            tma_load_2d(st + kAPart, &maps.bhi, kt * kTcBK, col0, &full_bar[s]);
            tma_load_2d(st + kAPart + kBBytes, &maps.blo, kt * kTcBK, col0, &full_bar[s]);
          }
        }
        if (abort_s != 0) {
          // something ran out: let the copies still in flight land before the CTA exits
          for (long long j = (it > STAGES ? it - STAGES : 0); j < it; ++j)
            mbar_wait(&full_bar[j % STAGES], (uint32_t)(j / STAGES) & 1);
        }
      }
    } else if (warp == kTcIssueWarp) {
      // ---------------- issuer
      if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_tf32(BN);
        long long it = 0, gi = 0;      // running k-tile and fold-group counters
        bool alive = true;
        for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
          for (int kt = 0; kt < KT; ++kt, ++it) {
            // FOLD consecutive k-tiles share one TMEM accumulator (a chain of 12 FOLD UMMAs)
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
            const uint32_t a_hi = smem_u32(stage_ptr(s));
            const uint32_t a_lo = a_hi + kTcABytes;
            const uint32_t b_hi = a_hi + kAPart;
            const uint32_t b_lo = b_hi + kBBytes;
            const uint32_t tacc = tmem_base + (uint32_t)(buf * BN);
#pragma unroll
            for (int k8 = 0; k8 < kTcBK / 8; ++k8) {
              const uint32_t off = k8 * 32;
              const uint64_t dah = umma_desc_sw128(a_hi + off);
              const uint64_t dbh = umma_desc_sw128(b_hi + off), dbl = umma_desc_sw128(b_lo + off);
              const uint32_t ta = tmem_base + (uint32_t)(s * kAColsPerStage + k8 * 8);
              if (ATM)
                umma_tf32_ts(tacc, ta + kColALo, dbh, idesc, (k8 > 0 || !first) ? 1u : 0u);
              else
                umma_tf32(tacc, umma_desc_sw128(a_lo + off), dbh, idesc, (k8 > 0 || !first) ? 1u : 0u);
              if (ATM == 2) {
                umma_tf32_ts(tacc, ta + kColAHi, dbl, idesc, 1u);
                umma_tf32_ts(tacc, ta + kColAHi, dbh, idesc, 1u);
              } else {
                umma_tf32(tacc, dah, dbl, idesc, 1u);
                umma_tf32(tacc, dah, dbh, idesc, 1u);
              }
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
  } else if (warp < kTcFoldWarp0) {
    if (ATM) asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    // ---------------- rewriters: A -> head (in place) + tail
    const int rt = tid - kTcRewriteWarp0 * 32;
    long long it = 0;
    bool alive = true;
    for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
      for (int kt = 0; kt < KT; ++kt, ++it) {
        const int s = (int)(it % STAGES);
        // warp-uniform outcome: the TMEM store below is a warp-wide instruction
        if (!__all_sync(0xffffffffu,
                        mbar_wait_abortable(&full_bar[s], (uint32_t)(it / STAGES) & 1, &abort_s))) {
          if (lane == 0) fail(kTcTimeoutLoad);
          alive = false;
          break;
        }
        if (ATM) {
          // thread = row of the tile = TMEM lane: its 128-byte row (eight 16-byte chunks, chunk c
          // at position c ^ (row & 7) of the 128-byte swizzle) is rounded in place, the tails go
          // to the stage's 32 TMEM columns
          float4* rowp = reinterpret_cast<float4*>(stage_ptr(s) + rt * 128);
          uint32_t tl[32], th[ATM == 2 ? 32 : 1];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const int pc = c ^ (rt & 7);
            const float4 x = rowp[pc];
            float4 h;
            h.x = __uint_as_float((__float_as_uint(x.x) + 0x1000u) & 0xFFFFE000u);
            h.y = __uint_as_float((__float_as_uint(x.y) + 0x1000u) & 0xFFFFE000u);
            h.z = __uint_as_float((__float_as_uint(x.z) + 0x1000u) & 0xFFFFE000u);
            h.w = __uint_as_float((__float_as_uint(x.w) + 0x1000u) & 0xFFFFE000u);
            if (ATM == 2) {
              th[(4 * c) % (ATM == 2 ? 32 : 1)] = __float_as_uint(h.x);
              th[(4 * c + 1) % (ATM == 2 ? 32 : 1)] = __float_as_uint(h.y);
              th[(4 * c + 2) % (ATM == 2 ? 32 : 1)] = __float_as_uint(h.z);
              th[(4 * c + 3) % (ATM == 2 ? 32 : 1)] = __float_as_uint(h.w);
            } else {
              rowp[pc] = h;
            }
            tl[4 * c] = __float_as_uint(x.x - h.x);
            tl[4 * c + 1] = __float_as_uint(x.y - h.y);
            tl[4 * c + 2] = __float_as_uint(x.z - h.z);
            tl[4 * c + 3] = __float_as_uint(x.w - h.w);
          }
          const uint32_t trow = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) +
                                (uint32_t)(s * kAColsPerStage);
          tmem_st32(trow + kColALo, tl);
          if (ATM == 2) tmem_st32(trow + kColAHi, reinterpret_cast<const uint32_t (&)[32]>(th));
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        } else {
        float4* hi = reinterpret_cast<float4*>(stage_ptr(s));
        float4* lo = reinterpret_cast<float4*>(stage_ptr(s) + kTcABytes);
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
    // ---------------- folders + epilogue
    const int q = warp & 3;
    const bool issuer_thread = (warp == kTcFoldWarp0 && lane == 0);
    bool ok = true;
    long long it = 0;                  // running fold-group counter
    const int groups = (KT + FOLD - 1) / FOLD;
    for (long long tile = blockIdx.x; tile < total; tile += gridDim.x) {
      const int row0 = (int)(tile / tiles_n) * kTcBM, col0 = (int)(tile % tiles_n) * BN;
      float acc[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      for (int kt = 0; kt < groups; ++kt, ++it) {
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
      // ---- epilogue of this tile, two 128 x 32 sub-tiles at a time
      const bool tma_out = (EPI != kEpiResidual) || (a.R == a.C);
      const int rloc = q * 32 + lane;
      const int row = row0 + rloc;
      const float* hrow = nullptr;
      if (EPI == kEpiNodeScale && row < a.M) hrow = a.h + (size_t)gemm_node_of_row(a, row) * a.N + col0;
      float* tilebuf = reinterpret_cast<float*>(epi);
#pragma unroll
      for (int half = 0; half < BN / 64; ++half) {
        // the bulk stores issued for the previous pair of sub-tiles must have read the buffer
        if (issuer_thread) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ok && tma_out) {
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            const int cb = half * 2 + sub;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const int j = cb * 32 + c * 4;
              float4 o = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
              if (EPI == kEpiNodeScale && hrow != nullptr) {
                const float4 hh = *reinterpret_cast<const float4*>(hrow + j);
                o.x *= hh.x; o.y *= hh.y; o.z *= hh.z; o.w *= hh.w;
              }
              *reinterpret_cast<float4*>(tilebuf + sub * 4096 + rloc * 32 + ((c ^ (rloc & 7)) << 2)) = o;
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer_thread && ok && tma_out && abort_s == 0) {
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            const int cb = half * 2 + sub;
            const uint32_t src = smem_u32(epi) + sub * 16384;
            if (EPI == kEpiScatter) {
              const int wk0 = (row0 / kTcBM) * 8;
              asm volatile(
                  "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                  ::"l"(reinterpret_cast<uint64_t>(&maps.c)), "r"(col0 + cb * 32), "r"(a.sc_j0), "r"(wk0),
                    "r"(src)
                  : "memory");
              asm volatile(
                  "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                  ::"l"(reinterpret_cast<uint64_t>(&maps.c2)), "r"(col0 + cb * 32), "r"(a.sc_u), "r"(wk0),
                    "r"(src + 96 * 128)
                  : "memory");
              asm volatile(
                  "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                  ::"l"(reinterpret_cast<uint64_t>(&maps.c2)), "r"(col0 + cb * 32), "r"(a.sc_l), "r"(wk0),
                    "r"(src + 104 * 128)
                  : "memory");
            } else if (EPI == kEpiResidual) {
              asm volatile(
                  "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                  ::"l"(reinterpret_cast<uint64_t>(&maps.c)), "r"(col0 + cb * 32), "r"(row0), "r"(src)
                  : "memory");
            } else {
              asm volatile(
                  "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                  ::"l"(reinterpret_cast<uint64_t>(&maps.c)), "r"(col0 + cb * 32), "r"(row0), "r"(src)
                  : "memory");
            }
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      if (ok && !tma_out && row < a.M) {
        float* crow = a.C + (size_t)row * a.ldc + col0;
#pragma unroll
        for (int j = 0; j < BN; j += 4) {
          const float4 rr = *reinterpret_cast<const float4*>(a.R + (size_t)row * a.ldc + col0 + j);
          *reinterpret_cast<float4*>(crow + j) =
              make_float4(acc[j] + rr.x, acc[j + 1] + rr.y, acc[j + 2] + rr.z, acc[j + 3] + rr.w);
        }
      }
    }
    if (issuer_thread) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

// B [K,N] row-major -> Bt_hi, Bt_lo [N,K] row-major (K contiguous), head/tail split.
static __global__ void split_transpose_kernel(const float* __restrict__ B, float* __restrict__ hi,
                                       float* __restrict__ lo, int K, int N) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, n = n0 + threadIdx.x;
    tile[r][threadIdx.x] = (k < K && n < N) ? B[(size_t)k * N + n] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) {
      const float x = tile[threadIdx.x][r];
      const float h = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
      hi[(size_t)n * K + k] = h;
      lo[(size_t)n * K + k] = x - h;
    }
  }
}

// ---- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static const EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(p);
    return nullptr;
  }();
  return fn;
}

// 2-D fp32 row-major [rows, cols] (cols contiguous, leading dimension ld), box [box_rows, 32].
inline bool make_map(CUtensorMap* m, const float* base, long long rows, long long cols,
                     long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)kTcBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D fp32 [walkers, rows, cols] (cols contiguous), box [box_walkers, box_rows, 32].
inline bool make_map3(CUtensorMap* m, const float* base, long long walkers, long long rows,
                      long long cols, int box_rows, int box_walkers) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)walkers};
  cuuint64_t strides[2] = {(cuuint64_t)cols * sizeof(float), (cuuint64_t)rows * cols * sizeof(float)};
  cuuint32_t box[3] = {(cuuint32_t)kTcBK, (cuuint32_t)box_rows, (cuuint32_t)box_walkers};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline bool gemm_tc_supported(const GemmArgs& a) {
  return a.K % kTcBK == 0 && a.N % 128 == 0 && a.lda % 4 == 0 && a.ldc % 4 == 0 &&
         (reinterpret_cast<uintptr_t>(a.A) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.C) & 15) == 0;
}

template <int BN, int STAGES>
int launch_gemm_tc_bn(int epi, const GemmArgs& a, const float* bt_hi, const float* bt_lo,
                      int* status, cudaStream_t stream) {
  TcMaps maps;
  if (!make_map(&maps.a, a.A, a.M, a.K, a.lda, kTcBM) ||
      !make_map(&maps.bhi, bt_hi, a.N, a.K, a.K, BN) ||
      !make_map(&maps.blo, bt_lo, a.N, a.K, a.K, BN))
    return HZ_ERR_CUDA;
  if (epi == kEpiScatter) {
    if (a.ldc != a.N ||
        !make_map3(&maps.c, a.C, a.sc_walkers, a.sc_rows, a.N, 12, 8) ||
        !make_map3(&maps.c2, a.C, a.sc_walkers, a.sc_rows, a.N, 1, 8))
      return HZ_ERR_CUDA;
  } else {
    if (!make_map(&maps.c, a.C, a.M, a.N, a.ldc, kTcBM)) return HZ_ERR_CUDA;
    maps.c2 = maps.c;
  }
  constexpr size_t smem = (size_t)STAGES * (2 * kTcABytes + 2 * BN * kTcBK * 4) + 1024;
  dim3 grid(a.N / BN, (a.M + kTcBM - 1) / kTcBM);
#define HZ_TC_LAUNCH(E)                                                                          \
  do {                                                                                           \
    const int hz_rc__ = ensure_kernel_attributes(                                                \
        reinterpret_cast<const void*>(gemm_tc_kernel<BN, STAGES, E>), (int)smem);                \
    if (hz_rc__ != HZ_OK) return hz_rc__;                                                        \
    gemm_tc_kernel<BN, STAGES, E><<<grid, kTcThreads, smem, stream>>>(maps, a, status);          \
  } while (0)
  switch (epi) {
    case kEpiStore: HZ_TC_LAUNCH(kEpiStore); break;
    case kEpiNodeScale: HZ_TC_LAUNCH(kEpiNodeScale); break;
    case kEpiScatter: HZ_TC_LAUNCH(kEpiScatter); break;
    default: HZ_TC_LAUNCH(kEpiResidual); break;
  }
#undef HZ_TC_LAUNCH
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

inline int tc_sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  return n;
}

// HZ_GEMM_TC=classic selects the one-tile-per-CTA kernel.
inline bool use_persistent_tc() {
  static const bool persistent = !env_equals("HZ_GEMM_TC", "classic");
  return persistent;
}

// Where the persistent kernel keeps the split A operand: 2 = head and tail in TMEM (default),
// 1 = tail in TMEM (HZ_GEMM_TC=tail), 0 = both in shared memory, three stages (HZ_GEMM_TC=ring3).
inline int tmem_operand_mode() {
  static const int mode = env_equals("HZ_GEMM_TC", "ring3") ? 0 : env_equals("HZ_GEMM_TC", "tail") ? 1 : 2;
  return mode;
}

template <int BN, int STAGES, int ATM, int FOLD>
int launch_gemm_tcp_bn(int epi, const GemmArgs& a, const float* bt_hi, const float* bt_lo,
                       int* status, cudaStream_t stream) {
  TcMaps maps;
  if (!make_map(&maps.a, a.A, a.M, a.K, a.lda, kTcBM) ||
      !make_map(&maps.bhi, bt_hi, a.N, a.K, a.K, BN) ||
      !make_map(&maps.blo, bt_lo, a.N, a.K, a.K, BN))
    return HZ_ERR_CUDA;
  if (epi == kEpiScatter) {
    if (a.ldc != a.N ||
        !make_map3(&maps.c, a.C, a.sc_walkers, a.sc_rows, a.N, 12, 8) ||
        !make_map3(&maps.c2, a.C, a.sc_walkers, a.sc_rows, a.N, 1, 8))
      return HZ_ERR_CUDA;
  } else {
    if (!make_map(&maps.c, a.C, a.M, a.N, a.ldc, kTcBM)) return HZ_ERR_CUDA;
    maps.c2 = maps.c;
  }
  constexpr size_t smem = (size_t)STAGES * ((ATM ? 1 : 2) * kTcABytes + 2 * BN * kTcBK * 4) + kTcEpiBytes + 1024;
  const long long total = (long long)(a.N / BN) * ((a.M + kTcBM - 1) / kTcBM);
  const int sms = tc_sm_count();
  const unsigned grid = (unsigned)(total < sms ? total : sms);
#define HZ_TCP_LAUNCH(E)                                                                         \
  do {                                                                                           \
    const int hz_rc__ = ensure_kernel_attributes(                                                \
        reinterpret_cast<const void*>(gemm_tcp_kernel<BN, STAGES, E, ATM, FOLD>), (int)smem);    \
    if (hz_rc__ != HZ_OK) return hz_rc__;                                                        \
    gemm_tcp_kernel<BN, STAGES, E, ATM, FOLD><<<grid, kTcThreads, smem, stream>>>(maps, a, status);         \
  } while (0)
  switch (epi) {
    case kEpiStore: HZ_TCP_LAUNCH(kEpiStore); break;
    case kEpiNodeScale: HZ_TCP_LAUNCH(kEpiNodeScale); break;
    case kEpiScatter: HZ_TCP_LAUNCH(kEpiScatter); break;
    default: HZ_TCP_LAUNCH(kEpiResidual); break;
  }
#undef HZ_TCP_LAUNCH
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// ------------------------------------------------------------------ FP16-split variant
// The same persistent GEMM on kind::f16 UMMAs: every fp32 operand is used as an FP16 head plus an
// FP16 tail, and a product is head*head + head*tail + tail*head (each exact to about 3 * 2^-22,
// like the three-term TF32 split), but one instruction contracts 16 elements instead of 8: half
// the tensor time and half the shared-memory traffic of B per k-tile.
//   * B (weights) is prepared once per call by pack_f16_kernel: transposed [N, K], every
//     k-tile of 32 entries stored as one 128-byte row [head(32) | tail(32)] of halves, every row n
//     (output column) scaled by its own power of two so that its largest entry lies in
//     [2^14, 2^15): tails then keep all their bits for entries down to 2^-18 of the row's largest.
//     The epilogue multiplies the scale back in.
//   * A (jet rows, unbounded range) is scaled per (row, k-tile) by a power of two taken from the
//     row's largest entry in that k-tile, into the same range - the rewriter thread owns the row,
//     so the maximum costs nothing - and lands in TMEM as [head | tail] (16 + 16 columns, two
//     halves per column). The folder thread of the same row undoes the scale when it adds the
//     k-tile's accumulator into its fp32 registers (one k-tile per TMEM accumulator).
//   * Two groups of rewriter warps take the k-tiles alternately (a single warp per scheduler
//     converting every k-tile was the critical path).
// Barriers and the abort path are those of gemm_tcp_kernel.
constexpr int kTfAColsPerStage = 32;      // 16 columns [head] + 16 columns [tail]
// 4 service + 8 rewriter + 4 folder warps. Registers: the CTA starts with 512 x 128; service warps
// drop to 40 and rewriters to 96 (19456 released) before the folders ask for 232 (13312 more).
constexpr int kTfThreads = 512, kTfFoldThreads = 128;
constexpr int kTfRegsService = 40, kTfRegsRewrite = 96, kTfRegsFold = 232;
// setmaxnreg.inc waits until the registers exist: the three roles together must fit in what the
// CTA was launched with (512 threads x 128, the cap that __launch_bounds__(512) gives ptxas)
static_assert(128 * kTfRegsService + 256 * kTfRegsRewrite + 128 * kTfRegsFold <= kTfThreads * 128,
              "register budget of the FP16-split GEMM roles");
constexpr int kTfFoldWarp0 = 12;
constexpr int kTfScaleRing = 8;           // (row, k-tile) scales in flight between rewriters and folders

__host__ __device__ constexpr uint32_t umma_idesc_f16_n(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
        "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
        "r"(v[15])
      : "memory");
}

// exponent e_n of every row n of B^T such that the row's largest entry times 2^-e_n lies in
// [2^14, 2^15): scale[n] = 2^e_n, expo[n] = e_n. One warp per row.
static __global__ void pack_f16_rowscale_kernel(const float* __restrict__ B, float* __restrict__ scale,
                                                int* __restrict__ expo, int K, int N, int transposed) {
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (n >= N) return;
  float m = 0.f;
  for (int k = lane; k < K; k += 32)
    m = fmaxf(m, fabsf(transposed ? B[(size_t)k * N + n] : B[(size_t)n * K + k]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) {
    int e = 0;
    if (m > 0.f && isfinite(m)) { frexpf(m, &e); e -= 15; }
    scale[n] = ldexpf(1.f, e);
    expo[n] = e;
  }
}

// B [K,N] row-major (transposed = 1) or [N,K] (0) -> packed [N][K/32][head(32) | tail(32)] halves of
// B^T[n][:] * 2^-e_n.
static __global__ void pack_f16_kernel(const float* __restrict__ B, __half* __restrict__ packed,
                                       const int* __restrict__ expo, int K, int N, int transposed) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    // tile[k][n]
    if (transposed) {
      const int k = k0 + r, n = n0 + threadIdx.x;
      tile[r][threadIdx.x] = (k < K && n < N) ? B[(size_t)k * N + n] : 0.f;
    } else {
      const int n = n0 + r, k = k0 + threadIdx.x;
      tile[threadIdx.x][r] = (k < K && n < N) ? B[(size_t)n * K + k] : 0.f;
    }
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) {
      const float x = ldexpf(tile[threadIdx.x][r], -expo[n]);
      const __half hi = __float2half_rn(x);
      __half* row = packed + ((size_t)n * (K / 32) + blockIdx.y) * 64;
      row[threadIdx.x] = hi;
      row[32 + threadIdx.x] = __float2half_rn(x - __half2float(hi));
    }
  }
}

// hi: packed halves (the bytes of one [N,K] fp32 matrix); lo[0, N): the row scales 2^e_n that the
// GEMM's epilogue multiplies back in, lo[N, 2N): the exponents.
inline int prepare_weights_f16(const float* B, float* hi, float* lo, int K, int N, bool transposed,
                               cudaStream_t stream) {
  int* expo = reinterpret_cast<int*>(lo + N);
  pack_f16_rowscale_kernel<<<(N + 7) / 8, 256, 0, stream>>>(B, lo, expo, K, N, transposed ? 1 : 0);
  pack_f16_kernel<<<dim3((N + 31) / 32, K / 32), dim3(32, 8), 0, stream>>>(
      B, reinterpret_cast<__half*>(hi), expo, K, N, transposed ? 1 : 0);
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// exponent of every row of A that brings the row's largest entry into [2^14, 2^15); one warp per row
static __global__ void gemm_row_expo_kernel(const float* __restrict__ A, int M, int K, int lda,
                                            int* __restrict__ expo) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const float4* p = reinterpret_cast<const float4*>(A + (size_t)row * lda);
  float mx = 0.f;
  for (int c = lane; c < K / 4; c += 32) {
    const float4 v = p[c];
    mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) {
    int e = 0;
    if (mx > 0.f && isfinite(mx)) e = max((int)((__float_as_uint(mx) >> 23) & 0xff) - 141, -126);
    expo[row] = e;
  }
}

// FOLD: k-tiles that share one TMEM accumulator between two folds into the folders' registers.
// FOLD > 1 needs one scale per row for the whole K (a.a_expo, filled by gemm_row_expo_kernel):
// the folders then read the accumulator once per FOLD k-tiles instead of once per k-tile - their
// tcgen05.ld traffic, 64 KB per k-tile of a 128 x 128 tile, is what bounded the kernel at about
// 1200 cycles per k-tile.
template <int BN, int STAGES, int EPI, int FOLD>
__global__ void __launch_bounds__(kTfThreads, 1)
gemm_tcf_kernel(const __grid_constant__ TcMaps maps, GemmArgs a, const float* __restrict__ b_scale,
                int* __restrict__ status) {
  constexpr int kBBytes = BN * kTcBK * 4;          // [BN rows][head(32) | tail(32)] halves
  constexpr int kStageBytes = kTcABytes + kBBytes;
  constexpr uint32_t kTmemCols = tc_tmem_cols(2 * BN + STAGES * kTfAColsPerStage);
  constexpr uint32_t kColA = 2 * BN;
  // each rewriter group must own its stages (a group that met a stage only every other use would
  // skip a phase of the stage's barrier and could pass a parity wait one use early)
  static_assert(STAGES % 2 == 0, "two rewriter groups need an even number of stages");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_base = smem + (size_t)STAGES * kStageBytes;
  __shared__ __align__(8) uint64_t full_bar[STAGES], conv_bar[STAGES], empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2], tfree_bar[2];
  __shared__ float scale_ring[kTfScaleRing][kTcBM];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KT = a.K / kTcBK;
  const int tiles_n = a.N / BN;
  const int tiles_m = (a.M + kTcBM - 1) / kTcBM;
  const long long total = (long long)tiles_m * tiles_n;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&conv_bar[s], kTcRewriteThreads);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tfree_bar[b], kTfFoldThreads); }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  auto stage_ptr = [&](int s) { return smem + (size_t)s * kStageBytes; };
  auto fail = [&](int code) { atomicExch(status, code); abort_s = 1; };

  if (warp < kTcRewriteWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      // ---------------- producer
      if (lane == 0) {
        long long it = 0;
        bool alive = true;
        for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
          const int row0 = (int)(tile / tiles_n) * kTcBM, col0 = (int)(tile % tiles_n) * BN;
          for (int kt = 0; kt < KT; ++kt, ++it) {
            const int s = (int)(it % STAGES);
            if (it >= STAGES &&
                !mbar_wait_abortable(&empty_bar[s], (uint32_t)((it / STAGES) - 1) & 1, &abort_s)) {
              fail(kTcTimeoutMma);
              alive = false;
              break;
            }
            uint8_t* st = stage_ptr(s);
            mbar_expect_tx(&full_bar[s], kTcABytes + kBBytes);
            tma_load_2d(st, &maps.a, kt * kTcBK, row0, &full_bar[s]);
            tma_load_2d(st + kTcABytes, &maps.bhi, kt * kTcBK, col0, &full_bar[s]);
          }
        }
        if (abort_s != 0)
          for (long long j = (it > STAGES ? it - STAGES : 0); j < it; ++j)
            mbar_wait(&full_bar[j % STAGES], (uint32_t)(j / STAGES) & 1);
      }
    } else if (warp == kTcIssueWarp) {
      // ---------------- issuer: six kind::f16 UMMAs per k-tile, one k-tile per accumulator
      if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_f16_n(BN);
        long long it = 0, fc = 0;      // k-tiles and folds issued so far
        bool alive = true;
        for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
          for (int kt = 0; kt < KT; ++kt, ++it) {
            const int s = (int)(it % STAGES), buf = (int)(fc & 1);
            const bool first = (kt % FOLD) == 0;
            if (!mbar_wait_abortable(&conv_bar[s], (uint32_t)(it / STAGES) & 1, &abort_s) ||
                (first && fc >= 2 &&
                 !mbar_wait_abortable(&tfree_bar[buf], (uint32_t)((fc >> 1) - 1) & 1, &abort_s))) {
              fail(kTcTimeoutMma);
              alive = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t b = smem_u32(stage_ptr(s)) + kTcABytes;
            const uint32_t tacc = tmem_base + (uint32_t)(buf * BN);
            const uint32_t ta = tmem_base + kColA + (uint32_t)(s * kTfAColsPerStage);
            // small terms first: tail x head, head x tail, then head x head
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
              umma_f16_ts(tacc, ta + 16 + ks * 8, umma_desc_sw128(b + ks * 32), idesc, (ks > 0 || !first) ? 1u : 0u);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
              umma_f16_ts(tacc, ta + ks * 8, umma_desc_sw128(b + 64 + ks * 32), idesc, 1u);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
              umma_f16_ts(tacc, ta + ks * 8, umma_desc_sw128(b + ks * 32), idesc, 1u);
            umma_commit(&empty_bar[s]);
            if ((kt % FOLD) == FOLD - 1 || kt == KT - 1) {
              umma_commit(&tfull_bar[buf]);
              ++fc;
            }
          }
        }
      }
    }
  } else if (warp < kTfFoldWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    // ---------------- rewriters: thread = row of the tile = TMEM lane; group g takes the k-tiles
    // with it % 2 == g
    const int rt = (warp & 3) * 32 + lane, rgrp = (warp - kTcRewriteWarp0) >> 2;
    long long it = 0;
    bool alive = true;
    for (long long tile = blockIdx.x; tile < total && alive; tile += gridDim.x) {
      int e_row = 0;
      if (FOLD > 1) {
        const int arow = (int)(tile / tiles_n) * kTcBM + rt;
        e_row = arow < a.M ? a.a_expo[arow] : 0;
      }
      for (int kt = 0; kt < KT; ++kt, ++it) {
        if ((int)(it & 1) != rgrp) continue;
        const int s = (int)(it % STAGES);
        if (!__all_sync(0xffffffffu,
                        mbar_wait_abortable(&full_bar[s], (uint32_t)(it / STAGES) & 1, &abort_s))) {
          if (lane == 0) fail(kTcTimeoutLoad);
          alive = false;
          break;
        }
        const float4* rowp = reinterpret_cast<const float4*>(stage_ptr(s) + rt * 128);
        float4 x[8];
        float mx = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          x[c] = rowp[c ^ (rt & 7)];
          mx = fmaxf(fmaxf(mx, fmaxf(fabsf(x[c].x), fabsf(x[c].y))), fmaxf(fabsf(x[c].z), fabsf(x[c].w)));
        }
        // power of two that brings the row's largest entry of this k-tile into [2^14, 2^15)
        // (the tails then keep their bits for entries down to 2^-18 of the largest)
        int e = 0;
        if (FOLD > 1) e = e_row;
        else if (mx > 0.f && isfinite(mx)) e = max((int)((__float_as_uint(mx) >> 23) & 0xff) - 141, -126);
        const float down = __uint_as_float((uint32_t)(127 - e) << 23);
        if (FOLD == 1) scale_ring[it & (kTfScaleRing - 1)][rt] = __uint_as_float((uint32_t)(127 + e) << 23);
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
        tmem_st32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + kColA +
                      (uint32_t)(s * kTfAColsPerStage), av);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(&conv_bar[s]);
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ---------------- folders + epilogue: thread = row of the tile, all BN accumulator columns
    const int q = warp & 3;
    const bool issuer_thread = (q == 0 && lane == 0);
    uint8_t* epi = epi_base;
    bool ok = true;
    long long it = 0;       // folds consumed so far (k-tiles when FOLD == 1)
    const int folds = (KT + FOLD - 1) / FOLD;
    for (long long tile = blockIdx.x; tile < total; tile += gridDim.x) {
      const int row0 = (int)(tile / tiles_n) * kTcBM, col0 = (int)(tile % tiles_n) * BN;
      float acc[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      // one scale per row for the whole K, applied in the epilogue
      float row_scale = 1.f;
      if (FOLD > 1 && row0 + q * 32 + lane < a.M)
        row_scale = __uint_as_float((uint32_t)(127 + a.a_expo[row0 + q * 32 + lane]) << 23);
      for (int kt = 0; kt < folds; ++kt, ++it) {
        if (!ok) continue;
        const int buf = (int)(it & 1);
        if (!mbar_wait_abortable(&tfull_bar[buf], (uint32_t)(it >> 1) & 1, &abort_s)) {
          if (lane == 0) fail(kTcTimeoutMma);
          ok = false;
          continue;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float sc = FOLD > 1 ? 1.f : scale_ring[it & (kTfScaleRing - 1)][q * 32 + lane];
        const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 64) {
          uint32_t v0[32], v1[32];
          tmem_ld32(v0, t0 + c0);
          tmem_ld32(v1, t0 + c0 + 32);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (c0 + 64 == BN) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&tfree_bar[buf]);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            acc[c0 + j] = fmaf(__uint_as_float(v0[j]), sc, acc[c0 + j]);
            acc[c0 + 32 + j] = fmaf(__uint_as_float(v1[j]), sc, acc[c0 + 32 + j]);
          }
        }
      }
      if (FOLD > 1) {
#pragma unroll
        for (int j = 0; j < BN; ++j) acc[j] *= row_scale;
      }
      // ---- epilogue of this tile, two 128 x 32 sub-tiles at a time
      const bool tma_out = (EPI != kEpiResidual) || (a.R == a.C);
      const int rloc = q * 32 + lane;
      const int row = row0 + rloc;
      const float* hrow = nullptr;
      if (EPI == kEpiNodeScale && row < a.M) hrow = a.h + (size_t)gemm_node_of_row(a, row) * a.N + col0;
      float* tilebuf = reinterpret_cast<float*>(epi);
#pragma unroll
      for (int half = 0; half < BN / 64; ++half) {
        // the bulk stores issued for the previous pair of sub-tiles must have read the buffer
        if (issuer_thread) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ok && tma_out) {
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const int j = (half * 2 + sub) * 32 + c * 4;
              const float4 w4 = *reinterpret_cast<const float4*>(b_scale + col0 + j);
              float4 o = make_float4(acc[j] * w4.x, acc[j + 1] * w4.y, acc[j + 2] * w4.z, acc[j + 3] * w4.w);
              if (EPI == kEpiNodeScale && hrow != nullptr) {
                const float4 hh = *reinterpret_cast<const float4*>(hrow + j);
                o.x *= hh.x; o.y *= hh.y; o.z *= hh.z; o.w *= hh.w;
              }
              *reinterpret_cast<float4*>(tilebuf + sub * 4096 + rloc * 32 + ((c ^ (rloc & 7)) << 2)) = o;
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer_thread && ok && tma_out && abort_s == 0) {
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            const int cx = col0 + (half * 2 + sub) * 32;
            const uint32_t src = smem_u32(epi) + sub * 16384;
            if (EPI == kEpiScatter) {
              const int wk0 = (row0 / kTcBM) * 8;
              asm volatile(
                  "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                  ::"l"(reinterpret_cast<uint64_t>(&maps.c)), "r"(cx), "r"(a.sc_j0), "r"(wk0), "r"(src)
                  : "memory");
              asm volatile(
                  "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                  ::"l"(reinterpret_cast<uint64_t>(&maps.c2)), "r"(cx), "r"(a.sc_u), "r"(wk0),
                    "r"(src + 96 * 128)
                  : "memory");
              asm volatile(
                  "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                  ::"l"(reinterpret_cast<uint64_t>(&maps.c2)), "r"(cx), "r"(a.sc_l), "r"(wk0),
                    "r"(src + 104 * 128)
                  : "memory");
            } else if (EPI == kEpiResidual) {
              asm volatile(
                  "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                  ::"l"(reinterpret_cast<uint64_t>(&maps.c)), "r"(cx), "r"(row0), "r"(src)
                  : "memory");
            } else {
              asm volatile(
                  "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                  ::"l"(reinterpret_cast<uint64_t>(&maps.c)), "r"(cx), "r"(row0), "r"(src)
                  : "memory");
            }
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      if (ok && !tma_out && row < a.M) {
        float* crow = a.C + (size_t)row * a.ldc + col0;
#pragma unroll
        for (int j = 0; j < BN; j += 4) {
          const float4 rr = *reinterpret_cast<const float4*>(a.R + (size_t)row * a.ldc + col0 + j);
          const float4 w4 = *reinterpret_cast<const float4*>(b_scale + col0 + j);
          *reinterpret_cast<float4*>(crow + j) =
              make_float4(fmaf(acc[j], w4.x, rr.x), fmaf(acc[j + 1], w4.y, rr.y),
                          fmaf(acc[j + 2], w4.z, rr.z), fmaf(acc[j + 3], w4.w, rr.w));
        }
      }
    }
    if (issuer_thread) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

template <int BN, int STAGES, int FOLD>
int launch_gemm_tcf_bn(int epi, const GemmArgs& a, const float* packed, const float* b_scale,
                       int* status, cudaStream_t stream) {
  if (FOLD > 1) {
    gemm_row_expo_kernel<<<(a.M + 7) / 8, 256, 0, stream>>>(a.A, a.M, a.K, a.lda, a.a_expo);
    HZ_CUDA_TRY(cudaGetLastError());
  }
  TcMaps maps;
  if (!make_map(&maps.a, a.A, a.M, a.K, a.lda, kTcBM) ||
      !make_map(&maps.bhi, packed, a.N, a.K, a.K, BN))
    return HZ_ERR_CUDA;
  maps.blo = maps.bhi;
  if (epi == kEpiScatter) {
    if (a.ldc != a.N ||
        !make_map3(&maps.c, a.C, a.sc_walkers, a.sc_rows, a.N, 12, 8) ||
        !make_map3(&maps.c2, a.C, a.sc_walkers, a.sc_rows, a.N, 1, 8))
      return HZ_ERR_CUDA;
  } else {
    if (!make_map(&maps.c, a.C, a.M, a.N, a.ldc, kTcBM)) return HZ_ERR_CUDA;
    maps.c2 = maps.c;
  }
  constexpr size_t smem = (size_t)STAGES * (kTcABytes + BN * kTcBK * 4) + kTcEpiBytes + 1024;
  const long long total = (long long)(a.N / BN) * ((a.M + kTcBM - 1) / kTcBM);
  const int sms = tc_sm_count();
  const unsigned grid = (unsigned)(total < sms ? total : sms);
#define HZ_TCF_LAUNCH(E)                                                                         \
  do {                                                                                           \
    const int hz_rc__ = ensure_kernel_attributes(                                                \
        reinterpret_cast<const void*>(gemm_tcf_kernel<BN, STAGES, E, FOLD>), (int)smem);         \
    if (hz_rc__ != HZ_OK) return hz_rc__;                                                        \
    gemm_tcf_kernel<BN, STAGES, E, FOLD><<<grid, kTfThreads, smem, stream>>>(maps, a, b_scale, status); \
  } while (0)
  switch (epi) {
    case kEpiStore: HZ_TCF_LAUNCH(kEpiStore); break;
    case kEpiNodeScale: HZ_TCF_LAUNCH(kEpiNodeScale); break;
    case kEpiScatter: HZ_TCF_LAUNCH(kEpiScatter); break;
    default: HZ_TCF_LAUNCH(kEpiResidual); break;
  }
#undef HZ_TCF_LAUNCH
  HZ_CUDA_TRY(cudaGetLastError());
  return HZ_OK;
}

// The FP16-split GEMM for weights prepared by prepare_weights_f16 (packed in `packed`, scale in
// b_scale[0]); HZ_GEMM_KIND=tf32 keeps every GEMM on the three-term TF32 split.
inline bool use_f16_gemm() {
  static const bool on = !env_equals("HZ_GEMM_KIND", "tf32");
  return on && use_persistent_tc();
}
inline int launch_gemm_tcf(int epi, const GemmArgs& a, const float* packed, const float* b_scale,
                           int* status, cudaStream_t stream) {
  if (a.M <= 0) return HZ_OK;
  // k-tiles per TMEM accumulator when the caller gave room for the row exponents: 8 by default
  // (chains of 48 UMMAs between two folds); HZ_GEMM_F16_FOLD = 1, 2 or 4 for A/B runs
  static const int fold = env_int("HZ_GEMM_F16_FOLD", 8);
  if (a.a_expo != nullptr && a.K % 4 == 0 && a.lda % 4 == 0) {
    if (fold == 8) return launch_gemm_tcf_bn<128, 4, 8>(epi, a, packed, b_scale, status, stream);
    if (fold == 4) return launch_gemm_tcf_bn<128, 4, 4>(epi, a, packed, b_scale, status, stream);
    if (fold == 2) return launch_gemm_tcf_bn<128, 4, 2>(epi, a, packed, b_scale, status, stream);
  }
  return launch_gemm_tcf_bn<128, 4, 1>(epi, a, packed, b_scale, status, stream);
}

// bt_hi / bt_lo: B transposed and split ([N,K] each). `status` is a device int that a kernel
// sets to a TcStatus value when one of its bounded waits runs out.
inline int launch_gemm_tc(int epi, const GemmArgs& a, const float* bt_hi, const float* bt_lo,
                          int* status, cudaStream_t stream) {
  if (a.M <= 0) return HZ_OK;
  if (use_persistent_tc()) {
    const int mode = tmem_operand_mode();
    // k-tiles that share one TMEM accumulator before the fold into fp32 registers: 2 by default
    // (chains of 24 UMMAs, truncation bias about 1e-6 of a result); HZ_GEMM_FOLD=1 or 4 for A/B runs
    static const int fold = env_int("HZ_GEMM_FOLD", 2);
    if (mode == 2 && fold == 2) return launch_gemm_tcp_bn<128, 4, 2, 2>(epi, a, bt_hi, bt_lo, status, stream);
    if (mode == 2 && fold == 4) return launch_gemm_tcp_bn<128, 4, 2, 4>(epi, a, bt_hi, bt_lo, status, stream);
    if (mode == 2) return launch_gemm_tcp_bn<128, 4, 2, 1>(epi, a, bt_hi, bt_lo, status, stream);
    if (mode == 1) return launch_gemm_tcp_bn<128, 4, 1, 1>(epi, a, bt_hi, bt_lo, status, stream);
    return launch_gemm_tcp_bn<128, 3, 0, 1>(epi, a, bt_hi, bt_lo, status, stream);
  }
  return launch_gemm_tc_bn<128, 3>(epi, a, bt_hi, bt_lo, status, stream);
}

}  // namespace hz
