// Warp-level tensor-core helpers shared by the hz_b200 kernels.
//
// All contractions on this path must stay within fp32 tolerance of an fp32
// reference, so each fp32 operand is split into a TF32 head and a TF32 tail and
// a product is formed from three TF32 MMAs (tail*head + head*tail + head*head)
// accumulated in fp32. The dropped tail*tail term is below 2^-22 relative.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hz {

// Round to TF32 (10 explicit mantissa bits) with two integer operations. The conversion
// instruction cvt.rna.tf32.f32 runs on the transcendental unit at a quarter of the ALU rate and
// was the measured limit of the split (that pipe busier than the tensor pipe); the integer form
// rounds half away from zero in the same way for every finite value that does not overflow.
__device__ __forceinline__ uint32_t to_tf32(float x) {
  return (__float_as_uint(x) + 0x1000u) & 0xFFFFE000u;
}

// x = hi + lo with hi, lo representable in TF32 (lo carries the next 11 bits, rounded: the
// tensor core would truncate an unrounded tail, a bias that adds up over long contractions).
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  hi = to_tf32(x);
  lo = to_tf32(x - __uint_as_float(hi));
}

// D(16x8) += A(16x8, row) * B(8x8, col), TF32 in, fp32 accumulate.
// Fragment ownership for lane = 4*g + t (g = lane>>2, t = lane&3):
//   a0:(g, t)  a1:(g+8, t)  a2:(g, t+4)  a3:(g+8, t+4)
//   b0:(k=t, n=g)  b1:(k=t+4, n=g)
//   c0:(g, 2t)  c1:(g, 2t+1)  c2:(g+8, 2t)  c3:(g+8, 2t+1)
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4],
                                         const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

struct FragA {
  uint32_t hi[4], lo[4];
  __device__ __forceinline__ void set(float a0, float a1, float a2, float a3) {
    split_tf32(a0, hi[0], lo[0]);
    split_tf32(a1, hi[1], lo[1]);
    split_tf32(a2, hi[2], lo[2]);
    split_tf32(a3, hi[3], lo[3]);
  }
};

struct FragB {
  uint32_t hi[2], lo[2];
  __device__ __forceinline__ void set(float b0, float b1) {
    split_tf32(b0, hi[0], lo[0]);
    split_tf32(b1, hi[1], lo[1]);
  }
};

// c += a*b to fp32 accuracy: small terms first.
__device__ __forceinline__ void mma3(float (&c)[4], const FragA& a, const FragB& b) {
  mma_tf32(c, a.lo, b.hi);
  mma_tf32(c, a.hi, b.lo);
  mma_tf32(c, a.hi, b.hi);
}

// D(16x8) += A(16x16, row) * B(16x8, col), FP16 in, fp32 accumulate. Fragments, lane = 4g + t:
//   a0:(g; 2t,2t+1)  a1:(g+8; 2t,2t+1)  a2:(g; 2t+8,2t+9)  a3:(g+8; 2t+8,2t+9)
//   b0:(k=2t,2t+1; n=g)  b1:(k=2t+8,2t+9; n=g); the lower k index sits in the low half
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4],
                                        const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// (x, y) -> packed FP16 heads and packed FP16 tails scaled by 2^11 (x in the low half). With the
// scaling a tail has the magnitude range of its head, so it does not underflow for small
// operands; the products that contain a tail are accumulated apart and weighted by 2^-11.
__device__ __forceinline__ void split_f16x2_scaled(float x, float y, uint32_t& hi, uint32_t& lo) {
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(y), "f"(x));
  float xh, yh;
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}"
      : "=f"(xh), "=f"(yh) : "r"(hi));
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"((y - yh) * 2048.f), "f"((x - xh) * 2048.f));
}

__device__ __forceinline__ float quad_max(float x) {
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
  return x;
}

__device__ __forceinline__ float quad_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

}  // namespace hz
