// The TF32 split of an fp32 value, x = hi + lo to 2^-22 relative with both parts exactly representable
// in TF32: shared by the operand-split kernels of the tensor-core GEMM and by the producers that write
// the planes of their own output while they still hold it in registers.
#pragma once

#include <cstdint>

namespace ntb {

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
// hi = tf32(x), except that a finite x whose rounding would overflow to infinity keeps the largest
// finite TF32 value (the remainder then fits in lo); lo = tf32(x - hi), or 0 when x is not finite
// (inf - inf would turn an infinity into a NaN before any product is formed).
__device__ __forceinline__ float split_hi(float x) {
  float h = tf32_round(x);
  if (isinf(h) && !isinf(x)) h = copysignf(__uint_as_float(0x7F7FE000u), x);
  return h;
}
__device__ __forceinline__ float split_lo(float x, float h) {
  return (__float_as_uint(h) & 0x7F800000u) == 0x7F800000u ? 0.0f : tf32_round(x - h);
}

} // namespace ntb
