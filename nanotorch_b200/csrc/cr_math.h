// fp32 tanh and sigmoid evaluated in double precision and rounded once.
//
// tanh: the result is the correctly rounded
// float except for a vanishing fraction of arguments, which keeps it within 2 ulp of the host libm's
// tanhf (glibc 2.39's tanhf is itself at most 2 ulp from the correctly rounded value; both facts are
// checked by tests/test_tanh_restatement.py over 10^8 arguments on the host).  One evaluation path
// for every finite argument, about 85 instructions per element instead of the 130 of the bit-exact
// restatement in tanh_exact.h:
//     |x| <  2^-6 :  x - x^3/3 + 2x^5/15 - 17x^7/315                    (truncation < 2^-53 relative)
//     otherwise   :  E = exp(-2|x|) = 2^k e^r (Cody-Waite, degree-13 Taylor), tanh|x| = (1 - E) / (1 + E)
// sigmoid: 1 / (1 + exp(-x)) in double, rounded once: the reference computes the same expression in three
// rounded fp32 steps on top of libm's expf (src/cpp/ops/unary_ops.cu:107; total error <= 1.5 ulp), so the
// correctly rounded value is within 2 ulp of it; where expf(-x) overflows (x <= -88.7228394) the reference returns
// 1/inf = 0 and so does this.
// Only IEEE double +, *, fma, rint, a correctly rounded fp32 reciprocal and an integer add on the exponent
// field are used, so host and device return the same bits.
#pragma once

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define NT_TF_HD __host__ __device__ __forceinline__
#else
#define NT_TF_HD static inline
#endif

// p * 2^k for a normal p and a k that keeps the result normal: one integer add on the exponent field
NT_TF_HD double nt_tf_scale(double p, int k) {
#if defined(__CUDA_ARCH__)
  return __hiloint2double(__double2hiint(p) + k * 1048576, __double2loint(p));
#else
  uint64_t bits;
  memcpy(&bits, &p, 8);
  bits += (uint64_t)(int64_t)k << 52;
  memcpy(&p, &bits, 8);
  return p;
#endif
}

// exp(a) for a in [-700, 0.5]: 2^k * e^r, Cody-Waite reduction, degree-13 Taylor (truncation < 2^-58)
NT_TF_HD double nt_tf_exp(double a) {
  const double kd = rint(a * 1.4426950408889634074);
  const double r = fma(kd, -1.90821492927058770002e-10, fma(kd, -6.93147180369123816490e-01, a));
  double p = 1.0 / 6227020800.0;
  p = fma(p, r, 1.0 / 479001600.0);
  p = fma(p, r, 1.0 / 39916800.0);
  p = fma(p, r, 1.0 / 3628800.0);
  p = fma(p, r, 1.0 / 362880.0);
  p = fma(p, r, 1.0 / 40320.0);
  p = fma(p, r, 1.0 / 5040.0);
  p = fma(p, r, 1.0 / 720.0);
  p = fma(p, r, 1.0 / 120.0);
  p = fma(p, r, 1.0 / 24.0);
  p = fma(p, r, 1.0 / 6.0);
  p = fma(p, r, 0.5);
  p = fma(p, r, 1.0);
  p = fma(p, r, 1.0);
  return nt_tf_scale(p, (int)kd); // p in [0.70, 1.42], k >= -1010: the result stays a normal double
}

// num / den for den in [1, 2]: a correctly rounded fp32 reciprocal as the seed, two residual corrections
// (each squares the relative error: 2^-23 -> 2^-46 -> below the rounding of the last fma).  Replaces the
// double-precision division, which is several times as many instructions on the GPU.
NT_TF_HD double nt_tf_div(double num, double den) {
#if defined(__CUDA_ARCH__)
  const double r = (double)__frcp_rn((float)den);
#else
  const double r = (double)(1.0f / (float)den);
#endif
  double q = num * r;
  q = fma(fma(-q, den, num), r, q);
  q = fma(fma(-q, den, num), r, q);
  return q;
}

NT_TF_HD float nt_sigmoid_f32(float xf) {
  if (!(xf == xf)) return xf + xf;                   // NaN
  if (xf <= -88.72283935546875f) return 0.0f;        // expf(-x) = inf in the reference from this float on: 1 / inf
  if (xf > 40.0f) return 1.0f;                       // 1 + exp(-x) rounds to 1 long before
  const double x = (double)xf;
  // exp of a non-positive argument only: sigmoid(x) = 1/(1+E) for x >= 0, E/(1+E) for x < 0, E = exp(-|x|)
  const double E = nt_tf_exp(-fabs(x));
  const double num = (xf >= 0.0f) ? 1.0 : E;
  return (float)nt_tf_div(num, 1.0 + E);
}

NT_TF_HD float nt_tanh_fast_f32(float xf) {
  if (!(xf == xf)) return xf + xf;            // NaN
  const double ax = fabs((double)xf);
  // small arguments: odd Taylor polynomial
  const double x2 = ax * ax;
  double ps = -17.0 / 315.0;
  ps = fma(ps, x2, 2.0 / 15.0);
  ps = fma(ps, x2, -1.0 / 3.0);
  ps = fma(ps, x2, 1.0);
  const double t_small = ax * ps;
  // E = exp(-2|x|); beyond |x| = 20 the quotient rounds to 1.0f whatever E is, so the argument is clamped
  const double E = nt_tf_exp(fmax(-2.0 * ax, -40.0));
  const double t_big = nt_tf_div(1.0 - E, 1.0 + E);
  const float tf = (float)((ax < 0.015625) ? t_small : t_big);
  return copysignf(tf, xf);                   // tanh is odd; keeps the sign of zero
}
