// fp32 tanh and sigmoid evaluated in double precision and rounded once.
//
// tanh: the result is the correctly rounded
// float except for a vanishing fraction of arguments, which keeps it within 2 ulp of the host libm's
// tanhf (glibc 2.39's tanhf is itself at most 2 ulp from the correctly rounded value; both facts are
// checked by tests/test_tanh_restatement.py over 10^8 arguments on the host).  One evaluation path
// for every finite argument, about 50 instructions per element instead of the 130 of the bit-exact
// restatement in tanh_exact.h:
//     |x| <  2^-6 :  x - x^3/3 + 2x^5/15 - 17x^7/315                    (truncation < 2^-53 relative)
//     otherwise   :  E = exp(-2|x|) = 2^k e^r (Cody-Waite, degree-13 Taylor), tanh|x| = (1 - E) / (1 + E)
// sigmoid: 1 / (1 + exp(-x)) in double, rounded once: the reference computes the same expression in three
// rounded fp32 steps on top of libm's expf (src/cpp/ops/unary_ops.cu:107; total error <= 1.5 ulp), so the
// correctly rounded value is within 2 ulp of it; where expf(-x) overflows (x < -88.72) the reference returns
// 1/inf = 0 and so does this.
// Only IEEE double +, *, /, fma and rint are used, so host and device return the same bits.
#pragma once

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define NT_TF_HD __host__ __device__ __forceinline__
#else
#define NT_TF_HD static inline
#endif

NT_TF_HD double nt_tf_pow2(int k) { // 2^k for k in [-1022, 1023]
  const uint64_t bits = (uint64_t)(1023 + k) << 52;
#if defined(__CUDA_ARCH__)
  return __longlong_as_double((long long)bits);
#else
  double d;
  memcpy(&d, &bits, 8);
  return d;
#endif
}

// exp(a) for a in [-745, 0.5]: 2^k * e^r, Cody-Waite reduction, degree-13 Taylor (truncation < 2^-58)
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
  const int k = (int)kd;
  const int k1 = k / 2;
  return (p * nt_tf_pow2(k1)) * nt_tf_pow2(k - k1);
}

NT_TF_HD float nt_sigmoid_f32(float xf) {
  if (!(xf == xf)) return xf + xf;                   // NaN
  if (xf < -88.72283935546875f) return 0.0f;         // expf(-x) = inf in the reference: 1 / inf
  if (xf > 40.0f) return 1.0f;                       // 1 + exp(-x) rounds to 1 long before
  const double x = (double)xf;
  // exp of a non-positive argument only: sigmoid(x) = 1/(1+E) for x >= 0, E/(1+E) for x < 0, E = exp(-|x|)
  const double E = nt_tf_exp(-fabs(x));
  const double num = (xf >= 0.0f) ? 1.0 : E;
  return (float)(num / (1.0 + E));
}

NT_TF_HD float nt_tanh_fast_f32(float xf) {
  if (!(xf == xf)) return xf + xf;            // NaN
  const double x = (double)xf;
  const double ax = fabs(x);
  double t;                                   // tanh(|x|)
  if (ax >= 10.0) {
    t = 1.0;                                  // 1 - 2e-9 rounds to 1.0f well before 10
  } else {
    // small arguments: odd Taylor polynomial
    const double x2 = ax * ax;
    double ps = -17.0 / 315.0;
    ps = fma(ps, x2, 2.0 / 15.0);
    ps = fma(ps, x2, -1.0 / 3.0);
    ps = fma(ps, x2, 1.0);
    const double t_small = ax * ps;
    const double E = nt_tf_exp(-2.0 * ax);   // argument in (-20, 0]
    const double t_big = (1.0 - E) / (1.0 + E);
    t = (ax < 0.015625) ? t_small : t_big;
  }
  const float tf = (float)t;
  return (xf < 0.0f) ? -tf : ((xf == 0.0f) ? xf : tf); // keeps the sign of zero
}
