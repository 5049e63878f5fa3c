// tanh for fp32, identical bit for bit to the fdlibm algorithm (tanh through expm1) that the host
// libm of the reference's CPU path implements (glibc 2.39: sysdeps/ieee754/flt-32/s_tanhf.c and
// s_expm1f.c are the fdlibm float versions).  Only IEEE-754 binary32 +, -, *, / and integer bit
// operations are used, so any conforming target -- the GPU's FADD/FMUL/div.rn included -- returns the
// same bits as long as no multiply-add is contracted (the library is built with --fmad=false; the host
// check with -ffp-contract=off).
//
// The published algorithm is a tree of branches (argument ranges, k == 0, k == +-1, k < 23, ...).  A
// warp executing it on N(0,1) data visits nearly every branch, and tanh's two call sites of expm1
// double the work.  This restatement evaluates ONE expm1 body per element with selects:
//   - tanh's two branches share one expm1 of a = (|x| >= 1 ? 2|x| : -2|x|) and one division q = num / (t + 2)
//     with num = (|x| >= 1 ? 2 : t):  z = |x| >= 1 ? 1 - q : -q   [-(t/d) == (-t)/d exactly];
//   - the argument reduction always takes the general form hi = a - k*ln2_hi, lo = k*ln2_lo, with k
//     forced to +-1 (resp. 0) in the ranges where the original special-cases it: for those k the general
//     form produces the very same hi, lo (k*ln2_hi is exact) and c;
//   - the k == 0 result x - (x*e - hxs) equals the general x - e' because c == 0 there.
// tests/test_tanh_restatement.py compiles this header for the host and compares it with the host
// libm's tanhf over a dense sweep of the whole float range.
#pragma once

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define NT_HD __host__ __device__ __forceinline__
#else
#define NT_HD static inline
#endif

NT_HD uint32_t nt_f2u(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
#endif
}
NT_HD float nt_u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}

// expm1(a) for the arguments tanh produces: a in [2, 44) or a in (-2, -0].  NaN/inf never reach it.
NT_HD float nt_expm1_for_tanh(float a) {
  const float ln2_hi = 6.9313812256e-01f, ln2_lo = 9.0580006145e-06f, invln2 = 1.4426950216e+00f,
              Q1 = -3.3333335072e-02f, Q2 = 1.5873016091e-03f, Q3 = -7.9365076090e-05f, Q4 = 4.0082177293e-06f,
              Q5 = -2.0109921195e-07f;
  const uint32_t ua = nt_f2u(a);
  const uint32_t hx = ua & 0x7fffffffu;
  const int neg = (ua >> 31) != 0;
  // k: 0 for |a| <= 0.5 ln2, +-1 for |a| < 1.5 ln2, else trunc(a / ln2 +- 0.5)
  int k = (int)(invln2 * a + (neg ? -0.5f : 0.5f));
  if (hx < 0x3F851592u) k = -1; // only negative arguments are this small (positive ones are >= 2)
  if (hx <= 0x3eb17218u) k = 0;
  const float t = (float)k;
  const float hi = a - t * ln2_hi;
  const float lo = t * ln2_lo;
  const float x = hi - lo;
  const float c = (hi - x) - lo;
  const float hfx = 0.5f * x;
  const float hxs = x * hfx;
  const float r1 = 1.0f + hxs * (Q1 + hxs * (Q2 + hxs * (Q3 + hxs * (Q4 + hxs * Q5))));
  const float tt = 3.0f - r1 * hfx;
  float e = hxs * ((r1 - tt) / (6.0f - x * tt));
  e = (x * (e - c) - c);
  e -= hxs;
  float res;
  if (k == 0) {
    res = x - e;
  } else if (k == -1) {
    res = 0.5f * (x - e) - 0.5f;
  } else if (k <= -2 || k > 56) { // (k == 1 cannot occur: a positive argument is >= 2, so k >= 3)
    float y = 1.0f - (e - x);
    y = nt_u2f(nt_f2u(y) + ((uint32_t)k << 23));
    res = y - 1.0f;
  } else if (k < 23) {
    const float s = nt_u2f(0x3f800000u - (0x1000000u >> k));
    float y = s - (e - x);
    res = nt_u2f(nt_f2u(y) + ((uint32_t)k << 23));
  } else {
    const float s = nt_u2f((uint32_t)(0x7f - k) << 23);
    float y = x - (e + s);
    y += 1.0f;
    res = nt_u2f(nt_f2u(y) + ((uint32_t)k << 23));
  }
  // |a| < 2^-25: the original returns a itself (after raising inexact)
  if (hx < 0x33000000u) res = a;
  // a < -27 ln2 cannot happen here (a > -2); a >= 27 ln2 with a > 0 runs the general path above
  return res;
}

NT_HD float nt_tanh_f32(float x) {
  const uint32_t jx = nt_f2u(x), ix = jx & 0x7fffffffu;
  const int negx = (jx >> 31) != 0;
  if (ix >= 0x7f800000u) return negx ? 1.0f / x - 1.0f : 1.0f / x + 1.0f; // inf -> +-1, NaN -> NaN
  const float ax = nt_u2f(ix);
  const int big = ix >= 0x3f800000u; // |x| >= 1
  // clamp the argument of the shared expm1 for lanes whose result is replaced below
  const float arg = big ? 2.0f * ax : -2.0f * ax;
  const float t = nt_expm1_for_tanh((ix < 0x41b00000u) ? arg : 2.0f);
  const float q = (big ? 2.0f : t) / (t + 2.0f);
  float z = big ? 1.0f - q : -q;
  if (ix >= 0x41b00000u) z = 1.0f;                 // |x| >= 22: 1 - tiny rounds to 1
  if (ix < 0x24000000u) return x * (1.0f + x);     // |x| < 2^-55 (covers x == +-0: returns x)
  return negx ? -z : z;
}
