// fp32 sigmoid in fp32 arithmetic: the reference's own three rounded steps, 1 / (1 + expf(-x))
// (src/cpp/ops/unary_ops.cu:107), on top of an exponential accurate to 0.52 ulp.
//
//   e = exp(-x):  N = round(-x * 64 / ln 2) by the add-a-large-constant trick, r = -x - N ln2/64 with a
//                 two-constant Cody-Waite reduction (the first product is exact), N = 64 k + j,
//                 2^(j/64) = hi + lo from a 64-entry table of float pairs, e^r - 1 = r + r^2 (1/2 + r/6)
//                 (|r| <= ln2/128, truncation below 2^-34), e = 2^k (hi + (lo + hi (e^r - 1))): one rounding of
//                 consequence, the last addition;
//   s = 1 + e, result = 1 / s: IEEE addition and a correctly rounded reciprocal, as the reference rounds them.
//
// Where this exponential and the host libm's expf round differently (1 argument in 9000, by one ulp: both are
// within 0.53 ulp of the true value) the result moves by at most 2 ulp -- except for exp(-x) in [2^24, 2^25),
// where 1 + e is always a rounding tie; all of x <= -16.625 therefore takes the double-precision evaluation
// of cr_math.h.  tests/test_tanh_restatement.py walks all 2^32 arguments on the host against the reference's
// expression on the host libm (NT_EXHAUSTIVE=1): worst distance 2 ulp.  Only fmaf, +, *, a correctly rounded
// reciprocal, a table look-up and integer operations: host and device return the same bits.
// The table is printed by gen_exp2f_table.py.
#pragma once

#include <math.h>
#include <stdint.h>
#include <string.h>

#include "cr_math.h"

#if defined(__CUDACC__)
#define NT_SG_HD __host__ __device__ __forceinline__
#else
#define NT_SG_HD static inline
#endif

#define NT_SG_EXP2F_TABLE \
  {0x1.0000000000000p+0f, 0x0.0p+0f}, \
  {0x1.02c9a40000000p+0f, -0x1.887fa00000000p-28f}, \
  {0x1.059b0e0000000p+0f, -0x1.9d4f520000000p-25f}, \
  {0x1.0874520000000p+0f, -0x1.e2990e0000000p-26f}, \
  {0x1.0b55860000000p+0f, 0x1.9f31220000000p-25f}, \
  {0x1.0e3ec40000000p+0f, -0x1.a585cc0000000p-25f}, \
  {0x1.11301e0000000p+0f, -0x1.fdb4960000000p-25f}, \
  {0x1.1429aa0000000p+0f, 0x1.d525bc0000000p-25f}, \
  {0x1.172b840000000p+0f, -0x1.c157420000000p-27f}, \
  {0x1.1a35be0000000p+0f, 0x1.6df96e0000000p-25f}, \
  {0x1.1d48740000000p+0f, -0x1.d2e8ca0000000p-25f}, \
  {0x1.2063b80000000p+0f, 0x1.0c519a0000000p-25f}, \
  {0x1.2387a60000000p+0f, 0x1.ceac480000000p-25f}, \
  {0x1.26b4560000000p+0f, 0x1.789f380000000p-26f}, \
  {0x1.29e9e00000000p+0f, -0x1.5c04240000000p-25f}, \
  {0x1.2d285a0000000p+0f, 0x1.b900c20000000p-26f}, \
  {0x1.306fe00000000p+0f, 0x1.4636e20000000p-25f}, \
  {0x1.33c08c0000000p+0f, -0x1.b37d200000000p-25f}, \
  {0x1.371a740000000p+0f, -0x1.18aac60000000p-25f}, \
  {0x1.3a7db40000000p+0f, -0x1.634c020000000p-25f}, \
  {0x1.3dea640000000p+0f, 0x1.8246840000000p-25f}, \
  {0x1.4160a20000000p+0f, 0x1.f72e2a0000000p-28f}, \
  {0x1.44e0860000000p+0f, 0x1.8624b40000000p-30f}, \
  {0x1.486a2c0000000p+0f, -0x1.47d8660000000p-25f}, \
  {0x1.4bfdae0000000p+0f, -0x1.593abc0000000p-25f}, \
  {0x1.4f9b280000000p+0f, -0x1.2c5a6c0000000p-25f}, \
  {0x1.5342b60000000p+0f, -0x1.2c56100000000p-25f}, \
  {0x1.56f4740000000p+0f, -0x1.295b040000000p-25f}, \
  {0x1.5ab07e0000000p+0f, -0x1.5bd5ec0000000p-27f}, \
  {0x1.5e76f20000000p+0f, -0x1.4a5bd60000000p-25f}, \
  {0x1.6247ec0000000p+0f, -0x1.f8b5500000000p-25f}, \
  {0x1.6623880000000p+0f, 0x1.2a91120000000p-27f}, \
  {0x1.6a09e60000000p+0f, 0x1.9fcef40000000p-26f}, \
  {0x1.6dfb240000000p+0f, -0x1.cd72e80000000p-27f}, \
  {0x1.71f75e0000000p+0f, 0x1.1d8bee0000000p-25f}, \
  {0x1.75feb60000000p+0f, -0x1.37b3060000000p-25f}, \
  {0x1.7a11480000000p+0f, -0x1.829fd00000000p-25f}, \
  {0x1.7e2f340000000p+0f, -0x1.2616340000000p-25f}, \
  {0x1.82589a0000000p+0f, -0x1.accc7c0000000p-26f}, \
  {0x1.868d9a0000000p+0f, -0x1.2edb440000000p-26f}, \
  {0x1.8ace540000000p+0f, 0x1.15506e0000000p-27f}, \
  {0x1.8f1aea0000000p+0f, -0x1.baa2320000000p-26f}, \
  {0x1.93737c0000000p+0f, -0x1.e647440000000p-25f}, \
  {0x1.97d82a0000000p+0f, -0x1.0d8d840000000p-31f}, \
  {0x1.9c49180000000p+0f, 0x1.51f8480000000p-27f}, \
  {0x1.a0c6680000000p+0f, -0x1.2886a60000000p-26f}, \
  {0x1.a5503c0000000p+0f, -0x1.b83b540000000p-25f}, \
  {0x1.a9e6b60000000p+0f, -0x1.50c0480000000p-25f}, \
  {0x1.ae89fa0000000p+0f, -0x1.a94b140000000p-26f}, \
  {0x1.b33a2c0000000p+0f, -0x1.ec3a820000000p-26f}, \
  {0x1.b7f7700000000p+0f, -0x1.a094380000000p-25f}, \
  {0x1.bcc1ea0000000p+0f, -0x1.f687c60000000p-25f}, \
  {0x1.c199be0000000p+0f, -0x1.3d56b20000000p-27f}, \
  {0x1.c67f120000000p+0f, 0x1.cafa2a0000000p-25f}, \
  {0x1.cb720e0000000p+0f, -0x1.8837cc0000000p-27f}, \
  {0x1.d072d40000000p+0f, 0x1.40f1300000000p-25f}, \
  {0x1.d5818e0000000p+0f, -0x1.822dbc0000000p-27f}, \
  {0x1.da9e600000000p+0f, 0x1.ed99420000000p-27f}, \
  {0x1.dfc9740000000p+0f, -0x1.908c940000000p-25f}, \
  {0x1.e502ee0000000p+0f, 0x1.e2cffe0000000p-26f}, \
  {0x1.ea4afa0000000p+0f, 0x1.52486c0000000p-27f}, \
  {0x1.efa1be0000000p+0f, 0x1.cc2b440000000p-25f}, \
  {0x1.f507660000000p+0f, -0x1.246eb00000000p-26f}, \
  {0x1.fa7c180000000p+0f, 0x1.9e90d80000000p-28f}, \


#if defined(__CUDACC__)
static __device__ const float2 nt_sg_exp2f_dev[64] = {NT_SG_EXP2F_TABLE};
#endif
static const float nt_sg_exp2f_host[64][2] = {NT_SG_EXP2F_TABLE};

// exp(a) for a in [-40, 17] (any a whose result is a normal float would do): see the file comment.
NT_SG_HD float nt_sg_expf(float a) {
  const float shift = 12582912.0f; // 1.5 * 2^23
  const float t = fmaf(a, 0x1.715476p+6f, shift);
  const float nf = t - shift;
  float r = fmaf(nf, -0x1.62cp-7f, a);        // exact: |N| < 2^14, the constant has 11 bits
  r = fmaf(nf, -0x1.217f7ep-18f, r);          // what is left of ln2/64 after these two is 2^-43: 2^-29 of the result at most
#if defined(__CUDA_ARCH__)
  const int n = __float_as_int(t) - 0x4B400000; // the low mantissa bits of t are N
  const float2 e = __ldg(nt_sg_exp2f_dev + (n & 63));
  const float hi = e.x, lo = e.y;
#else
  int32_t tb;
  memcpy(&tb, &t, 4);
  const int n = tb - 0x4B400000;
  const float hi = nt_sg_exp2f_host[n & 63][0], lo = nt_sg_exp2f_host[n & 63][1];
#endif
  const int k = n >> 6;
  const float r2 = r * r;
  const float h = fmaf(r, 0x1.555556p-3f, 0.5f); // 1/2 + r/6; the next term, r^4/24, is below 2^-34
  const float p = fmaf(r2, h, r);              // e^r - 1
  const float v = hi + fmaf(hi, p, lo);        // 2^(j/64) e^r in [1, 2)
#if defined(__CUDA_ARCH__)
  return __int_as_float(__float_as_int(v) + (k << 23));
#else
  int32_t vb;
  memcpy(&vb, &v, 4);
  vb += k * (1 << 23);
  float out;
  memcpy(&out, &vb, 4);
  return out;
#endif
}

// Everything else takes the double-precision evaluation of cr_math.h (within 2 ulp of the reference for every
// argument): NaN, x >= 40 (1), and x <= -16.625.  The last is not about range: for exp(-x) in [2^24, 2^25)
// 1 + e is a rounding tie for every e, so one ulp of e moves the quotient by up to 4 ulp (102 arguments of
// that window end up 3 or 4 ulp from the reference with the fp32 exponential); one comparison covers the
// window, the results below the normal range and the zeros together.  One out-of-line copy on the device:
// inlined into every element slot of a kernel it would multiply the code size for a path that few arguments take.
#if defined(__CUDACC__)
static __device__ __noinline__ float nt_sg_rare(float x) { return nt_sigmoid_cr_f32(x); }
#endif

NT_SG_HD float nt_sigmoid_f32(float x) {
  if (!(fabsf(x - 11.6875f) < 28.3125f)) { // x outside (-16.625, 40), or NaN
#if defined(__CUDA_ARCH__)
    return nt_sg_rare(x);
#else
    return nt_sigmoid_cr_f32(x);
#endif
  }
  const float s = 1.0f + nt_sg_expf(-x);
#if defined(__CUDA_ARCH__)
  return __frcp_rn(s);
#else
  return 1.0f / s;
#endif
}
