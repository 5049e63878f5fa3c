// fp32 tanh evaluated in double precision and rounded once.
//
// tanh: float(tanh(double(x))) for every float argument -- checked exhaustively on the host by
// tests/test_tanh_restatement.py (NT_EXHAUSTIVE=1), which also finds the host libm's tanhf (what the
// reference's CPU path calls, src/cpp/ops/unary_ops.cu:106) never more than 2 ulp away from it.  One
// evaluation path for every finite argument:
//     E - 1 = exp(-2|x|) - 1 from a 64-entry table of 2^(j/64) and a degree-6 polynomial, formed without
//     cancellation near 0;  tanh|x| = -(E - 1) / (2 + (E - 1)).
// (The sigmoid lives in sigmoid_f32.h: fp32 arithmetic, the reference's three rounded steps.)
// Only IEEE double +, *, fma, a correctly rounded fp32 reciprocal, a table look-up and integer adds on the
// exponent field are used, so host and device return the same bits.  About 45 instructions per element
// (the degree-13 polynomial this replaces took 99; the bit-exact restatement in tanh_exact.h takes 130).
#pragma once

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define NT_TF_HD __host__ __device__ __forceinline__
#else
#define NT_TF_HD static inline
#endif

// 2^(j/64), j = 0..63, as an unevaluated sum hi + lo of two doubles (hi = the nearest double, lo = the rest):
// {hi, lo} pairs, one 16-byte load per element.
#define NT_TF_EXP2_TABLE \
  0x1.0000000000000p+0, 0x0.0p+0, \
  0x1.02c9a3e778061p+0, -0x1.19083535b085dp-56, \
  0x1.059b0d3158574p+0, 0x1.d73e2a475b465p-55, \
  0x1.0874518759bc8p+0, 0x1.186be4bb284ffp-57, \
  0x1.0b5586cf9890fp+0, 0x1.8a62e4adc610bp-54, \
  0x1.0e3ec32d3d1a2p+0, 0x1.03a1727c57b53p-59, \
  0x1.11301d0125b51p+0, -0x1.6c51039449b3ap-54, \
  0x1.1429aaea92de0p+0, -0x1.32fbf9af1369ep-54, \
  0x1.172b83c7d517bp+0, -0x1.19041b9d78a76p-55, \
  0x1.1a35beb6fcb75p+0, 0x1.e5b4c7b4968e4p-55, \
  0x1.1d4873168b9aap+0, 0x1.e016e00a2643cp-54, \
  0x1.2063b88628cd6p+0, 0x1.dc775814a8495p-55, \
  0x1.2387a6e756238p+0, 0x1.9b07eb6c70573p-54, \
  0x1.26b4565e27cddp+0, 0x1.2bd339940e9d9p-55, \
  0x1.29e9df51fdee1p+0, 0x1.612e8afad1255p-55, \
  0x1.2d285a6e4030bp+0, 0x1.0024754db41d5p-54, \
  0x1.306fe0a31b715p+0, 0x1.6f46ad23182e4p-55, \
  0x1.33c08b26416ffp+0, 0x1.32721843659a6p-54, \
  0x1.371a7373aa9cbp+0, -0x1.63aeabf42eae2p-54, \
  0x1.3a7db34e59ff7p+0, -0x1.5e436d661f5e3p-56, \
  0x1.3dea64c123422p+0, 0x1.ada0911f09ebcp-55, \
  0x1.4160a21f72e2ap+0, -0x1.ef3691c309278p-58, \
  0x1.44e086061892dp+0, 0x1.89b7a04ef80d0p-59, \
  0x1.486a2b5c13cd0p+0, 0x1.3c1a3b69062f0p-56, \
  0x1.4bfdad5362a27p+0, 0x1.d4397afec42e2p-56, \
  0x1.4f9b2769d2ca7p+0, -0x1.4b309d25957e3p-54, \
  0x1.5342b569d4f82p+0, -0x1.07abe1db13cadp-55, \
  0x1.56f4736b527dap+0, 0x1.9bb2c011d93adp-54, \
  0x1.5ab07dd485429p+0, 0x1.6324c054647adp-54, \
  0x1.5e76f15ad2148p+0, 0x1.ba6f93080e65ep-54, \
  0x1.6247eb03a5585p+0, -0x1.383c17e40b497p-54, \
  0x1.6623882552225p+0, -0x1.bb60987591c34p-54, \
  0x1.6a09e667f3bcdp+0, -0x1.bdd3413b26456p-54, \
  0x1.6dfb23c651a2fp+0, -0x1.bbe3a683c88abp-57, \
  0x1.71f75e8ec5f74p+0, -0x1.16e4786887a99p-55, \
  0x1.75feb564267c9p+0, -0x1.0245957316dd3p-54, \
  0x1.7a11473eb0187p+0, -0x1.41577ee04992fp-55, \
  0x1.7e2f336cf4e62p+0, 0x1.05d02ba15797ep-56, \
  0x1.82589994cce13p+0, -0x1.d4c1dd41532d8p-54, \
  0x1.868d99b4492edp+0, -0x1.fc6f89bd4f6bap-54, \
  0x1.8ace5422aa0dbp+0, 0x1.6e9f156864b27p-54, \
  0x1.8f1ae99157736p+0, 0x1.5cc13a2e3976cp-55, \
  0x1.93737b0cdc5e5p+0, -0x1.75fc781b57ebcp-57, \
  0x1.97d829fde4e50p+0, -0x1.d185b7c1b85d1p-54, \
  0x1.9c49182a3f090p+0, 0x1.c7c46b071f2bep-56, \
  0x1.a0c667b5de565p+0, -0x1.359495d1cd533p-54, \
  0x1.a5503b23e255dp+0, -0x1.d2f6edb8d41e1p-54, \
  0x1.a9e6b5579fdbfp+0, 0x1.0fac90ef7fd31p-54, \
  0x1.ae89f995ad3adp+0, 0x1.7a1cd345dcc81p-54, \
  0x1.b33a2b84f15fbp+0, -0x1.2805e3084d708p-57, \
  0x1.b7f76f2fb5e47p+0, -0x1.5584f7e54ac3bp-56, \
  0x1.bcc1e904bc1d2p+0, 0x1.23dd07a2d9e84p-55, \
  0x1.c199bdd85529cp+0, 0x1.11065895048ddp-55, \
  0x1.c67f12e57d14bp+0, 0x1.2884dff483cadp-54, \
  0x1.cb720dcef9069p+0, 0x1.503cbd1e949dbp-56, \
  0x1.d072d4a07897cp+0, -0x1.cbc3743797a9cp-54, \
  0x1.d5818dcfba487p+0, 0x1.2ed02d75b3707p-55, \
  0x1.da9e603db3285p+0, 0x1.c2300696db532p-54, \
  0x1.dfc97337b9b5fp+0, -0x1.1a5cd4f184b5cp-54, \
  0x1.e502ee78b3ff6p+0, 0x1.39e8980a9cc8fp-55, \
  0x1.ea4afa2a490dap+0, -0x1.e9c23179c2893p-54, \
  0x1.efa1bee615a27p+0, 0x1.dc7f486a4b6b0p-54, \
  0x1.f50765b6e4540p+0, 0x1.9d3e12dd8a18bp-54, \
  0x1.fa7c1819e90d8p+0, 0x1.74853f3a5931ep-55, \

#if defined(__CUDACC__)
static __device__ const double nt_tf_exp2_dev[128] = {NT_TF_EXP2_TABLE};
#endif
static const double nt_tf_exp2_host[128] = {NT_TF_EXP2_TABLE};

// exp(a) for a in [-90, 0] in three pieces, exp(a) = s + slo + s * p:
//   N = round(a * 64 / ln 2) by the add-a-large-constant trick (its low word is N, no conversion),
//   r = a - N ln2/64 (two-constant Cody-Waite, |r| <= ln2/128),  N = 64 k + j,
//   s + slo = 2^k * 2^(j/64) from the table,  p = e^r - 1 by a degree-6 polynomial (truncation r^7/5040 < 2^-65).
// Keeping s apart lets tanh form e^a - 1 = (s - 1) + (slo + s p) without cancellation when a is small
// (s = 1 and slo = 0 exactly for N = 0).
NT_TF_HD void nt_tf_exp_parts(double a, double *s_out, double *u_out) {
  const double shift = 6755399441055744.0; // 1.5 * 2^52
  const double t = fma(a, 0x1.71547652b82fep+6, shift);
  const double nd = t - shift;
#if defined(__CUDA_ARCH__)
  const int n = __double2loint(t);
#else
  uint64_t tb;
  memcpy(&tb, &t, 8);
  const int n = (int)(uint32_t)tb;
#endif
  double r = fma(nd, -0x1.62e42fefa0000p-7, a); // exact: nd has at most 14 bits, the constant 38
  r = fma(nd, -0x1.cf79abc9e3b3ap-46, r);
  const int j = n & 63, k = n >> 6;
#if defined(__CUDA_ARCH__)
  const double2 e = __ldg(reinterpret_cast<const double2 *>(nt_tf_exp2_dev) + j);
  const double hi = e.x, lo = e.y;
  const double s = __hiloint2double(__double2hiint(hi) + (k << 20), __double2loint(hi));
  const double slo = (lo == 0.0) ? 0.0 : __hiloint2double(__double2hiint(lo) + (k << 20), __double2loint(lo));
#else
  const double hi = nt_tf_exp2_host[2 * j], lo = nt_tf_exp2_host[2 * j + 1];
  uint64_t hb, lb;
  memcpy(&hb, &hi, 8);
  memcpy(&lb, &lo, 8);
  hb += (uint64_t)(int64_t)k << 52;
  if (lo != 0.0) lb += (uint64_t)(int64_t)k << 52;
  double s, slo;
  memcpy(&s, &hb, 8);
  memcpy(&slo, &lb, 8);
#endif
  const double r2 = r * r;
  double q = fma(r, 1.0 / 720.0, 1.0 / 120.0);
  q = fma(q, r, 1.0 / 24.0);
  q = fma(q, r, 1.0 / 6.0);
  q = fma(q, r, 0.5);
  const double p = fma(r2, q, r);
  *s_out = s;
  *u_out = fma(s, p, slo);
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

// 1 / (1 + exp(-x)) evaluated in double and rounded once (sigmoid_f32.h uses it for the one window of
// arguments where the reference's three fp32 steps amplify a one-ulp difference of the exponential).
NT_TF_HD float nt_sigmoid_cr_f32(float xf) {
  if (!(xf == xf)) return xf + xf;                   // NaN
  if (xf <= -88.72283935546875f) return 0.0f;        // expf(-x) = inf in the reference from this float on: 1 / inf
  if (xf > 40.0f) return 1.0f;                       // 1 + exp(-x) rounds to 1 long before
  // exp of a non-positive argument only: sigmoid(x) = 1/(1+E) for x >= 0, E/(1+E) for x < 0, E = exp(-|x|)
  double s, u;
  nt_tf_exp_parts(-(double)fabsf(xf), &s, &u);
  const double E = s + u;
  const double num = (xf >= 0.0f) ? 1.0 : E;
  return (float)nt_tf_div(num, 1.0 + E);
}

NT_TF_HD float nt_tanh_fast_f32(float xf) {
  if (!(xf == xf)) return xf + xf;            // NaN
  // beyond |x| = 20 the quotient rounds to 1.0f whatever exp(-2|x|) is, so the argument is clamped
  const double a = -2.0 * (double)fminf(fabsf(xf), 20.0f);
  double s, u;
  nt_tf_exp_parts(a, &s, &u);
  const double em1 = (s - 1.0) + u;           // exp(-2|x|) - 1, no cancellation: s - 1 is exact near a = 0
  const float tf = (float)nt_tf_div(-em1, 2.0 + em1);   // tanh|x| = (1 - E) / (1 + E)
  return copysignf(tf, xf);                   // tanh is odd; keeps the sign of zero
}
