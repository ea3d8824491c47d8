// fp32 transcendental building blocks for the eltwise kernels, accurate to well under 1 ulp.
//
// The CUDA math library's expf/tanhf are 2-3 ulp off the correctly rounded value on parts of
// their range, and 1/(1+expf(-x)) compounds that; the parity bar for logistic/tanh/elu is 2 ulp.
// Everything below is built from one exp kernel that returns its result as an unevaluated sum
// hi + lo (about 2^-31 relative), followed by quotient evaluation with one residual correction,
// so the only full-size rounding error is the final one.
//
// exp(x), x <= 0:  n = rint(x*log2(e)),  r = x - n*ln2 (two FMAs, ln2 split so the first is exact),
//                  exp(r) - 1 = r + r^2*g(r), g a degree-5 polynomial fitted by least squares on
//                  Chebyshev nodes over |r| <= 1.02*ln2/2 (max error 1.6e-9 in g, 2e-10 in exp);
//                  result = (1 + t) * 2^n with the rounding error of 1 + t kept as the low word.
#pragma once
#include <cuda_runtime.h>

#define DD_LN2_HI 0.693145751953125f       // ln 2 with the low 9 mantissa bits cleared
#define DD_LN2_LO 1.428606765330187e-06f   // ln 2 - DD_LN2_HI
#define DD_LOG2E 1.4426950216293335f

__device__ __forceinline__ float dd_rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// exp(x) = (p + pl) * 2^n for x in [-104, 0] (callers clamp): p in [0.7, 1.43] is the rounded
// mantissa part, pl its rounding error, n in [-150, 0].  `nbits` is the raw bit pattern of the
// rounding helper, 0x4B400000 + n: shifted left by 23 it is n << 23 (every set bit of 0x4B400000
// falls off the top), which is how the callers build 2^(n+k) in two integer instructions.
__device__ __forceinline__ void dd_exp_neg_raw(float x, float &p, float &pl, int &nbits) {
  // n = rint(x * log2 e) by the add-a-big-constant trick: both the rounded float and the integer
  // come out of one FMA (no round / float-to-int conversions, which run on the quarter-rate unit)
  const float big = fmaf(x, DD_LOG2E, 12582912.0f);  // 1.5 * 2^23: the sum's low mantissa bits are n
  const float fn = __fsub_rn(big, 12582912.0f);
  float r = fmaf(fn, -DD_LN2_HI, x);
  r = fmaf(fn, -DD_LN2_LO, r);
  float g = 0.00019901622727047652f;
  g = fmaf(g, r, 0.0013935454189777374f);
  g = fmaf(g, r, 0.008333295583724976f);
  g = fmaf(g, r, 0.04166644811630249f);
  g = fmaf(g, r, 0.1666666716337204f);
  g = fmaf(g, r, 0.5f);
  const float t = fmaf(__fmul_rn(r, r), g, r);  // exp(r) - 1, |t| <= 0.43
  p = __fadd_rn(1.0f, t);
  pl = __fsub_rn(t, __fsub_rn(p, 1.0f));        // exact: 1 + t = p + pl
  nbits = __float_as_int(big);
}

// 2^(n + k) as a float from nbits = 0x4B400000 + n; n + k must be in [-126, 127].
__device__ __forceinline__ float dd_pow2_from_bits(int nbits, int k) {
  return __int_as_float((int)(((unsigned)nbits << 23) + ((unsigned)(127 + k) << 23)));
}

// exp(x) for x in [-104, 0] reaches 2^-150, below the normal range.  To stay branch-free the kernels
// carry E = exp(x) * 2^64 (always a normal float, scaled exactly by one factor) wherever exp(x) is a
// NUMERATOR and multiply the final quotient by 2^-64 (exact unless the result is denormal, where it
// is the single rounding), and the plain e = E * 2^-64 only where it is added to 1.
#define DD_EXP_BIAS 64
#define DD_UNBIAS 5.421010862427522e-20f  // 2^-64

__device__ __forceinline__ void dd_exp_neg_biased(float x, float &Eh, float &El) {
  float p, pl;
  int nbits;
  dd_exp_neg_raw(x, p, pl, nbits);
  const float sc = dd_pow2_from_bits(nbits, DD_EXP_BIAS);
  Eh = __fmul_rn(p, sc);
  El = __fmul_rn(pl, sc);
}

// (nh + nl) / (dh + dl) with dh in [1, 2]: approximate quotient + one residual correction.
__device__ __forceinline__ float dd_quot(float nh, float nl, float dh, float dl) {
  const float r0 = dd_rcp_approx(dh);
  const float q = __fmul_rn(nh, r0);
  float res = fmaf(-dh, q, nh);  // exact remainder of the leading terms
  res = __fadd_rn(fmaf(-dl, q, res), nl);
  return fmaf(res, r0, q);
}

// 1 + e as an exact pair (e = eh + el in [0, 1])
__device__ __forceinline__ void dd_one_plus(float eh, float el, float &dh, float &dl) {
  dh = __fadd_rn(1.0f, eh);
  dl = __fadd_rn(__fadd_rn(__fsub_rn(1.0f, dh), eh), el);
}

// The same from the biased pair E = e * 2^64: the un-biasing multiplications ride inside FMAs
// (fma(Eh, 2^-64, 1) rounds 1 + eh once, exactly like the addition above).
__device__ __forceinline__ void dd_one_plus_biased(float Eh, float El, float &dh, float &dl) {
  dh = fmaf(Eh, DD_UNBIAS, 1.0f);
  dl = fmaf(El, DD_UNBIAS, fmaf(Eh, DD_UNBIAS, __fsub_rn(1.0f, dh)));
}

__device__ __forceinline__ float dd_sigmoid_f32(float x) {
  float Eh, El, dh, dl;
  dd_exp_neg_biased(fmaxf(-fabsf(x), -104.0f), Eh, El);
  dd_one_plus_biased(Eh, El, dh, dl);
  const bool pos = x >= 0.0f;
  // numerator 1 (as 2^64) or e (as E = e * 2^64); one exact un-biasing multiplication at the end
  const float s = __fmul_rn(dd_quot(pos ? 18446744073709551616.0f : Eh, pos ? 0.0f : El, dh, dl), DD_UNBIAS);
  return x != x ? x : s;
}

// 2^K * e / (1 + e)^2 for e = exp(xneg), xneg in [-104, 0]: the derivative kernel of both logistic
// (K = 0, e = exp(-|x|): s*(1-s)) and tanh (K = 2, e = exp(-2|x|): 1 - tanh^2).
template <int K>
__device__ __forceinline__ float dd_e_over_one_plus_e_sq(float xneg) {
  float Eh, El, dh, dl;
  dd_exp_neg_biased(xneg, Eh, El);
  dd_one_plus_biased(Eh, El, dh, dl);
  const float nh = Eh * (float)(1 << K), nl = El * (float)(1 << K);  // exact
  const float r0 = dd_rcp_approx(dh);
  const float rr = __fmul_rn(r0, r0);
  const float q = __fmul_rn(nh, rr);
  // residual nh + nl - q*(dh+dl)^2, with w = q*dh split into a rounded part and its error
  const float w = __fmul_rn(q, dh);
  const float wl = fmaf(q, dh, -w);
  float res = fmaf(-w, dh, nh);
  res = fmaf(-wl, dh, res);
  res = fmaf(-2.0f * w, dl, res);
  res = __fadd_rn(res, nl);
  return __fmul_rn(fmaf(res, rr, q), DD_UNBIAS);
}

// tanh(x) = (1 - e) / (1 + e), e = exp(-2|x|).  No separate small-|x| branch: 1 - e is formed from
// the hi/lo pair, and for |x| < 0.17 (n == 0) that difference is exactly -(exp(r) - 1), which the
// exp kernel computed without cancellation.  Here e only ever meets 1, so the argument is clamped at
// -87 (n >= -126: 2^n stays a normal float; tanh is 1 to the last bit from |x| = 9.1 on anyway).
__device__ __forceinline__ float dd_tanh_f32(float x) {
  float p, pl, dh, dl;
  int nbits;
  dd_exp_neg_raw(fmaxf(-2.0f * fabsf(x), -87.0f), p, pl, nbits);
  const float sc = dd_pow2_from_bits(nbits, 0);
  const float eh = __fmul_rn(p, sc), el = __fmul_rn(pl, sc);
  dd_one_plus(eh, el, dh, dl);
  // 1 - e = 2 - (1 + e) exactly: 2 - dh is exact (dh in [1, 2]) and the low word just changes sign.
  // The pair is not normalised, which dd_quot does not need: its residual is formed exactly.
  const float t = copysignf(dd_quot(__fsub_rn(2.0f, dh), -dl, dh, dl), x);
  return x != x ? x : t;
}

// exp(x) rounded once, for x <= 0 (elu backward)
__device__ __forceinline__ float dd_exp_neg_rounded(float x) {
  float Eh, El;
  dd_exp_neg_biased(fmaxf(x, -104.0f), Eh, El);
  return x != x ? x : __fmul_rn(__fadd_rn(Eh, El), DD_UNBIAS);
}

// exp(x) - 1 for x <= 0 (elu forward): (eh - 1) + el.  For |x| < 0.35 the reduction has n = 0, so
// eh - 1 is exact and the sum is the cancellation-free exp(r) - 1 the exp kernel produced; further
// out exp(x) <= 0.71 and the subtraction does not cancel.
__device__ __forceinline__ float dd_expm1_neg(float x) {
  float p, pl;
  int nbits;
  dd_exp_neg_raw(fmaxf(x, -87.0f), p, pl, nbits);  // exp(-87) - 1 is already -1 to the last bit
  const float sc = dd_pow2_from_bits(nbits, 0);
  const float r = __fadd_rn(__fsub_rn(__fmul_rn(p, sc), 1.0f), __fmul_rn(pl, sc));
  return x != x ? x : r;
}
