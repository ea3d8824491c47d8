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
//
// Every function is written once over a lane type F: `float` (one element) or `float2` (two
// elements in a 64-bit register pair).  On sm_100 the float2 form issues the packed
// fma/add/mul.rn.f32x2 instructions, one per TWO elements; each lane of a packed instruction is the
// same IEEE round-to-nearest operation as its scalar twin, so both forms return identical bits.
// Only what has no packed form stays per lane: the clamp, the reciprocal seed, the exponent
// integer arithmetic and the selects.  Subtractions are written as fma(u, -1, t) or as additions of
// negated constants so that no separate negation is needed on a packed operand.
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

// max(a, b) that returns NaN when a is NaN (fmaxf would return b): lets a NaN input run through
// the arithmetic below and come out as NaN without a select at the end.
__device__ __forceinline__ float dd_max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// 2^(n + k) as a float from the rounding helper big = 1.5*2^23 + n (bit pattern 0x4B400000 + n):
// shifted left by 23 it is n << 23 (every set bit of 0x4B400000 falls off the top); n + k must be
// in [-126, 127].
__device__ __forceinline__ float dd_pow2_from_big(float big, int k) {
  return __int_as_float((int)(((unsigned)__float_as_int(big) << 23) + ((unsigned)(127 + k) << 23)));
}

template <typename F> struct dd_lane;

template <> struct dd_lane<float> {
  static __device__ __forceinline__ float bc(float c) { return c; }
  static __device__ __forceinline__ float fma(float a, float b, float c) { return fmaf(a, b, c); }
  static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
  static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
  static __device__ __forceinline__ float nrcp(float a) { return dd_rcp_approx(-a); }  // about -1/a
  // max(-S*|x|, lo); NaN stays NaN
  template <int S> static __device__ __forceinline__ float neg_abs_clamped(float x, float lo) {
    return dd_max_nan(S == 1 ? -fabsf(x) : -(float)S * fabsf(x), lo);
  }
  static __device__ __forceinline__ float clamped(float x, float lo) { return dd_max_nan(x, lo); }
  static __device__ __forceinline__ float pow2(float big, int k) { return dd_pow2_from_big(big, k); }
  static __device__ __forceinline__ float sel_nonneg(float x, float a, float b) { return x >= 0.0f ? a : b; }
  static __device__ __forceinline__ float sel_pos(float x, float a, float b) { return x > 0.0f ? a : b; }
  static __device__ __forceinline__ float copysign(float m, float sgn) { return copysignf(m, sgn); }
};

template <> struct dd_lane<float2> {
  typedef dd_lane<float> S1;
  static __device__ __forceinline__ float2 bc(float c) { return make_float2(c, c); }
  static __device__ __forceinline__ float2 fma(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
  static __device__ __forceinline__ float2 add(float2 a, float2 b) { return __fadd2_rn(a, b); }
  static __device__ __forceinline__ float2 mul(float2 a, float2 b) { return __fmul2_rn(a, b); }
  static __device__ __forceinline__ float2 nrcp(float2 a) { return make_float2(S1::nrcp(a.x), S1::nrcp(a.y)); }
  template <int S> static __device__ __forceinline__ float2 neg_abs_clamped(float2 x, float lo) {
    return make_float2(S1::neg_abs_clamped<S>(x.x, lo), S1::neg_abs_clamped<S>(x.y, lo));
  }
  static __device__ __forceinline__ float2 clamped(float2 x, float lo) {
    return make_float2(dd_max_nan(x.x, lo), dd_max_nan(x.y, lo));
  }
  static __device__ __forceinline__ float2 pow2(float2 big, int k) {
    return make_float2(dd_pow2_from_big(big.x, k), dd_pow2_from_big(big.y, k));
  }
  static __device__ __forceinline__ float2 sel_nonneg(float2 x, float2 a, float2 b) {
    return make_float2(x.x >= 0.0f ? a.x : b.x, x.y >= 0.0f ? a.y : b.y);
  }
  static __device__ __forceinline__ float2 sel_pos(float2 x, float2 a, float2 b) {
    return make_float2(x.x > 0.0f ? a.x : b.x, x.y > 0.0f ? a.y : b.y);
  }
  static __device__ __forceinline__ float2 copysign(float2 m, float2 sgn) {
    return make_float2(copysignf(m.x, sgn.x), copysignf(m.y, sgn.y));
  }
};

// exp(x) = (p + pl) * 2^n for x in [-104, 0] (callers clamp): p in [0.7, 1.43] is the rounded
// mantissa part, pl its rounding error, n in [-150, 0] sits in the low mantissa bits of `big`.
template <typename F>
__device__ __forceinline__ void dd_exp_neg_raw(F x, F &p, F &pl, F &big) {
  typedef dd_lane<F> L;
  // n = rint(x * log2 e) by the add-a-big-constant trick: both the rounded float and the integer
  // come out of one FMA (no round / float-to-int conversions, which run on the quarter-rate unit)
  big = L::fma(x, L::bc(DD_LOG2E), L::bc(12582912.0f));  // 1.5 * 2^23: the sum's low mantissa bits are n
  const F fn = L::add(big, L::bc(-12582912.0f));
  F r = L::fma(fn, L::bc(-DD_LN2_HI), x);
  r = L::fma(fn, L::bc(-DD_LN2_LO), r);
  F g = L::bc(0.00019901622727047652f);
  g = L::fma(g, r, L::bc(0.0013935454189777374f));
  g = L::fma(g, r, L::bc(0.008333295583724976f));
  g = L::fma(g, r, L::bc(0.04166644811630249f));
  g = L::fma(g, r, L::bc(0.1666666716337204f));
  g = L::fma(g, r, L::bc(0.5f));
  const F t = L::fma(L::mul(r, r), g, r);  // exp(r) - 1, |t| <= 0.43
  p = L::add(L::bc(1.0f), t);
  pl = L::fma(L::add(p, L::bc(-1.0f)), L::bc(-1.0f), t);  // t - (p - 1), exact: 1 + t = p + pl
}

// exp(x) for x in [-104, 0] reaches 2^-150, below the normal range.  To stay branch-free the kernels
// carry E = exp(x) * 2^64 (always a normal float, scaled exactly by one factor) wherever exp(x) is a
// NUMERATOR and multiply the final quotient by 2^-64 (exact unless the result is denormal, where it
// is the single rounding), and the plain e = E * 2^-64 only where it is added to 1.  KX extra powers
// of two can ride in the same scale factor (the derivative kernels want 2^K * e).
#define DD_EXP_BIAS 64
#define DD_UNBIAS 5.421010862427522e-20f  // 2^-64

template <typename F, int KX = 0>
__device__ __forceinline__ void dd_exp_neg_biased(F x, F &Eh, F &El) {
  typedef dd_lane<F> L;
  F p, pl, big;
  dd_exp_neg_raw<F>(x, p, pl, big);
  const F sc = L::pow2(big, DD_EXP_BIAS + KX);
  Eh = L::mul(p, sc);
  El = L::mul(pl, sc);
}

// MINUS (nh + nl) / (dh + dl) with dh in [1, 2]: approximate quotient + one residual correction,
// carried negated (nr0 is about -1/dh) so that every step is a plain fma; callers fold the sign into
// their last operation.  Each step is the exact mirror image of the positive form, so the magnitude
// has the same bits.
template <typename F>
__device__ __forceinline__ F dd_neg_quot(F nh, F nl, F dh, F dl) {
  typedef dd_lane<F> L;
  const F nr0 = L::nrcp(dh);
  const F nq = L::mul(nh, nr0);
  F res = L::fma(dh, nq, nh);  // exact remainder of the leading terms
  res = L::add(L::fma(dl, nq, res), nl);
  return L::fma(res, nr0, nq);
}

// 1 + e as an exact pair (e = eh + el in [0, 1])
template <typename F>
__device__ __forceinline__ void dd_one_plus(F eh, F el, F &dh, F &dl) {
  typedef dd_lane<F> L;
  dh = L::add(L::bc(1.0f), eh);
  dl = L::add(L::add(L::fma(dh, L::bc(-1.0f), L::bc(1.0f)), eh), el);
}

// The same from the biased pair E = e / unb: the un-biasing multiplications ride inside FMAs
// (fma(Eh, unb, 1) rounds 1 + eh once, exactly like the addition above).
template <typename F>
__device__ __forceinline__ void dd_one_plus_biased(F Eh, F El, float unb, F &dh, F &dl) {
  typedef dd_lane<F> L;
  dh = L::fma(Eh, L::bc(unb), L::bc(1.0f));
  dl = L::fma(El, L::bc(unb), L::fma(Eh, L::bc(unb), L::fma(dh, L::bc(-1.0f), L::bc(1.0f))));
}

// logistic(x) = 1 / (1 + e) for x >= 0, e / (1 + e) for x < 0, e = exp(-|x|).  NaN in, NaN out.
template <typename F>
__device__ __forceinline__ F dd_sigmoid(F x) {
  typedef dd_lane<F> L;
  F Eh, El, dh, dl;
  dd_exp_neg_biased<F>(L::template neg_abs_clamped<1>(x, -104.0f), Eh, El);
  dd_one_plus_biased<F>(Eh, El, DD_UNBIAS, dh, dl);
  // numerator 1 (as 2^64) or e (as E = e * 2^64); one exact un-biasing multiplication at the end
  const F nh = L::sel_nonneg(x, L::bc(18446744073709551616.0f), Eh);
  const F nl = L::sel_nonneg(x, L::bc(0.0f), El);
  return L::mul(dd_neg_quot<F>(nh, nl, dh, dl), L::bc(-DD_UNBIAS));
}

// 2^K * e / (1 + e)^2 for e = exp(xneg), xneg in [-104, 0]: the derivative kernel of both logistic
// (K = 0, e = exp(-|x|): s*(1-s)) and tanh (K = 2, e = exp(-2|x|): 1 - tanh^2).
template <typename F, int K>
__device__ __forceinline__ F dd_e_over_one_plus_e_sq(F xneg) {
  typedef dd_lane<F> L;
  constexpr float unb = DD_UNBIAS / (float)(1 << K);  // the numerator carries 2^(64+K)
  F nh, nl, dh, dl;
  dd_exp_neg_biased<F, K>(xneg, nh, nl);
  dd_one_plus_biased<F>(nh, nl, unb, dh, dl);
  const F ndh = L::mul(dh, L::bc(-1.0f));
  const F r0 = L::nrcp(dh);
  const F rr = L::mul(r0, r0);
  const F q = L::mul(nh, rr);
  // residual nh + nl - q*(dh+dl)^2, with w = q*dh split into a rounded part and its error
  const F nw = L::mul(q, ndh);           // -w
  const F wl = L::fma(q, dh, nw);
  F res = L::fma(nw, dh, nh);
  res = L::fma(wl, ndh, res);
  res = L::fma(L::mul(nw, L::bc(2.0f)), dl, res);
  res = L::add(res, nl);
  return L::mul(L::fma(res, rr, q), L::bc(DD_UNBIAS));
}

// tanh(x) = (1 - e) / (1 + e), e = exp(-2|x|).  No separate small-|x| branch: 1 - e is formed from
// the hi/lo pair, and for |x| < 0.17 (n == 0) that difference is exactly -(exp(r) - 1), which the
// exp kernel computed without cancellation.  Here e only ever meets 1, so the argument is clamped at
// -87 (n >= -126: 2^n stays a normal float; tanh is 1 to the last bit from |x| = 9.1 on anyway).
template <typename F>
__device__ __forceinline__ F dd_tanh(F x) {
  typedef dd_lane<F> L;
  F p, pl, big, dh, dl;
  dd_exp_neg_raw<F>(L::template neg_abs_clamped<2>(x, -87.0f), p, pl, big);
  const F sc = L::pow2(big, 0);
  dd_one_plus<F>(L::mul(p, sc), L::mul(pl, sc), dh, dl);
  // 1 - e = 2 - (1 + e) exactly: 2 - dh is exact (dh in [1, 2]) and the low word just changes sign.
  // The pair is not normalised, which the quotient does not need: its residual is formed exactly.
  const F q = dd_neg_quot<F>(L::fma(dh, L::bc(-1.0f), L::bc(2.0f)), L::mul(dl, L::bc(-1.0f)), dh, dl);
  return L::copysign(q, x);  // the quotient's own sign (negated form) is replaced by x's
}

// exp(x) rounded once, for x <= 0 (elu backward)
template <typename F>
__device__ __forceinline__ F dd_exp_neg_rounded(F x) {
  typedef dd_lane<F> L;
  F Eh, El;
  dd_exp_neg_biased<F>(L::clamped(x, -104.0f), Eh, El);
  return L::mul(L::add(Eh, El), L::bc(DD_UNBIAS));
}

// exp(x) - 1 for x <= 0 (elu forward): (eh - 1) + el.  For |x| < 0.35 the reduction has n = 0, so
// eh - 1 is exact and the sum is the cancellation-free exp(r) - 1 the exp kernel produced; further
// out exp(x) <= 0.71 and the subtraction does not cancel.
template <typename F>
__device__ __forceinline__ F dd_expm1_neg(F x) {
  typedef dd_lane<F> L;
  F p, pl, big;
  dd_exp_neg_raw<F>(L::clamped(x, -87.0f), p, pl, big);  // exp(-87) - 1 is already -1 to the last bit
  const F sc = L::pow2(big, 0);
  return L::add(L::add(L::mul(p, sc), L::bc(-1.0f)), L::mul(pl, sc));
}

// log(x) for two positive, normal, finite inputs at once (the cross-entropy cost needs log(a) and
// log(1 - a) of every element).  x = m * 2^e with m in [sqrt(1/2), sqrt(2)); t = m - 1 exactly;
// log(m) = t - t^2/2 + t^3 * P(t) with P a degree-7 polynomial fitted by least squares on Chebyshev
// nodes (0.84 ulp of log(m) in a float32 emulation over 2 million points); the result is assembled
// small terms first as e*ln2_hi + (t + (t^3*P - t^2/2 + e*ln2_lo)), e*ln2_hi being exact.  Anything
// else (zero, negative, denormal, infinite, NaN) takes the library's logf for that lane.
__device__ __forceinline__ float2 dd_log_pair(float2 x) {
  typedef dd_lane<float2> L;
  const int ix = __float_as_int(x.x), iy = __float_as_int(x.y);
  const int ex = (ix - 0x3f3504f3) >> 23, ey = (iy - 0x3f3504f3) >> 23;
  const float2 m = make_float2(__int_as_float(ix - (ex << 23)), __int_as_float(iy - (ey << 23)));
  // e as a float without an integer-to-float conversion (an eighth-rate instruction): 1.5*2^23 + e
  // has e in its low mantissa bits, and subtracting 1.5*2^23 is exact
  const float2 fe = L::add(make_float2(__int_as_float(0x4B400000 + ex), __int_as_float(0x4B400000 + ey)),
                           L::bc(-12582912.0f));
  const float2 t = L::add(m, L::bc(-1.0f));
  float2 P = L::bc(-0.0733518898487091f);
  P = L::fma(P, t, L::bc(0.12697939574718475f));
  P = L::fma(P, t, L::bc(-0.13257159292697906f));
  P = L::fma(P, t, L::bc(0.1422044187784195f));
  P = L::fma(P, t, L::bc(-0.16613943874835968f));
  P = L::fma(P, t, L::bc(0.1999974548816681f));
  P = L::fma(P, t, L::bc(-0.25001105666160583f));
  P = L::fma(P, t, L::bc(0.3333336412906647f));
  const float2 t2 = L::mul(t, t);
  float2 s = L::fma(L::bc(-0.5f), t2, L::mul(L::mul(t2, t), P));
  s = L::fma(fe, L::bc(DD_LN2_LO), s);
  float2 r = L::fma(fe, L::bc(DD_LN2_HI), L::add(t, s));
  // 0x00800000 <= bits < 0x7f800000: positive, normal, finite
  if ((unsigned)(ix - 0x00800000) >= 0x7f000000u) r.x = logf(x.x);
  if ((unsigned)(iy - 0x00800000) >= 0x7f000000u) r.y = logf(x.y);
  return r;
}

// ---- 16-bit element types --------------------------------------------------------------------
// A result that is going to be rounded to f16 (11 significant bits) or bf16 (8) does not need the
// sub-ulp float evaluation above: the special function unit's exp2 and reciprocal (about 2^-22
// relative) leave the 16-bit rounding right except within 2^-21 of a tie, i.e. at most one unit of
// the 16-bit type off, at a fraction of the instructions.  Differences that would cancel (1 - e
// and e - 1 near 0) are replaced by short series there.  Denormals are kept (no .ftz).
__device__ __forceinline__ float dd_ex2_sfu(float x) {
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float dd_rcp_sfu(float x) {
  float r;
  asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
#define DD_LOG2E_F 1.4426950408889634f

__device__ __forceinline__ float dd_sigmoid_light(float x) {
  const float e = dd_ex2_sfu(-fabsf(x) * DD_LOG2E_F);  // exp(-|x|); NaN stays NaN
  const float r = dd_rcp_sfu(1.0f + e);
  return x >= 0.0f ? r : e * r;
}
// s * (1 - s) = e / (1 + e)^2, e = exp(-|x|)
__device__ __forceinline__ float dd_dsigmoid_light(float x) {
  const float e = dd_ex2_sfu(-fabsf(x) * DD_LOG2E_F);
  const float r = dd_rcp_sfu(1.0f + e);
  return e * r * r;
}
__device__ __forceinline__ float dd_tanh_light(float x) {
  const float ax = fabsf(x);
  const float e = dd_ex2_sfu(ax * (-2.0f * DD_LOG2E_F));  // exp(-2|x|)
  float t = (1.0f - e) * dd_rcp_sfu(1.0f + e);
  const float x2 = ax * ax;  // |x| < 0.25: x (1 - x^2/3 + 2 x^4/15 - 17 x^6/315), next term below 2^-19 relative
  const float p = ax * fmaf(x2, fmaf(x2, fmaf(x2, -0.05396825397f, 0.13333333333f), -0.33333333333f), 1.0f);
  t = ax < 0.25f ? p : t;
  return copysignf(t, x);
}
// 1 - tanh^2 = 4 e / (1 + e)^2, e = exp(-2|x|)
__device__ __forceinline__ float dd_dtanh_light(float x) {
  const float e = dd_ex2_sfu(fabsf(x) * (-2.0f * DD_LOG2E_F));
  const float r = dd_rcp_sfu(1.0f + e);
  return 4.0f * e * r * r;
}
// exp(x) - 1 for x <= 0
__device__ __forceinline__ float dd_expm1_neg_light(float x) {
  const float e = dd_ex2_sfu(x * DD_LOG2E_F) - 1.0f;
  // |x| < 0.25: x + x^2/2 + x^3/6 + x^4/24 + x^5/120, next term below 2^-19 relative
  const float p = x * fmaf(x, fmaf(x, fmaf(x, fmaf(x, 0.00833333333f, 0.04166666667f), 0.16666666667f), 0.5f), 1.0f);
  return x > -0.25f ? p : e;
}
__device__ __forceinline__ float dd_exp_neg_light(float x) { return dd_ex2_sfu(x * DD_LOG2E_F); }

// bf16 results (8 significant bits) can take tanh from the special function unit directly: its
// error of about 2^-11 relative keeps the rounded result within one bf16 unit of the true value.
__device__ __forceinline__ float dd_tanh_sfu(float x) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
