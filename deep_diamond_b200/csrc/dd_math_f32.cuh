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
// tanh(x), |x| < 0.3:  x + x^3*q(x^2), q a degree-3 least-squares fit (error 4e-10 relative).
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

// v * 2^n for n in [-152, 2], in two normal factors so that a denormal result rounds once.
__device__ __forceinline__ float dd_scale2(float v, int n) {
  const int n1 = n >> 1, n2 = n - n1;
  const float s1 = __int_as_float((n1 + 127) << 23), s2 = __int_as_float((n2 + 127) << 23);
  return __fmul_rn(__fmul_rn(v, s1), s2);
}

// exp(x) = (p + pl) * 2^n for x in [-104, 0] (callers clamp): p in [0.7, 1.43] is the rounded
// mantissa part, pl its rounding error, n in [-150, 0].
__device__ __forceinline__ void dd_exp_neg_raw(float x, float &p, float &pl, int &n) {
  const float fn = rintf(__fmul_rn(x, DD_LOG2E));
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
  n = (int)fn;
}

// exp(x) = hi + lo: hi carries the rounded value, lo its error.
__device__ __forceinline__ void dd_exp_neg(float x, float &hi, float &lo) {
  float p, pl;
  int n;
  dd_exp_neg_raw(x, p, pl, n);
  hi = dd_scale2(p, n);
  lo = dd_scale2(pl, n);
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

__device__ __forceinline__ float dd_sigmoid_f32(float x) {
  const float xc = fmaxf(-fabsf(x), -104.0f);
  float eh, el, dh, dl;
  dd_exp_neg(xc, eh, el);
  dd_one_plus(eh, el, dh, dl);
  const bool pos = x >= 0.0f;
  const float s = dd_quot(pos ? 1.0f : eh, pos ? 0.0f : el, dh, dl);
  return x != x ? x : s;
}

// 2^k * e / (1 + e)^2 for e = exp(xneg), xneg in [-104, 0]: the derivative kernel of both logistic
// (k = 0, e = exp(-|x|): s*(1-s)) and tanh (k = 2, e = exp(-2|x|): 1 - tanh^2).  The factor 2^k goes
// into the numerator's exponent so that results near the denormal range still round once.
__device__ __forceinline__ float dd_e_over_one_plus_e_sq(float xneg, int k) {
  float p, pl, dh, dl;
  int n;
  dd_exp_neg_raw(xneg, p, pl, n);
  dd_one_plus(dd_scale2(p, n), dd_scale2(pl, n), dh, dl);
  const float nh = dd_scale2(p, n + k), nl = dd_scale2(pl, n + k);
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
  return fmaf(res, rr, q);
}

__device__ __forceinline__ float dd_tanh_f32(float x) {
  const float ax = fabsf(x);
  float t;
  if (ax < 0.3f) {
    const float z = __fmul_rn(x, x);
    float q = 0.0203524362295866f;
    q = fmaf(q, z, -0.053884357213974f);
    q = fmaf(q, z, 0.13333183526992798f);
    q = fmaf(q, z, -0.3333333432674408f);
    t = fmaf(__fmul_rn(x, z), q, x);
  } else {
    float eh, el, dh, dl;
    dd_exp_neg(fmaxf(-2.0f * ax, -104.0f), eh, el);
    dd_one_plus(eh, el, dh, dl);
    const float nh = __fsub_rn(1.0f, eh);                                    // 1 - e as a pair
    const float nl = __fsub_rn(__fsub_rn(__fsub_rn(1.0f, nh), eh), el);
    t = copysignf(dd_quot(nh, nl, dh, dl), x);
  }
  return x != x ? x : t;
}

// exp(x) rounded once, for x <= 0 (elu backward)
__device__ __forceinline__ float dd_exp_neg_rounded(float x) {
  float eh, el;
  dd_exp_neg(fmaxf(x, -104.0f), eh, el);
  return x != x ? x : __fadd_rn(eh, el);
}
