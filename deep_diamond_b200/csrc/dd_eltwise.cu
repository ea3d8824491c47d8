// Eltwise activation forward / backward (the bodies of ddActivationForward / ddActivationBackward).
//
//   forward   y  = alpha*act(x)       + beta*y       algorithmic bytes/element: 2*sizeof(T)
//   backward  dx = alpha*act'(x)*dy   + beta*dx      algorithmic bytes/element: 3*sizeof(T)
//
// Dense tensors with identical strides (the layer case) run as a flat 16-byte vector stream;
// anything else goes through the strided kernel.  Both are HBM-bound.
//
// Arithmetic follows oneDNN's documented eltwise definitions (the reference binds them in
// dnnl/impl.clj:324-341, algorithm keywords dnnl/constants.clj:277-308), evaluated in fp32 (fp64
// for double tensors) with the derivative taken from the forward source:
//   relu      f = x>0 ? x : a*x            f' = x>0 ? 1 : a
//   logistic  f = 1/(1+exp(-x))            f' = f*(1-f)
//   tanh      f = tanh(x)                  f' = 1-f^2
//   elu       f = x>0 ? x : a*(exp(x)-1)   f' = x>0 ? 1 : a*exp(x)
//   linear    f = a*x+b                    f' = a
//   clip-relu f = min(max(x,0),a)          f' = 0<x<=a ? 1 : 0
//   abs       f = |x|                      f' = sign(x)
// and the rest of the reference's oneDNN table (dnnl/constants.clj:277-308; a = coef, b = shift):
//   square x^2 | sqrt | exp | log | soft-relu log(1+exp(a x))/a | swish x*sigma(a x) |
//   gelu-tanh x*sigma(2 g), g = sqrt(2/pi) x (1 + 0.044715 x^2)  (= 0.5 x (1 + tanh g)) |
//   gelu-erf 0.5 x erfc(-x/sqrt 2)  (= 0.5 x (1 + erf(x/sqrt 2))) | hardswish x*max(0,min(1,a x+b)) |
//   clip, clip-v2 min(max(x,a),b) | pow a*x^b | mish x*tanh(log(1+exp x)) | round (to nearest even)
// each with oneDNN's documented derivative, written so that nothing cancels (sigma(2g) for
// 1 + tanh g, erfc for 1 + erf, e(e+2)/(e(e+2)+2) for tanh(softplus)).  The *-dst-bwd kinds run the
// same forward and take the derivative from the forward RESULT: relu, tanh 1-y^2, elu y+a,
// sqrt 1/(2y), logistic y(1-y), exp y, clip-v2.  These kinds run as two kernel families whose
// arithmetic is selected by a grid-uniform switch (one instantiation per family, not per kind).
// f*(1-f) and 1-f^2 are evaluated as e/(1+e)^2 forms (no cancellation near saturation); the fp32
// exp/logistic/tanh come from dd_math_f32.cuh (under 1 ulp), not from the CUDA math library.
#include "dd_internal.cuh"
#include "dd_math_f32.cuh"

template <typename C> struct dd_math;
template <> struct dd_math<float> {
  static __device__ __forceinline__ float exp(float x) { return expf(x); }
  static __device__ __forceinline__ float expm1(float x) { return expm1f(x); }
  static __device__ __forceinline__ float expm1_neg(float x) { return dd_expm1_neg<float>(x); }
  static __device__ __forceinline__ float tanh(float x) { return tanhf(x); }
  static __device__ __forceinline__ float abs(float x) { return fabsf(x); }
  static __device__ __forceinline__ float fma(float a, float b, float c) { return fmaf(a, b, c); }
  static __device__ __forceinline__ float max(float a, float b) { return fmaxf(a, b); }
  static __device__ __forceinline__ float min(float a, float b) { return fminf(a, b); }
  static __device__ __forceinline__ float div(float a, float b) { return __fdiv_rn(a, b); }
  static __device__ __forceinline__ float sigmoid(float x) { return dd_sigmoid<float>(x); }
  // s*(1-s) = e/(1+e)^2 with e = exp(-|x|)
  static __device__ __forceinline__ float dsigmoid(float x) {
    return dd_e_over_one_plus_e_sq<float, 0>(dd_lane<float>::neg_abs_clamped<1>(x, -104.0f));
  }
  static __device__ __forceinline__ float tanh_(float x) { return dd_tanh<float>(x); }
  // 1 - tanh^2 = 4e/(1+e)^2 with e = exp(-2|x|)
  static __device__ __forceinline__ float dtanh(float x) {
    return dd_e_over_one_plus_e_sq<float, 2>(dd_lane<float>::neg_abs_clamped<2>(x, -104.0f));
  }
  static __device__ __forceinline__ float exp_neg(float x) { return dd_exp_neg_rounded<float>(x); }
  static __device__ __forceinline__ float log(float x) { return logf(x); }
  static __device__ __forceinline__ float log1p(float x) { return log1pf(x); }
  static __device__ __forceinline__ float erfc(float x) { return erfcf(x); }
  static __device__ __forceinline__ float pow(float a, float b) { return powf(a, b); }
  static __device__ __forceinline__ float sqrt(float x) { return __fsqrt_rn(x); }
  static __device__ __forceinline__ float rint(float x) { return rintf(x); }
};
template <> struct dd_math<double> {
  static __device__ __forceinline__ double exp(double x) { return ::exp(x); }
  static __device__ __forceinline__ double expm1(double x) { return ::expm1(x); }
  static __device__ __forceinline__ double expm1_neg(double x) { return ::expm1(x); }
  static __device__ __forceinline__ double tanh(double x) { return ::tanh(x); }
  static __device__ __forceinline__ double abs(double x) { return ::fabs(x); }
  static __device__ __forceinline__ double fma(double a, double b, double c) { return ::fma(a, b, c); }
  static __device__ __forceinline__ double max(double a, double b) { return ::fmax(a, b); }
  static __device__ __forceinline__ double min(double a, double b) { return ::fmin(a, b); }
  static __device__ __forceinline__ double div(double a, double b) { return __ddiv_rn(a, b); }
  static __device__ __forceinline__ double sigmoid(double x) {
    double e = ::exp(-::fabs(x));
    double r = 1.0 / (1.0 + e);
    return x != x ? x : (x >= 0.0 ? r : e * r);
  }
  static __device__ __forceinline__ double dsigmoid(double x) {
    double e = ::exp(-::fabs(x));
    double r = 1.0 / (1.0 + e);
    return x != x ? x : e * r * r;
  }
  static __device__ __forceinline__ double tanh_(double x) { return ::tanh(x); }
  static __device__ __forceinline__ double dtanh(double x) {
    double e = ::exp(-2.0 * ::fabs(x));
    double r = 1.0 / (1.0 + e);
    return x != x ? x : 4.0 * e * r * r;
  }
  static __device__ __forceinline__ double exp_neg(double x) { return ::exp(x); }
  static __device__ __forceinline__ double log(double x) { return ::log(x); }
  static __device__ __forceinline__ double log1p(double x) { return ::log1p(x); }
  static __device__ __forceinline__ double erfc(double x) { return ::erfc(x); }
  static __device__ __forceinline__ double pow(double a, double b) { return ::pow(a, b); }
  static __device__ __forceinline__ double sqrt(double x) { return __dsqrt_rn(x); }
  static __device__ __forceinline__ double rint(double x) { return ::rint(x); }
};

struct ddActArgs {
  double coef, shift;
  int nanProp;
  int kind;  // the families below: which of their kinds (a ddActivationMode_t), the same for the whole grid
};

// Kernel families of the oneDNN-only kinds: one template instantiation each, the kind chosen at run
// time.  CHEAP: a few arithmetic instructions.  TRANS: exp / log / erfc / pow inside.
enum { DD_ACT_FAM_CHEAP = 100, DD_ACT_FAM_TRANS = 101 };

template <typename C>
__device__ __forceinline__ C dd_ext_cheap_fwd(int kind, C x, C a, C b) {
  typedef dd_math<C> M;
  switch (kind) {
    case DD_ACTIVATION_SQUARE: return dd_mul_rn(x, x);
    case DD_ACTIVATION_SQRT: return M::sqrt(x);
    case DD_ACTIVATION_CLIP: case DD_ACTIVATION_CLIP_V2: return x <= a ? a : (x > b ? b : x);
    case DD_ACTIVATION_HARDSWISH: {
      const C t = M::fma(a, x, b);
      return dd_mul_rn(x, t <= (C)0 ? (C)0 : (t >= (C)1 ? (C)1 : t));
    }
    default: return M::rint(x);  // ROUND
  }
}

// x is the forward source, or the forward result for the *_DST kinds
template <typename C>
__device__ __forceinline__ C dd_ext_cheap_bwd(int kind, C x, C dy, C a, C b) {
  typedef dd_math<C> M;
  switch (kind) {
    case DD_ACTIVATION_SQUARE: return dd_mul_rn(dy, dd_add_rn(x, x));
    case DD_ACTIVATION_SQRT: case DD_ACTIVATION_SQRT_DST_BWD: {
      const C r = kind == DD_ACTIVATION_SQRT ? M::sqrt(x) : x;
      return M::div(dy, dd_add_rn(r, r));
    }
    case DD_ACTIVATION_CLIP: return (x > a && x <= b) ? dy : (C)0;
    case DD_ACTIVATION_CLIP_V2: return (x > a && x < b) ? dy : (C)0;
    case DD_ACTIVATION_HARDSWISH: {
      const C t = M::fma(a, x, b);
      return t <= (C)0 ? (C)0 : (t >= (C)1 ? dy : dd_mul_rn(dy, M::fma(dd_add_rn(a, a), x, b)));
    }
    case DD_ACTIVATION_TANH_DST_BWD: return dd_mul_rn(dy, M::fma(-x, x, (C)1));
    case DD_ACTIVATION_ELU_DST_BWD: return x > (C)0 ? dy : dd_mul_rn(dy, dd_add_rn(x, a));
    case DD_ACTIVATION_LOGISTIC_DST_BWD: return dd_mul_rn(dy, dd_mul_rn(x, dd_add_rn((C)1, -x)));
    default: return dd_mul_rn(dy, x);  // EXP_DST_BWD
  }
}

template <typename C>
__device__ __forceinline__ C dd_ext_trans_fwd(int kind, C x, C a, C b) {
  typedef dd_math<C> M;
  switch (kind) {
    case DD_ACTIVATION_EXP: return M::exp(x);
    case DD_ACTIVATION_LOG: return M::log(x);
    case DD_ACTIVATION_SOFT_RELU: {
      const C t = dd_mul_rn(a, x);
      const C sp = t > (C)0 ? dd_add_rn(t, M::log1p(M::exp(-t))) : M::log1p(M::exp(t));
      return M::div(sp, a);
    }
    case DD_ACTIVATION_SWISH: return dd_mul_rn(x, M::sigmoid(dd_mul_rn(a, x)));
    case DD_ACTIVATION_GELU_TANH: {
      const C g = dd_mul_rn(dd_mul_rn((C)0.7978845608028654, x), M::fma((C)0.044715, dd_mul_rn(x, x), (C)1));
      return dd_mul_rn(x, M::sigmoid(dd_add_rn(g, g)));
    }
    case DD_ACTIVATION_GELU_ERF:
      return dd_mul_rn(dd_mul_rn((C)0.5, x), M::erfc(dd_mul_rn((C)-0.7071067811865476, x)));
    case DD_ACTIVATION_POW: return dd_mul_rn(a, M::pow(x, b));
    default: {  // MISH: tanh(log(1 + e)) = e(e+2) / (e(e+2) + 2)
      if (x > (C)20) return x;
      const C e = M::exp(x);
      const C n = dd_mul_rn(e, dd_add_rn(e, (C)2));
      return dd_mul_rn(x, M::div(n, dd_add_rn(n, (C)2)));
    }
  }
}

template <typename C>
__device__ __forceinline__ C dd_ext_trans_bwd(int kind, C x, C dy, C a, C b) {
  typedef dd_math<C> M;
  switch (kind) {
    case DD_ACTIVATION_EXP: return dd_mul_rn(dy, M::exp(x));
    case DD_ACTIVATION_LOG: return M::div(dy, x);
    case DD_ACTIVATION_SOFT_RELU: return dd_mul_rn(dy, M::sigmoid(dd_mul_rn(a, x)));
    case DD_ACTIVATION_SWISH: {  // s + a x s (1 - s)
      const C t = dd_mul_rn(a, x);
      return dd_mul_rn(dy, M::fma(t, M::dsigmoid(t), M::sigmoid(t)));
    }
    case DD_ACTIVATION_GELU_TANH: {  // s + 2 x s (1 - s) g',  s = sigma(2g)
      const C x2 = dd_mul_rn(x, x);
      const C g = dd_mul_rn(dd_mul_rn((C)0.7978845608028654, x), M::fma((C)0.044715, x2, (C)1));
      const C gp = dd_mul_rn((C)0.7978845608028654, M::fma((C)0.134145, x2, (C)1));
      const C g2 = dd_add_rn(g, g);
      return dd_mul_rn(dy, M::fma(dd_mul_rn(dd_add_rn(x, x), gp), M::dsigmoid(g2), M::sigmoid(g2)));
    }
    case DD_ACTIVATION_GELU_ERF: {  // 0.5 erfc(-x/sqrt 2) + x exp(-x^2/2)/sqrt(2 pi)
      const C h = dd_mul_rn((C)0.5, M::erfc(dd_mul_rn((C)-0.7071067811865476, x)));
      const C q = dd_mul_rn(dd_mul_rn((C)0.3989422804014327, x), M::exp(dd_mul_rn((C)-0.5, dd_mul_rn(x, x))));
      return dd_mul_rn(dy, dd_add_rn(h, q));
    }
    case DD_ACTIVATION_POW: return dd_mul_rn(dy, dd_mul_rn(dd_mul_rn(a, b), M::pow(x, dd_add_rn(b, (C)-1))));
    default: {  // MISH: e w / d^2,  w = 4(x+1) + 4e^2 + e^3 + e(4x+6),  d = e^2 + 2e + 2
      if (x > (C)20) return dy;
      const C e = M::exp(x);
      const C d = M::fma(e, dd_add_rn(e, (C)2), (C)2);
      const C w = M::fma(e, M::fma(e, dd_add_rn(e, (C)4), M::fma((C)4, x, (C)6)), dd_mul_rn((C)4, dd_add_rn(x, (C)1)));
      return dd_mul_rn(dy, M::div(dd_mul_rn(e, w), dd_mul_rn(d, d)));
    }
  }
}

// The result of a 16-bit element type takes the special-function-unit forms of dd_math_f32.cuh for
// the transcendental modes (at most one unit of the 16-bit type off).
// LIGHT: 0 = full float accuracy, 1 = f16 result, 2 = bf16 result
template <typename T> struct dd_light { static constexpr int value = 0; };
template <> struct dd_light<__half> { static constexpr int value = 1; };
template <> struct dd_light<__nv_bfloat16> { static constexpr int value = 2; };

template <typename C, int MODE, int LIGHT = 0>
__device__ __forceinline__ C dd_act_fwd(C x, C coef, C shift, bool nanProp, int kind = 0) {
  typedef dd_math<C> M;
  if (MODE == DD_ACT_FAM_CHEAP) return dd_ext_cheap_fwd<C>(kind, x, coef, shift);
  if (MODE == DD_ACT_FAM_TRANS) return dd_ext_trans_fwd<C>(kind, x, coef, shift);
  // swish and gelu-tanh have kernels of their own (packed fp32 forms below); this is their scalar form
  if (MODE == DD_ACTIVATION_SWISH || MODE == DD_ACTIVATION_GELU_TANH) return dd_ext_trans_fwd<C>(MODE, x, coef, shift);
  if constexpr (LIGHT != 0 && sizeof(C) == 4) {
    if (MODE == DD_ACTIVATION_SIGMOID) return dd_sigmoid_light(x);
    if (MODE == DD_ACTIVATION_TANH) return LIGHT == 2 ? dd_tanh_sfu(x) : dd_tanh_light(x);
    if (MODE == DD_ACTIVATION_ELU) return x > 0.0f ? x : dd_mul_rn(coef, dd_expm1_neg_light(x));
  }
  if (MODE == DD_ACTIVATION_RELU) {
    if (coef == (C)0) {
      if (nanProp && x != x) return x;
      return M::max(x, (C)0);
    }
    return x > (C)0 ? x : dd_mul_rn(coef, x);
  } else if (MODE == DD_ACTIVATION_SIGMOID) {
    return M::sigmoid(x);
  } else if (MODE == DD_ACTIVATION_TANH) {
    return M::tanh_(x);
  } else if (MODE == DD_ACTIVATION_ELU) {
    return x > (C)0 ? x : dd_mul_rn(coef, M::expm1_neg(x));
  } else if (MODE == DD_ACTIVATION_LINEAR) {
    return M::fma(coef, x, shift);
  } else if (MODE == DD_ACTIVATION_CLIPPED_RELU) {
    if (nanProp && x != x) return x;
    return M::min(M::max(x, (C)0), coef);
  } else {  // ABS
    return M::abs(x);
  }
}

// returns act'(x) * dy
template <typename C, int MODE, int LIGHT = 0>
__device__ __forceinline__ C dd_act_bwd(C x, C dy, C coef, C shift = (C)0, int kind = 0) {
  typedef dd_math<C> M;
  if (MODE == DD_ACT_FAM_CHEAP) return dd_ext_cheap_bwd<C>(kind, x, dy, coef, shift);
  if (MODE == DD_ACT_FAM_TRANS) return dd_ext_trans_bwd<C>(kind, x, dy, coef, shift);
  if (MODE == DD_ACTIVATION_SWISH || MODE == DD_ACTIVATION_GELU_TANH) return dd_ext_trans_bwd<C>(MODE, x, dy, coef, shift);
  if constexpr (LIGHT != 0 && sizeof(C) == 4) {
    if (MODE == DD_ACTIVATION_SIGMOID) return dd_mul_rn(dy, dd_dsigmoid_light(x));
    if (MODE == DD_ACTIVATION_TANH) return dd_mul_rn(dy, dd_dtanh_light(x));
    if (MODE == DD_ACTIVATION_ELU) return x > 0.0f ? dy : dd_mul_rn(dy, dd_mul_rn(coef, dd_exp_neg_light(x)));
  }
  if (MODE == DD_ACTIVATION_RELU) {
    return x > (C)0 ? dy : dd_mul_rn(coef, dy);
  } else if (MODE == DD_ACTIVATION_SIGMOID) {
    return dd_mul_rn(dy, M::dsigmoid(x));
  } else if (MODE == DD_ACTIVATION_TANH) {
    return dd_mul_rn(dy, M::dtanh(x));
  } else if (MODE == DD_ACTIVATION_ELU) {
    return x > (C)0 ? dy : dd_mul_rn(dy, dd_scale(coef, M::exp_neg(x)));
  } else if (MODE == DD_ACTIVATION_LINEAR) {
    return dd_mul_rn(coef, dy);
  } else if (MODE == DD_ACTIVATION_CLIPPED_RELU) {
    return (x > (C)0 && x <= coef) ? dy : (C)0;
  } else {  // ABS
    return x > (C)0 ? dy : (x < (C)0 ? -dy : (C)0);
  }
}

// The transcendental modes on TWO fp32 elements at a time (packed f32x2 arithmetic): the same
// formulas as above, lane for lane, with identical results.
template <int MODE> struct dd_act_packed { static constexpr bool value = false; };
template <> struct dd_act_packed<DD_ACTIVATION_SIGMOID> { static constexpr bool value = true; };
template <> struct dd_act_packed<DD_ACTIVATION_TANH> { static constexpr bool value = true; };
template <> struct dd_act_packed<DD_ACTIVATION_ELU> { static constexpr bool value = true; };
template <> struct dd_act_packed<DD_ACTIVATION_SWISH> { static constexpr bool value = true; };
template <> struct dd_act_packed<DD_ACTIVATION_GELU_TANH> { static constexpr bool value = true; };

// g and g' of gelu-tanh on two lanes: g = sqrt(2/pi) x (1 + 0.044715 x^2)
__device__ __forceinline__ float2 dd_gelu_g2(float2 x, float2 x2) {
  typedef dd_lane<float2> L;
  return L::mul(L::mul(L::bc(0.7978845608028654f), x), L::fma(L::bc(0.044715f), x2, L::bc(1.0f)));
}

template <int MODE>
__device__ __forceinline__ float2 dd_act_fwd2(float2 x, float coef) {
  typedef dd_lane<float2> L;
  if (MODE == DD_ACTIVATION_SIGMOID) return dd_sigmoid<float2>(x);
  if (MODE == DD_ACTIVATION_TANH) return dd_tanh<float2>(x);
  if (MODE == DD_ACTIVATION_SWISH) return L::mul(x, dd_sigmoid<float2>(L::mul(L::bc(coef), x)));
  if (MODE == DD_ACTIVATION_GELU_TANH) {
    const float2 g = dd_gelu_g2(x, L::mul(x, x));
    return L::mul(x, dd_sigmoid<float2>(L::add(g, g)));
  }
  return L::sel_pos(x, x, L::mul(L::bc(coef), dd_expm1_neg<float2>(x)));  // ELU
}

template <int MODE>
__device__ __forceinline__ float2 dd_act_bwd2(float2 x, float2 dy, float coef) {
  typedef dd_lane<float2> L;
  if (MODE == DD_ACTIVATION_SIGMOID)
    return L::mul(dy, dd_e_over_one_plus_e_sq<float2, 0>(L::neg_abs_clamped<1>(x, -104.0f)));
  if (MODE == DD_ACTIVATION_TANH)
    return L::mul(dy, dd_e_over_one_plus_e_sq<float2, 2>(L::neg_abs_clamped<2>(x, -104.0f)));
  if (MODE == DD_ACTIVATION_SWISH) {  // s + t s (1 - s), t = a x
    const float2 t = L::mul(L::bc(coef), x);
    const float2 ds = dd_e_over_one_plus_e_sq<float2, 0>(L::neg_abs_clamped<1>(t, -104.0f));
    return L::mul(dy, L::fma(t, ds, dd_sigmoid<float2>(t)));
  }
  if (MODE == DD_ACTIVATION_GELU_TANH) {  // s + 2 x g' s (1 - s), s = sigma(2g)
    const float2 x2 = L::mul(x, x);
    const float2 g = dd_gelu_g2(x, x2);
    const float2 gp = L::mul(L::bc(0.7978845608028654f), L::fma(L::bc(0.134145f), x2, L::bc(1.0f)));
    const float2 g2 = L::add(g, g);
    const float2 ds = dd_e_over_one_plus_e_sq<float2, 0>(L::neg_abs_clamped<1>(g2, -104.0f));
    return L::mul(dy, L::fma(L::mul(L::add(x, x), gp), ds, dd_sigmoid<float2>(g2)));
  }
  return L::sel_pos(x, dy, L::mul(dy, L::mul(L::bc(coef), dd_exp_neg_rounded<float2>(x))));  // ELU
}

// alpha*v + beta*old.  Multiplying by exactly 1 is exact, so alpha is applied unconditionally.
template <typename C>
__device__ __forceinline__ C dd_blend(C alpha, C v, C beta, C old, bool useOld) {
  C t = dd_mul_rn(alpha, v);
  return useOld ? dd_add_rn(t, dd_mul_rn(beta, old)) : t;
}

struct ddEltFlatParams {
  const void *x;   // forward: source.  backward: forward source
  const void *dy;  // backward only
  void *out;       // forward: y.  backward: dx
  int64_t n;
  double alpha, beta;
  ddActArgs act;
  int vec;
};

// PLAIN: alpha == 1 and beta == 0 (what every layer passes): no blend arithmetic at all.
// (the run-time-switched transcendental family gets 64 registers: the math library's slow paths spill at 32)
template <typename T, typename C, int MODE, bool BWD, bool PLAIN>
__global__ void __launch_bounds__(256, MODE == DD_ACT_FAM_TRANS ? 4 : 8) dd_elt_flat_kernel(ddEltFlatParams p) {
  dd_pdl_prologue();
  constexpr int V = 16 / sizeof(T);
  const T *x = (const T *)p.x;
  const T *dy = (const T *)p.dy;
  T *out = (T *)p.out;
  const C alpha = (C)p.alpha, beta = (C)p.beta, coef = (C)p.act.coef, shift = (C)p.act.shift;
  const bool useOld = p.beta != 0.0, nanProp = p.act.nanProp != 0;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  int64_t done = 0;
  if (p.vec) {
    const int64_t nv = p.n / V;
    for (int64_t i = tid; i < nv; i += nthreads) {
      uint4 xin = *(const uint4 *)(x + i * V);
      uint4 din = BWD ? *(const uint4 *)(dy + i * V) : make_uint4(0, 0, 0, 0);
      uint4 oin = make_uint4(0, 0, 0, 0);
      if (!PLAIN && useOld) oin = *(const uint4 *)(out + i * V);
      uint4 res;
      const T *xv = (const T *)&xin, *dv = (const T *)&din, *ov = (const T *)&oin;
      T *rv = (T *)&res;
      if constexpr (sizeof(C) == 4 && sizeof(T) == 4 && dd_act_packed<MODE>::value) {
#pragma unroll
        for (int k = 0; k < V; k += 2) {
          const float2 xc = make_float2(dd_load<float, T>(xv[k]), dd_load<float, T>(xv[k + 1]));
          float2 v;
          if (BWD) v = dd_act_bwd2<MODE>(xc, make_float2(dd_load<float, T>(dv[k]), dd_load<float, T>(dv[k + 1])), coef);
          else v = dd_act_fwd2<MODE>(xc, coef);
          rv[k] = PLAIN ? dd_store<T, float>(v.x) : dd_store<T, float>(dd_blend(alpha, v.x, beta, dd_load<float, T>(ov[k]), useOld));
          rv[k + 1] = PLAIN ? dd_store<T, float>(v.y) : dd_store<T, float>(dd_blend(alpha, v.y, beta, dd_load<float, T>(ov[k + 1]), useOld));
        }
      } else {
        C vals[V];
#pragma unroll
        for (int k = 0; k < V; k++) {
          C xc = dd_load<C, T>(xv[k]);
          C v = BWD ? dd_act_bwd<C, MODE, dd_light<T>::value>(xc, dd_load<C, T>(dv[k]), coef, shift, p.act.kind)
                    : dd_act_fwd<C, MODE, dd_light<T>::value>(xc, coef, shift, nanProp, p.act.kind);
          vals[k] = PLAIN ? v : dd_blend(alpha, v, beta, dd_load<C, T>(ov[k]), useOld);
        }
        dd_store_n<T, C, V>(rv, vals);
      }
      *(uint4 *)(out + i * V) = res;
    }
    done = nv * V;
  }
  for (int64_t i = done + tid; i < p.n; i += nthreads) {
    C xc = dd_load<C, T>(x[i]);
    C v = BWD ? dd_act_bwd<C, MODE, dd_light<T>::value>(xc, dd_load<C, T>(dy[i]), coef, shift, p.act.kind)
              : dd_act_fwd<C, MODE, dd_light<T>::value>(xc, coef, shift, nanProp, p.act.kind);
    C old = useOld ? dd_load<C, T>(out[i]) : (C)0;
    out[i] = dd_store<T, C>(dd_blend(alpha, v, beta, old, useOld));
  }
}

// The fp32 transcendental modes (logistic, tanh, elu; alpha == 1, beta == 0, 16-byte aligned) with U
// 16-byte vectors per thread-iteration: all U loads (2 U backward) go out before the first result is
// computed, so a thread keeps U times the bytes in flight while it works through some twenty
// instructions per element.  64 registers, 4 CTAs of 256 threads per SM.
template <int MODE, bool BWD, int U>
__global__ void __launch_bounds__(256, 4) dd_elt_flat_multi_kernel(ddEltFlatParams p) {
  dd_pdl_prologue();
  const float *x = (const float *)p.x;
  const float *dy = (const float *)p.dy;
  float *out = (float *)p.out;
  const float coef = (float)p.act.coef, shift = (float)p.act.shift;
  const bool nanProp = p.act.nanProp != 0;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int64_t nv = p.n / 4;
  for (int64_t base = tid; base < nv; base += (int64_t)U * nthreads) {
    float4 xin[U], din[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int64_t i = base + (int64_t)u * nthreads;
      if (i < nv) {
        xin[u] = *(const float4 *)(x + i * 4);
        if (BWD) din[u] = *(const float4 *)(dy + i * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int64_t i = base + (int64_t)u * nthreads;
      if (i < nv) {
        float2 lo, hi;
        if (BWD) {
          lo = dd_act_bwd2<MODE>(make_float2(xin[u].x, xin[u].y), make_float2(din[u].x, din[u].y), coef);
          hi = dd_act_bwd2<MODE>(make_float2(xin[u].z, xin[u].w), make_float2(din[u].z, din[u].w), coef);
        } else {
          lo = dd_act_fwd2<MODE>(make_float2(xin[u].x, xin[u].y), coef);
          hi = dd_act_fwd2<MODE>(make_float2(xin[u].z, xin[u].w), coef);
        }
        *(float4 *)(out + i * 4) = make_float4(lo.x, lo.y, hi.x, hi.y);
      }
    }
  }
  for (int64_t i = nv * 4 + tid; i < p.n; i += nthreads) {
    const float xc = x[i];
    out[i] = BWD ? dd_act_bwd<float, MODE, false>(xc, dy[i], coef) : dd_act_fwd<float, MODE, false>(xc, coef, shift, nanProp, p.act.kind);
  }
}

struct ddEltStridedParams {
  const void *x;
  const void *dy;
  void *out;
  ddStridedParams<3> sp;  // operands: 0 = x, 1 = dy (backward), 2 = out
  double alpha, beta;
  ddActArgs act;
};

template <typename T, typename C, int MODE, bool BWD>
__global__ void __launch_bounds__(256) dd_elt_strided_kernel(ddEltStridedParams p) {
  const T *x = (const T *)p.x;
  const T *dy = (const T *)p.dy;
  T *out = (T *)p.out;
  const C alpha = (C)p.alpha, beta = (C)p.beta, coef = (C)p.act.coef, shift = (C)p.act.shift;
  const bool useOld = p.beta != 0.0, nanProp = p.act.nanProp != 0;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.sp.total; i += nthreads) {
    int64_t off[3];
    dd_offsets<3, int64_t>(p.sp, i, off);
    C xc = dd_load<C, T>(x[off[0]]);
    C v = BWD ? dd_act_bwd<C, MODE, dd_light<T>::value>(xc, dd_load<C, T>(dy[off[1]]), coef, shift, p.act.kind)
              : dd_act_fwd<C, MODE, dd_light<T>::value>(xc, coef, shift, nanProp, p.act.kind);
    C old = useOld ? dd_load<C, T>(out[off[2]]) : (C)0;
    out[off[2]] = dd_store<T, C>(dd_blend(alpha, v, beta, old, useOld));
  }
}

// Rows: views whose innermost dim is contiguous for every operand (a channel window, a batch slice
// with its own pitch): the strided walk over 16-byte vectors.  `sp` counts the innermost dim in
// vectors of V elements (extent / V, stride V).
template <typename T, typename C, int MODE, bool BWD>
__global__ void __launch_bounds__(256) dd_elt_rows_kernel(ddEltStridedParams p) {
  constexpr int V = 16 / sizeof(T);
  const T *x = (const T *)p.x;
  const T *dy = (const T *)p.dy;
  T *out = (T *)p.out;
  const C alpha = (C)p.alpha, beta = (C)p.beta, coef = (C)p.act.coef, shift = (C)p.act.shift;
  const bool useOld = p.beta != 0.0, nanProp = p.act.nanProp != 0;
  const uint32_t total = (uint32_t)p.sp.total, nthreads = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nthreads) {
    int64_t off[3];
    dd_offsets32<3>(p.sp, i, off);
    uint4 xin = *(const uint4 *)(x + off[0]);
    uint4 din = BWD ? *(const uint4 *)(dy + off[1]) : make_uint4(0, 0, 0, 0);
    uint4 oin = make_uint4(0, 0, 0, 0);
    if (useOld) oin = *(const uint4 *)(out + off[2]);
    uint4 res;
    const T *xv = (const T *)&xin, *dv = (const T *)&din, *ov = (const T *)&oin;
    T *rv = (T *)&res;
    C vals[V];
#pragma unroll
    for (int k = 0; k < V; k++) {
      C xc = dd_load<C, T>(xv[k]);
      C v = BWD ? dd_act_bwd<C, MODE, dd_light<T>::value>(xc, dd_load<C, T>(dv[k]), coef, shift, p.act.kind)
                : dd_act_fwd<C, MODE, dd_light<T>::value>(xc, coef, shift, nanProp, p.act.kind);
      vals[k] = dd_blend(alpha, v, beta, dd_load<C, T>(ov[k]), useOld);
    }
    dd_store_n<T, C, V>(rv, vals);
    *(uint4 *)(out + off[2]) = res;
  }
}

// True when every operand's innermost dim is contiguous and every vector start is 16-byte aligned.
template <typename T, bool BWD>
static bool dd_elt_rows_ok(const ddCanon &c, const void *x, const void *dy, const void *out) {
  constexpr int V = 16 / (int)sizeof(T);
  const int last = c.nd - 1;
  if (c.nd < 2 || c.dims[last] % V != 0 || c.total / V >= 0x7fffffffLL) return false;
  uintptr_t bits = (uintptr_t)x | (uintptr_t)out | (BWD ? (uintptr_t)dy : 0);
  if (bits & 15) return false;
  for (int o = 0; o < 3; o++) {
    if (o == 1 && !BWD) continue;
    if (c.st[o][last] != 1) return false;
    for (int i = 0; i < last; i++)
      if ((c.st[o][i] * (int64_t)sizeof(T)) % 16 != 0) return false;
  }
  return true;
}

template <typename T, typename C, int MODE, bool BWD>
static ddStatus_t launch_elt(ddHandle_t h, const ddCanon &c, const void *x, const void *dy, void *out,
                             double alpha, double beta, const ddActArgs &act) {
  bool dense = c.nd == 1 && c.st[0][0] == 1 && c.st[2][0] == 1 && (!BWD || c.st[1][0] == 1);
  if (dense) {
    ddEltFlatParams p;
    p.x = x;
    p.dy = dy;
    p.out = out;
    p.n = c.total;
    p.alpha = alpha;
    p.beta = beta;
    p.act = act;
    uintptr_t bits = (uintptr_t)x | (uintptr_t)out | (BWD ? (uintptr_t)dy : 0);
    p.vec = (bits & 15) == 0;
    constexpr int V = 16 / sizeof(T);
    if constexpr (sizeof(T) == 4 && sizeof(C) == 4 && dd_act_packed<MODE>::value) {
      // backward (two loads per vector): two vectors per thread-iteration measured 4-5 % faster than one
      // on [256,256,28,28] (tanh 96.7 us against 100.6-105.0, logistic 94.6-95.9 against 100.1-104.2);
      // forward measured the same or slower with 2, 3 or 4 and keeps the one-vector kernel
      const int U = BWD ? dd_tune("DD_ELT_U_BWD", 2) : dd_tune("DD_ELT_U_FWD", 1);
      if (U > 1 && p.vec && alpha == 1.0 && beta == 0.0) {
        const int cps = dd_tune("DD_ELT_MULTI_CPS", 24);  // 8 -> 24: gelu-tanh / swish backward +2 %
        unsigned g = dd_flat_grid(h, (p.n / 4 + U - 1) / U, 256, cps);
        if (U == 2) dd_launch_pdl(dd_elt_flat_multi_kernel<MODE, BWD, 2>, g, 256, h->stream, p);
        else if (U == 3) dd_launch_pdl(dd_elt_flat_multi_kernel<MODE, BWD, 3>, g, 256, h->stream, p);
        else dd_launch_pdl(dd_elt_flat_multi_kernel<MODE, BWD, 4>, g, 256, h->stream, p);
        DD_LAUNCHED(h, BWD ? "activation-bwd/flat-multi" : "activation-fwd/flat-multi");
        return DD_STATUS_SUCCESS;
      }
    }
    // 48 CTAs per SM (six times the resident eight): on [256,256,28,28] the whole forward + backward step
    // measured 6154-6160 GB/s with 16, 6196 with 32, 6240 with 48 or 64, 6209 with 128 (same box, same
    // clocks); shorter CTAs shorten the tail of each launch, relu backward most (6070 -> 6320 GB/s)
    // backward (three streams) keeps gaining up to 160-190 CTAs per SM (relu backward 6070 GB/s with 16, 6320 with
    // 48, 6490 with 128; hardswish backward 6595 / 6850 / 6946 with 48 / 96 / 192); forward peaks at 48-64
    unsigned grid = dd_flat_grid(h, (p.n + V - 1) / V, 256, BWD ? dd_tune("DD_ELTFLAT_CPS_BWD", 160) : dd_tune("DD_ELTFLAT_CPS", 48));
    if (alpha == 1.0 && beta == 0.0) dd_launch_pdl(dd_elt_flat_kernel<T, C, MODE, BWD, true>, grid, 256, h->stream, p);
    else dd_launch_pdl(dd_elt_flat_kernel<T, C, MODE, BWD, false>, grid, 256, h->stream, p);
    DD_LAUNCHED(h, BWD ? "activation-bwd/flat" : "activation-fwd/flat");
  } else if (dd_elt_rows_ok<T, BWD>(c, x, dy, out)) {
    constexpr int V = 16 / (int)sizeof(T);
    ddCanon v = c;
    const int last = c.nd - 1;
    v.dims[last] = c.dims[last] / V;
    for (int o = 0; o < 3; o++) v.st[o][last] = V;
    v.total = c.total / V;
    ddEltStridedParams p;
    p.x = x;
    p.dy = dy;
    p.out = out;
    p.sp = dd_strided_params<3>(v);
    p.alpha = alpha;
    p.beta = beta;
    p.act = act;
    unsigned grid = dd_flat_grid(h, v.total, 256, 64);
    dd_elt_rows_kernel<T, C, MODE, BWD><<<grid, 256, 0, h->stream>>>(p);
    DD_LAUNCHED(h, BWD ? "activation-bwd/rows" : "activation-fwd/rows");
  } else {
    ddEltStridedParams p;
    p.x = x;
    p.dy = dy;
    p.out = out;
    p.sp = dd_strided_params<3>(c);
    p.alpha = alpha;
    p.beta = beta;
    p.act = act;
    unsigned grid = dd_flat_grid(h, c.total, 256, 16);
    dd_elt_strided_kernel<T, C, MODE, BWD><<<grid, 256, 0, h->stream>>>(p);
    DD_LAUNCHED(h, BWD ? "activation-bwd/strided" : "activation-fwd/strided");
  }
  return DD_STATUS_SUCCESS;
}

template <typename T, typename C, bool BWD>
static ddStatus_t dispatch_mode(ddHandle_t h, int mode, const ddCanon &c, const void *x,
                                const void *dy, void *out, double alpha, double beta,
                                const ddActArgs &act) {
  switch (mode) {
    case DD_ACTIVATION_SIGMOID: return launch_elt<T, C, DD_ACTIVATION_SIGMOID, BWD>(h, c, x, dy, out, alpha, beta, act);
    case DD_ACTIVATION_RELU: return launch_elt<T, C, DD_ACTIVATION_RELU, BWD>(h, c, x, dy, out, alpha, beta, act);
    case DD_ACTIVATION_TANH: return launch_elt<T, C, DD_ACTIVATION_TANH, BWD>(h, c, x, dy, out, alpha, beta, act);
    case DD_ACTIVATION_CLIPPED_RELU: return launch_elt<T, C, DD_ACTIVATION_CLIPPED_RELU, BWD>(h, c, x, dy, out, alpha, beta, act);
    case DD_ACTIVATION_ELU: return launch_elt<T, C, DD_ACTIVATION_ELU, BWD>(h, c, x, dy, out, alpha, beta, act);
    case DD_ACTIVATION_LINEAR: return launch_elt<T, C, DD_ACTIVATION_LINEAR, BWD>(h, c, x, dy, out, alpha, beta, act);
    case DD_ACTIVATION_ABS: return launch_elt<T, C, DD_ACTIVATION_ABS, BWD>(h, c, x, dy, out, alpha, beta, act);
    case DD_ACTIVATION_ROUND:
      if (BWD) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "activation: round has no backward (oneDNN defines it forward only)");
    case DD_ACTIVATION_SQUARE: case DD_ACTIVATION_SQRT: case DD_ACTIVATION_HARDSWISH: case DD_ACTIVATION_CLIP:
    case DD_ACTIVATION_CLIP_V2: case DD_ACTIVATION_TANH_DST_BWD: case DD_ACTIVATION_ELU_DST_BWD:
    case DD_ACTIVATION_SQRT_DST_BWD: case DD_ACTIVATION_LOGISTIC_DST_BWD: case DD_ACTIVATION_EXP_DST_BWD:
      return launch_elt<T, C, DD_ACT_FAM_CHEAP, BWD>(h, c, x, dy, out, alpha, beta, act);
    case DD_ACTIVATION_SWISH: return launch_elt<T, C, DD_ACTIVATION_SWISH, BWD>(h, c, x, dy, out, alpha, beta, act);
    case DD_ACTIVATION_GELU_TANH: return launch_elt<T, C, DD_ACTIVATION_GELU_TANH, BWD>(h, c, x, dy, out, alpha, beta, act);
    case DD_ACTIVATION_EXP: case DD_ACTIVATION_LOG: case DD_ACTIVATION_SOFT_RELU:
    case DD_ACTIVATION_GELU_ERF: case DD_ACTIVATION_POW: case DD_ACTIVATION_MISH:
      return launch_elt<T, C, DD_ACT_FAM_TRANS, BWD>(h, c, x, dy, out, alpha, beta, act);
  }
  DD_FAIL(h, DD_STATUS_BAD_PARAM, "activation: unknown mode %d", mode);
}

template <bool BWD>
static ddStatus_t dispatch_type(ddHandle_t h, ddDataType_t t, int mode, const ddCanon &c,
                                const void *x, const void *dy, void *out, double alpha, double beta,
                                const ddActArgs &act) {
  switch (t) {
    case DD_DATA_FLOAT: return dispatch_mode<float, float, BWD>(h, mode, c, x, dy, out, alpha, beta, act);
    case DD_DATA_DOUBLE: return dispatch_mode<double, double, BWD>(h, mode, c, x, dy, out, alpha, beta, act);
    case DD_DATA_HALF: return dispatch_mode<__half, float, BWD>(h, mode, c, x, dy, out, alpha, beta, act);
    case DD_DATA_BFLOAT16: return dispatch_mode<__nv_bfloat16, float, BWD>(h, mode, c, x, dy, out, alpha, beta, act);
    default: break;
  }
  DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "activation: data type must be floating point");
}

ddStatus_t dd_activation_fwd_impl(ddHandle_t h, const ddActivationStruct *a, double alpha,
                                  const ddTensorStruct *xd, const void *x, double beta,
                                  const ddTensorStruct *yd, void *y) {
  int64_t st[3][DD_DIM_MAX];
  for (int i = 0; i < xd->nd; i++) {
    st[0][i] = xd->strides[i];
    st[1][i] = xd->strides[i];
    st[2][i] = yd->strides[i];
  }
  ddCanon c;
  dd_canonicalize(&c, xd->nd, xd->dims, 3, st, 2);
  // a *-dst-bwd kind runs the forward of the kind it is named after
  int mode = a->mode;
  switch (mode) {
    case DD_ACTIVATION_RELU_DST_BWD: mode = DD_ACTIVATION_RELU; break;
    case DD_ACTIVATION_TANH_DST_BWD: mode = DD_ACTIVATION_TANH; break;
    case DD_ACTIVATION_ELU_DST_BWD: mode = DD_ACTIVATION_ELU; break;
    case DD_ACTIVATION_SQRT_DST_BWD: mode = DD_ACTIVATION_SQRT; break;
    case DD_ACTIVATION_LOGISTIC_DST_BWD: mode = DD_ACTIVATION_SIGMOID; break;
    case DD_ACTIVATION_EXP_DST_BWD: mode = DD_ACTIVATION_EXP; break;
    case DD_ACTIVATION_CLIP_V2_DST_BWD: mode = DD_ACTIVATION_CLIP_V2; break;
    default: break;
  }
  ddActArgs act = {a->coef, a->shift, a->nan == DD_PROPAGATE_NAN, mode};
  return dispatch_type<false>(h, xd->dtype, mode, c, x, nullptr, y, alpha, beta, act);
}

ddStatus_t dd_activation_bwd_impl(ddHandle_t h, const ddActivationStruct *a, double alpha,
                                  const ddTensorStruct *dyd, const void *dy,
                                  const ddTensorStruct *xd, const void *x, double beta,
                                  const ddTensorStruct *dxd, void *dx) {
  int64_t st[3][DD_DIM_MAX];
  for (int i = 0; i < xd->nd; i++) {
    st[0][i] = xd->strides[i];
    st[1][i] = dyd->strides[i];
    st[2][i] = dxd->strides[i];
  }
  ddCanon c;
  dd_canonicalize(&c, xd->nd, xd->dims, 3, st, 2);
  // `x` is the forward result for the *-dst-bwd kinds (the caller has put y in its place); relu and
  // clip-v2 have the same derivative written in terms of either
  int mode = a->mode;
  if (mode == DD_ACTIVATION_RELU_DST_BWD) mode = DD_ACTIVATION_RELU;
  if (mode == DD_ACTIVATION_CLIP_V2_DST_BWD) mode = DD_ACTIVATION_CLIP_V2;
  ddActArgs act = {a->coef, a->shift, a->nan == DD_PROPAGATE_NAN, mode};
  return dispatch_type<true>(h, xd->dtype, mode, c, x, dy, dx, alpha, beta, act);
}
