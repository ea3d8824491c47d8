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
};

struct ddActArgs {
  double coef, shift;
  int nanProp;
};

// The result of a 16-bit element type takes the special-function-unit forms of dd_math_f32.cuh for
// the transcendental modes (at most one unit of the 16-bit type off).
// LIGHT: 0 = full float accuracy, 1 = f16 result, 2 = bf16 result
template <typename T> struct dd_light { static constexpr int value = 0; };
template <> struct dd_light<__half> { static constexpr int value = 1; };
template <> struct dd_light<__nv_bfloat16> { static constexpr int value = 2; };

template <typename C, int MODE, int LIGHT = 0>
__device__ __forceinline__ C dd_act_fwd(C x, C coef, C shift, bool nanProp) {
  typedef dd_math<C> M;
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
__device__ __forceinline__ C dd_act_bwd(C x, C dy, C coef) {
  typedef dd_math<C> M;
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

template <int MODE>
__device__ __forceinline__ float2 dd_act_fwd2(float2 x, float coef) {
  typedef dd_lane<float2> L;
  if (MODE == DD_ACTIVATION_SIGMOID) return dd_sigmoid<float2>(x);
  if (MODE == DD_ACTIVATION_TANH) return dd_tanh<float2>(x);
  return L::sel_pos(x, x, L::mul(L::bc(coef), dd_expm1_neg<float2>(x)));  // ELU
}

template <int MODE>
__device__ __forceinline__ float2 dd_act_bwd2(float2 x, float2 dy, float coef) {
  typedef dd_lane<float2> L;
  if (MODE == DD_ACTIVATION_SIGMOID)
    return L::mul(dy, dd_e_over_one_plus_e_sq<float2, 0>(L::neg_abs_clamped<1>(x, -104.0f)));
  if (MODE == DD_ACTIVATION_TANH)
    return L::mul(dy, dd_e_over_one_plus_e_sq<float2, 2>(L::neg_abs_clamped<2>(x, -104.0f)));
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
template <typename T, typename C, int MODE, bool BWD, bool PLAIN>
__global__ void __launch_bounds__(256, 8) dd_elt_flat_kernel(ddEltFlatParams p) {
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
#pragma unroll
        for (int k = 0; k < V; k++) {
          C xc = dd_load<C, T>(xv[k]);
          C v = BWD ? dd_act_bwd<C, MODE, dd_light<T>::value>(xc, dd_load<C, T>(dv[k]), coef)
                    : dd_act_fwd<C, MODE, dd_light<T>::value>(xc, coef, shift, nanProp);
          rv[k] = PLAIN ? dd_store<T, C>(v) : dd_store<T, C>(dd_blend(alpha, v, beta, dd_load<C, T>(ov[k]), useOld));
        }
      }
      *(uint4 *)(out + i * V) = res;
    }
    done = nv * V;
  }
  for (int64_t i = done + tid; i < p.n; i += nthreads) {
    C xc = dd_load<C, T>(x[i]);
    C v = BWD ? dd_act_bwd<C, MODE, dd_light<T>::value>(xc, dd_load<C, T>(dy[i]), coef)
              : dd_act_fwd<C, MODE, dd_light<T>::value>(xc, coef, shift, nanProp);
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
    out[i] = BWD ? dd_act_bwd<float, MODE, false>(xc, dy[i], coef) : dd_act_fwd<float, MODE, false>(xc, coef, shift, nanProp);
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
    C v = BWD ? dd_act_bwd<C, MODE, dd_light<T>::value>(xc, dd_load<C, T>(dy[off[1]]), coef)
              : dd_act_fwd<C, MODE, dd_light<T>::value>(xc, coef, shift, nanProp);
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
#pragma unroll
    for (int k = 0; k < V; k++) {
      C xc = dd_load<C, T>(xv[k]);
      C v = BWD ? dd_act_bwd<C, MODE, dd_light<T>::value>(xc, dd_load<C, T>(dv[k]), coef)
                : dd_act_fwd<C, MODE, dd_light<T>::value>(xc, coef, shift, nanProp);
      rv[k] = dd_store<T, C>(dd_blend(alpha, v, beta, dd_load<C, T>(ov[k]), useOld));
    }
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
        const int cps = dd_tune("DD_ELT_MULTI_CPS", 8);
        unsigned g = dd_flat_grid(h, (p.n / 4 + U - 1) / U, 256, cps);
        if (U == 2) dd_launch_pdl(dd_elt_flat_multi_kernel<MODE, BWD, 2>, g, 256, h->stream, p);
        else if (U == 3) dd_launch_pdl(dd_elt_flat_multi_kernel<MODE, BWD, 3>, g, 256, h->stream, p);
        else dd_launch_pdl(dd_elt_flat_multi_kernel<MODE, BWD, 4>, g, 256, h->stream, p);
        DD_LAUNCHED(h, BWD ? "activation-bwd/flat-multi" : "activation-fwd/flat-multi");
        return DD_STATUS_SUCCESS;
      }
    }
    unsigned grid = dd_flat_grid(h, (p.n + V - 1) / V, 256, dd_tune("DD_ELTFLAT_CPS", 16));
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
    unsigned grid = dd_flat_grid(h, v.total, 256, 16);
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
  ddActArgs act = {a->coef, a->shift, a->nan == DD_PROPAGATE_NAN};
  return dispatch_type<false>(h, xd->dtype, a->mode, c, x, nullptr, y, alpha, beta, act);
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
  ddActArgs act = {a->coef, a->shift, a->nan == DD_PROPAGATE_NAN};
  return dispatch_type<true>(h, xd->dtype, a->mode, c, x, dy, dx, alpha, beta, act);
}
