/*
 * dd_oracle.c -- TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C, CPU restatement of what the reference's DNNL backend computes on the tensor hot path
 * (reorder with data type conversion, eltwise forward/backward, binary with broadcast, scaled sum,
 * reduction).  Only tests, the smoke check and the CPU-baseline leg of the benchmark may load it;
 * the GPU library never does.
 *
 * PARITY PINNING.  The reference (Clojure on the JVM calling oneDNN 3.13 through the bytedeco
 * preset `dnnl-platform 3.13-1.5.14`, deep-diamond-dnnl/project.clj:17) holds no arithmetic of its
 * own for these ops: it builds descriptors and calls oneDNN, which is not vendored in the reference
 * tree and cannot be run without a JVM.  This file therefore restates oneDNN's published
 * definitions of the primitives and is pinned by
 *   (1) every known-answer vector the reference's own tests hold for the path
 *       (tests/test_oracle_golden.py lists them with file:line), and
 *   (2) outputs of real oneDNN (the build bundled with PyTorch) for eltwise forward, same-shape
 *       add/mul and f32->bf16 conversion, committed under tests/golden/ with their generator.
 * Not pinned by either: elu, eltwise backward on non-trivial data, broadcast binary, mean, and
 * reductions on non-trivial floating data ("parity unpinned" for those).
 *
 * What each function follows in the reference (paths relative to the reference project):
 *   oracle_reorder      dnnl/core.clj:523-529 `reorder` + dnnl/impl.clj:372-376 (attr = NULL: no
 *                       scales) as used by DnnlTransformer, dnnl/tensor.clj:102-151; the alpha/beta
 *                       blend is cuDNN's transform-tensor form, cudnn/core.clj:131-144.
 *   oracle_eltwise_fwd  dnnl/core.clj:345-362 `eltwise-fwd`, dnnl/impl.clj:324-331; algorithm
 *                       keywords dnnl/constants.clj:277-308; alpha/beta defaults base/dnn.clj:79-82.
 *   oracle_eltwise_bwd  dnnl/core.clj:364-388 `eltwise-bwd` with args SRC, DIFF_DST, DIFF_SRC:
 *                       the derivative is taken from the forward SOURCE.
 *   oracle_binary       dnnl/core.clj:430-447 `binary` (+ cudnn/core.clj:117-129 add-tensor form).
 *   oracle_sum          dnnl/core.clj:392-426 `sum!`.
 *   oracle_reduce       dnnl/core.clj:796-803 `reduction`, kinds dnnl/constants.clj:393-402
 *                       (+ cudnn/core.clj:213-231 reduce-tensor's alpha/beta and op set).
 * (prefix dnnl/ = deep-diamond-dnnl/src/uncomplicate/diamond/internal/dnnl/,
 *  cudnn/ = deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/,
 *  base/ = deep-diamond-base/src/uncomplicate/diamond/.)
 *
 * Arithmetic rules (shared with the GPU kernels so that "bit-exact" is well defined):
 *   - conversions: to bf16/f16 round-to-nearest-even; to s8/u8/s32/s64 saturate then
 *     round-to-nearest-even, NaN -> 0; compute type float unless a 64-bit type (or an s32 source)
 *     is involved, then double.
 *   - alpha*v + beta*old: each product and the sum rounded separately (compile with
 *     -ffp-contract=off), a factor of exactly 1 skipped, beta == 0 does not read `old`.
 *   - transcendental eltwise (logistic, tanh, elu) in fp32: oneDNN's documented definition
 *     evaluated in double and rounded to float once -- the value every fp32 implementation
 *     (oneDNN's JIT polynomial, its libm-based reference, the GPU kernel) approximates to within
 *     its own few ulp; measured: oneDNN 3.10.2 is within 2 ulp of it for logistic, 1 for tanh.
 *     Backward = that rounded derivative times dy in fp32.  *_truth variants return doubles.
 *   - sum-type reductions add in pairwise order in the compute type over the logical (row-major)
 *     order of the reduced dims; max/min/mul run left to right; *_truth accumulates in long double.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -fPIC -shared -o oracle/libdd_oracle.so oracle/dd_oracle.c -lm
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { T_F32 = 0, T_F64 = 1, T_F16 = 2, T_S8 = 3, T_S32 = 4, T_U8 = 6, T_BF16 = 9, T_S64 = 15 };
#define MAXD 8

static int tsize(int t) {
  switch (t) {
    case T_F32: case T_S32: return 4;
    case T_F64: case T_S64: return 8;
    case T_F16: case T_BF16: return 2;
    case T_S8: case T_U8: return 1;
  }
  return 0;
}

/* ------------------------------------------------------------ scalar conversions ------------ */

static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static uint16_t f32_to_bf16(float f) { /* round-to-nearest-even; NaN stays NaN (quiet) */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

static float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else { /* subnormal: normalise */
      int e = -1;
      do { e++; man <<= 1; } while (!(man & 0x400u));
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
  else u = sign | ((exp + 112u) << 23) | (man << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static uint16_t f32_to_f16(float f) { /* round-to-nearest-even */
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t sign = (u >> 16) & 0x8000u;
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((a >> 13) & 0x1ffu)); /* NaN */
  if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);                        /* >= 65536: inf (65520 rounds below) */
  if (a < 0x38800000u) { /* result is subnormal or zero: value < 2^-14 */
    if (a < 0x33000000u) return (uint16_t)sign; /* < 2^-25 rounds to 0 */
    uint32_t exp = a >> 23;
    uint32_t man = (a & 0x7fffffu) | 0x800000u;
    uint32_t shift = 126u - exp; /* 14..24 */
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half & 1u))) half++;
    return (uint16_t)(sign | half);
  }
  uint32_t exp = (a >> 23) - 112u;
  uint32_t man = a & 0x7fffffu;
  uint32_t half = (exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++; /* may carry into exp: correct */
  return (uint16_t)(sign | half);
}

static uint16_t f64_to_f16(double d) { /* single rounding from double */
  /* round d to the f16 grid directly: go through float only when exact */
  float f = (float)d;
  if ((double)f == d) return f32_to_f16(f);
  /* inexact in float: nudge toward d so that the float keeps a sticky bit */
  uint16_t lo = f32_to_f16(nextafterf(f, (double)f < d ? INFINITY : -INFINITY));
  uint16_t hi = f32_to_f16(f);
  /* if both neighbours agree the result is settled; otherwise pick by distance in double */
  if (lo == hi) return hi;
  double dlo = fabs((double)f16_to_f32(lo) - d), dhi = fabs((double)f16_to_f32(hi) - d);
  if (dlo < dhi) return lo;
  if (dhi < dlo) return hi;
  return (lo & 1u) ? hi : lo;
}

static uint16_t f64_to_bf16(double d) {
  float f = (float)d;
  if ((double)f == d) return f32_to_bf16(f);
  uint16_t a = f32_to_bf16(f);
  uint16_t b = f32_to_bf16(nextafterf(f, (double)f < d ? INFINITY : -INFINITY));
  if (a == b) return a;
  double da = fabs((double)bf16_to_f32(a) - d), db = fabs((double)bf16_to_f32(b) - d);
  if (da < db) return a;
  if (db < da) return b;
  return (a & 1u) ? b : a;
}

static double load_as_double(const void *p, int t, int64_t i) {
  switch (t) {
    case T_F32: return ((const float *)p)[i];
    case T_F64: return ((const double *)p)[i];
    case T_F16: return f16_to_f32(((const uint16_t *)p)[i]);
    case T_BF16: return bf16_to_f32(((const uint16_t *)p)[i]);
    case T_S8: return ((const int8_t *)p)[i];
    case T_U8: return ((const uint8_t *)p)[i];
    case T_S32: return ((const int32_t *)p)[i];
    case T_S64: return (double)((const int64_t *)p)[i];
  }
  return 0;
}
static float load_as_float(const void *p, int t, int64_t i) { return (float)load_as_double(p, t, i); }

static void store_from_float(void *p, int t, int64_t i, float v) {
  switch (t) {
    case T_F32: ((float *)p)[i] = v; break;
    case T_F64: ((double *)p)[i] = v; break;
    case T_F16: ((uint16_t *)p)[i] = f32_to_f16(v); break;
    case T_BF16: ((uint16_t *)p)[i] = f32_to_bf16(v); break;
    case T_S8: ((int8_t *)p)[i] = v != v ? 0 : (int8_t)nearbyintf(fminf(fmaxf(v, -128.f), 127.f)); break;
    case T_U8: ((uint8_t *)p)[i] = v != v ? 0 : (uint8_t)nearbyintf(fminf(fmaxf(v, 0.f), 255.f)); break;
    case T_S32:
      if (v != v) ((int32_t *)p)[i] = 0;
      else if (v >= 2147483648.f) ((int32_t *)p)[i] = INT32_MAX;
      else if (v <= -2147483648.f) ((int32_t *)p)[i] = INT32_MIN;
      else ((int32_t *)p)[i] = (int32_t)nearbyintf(v);
      break;
    case T_S64:
      if (v != v) ((int64_t *)p)[i] = 0;
      else if (v >= 9223372036854775808.f) ((int64_t *)p)[i] = INT64_MAX;
      else if (v <= -9223372036854775808.f) ((int64_t *)p)[i] = INT64_MIN;
      else ((int64_t *)p)[i] = (int64_t)nearbyintf(v);
      break;
  }
}

static void store_from_double(void *p, int t, int64_t i, double v) {
  switch (t) {
    case T_F32: ((float *)p)[i] = (float)v; break;
    case T_F64: ((double *)p)[i] = v; break;
    case T_F16: ((uint16_t *)p)[i] = f64_to_f16(v); break;
    case T_BF16: ((uint16_t *)p)[i] = f64_to_bf16(v); break;
    case T_S8: ((int8_t *)p)[i] = v != v ? 0 : (int8_t)nearbyint(fmin(fmax(v, -128.0), 127.0)); break;
    case T_U8: ((uint8_t *)p)[i] = v != v ? 0 : (uint8_t)nearbyint(fmin(fmax(v, 0.0), 255.0)); break;
    case T_S32:
      if (v != v) ((int32_t *)p)[i] = 0;
      else if (v >= 2147483647.0) ((int32_t *)p)[i] = INT32_MAX;
      else if (v <= -2147483648.0) ((int32_t *)p)[i] = INT32_MIN;
      else ((int32_t *)p)[i] = (int32_t)nearbyint(v);
      break;
    case T_S64:
      if (v != v) ((int64_t *)p)[i] = 0;
      else if (v >= 9223372036854775808.0) ((int64_t *)p)[i] = INT64_MAX;
      else if (v <= -9223372036854775808.0) ((int64_t *)p)[i] = INT64_MIN;
      else ((int64_t *)p)[i] = (int64_t)nearbyint(v);
      break;
  }
}

static int compute_is_double(int st, int dt) { return tsize(st) == 8 || tsize(dt) == 8 || st == T_S32; }

/* ------------------------------------------------------------ index helpers ------------------ */

static int64_t total_of(int nd, const int64_t *dims) {
  int64_t n = 1;
  for (int i = 0; i < nd; i++) n *= dims[i];
  return n;
}

/* logical (row-major) linear index -> element offset under `st` */
static int64_t offset_of(int nd, const int64_t *dims, const int64_t *st, int64_t idx) {
  int64_t off = 0;
  for (int d = nd - 1; d >= 0; d--) {
    int64_t q = idx / dims[d];
    off += (idx - q * dims[d]) * st[d];
    idx = q;
  }
  return off;
}

/* ------------------------------------------------------------ reorder ------------------------ */

int oracle_reorder(int nd, const int64_t *dims, int st, const int64_t *sst, const void *src, int dt,
                   const int64_t *dst_st, void *dst, double alpha, double beta) {
  if (nd < 1 || nd > MAXD) return 1;
  const int64_t n = total_of(nd, dims);
  const int64_t inner = dims[nd - 1], outer = n / (inner ? inner : 1);
  const int dbl = compute_is_double(st, dt);
  const int raw = (st == dt && alpha == 1.0 && beta == 0.0);
  const int w = tsize(st);
#pragma omp parallel for schedule(static)
  for (int64_t o = 0; o < outer; o++) {
    int64_t so = offset_of(nd - 1, dims, sst, o), dof = offset_of(nd - 1, dims, dst_st, o);
    for (int64_t i = 0; i < inner; i++) {
      int64_t si = so + i * sst[nd - 1], di = dof + i * dst_st[nd - 1];
      if (raw) {
        memcpy((char *)dst + di * w, (const char *)src + si * w, (size_t)w);
      } else if (dbl) {
        double v = load_as_double(src, st, si);
        if (alpha != 1.0) v = alpha * v;
        if (beta != 0.0) {
          double u = load_as_double(dst, dt, di);
          if (beta != 1.0) u = beta * u;
          v = v + u;
        }
        store_from_double(dst, dt, di, v);
      } else {
        float v = load_as_float(src, st, si);
        if (alpha != 1.0) v = (float)alpha * v;
        if (beta != 0.0) {
          float u = load_as_float(dst, dt, di);
          if (beta != 1.0) u = (float)beta * u;
          v = v + u;
        }
        store_from_float(dst, dt, di, v);
      }
    }
  }
  return 0;
}

/* ------------------------------------------------------------ eltwise ------------------------ */

/* A_ELU_FP32: elu as oneDNN's fp32 kernels form it, alpha * (exp(x) - 1) with exp(x) rounded to
 * float BEFORE the subtraction (what dnnl/constants.clj:277-308 `:elu` binds).  Near zero the
 * subtraction cancels: the result keeps only the bits of exp(x) above 1.  Oracle-only: it exists so
 * that the tests can state how far the library's elu (alpha * expm1(x), no cancellation) sits from it. */
enum { A_SIGMOID = 0, A_RELU = 1, A_TANH = 2, A_CLIP = 3, A_ELU = 4, A_LINEAR = 5, A_ABS = 6, A_ELU_FP32 = 7,
       /* the rest of the reference's oneDNN table, dnnl/constants.clj:277-308, by oneDNN's documented
        * definitions (a = alpha, b = beta of the primitive); X_DST = derivative from the forward result */
       X_SQUARE = 20, X_SQRT, X_EXP, X_LOG, X_SOFT_RELU, X_SWISH, X_GELU_TANH, X_GELU_ERF, X_HARDSWISH,
       X_CLIP, X_CLIP_V2, X_POW, X_MISH, X_ROUND,
       X_RELU_DST, X_TANH_DST, X_ELU_DST, X_SQRT_DST, X_LOGISTIC_DST, X_EXP_DST, X_CLIP_V2_DST };

/* forward kind behind a *-dst-bwd kind */
static int fwd_alg_of(int alg) {
  switch (alg) {
    case X_RELU_DST: return A_RELU;
    case X_TANH_DST: return A_TANH;
    case X_ELU_DST: return A_ELU;
    case X_SQRT_DST: return X_SQRT;
    case X_LOGISTIC_DST: return A_SIGMOID;
    case X_EXP_DST: return X_EXP;
    case X_CLIP_V2_DST: return X_CLIP_V2;
  }
  return alg;
}

#define SQRT_2_OVER_PI 0.7978845608028654
#define GELU_C 0.044715

/* the transcendental kinds of the table in double (x, a, b already double) */
static double ext_fwd_d(int alg, double x, double a, double b) {
  switch (alg) {
    case X_SQUARE: return x * x;
    case X_SQRT: return sqrt(x);
    case X_EXP: return exp(x);
    case X_LOG: return log(x);
    case X_SOFT_RELU: { double t = a * x; return (t > 0 ? t + log1p(exp(-t)) : log1p(exp(t))) / a; }
    case X_SWISH: return x / (1.0 + exp(-a * x));
    case X_GELU_TANH: { double g = SQRT_2_OVER_PI * x * (1.0 + GELU_C * x * x); return x / (1.0 + exp(-2.0 * g)); }
    case X_GELU_ERF: return 0.5 * x * erfc(-x * M_SQRT1_2);
    case X_HARDSWISH: { double t = fma(a, x, b); return x * (t <= 0 ? 0.0 : (t >= 1 ? 1.0 : t)); }
    case X_CLIP: case X_CLIP_V2: return x <= a ? a : (x > b ? b : x);
    case X_POW: return a * pow(x, b);
    case X_MISH: { if (x > 20) return x; double e = exp(x), n = e * (e + 2.0); return x * (n / (n + 2.0)); }
    case X_ROUND: return rint(x);
  }
  return NAN;
}

/* derivative (not yet times dy); x is the forward source, or the forward result for X_*_DST */
static double ext_der_d(int alg, double x, double a, double b) {
  switch (alg) {
    case X_SQUARE: return x + x;
    case X_SQRT: return 1.0 / (2.0 * sqrt(x));
    case X_EXP: return exp(x);
    case X_LOG: return 1.0 / x;
    case X_SOFT_RELU: return 1.0 / (1.0 + exp(-a * x));
    case X_SWISH: { double s = 1.0 / (1.0 + exp(-a * x)); return s * (1.0 + a * x * (1.0 - s)); }
    case X_GELU_TANH: {
      double g = SQRT_2_OVER_PI * x * (1.0 + GELU_C * x * x), gp = SQRT_2_OVER_PI * (1.0 + 3.0 * GELU_C * x * x);
      double e = exp(-2.0 * fabs(g)), r = 1.0 / (1.0 + e), s = g >= 0 ? r : e * r;
      return s + 2.0 * x * gp * (e * r * r);
    }
    case X_GELU_ERF: return 0.5 * erfc(-x * M_SQRT1_2) + x * exp(-0.5 * x * x) * 0.3989422804014327;
    case X_HARDSWISH: { double t = fma(a, x, b); return t <= 0 ? 0.0 : (t >= 1 ? 1.0 : fma(a + a, x, b)); }
    case X_CLIP: return (x > a && x <= b) ? 1.0 : 0.0;
    case X_CLIP_V2: case X_CLIP_V2_DST: return (x > a && x < b) ? 1.0 : 0.0;
    case X_POW: return a * b * pow(x, b - 1.0);
    case X_MISH: {
      if (x > 20) return 1.0;
      double e = exp(x), d = e * e + 2.0 * e + 2.0;
      double w = 4.0 * (x + 1.0) + 4.0 * e * e + e * e * e + e * (4.0 * x + 6.0);
      return e * w / (d * d);
    }
    case X_TANH_DST: return 1.0 - x * x;
    case X_ELU_DST: return x > 0 ? 1.0 : x + a;
    case X_SQRT_DST: return 1.0 / (2.0 * x);
    case X_LOGISTIC_DST: return x * (1.0 - x);
    case X_EXP_DST: return x;
  }
  return NAN;
}

static float act_fwd_f(int alg, float x, float a, float b, int nanprop) {
  switch (alg) {
    case A_RELU:
      if (a == 0.f) {
        if (nanprop && x != x) return x;
        return fmaxf(x, 0.f);
      }
      return x > 0.f ? x : a * x;
    /* transcendental modes: the definition evaluated in double, rounded to float once */
    case A_SIGMOID: { double e = exp(-fabs((double)x)); double r = 1.0 / (1.0 + e); return (float)(x >= 0.f ? r : e * r); }
    case A_TANH: return (float)tanh((double)x);
    case A_ELU: return x > 0.f ? x : a * (float)expm1((double)x);
    case A_ELU_FP32: return x > 0.f ? x : a * ((float)exp((double)x) - 1.f);
    case A_LINEAR: return fmaf(a, x, b);
    case A_CLIP:
      if (nanprop && x != x) return x;
      return fminf(fmaxf(x, 0.f), a);
    case A_ABS: return fabsf(x);
    /* the few-instruction kinds in the float arithmetic the definition spells out (so bit-exact) */
    case X_SQUARE: return x * x;
    case X_SQRT: return sqrtf(x);
    case X_CLIP: case X_CLIP_V2: return x <= a ? a : (x > b ? b : x);
    case X_HARDSWISH: { float t = fmaf(a, x, b); return x * (t <= 0.f ? 0.f : (t >= 1.f ? 1.f : t)); }
    case X_ROUND: return rintf(x);
  }
  /* the transcendental kinds: the definition in double on the float arguments, rounded once */
  if (alg >= X_SQUARE) return (float)ext_fwd_d(alg, (double)x, (double)a, (double)b);
  return NAN;
}

static double act_fwd_d(int alg, double x, double a, double b, int nanprop) {
  switch (alg) {
    case A_RELU:
      if (a == 0.0) {
        if (nanprop && x != x) return x;
        return fmax(x, 0.0);
      }
      return x > 0.0 ? x : a * x;
    case A_SIGMOID: return 1.0 / (1.0 + exp(-x));
    case A_TANH: return tanh(x);
    case A_ELU: return x > 0.0 ? x : a * expm1(x);
    case A_ELU_FP32: return x > 0.0 ? x : a * (exp(x) - 1.0);
    case A_LINEAR: return fma(a, x, b);
    case A_CLIP:
      if (nanprop && x != x) return x;
      return fmin(fmax(x, 0.0), a);
    case A_ABS: return fabs(x);
  }
  if (alg >= X_SQUARE) return ext_fwd_d(alg, x, a, b);
  return NAN;
}

/* derivative times dy, from the forward source */
static float act_bwd_f(int alg, float x, float dy, float a, float b) {
  switch (alg) {
    case X_RELU_DST: return x > 0.f ? dy : a * dy;
    case X_SQUARE: return dy * (x + x);
    case X_SQRT: { float r = sqrtf(x); return dy / (r + r); }
    case X_SQRT_DST: return dy / (x + x);
    case X_CLIP: return (x > a && x <= b) ? dy : 0.f;
    case X_CLIP_V2: case X_CLIP_V2_DST: return (x > a && x < b) ? dy : 0.f;
    case X_HARDSWISH: { float t = fmaf(a, x, b); return t <= 0.f ? 0.f : (t >= 1.f ? dy : dy * fmaf(a + a, x, b)); }
    case X_TANH_DST: return dy * fmaf(-x, x, 1.f);
    case X_ELU_DST: return x > 0.f ? dy : dy * (x + a);
    case X_LOGISTIC_DST: return dy * (x * (1.f - x));
    case X_EXP_DST: return dy * x;
    case X_LOG: return dy / x;
    case A_RELU: return x > 0.f ? dy : a * dy;
    /* derivative evaluated in double and rounded once, then one fp32 product with dy */
    case A_SIGMOID: { double e = exp(-fabs((double)x)); double r = 1.0 / (1.0 + e); return dy * (float)(e * r * r); }
    case A_TANH: { double e = exp(-2.0 * fabs((double)x)); double r = 1.0 / (1.0 + e); return dy * (float)(4.0 * e * r * r); }
    case A_ELU: { float ex = (float)exp((double)x); return x > 0.f ? dy : dy * (a == 1.f ? ex : a * ex); }
    case A_LINEAR: return a * dy;
    case A_CLIP: return (x > 0.f && x <= a) ? dy : 0.f;
    case A_ABS: return x > 0.f ? dy : (x < 0.f ? -dy : 0.f);
  }
  /* transcendental kinds: the derivative in double, rounded once, then one fp32 product with dy */
  if (alg >= X_SQUARE) return dy * (float)ext_der_d(alg, (double)x, (double)a, (double)b);
  return NAN;
}

static double act_bwd_d(int alg, double x, double dy, double a, double b) {
  switch (alg) {
    case X_RELU_DST: return x > 0.0 ? dy : a * dy;
    case X_LOG: return dy / x;
    case X_SQRT: { double r = sqrt(x); return dy / (r + r); }
    case X_SQRT_DST: return dy / (x + x);
    case A_RELU: return x > 0.0 ? dy : a * dy;
    case A_SIGMOID: { double e = exp(-fabs(x)); double r = 1.0 / (1.0 + e); return dy * (e * r * r); }
    case A_TANH: { double e = exp(-2.0 * fabs(x)); double r = 1.0 / (1.0 + e); return dy * (4.0 * e * r * r); }
    case A_ELU: return x > 0.0 ? dy : dy * (a * exp(x));
    case A_LINEAR: return a * dy;
    case A_CLIP: return (x > 0.0 && x <= a) ? dy : 0.0;
    case A_ABS: return x > 0.0 ? dy : (x < 0.0 ? -dy : 0.0);
  }
  if (alg >= X_SQUARE) return dy * ext_der_d(alg, x, a, b);
  return NAN;
}

static float blend_f(float alpha, float v, float beta, const void *y, int t, int64_t off) {
  if (alpha != 1.f) v = alpha * v;
  if (beta != 0.f) v = v + beta * load_as_float(y, t, off);
  return v;
}
static double blend_d(double alpha, double v, double beta, const void *y, int t, int64_t off) {
  if (alpha != 1.0) v = alpha * v;
  if (beta != 0.0) v = v + beta * load_as_double(y, t, off);
  return v;
}

/* 1 if `st` is the row-major (dense, default) stride vector of `dims` */
static int is_default(int nd, const int64_t *dims, const int64_t *st) {
  int64_t run = 1;
  for (int d = nd - 1; d >= 0; d--) {
    if (dims[d] != 1 && st[d] != run) return 0;
    run *= dims[d];
  }
  return 1;
}

int oracle_eltwise_fwd(int alg, double coef, double shift, int nanprop, int t, int nd,
                       const int64_t *dims, const int64_t *xst, const void *x, const int64_t *yst,
                       void *y, double alpha, double beta) {
  const int64_t n = total_of(nd, dims);
  const int dense = is_default(nd, dims, xst) && is_default(nd, dims, yst);
  alg = fwd_alg_of(alg);
  if (dense && t == T_F32 && alpha == 1.0 && beta == 0.0) {
    /* the common case (dense fp32, no blend) without the per-element type and layout dispatch; the
     * arithmetic is act_fwd_f's, so the results are the same bits */
    const float *xf = (const float *)x;
    float *yf = (float *)y;
    const float a = (float)coef, b = (float)shift;
    if (alg == A_RELU && a == 0.f) {
#pragma omp parallel for simd schedule(static)
      for (int64_t i = 0; i < n; i++) {
        const float v = xf[i];
        yf[i] = (nanprop && v != v) ? v : fmaxf(v, 0.f);
      }
      return 0;
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) yf[i] = act_fwd_f(alg, xf[i], a, b, nanprop);
    return 0;
  }
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    int64_t xo = dense ? i : offset_of(nd, dims, xst, i), yo = dense ? i : offset_of(nd, dims, yst, i);
    if (t == T_F64) {
      double v = act_fwd_d(alg, ((const double *)x)[xo], coef, shift, nanprop);
      ((double *)y)[yo] = blend_d(alpha, v, beta, y, t, yo);
    } else {
      float v = act_fwd_f(alg, load_as_float(x, t, xo), (float)coef, (float)shift, nanprop);
      store_from_float(y, t, yo, blend_f((float)alpha, v, (float)beta, y, t, yo));
    }
  }
  return 0;
}

/* `x` is the forward source; for the X_*_DST kinds the caller passes the forward result there */
int oracle_eltwise_bwd_ex(int alg, double coef, double shift, int t, int nd, const int64_t *dims,
                          const int64_t *xst, const void *x, const int64_t *dyst, const void *dy,
                          const int64_t *dxst, void *dx, double alpha, double beta) {
  const int64_t n = total_of(nd, dims);
  const int dense = is_default(nd, dims, xst) && is_default(nd, dims, dyst) && is_default(nd, dims, dxst);
  if (dense && t == T_F32 && alpha == 1.0 && beta == 0.0) {
    const float *xf = (const float *)x, *gf = (const float *)dy;
    float *of = (float *)dx;
    const float a = (float)coef;
    if (alg == A_RELU) {
#pragma omp parallel for simd schedule(static)
      for (int64_t i = 0; i < n; i++) of[i] = xf[i] > 0.f ? gf[i] : a * gf[i];
      return 0;
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) of[i] = act_bwd_f(alg, xf[i], gf[i], a, (float)shift);
    return 0;
  }
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    int64_t xo = dense ? i : offset_of(nd, dims, xst, i), go = dense ? i : offset_of(nd, dims, dyst, i),
            oo = dense ? i : offset_of(nd, dims, dxst, i);
    if (t == T_F64) {
      double v = act_bwd_d(alg, ((const double *)x)[xo], ((const double *)dy)[go], coef, shift);
      ((double *)dx)[oo] = blend_d(alpha, v, beta, dx, t, oo);
    } else {
      float v = act_bwd_f(alg, load_as_float(x, t, xo), load_as_float(dy, t, go), (float)coef, (float)shift);
      store_from_float(dx, t, oo, blend_f((float)alpha, v, (float)beta, dx, t, oo));
    }
  }
  return 0;
}

int oracle_eltwise_bwd(int alg, double coef, int t, int nd, const int64_t *dims, const int64_t *xst,
                       const void *x, const int64_t *dyst, const void *dy, const int64_t *dxst,
                       void *dx, double alpha, double beta) {
  return oracle_eltwise_bwd_ex(alg, coef, 0.0, t, nd, dims, xst, x, dyst, dy, dxst, dx, alpha, beta);
}

/* The same definitions evaluated in double on float inputs (error attribution). */
int oracle_eltwise_fwd_truth(int alg, double coef, double shift, int64_t n, const float *x, double *out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) out[i] = act_fwd_d(fwd_alg_of(alg), (double)x[i], coef, shift, 1);
  return 0;
}
int oracle_eltwise_bwd_truth(int alg, double coef, int64_t n, const float *x, const float *dy, double *out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) out[i] = act_bwd_d(alg, (double)x[i], (double)dy[i], coef, 0.0);
  return 0;
}
int oracle_eltwise_bwd_truth_ex(int alg, double coef, double shift, int64_t n, const float *x, const float *dy, double *out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) out[i] = act_bwd_d(alg, (double)x[i], (double)dy[i], coef, shift);
  return 0;
}

/* ------------------------------------------------------------ binary / sum ------------------- */

/* 6..11: oneDNN's comparison kinds (dnnl/constants.clj:359-371 :ge :gt :le :lt :eq :ne): 1 where the
 * relation holds, else 0, in the destination's type. */
enum { B_ADD = 0, B_MUL = 1, B_MIN = 2, B_MAX = 3, B_SUB = 4, B_DIV = 5, B_GE = 6, B_GT = 7, B_LE = 8, B_LT = 9,
       B_EQ = 10, B_NE = 11 };

/* C = op(alpha1*A, alpha2*bcast(B)) + beta*C; bdims[i] is dims[i] or 1. */
int oracle_binary(int op, int t, int nd, const int64_t *dims, double alpha1, const int64_t *ast,
                  const void *A, double alpha2, const int64_t *bdims, const int64_t *bst,
                  const void *B, double beta, const int64_t *cst, void *C) {
  const int64_t n = total_of(nd, dims);
  int64_t bs[MAXD];
  for (int i = 0; i < nd; i++) bs[i] = (bdims[i] == 1 && dims[i] != 1) ? 0 : bst[i];
  const int dbl = (t == T_F64 || t == T_S32);
  const int readA = !(alpha1 == 0.0 && op == B_ADD);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    int64_t ao = offset_of(nd, dims, ast, i), bo = offset_of(nd, dims, bs, i),
            co = offset_of(nd, dims, cst, i);
    if (dbl) {
      double a = readA ? load_as_double(A, t, ao) : 0.0, b = load_as_double(B, t, bo), r;
      if (readA && alpha1 != 1.0) a = alpha1 * a;
      if (alpha2 != 1.0) b = alpha2 * b;
      switch (op) {
        case B_ADD: r = a + b; break;
        case B_MUL: r = a * b; break;
        case B_MIN: r = a < b ? a : b; break;
        case B_MAX: r = a > b ? a : b; break;
        case B_SUB: r = a - b; break;
        case B_GE: r = a >= b ? 1.0 : 0.0; break;
        case B_GT: r = a > b ? 1.0 : 0.0; break;
        case B_LE: r = a <= b ? 1.0 : 0.0; break;
        case B_LT: r = a < b ? 1.0 : 0.0; break;
        case B_EQ: r = a == b ? 1.0 : 0.0; break;
        case B_NE: r = a != b ? 1.0 : 0.0; break;
        default: r = a / b; break;
      }
      if (beta != 0.0) r = r + beta * load_as_double(C, t, co);
      store_from_double(C, t, co, r);
    } else {
      float a = readA ? load_as_float(A, t, ao) : 0.f, b = load_as_float(B, t, bo), r;
      if (readA && alpha1 != 1.0) a = (float)alpha1 * a;
      if (alpha2 != 1.0) b = (float)alpha2 * b;
      switch (op) {
        case B_ADD: r = a + b; break;
        case B_MUL: r = a * b; break;
        case B_MIN: r = a < b ? a : b; break;
        case B_MAX: r = a > b ? a : b; break;
        case B_SUB: r = a - b; break;
        case B_GE: r = a >= b ? 1.f : 0.f; break;
        case B_GT: r = a > b ? 1.f : 0.f; break;
        case B_LE: r = a <= b ? 1.f : 0.f; break;
        case B_LT: r = a < b ? 1.f : 0.f; break;
        case B_EQ: r = a == b ? 1.f : 0.f; break;
        case B_NE: r = a != b ? 1.f : 0.f; break;
        default: r = a / b; break;
      }
      if (beta != 0.0) r = r + (float)beta * load_as_float(C, t, co);
      store_from_float(C, t, co, r);
    }
  }
  return 0;
}

/* dst = ((s0*x0) + s1*x1) + ... over n dense same-layout sources; dst may alias srcs[0]. */
int oracle_sum(int n, const float *scales, int t, int64_t total, const void *const *srcs, void *dst) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < total; i++) {
    if (t == T_F64) {
      double acc = 0;
      for (int s = 0; s < n; s++) {
        double v = ((const double *)srcs[s])[i];
        if (scales[s] != 1.f) v = (double)scales[s] * v;
        acc = s == 0 ? v : acc + v;
      }
      ((double *)dst)[i] = acc;
    } else {
      float acc = 0;
      for (int s = 0; s < n; s++) {
        float v = load_as_float(srcs[s], t, i);
        if (scales[s] != 1.f) v = scales[s] * v;
        acc = s == 0 ? v : acc + v;
      }
      store_from_float(dst, t, i, acc);
    }
  }
  return 0;
}

/* ------------------------------------------------------------ reduction ---------------------- */

enum { R_ADD = 0, R_MUL = 1, R_MIN = 2, R_MAX = 3, R_AMAX = 4, R_AVG = 5, R_NORM1 = 6, R_NORM2 = 7, R_MULNZ = 8,
       /* oneDNN's norm kinds with their p and epsilon (dnnl/constants.clj:393-402, `reduction` in
        * dnnl/core.clj:796-803), S = sum of |x|^p:  max(S,eps)^(1/p), (S+eps)^(1/p), max(S,eps), S+eps */
       R_LP_MAX = 9, R_LP_SUM = 10, R_LP_POWER_P_MAX = 11, R_LP_POWER_P_SUM = 12 };
#define R_IS_LP(op) ((op) >= R_LP_MAX && (op) <= R_LP_POWER_P_SUM)

static double minmax_d(int op, double a, double b, int nanprop) {
  double r = (op == R_MIN) ? (a < b ? a : b) : (a > b ? a : b);
  if (a != a) r = nanprop ? a : b;
  if (b != b) r = nanprop ? b : (a != a ? b : a);
  return r;
}

/* Sum-type reductions (sum, mean, norm1, norm2) add in pairwise (binary tree) order over the
 * logical order of the reduced elements, leaves of <= 8 elements added left to right: a fixed,
 * reproducible fp32 order whose error grows with log(n), like the vectorised/blocked orders real
 * implementations use (a single left-to-right fp32 accumulator is off by 5e-4 relative at 2^20
 * terms and is nobody's algorithm).  max/min/mul run left to right. */
typedef struct {
  int op, t, nr;
  const int64_t *rd, *rx;
  const void *x;
  int64_t xo;
  double p;
} red_ctx;

/* |v|^p of one element, in the arithmetic of the accumulator */
static float lp_term_f(float v, double p) {
  if (p == 1.0) return fabsf(v);
  if (p == 2.0) return v * v;
  if (p == 3.0) return v * v * fabsf(v);
  if (p == 4.0) return (v * v) * (v * v);
  return powf(fabsf(v), (float)p);
}
static double lp_term_d(double v, double p) { return p == 1.0 ? fabs(v) : (p == 2.0 ? v * v : pow(fabs(v), p)); }

static double red_value(const red_ctx *c, int64_t r) {
  return load_as_double(c->x, c->t, c->xo + offset_of(c->nr, c->rd, c->rx, r));
}

static float pair_f(const red_ctx *c, int64_t lo, int64_t hi) {
  if (hi - lo <= 8) {
    float acc = 0.f;
    for (int64_t r = lo; r < hi; r++) {
      float v = (float)red_value(c, r);
      acc += R_IS_LP(c->op) ? lp_term_f(v, c->p) : (c->op == R_NORM1 ? fabsf(v) : (c->op == R_NORM2 ? v * v : v));
    }
    return acc;
  }
  int64_t mid = lo + (hi - lo) / 2;
  return pair_f(c, lo, mid) + pair_f(c, mid, hi);
}

static double pair_d(const red_ctx *c, int64_t lo, int64_t hi) {
  if (hi - lo <= 8) {
    double acc = 0.0;
    for (int64_t r = lo; r < hi; r++) {
      double v = red_value(c, r);
      acc += R_IS_LP(c->op) ? lp_term_d(v, c->p) : (c->op == R_NORM1 ? fabs(v) : (c->op == R_NORM2 ? v * v : v));
    }
    return acc;
  }
  int64_t mid = lo + (hi - lo) / 2;
  return pair_d(c, lo, mid) + pair_d(c, mid, hi);
}

/* y = alpha*reduce(x) + beta*y; reduced dims are those with ydims == 1 and xdims != 1.
 * `truth`, if not NULL, receives the reduction (before alpha/beta) accumulated in long double, one
 * value per output in logical order of y. */
static int reduce_core(int op, int t, int nanprop, int nd, const int64_t *xdims, const int64_t *xst,
                       const void *x, const int64_t *ydims, const int64_t *yst, void *y, double alpha,
                       double beta, double *truth, double p, double eps) {
  int64_t kd[MAXD], rd[MAXD], kx[MAXD], rx[MAXD], ky[MAXD];
  int nk = 0, nr = 0;
  for (int i = 0; i < nd; i++) {
    if (ydims[i] == 1 && xdims[i] != 1) { rd[nr] = xdims[i]; rx[nr] = xst[i]; nr++; }
    else { kd[nk] = xdims[i]; kx[nk] = xst[i]; ky[nk] = yst[i]; nk++; }
  }
  const int64_t nout = total_of(nk, kd), nred = total_of(nr, rd);
  const int dbl = (t == T_F64);
  const int sumlike = (op == R_ADD || op == R_AVG || op == R_NORM1 || op == R_NORM2 || R_IS_LP(op));
#pragma omp parallel for schedule(static)
  for (int64_t o = 0; o < nout; o++) {
    const int64_t xo = offset_of(nk, kd, kx, o), yo = offset_of(nk, kd, ky, o);
    double accd;
    float accf;
    long double acct;
    switch (op) {
      case R_MUL: case R_MULNZ: accd = 1; accf = 1; acct = 1; break;
      case R_MIN: accd = INFINITY; accf = INFINITY; acct = INFINITY; break;
      case R_MAX: accd = -INFINITY; accf = -INFINITY; acct = -INFINITY; break;
      default: accd = 0; accf = 0; acct = 0; break;
    }
    if (sumlike) {
      red_ctx c = {op, t, nr, rd, rx, x, xo, p};
      if (dbl) accd = pair_d(&c, 0, nred);
      else accf = pair_f(&c, 0, nred);
    }
    for (int64_t r = 0; r < nred; r++) {
      const int64_t off = xo + offset_of(nr, rd, rx, r);
      const double vd = load_as_double(x, t, off);
      const float vf = (float)vd;
      switch (op) {
        case R_ADD: case R_AVG: acct += vd; break;
        case R_NORM1: acct += fabs(vd); break;
        case R_NORM2: acct += (long double)vd * vd; break;
        case R_LP_MAX: case R_LP_SUM: case R_LP_POWER_P_MAX: case R_LP_POWER_P_SUM:
          acct += powl(fabsl((long double)vd), (long double)p); break;
        case R_MUL: accd *= vd; accf *= vf; acct *= vd; break;
        case R_MULNZ: if (vd != 0) { accd *= vd; accf *= vf; acct *= vd; } break;
        case R_MIN: case R_MAX:
          accd = minmax_d(op, accd, vd, nanprop); accf = (float)minmax_d(op, accf, vf, nanprop);
          acct = minmax_d(op, (double)acct, vd, nanprop); break;
        case R_AMAX:
          accd = minmax_d(R_MAX, accd, fabs(vd), nanprop); accf = (float)minmax_d(R_MAX, accf, fabsf(vf), nanprop);
          acct = minmax_d(R_MAX, (double)acct, fabs(vd), nanprop); break;
      }
    }
    if (op == R_AVG) { accd = accd / (double)nred; accf = accf / (float)nred; acct = acct / (long double)nred; }
    if (op == R_NORM2) { accd = sqrt(accd); accf = sqrtf(accf); acct = sqrtl(acct); }
    if (R_IS_LP(op)) {
      if (op == R_LP_MAX || op == R_LP_POWER_P_MAX) {
        accd = accd > eps ? accd : eps; accf = accf > (float)eps ? accf : (float)eps;
        acct = acct > (long double)eps ? acct : (long double)eps;
      } else {
        accd += eps; accf += (float)eps; acct += (long double)eps;
      }
      if (op == R_LP_MAX || op == R_LP_SUM) {
        if (p == 2.0) { accd = sqrt(accd); accf = sqrtf(accf); acct = sqrtl(acct); }
        else if (p != 1.0) {
          accd = pow(accd, 1.0 / p); accf = powf(accf, (float)(1.0 / p)); acct = powl(acct, 1.0L / (long double)p);
        }
      }
    }
    if (truth) truth[o] = (double)acct;
    if (dbl) {
      store_from_double(y, t, yo, blend_d(alpha, accd, beta, y, t, yo));
    } else {
      store_from_float(y, t, yo, blend_f((float)alpha, accf, (float)beta, y, t, yo));
    }
  }
  return 0;
}

int oracle_reduce(int op, int t, int nanprop, int nd, const int64_t *xdims, const int64_t *xst,
                  const void *x, const int64_t *ydims, const int64_t *yst, void *y, double alpha,
                  double beta, double *truth) {
  if (R_IS_LP(op)) return -1;
  return reduce_core(op, t, nanprop, nd, xdims, xst, x, ydims, yst, y, alpha, beta, truth, 2.0, 0.0);
}

/* The norm kinds of oneDNN's reduction with p >= 1 and epsilon, as the reference's `reduction`
 * passes them (dnnl/core.clj:796-803; the known answer at dnnl-t/core_test.clj:926-943 is
 * norm-lp-sum with p = 2, eps = 0). */
int oracle_reduce_lp(int op, double p, double eps, int t, int nd, const int64_t *xdims, const int64_t *xst,
                     const void *x, const int64_t *ydims, const int64_t *yst, void *y, double alpha,
                     double beta, double *truth) {
  if (!R_IS_LP(op) || !(p >= 1.0)) return -1;
  return reduce_core(op, t, 1, nd, xdims, xst, x, ydims, yst, y, alpha, beta, truth, p, eps);
}

/* any-mismatch over two strided views (typed compare) -- restates blas-plus.cu:9-101 of the
 * reference (deep-diamond-cuda/src/device/uncomplicate/diamond/internal/cuda/). */
int oracle_equals(int t, int nd, const int64_t *dims, const int64_t *xst, const void *x,
                  const int64_t *yst, const void *y) {
  const int64_t n = total_of(nd, dims);
  int diff = 0;
  for (int64_t i = 0; i < n && !diff; i++) {
    double a = load_as_double(x, t, offset_of(nd, dims, xst, i));
    double b = load_as_double(y, t, offset_of(nd, dims, yst, i));
    if (a != b) diff = 1;
  }
  return !diff;
}

/* Cost functions over dense vectors of n floats, following
 * deep-diamond-base/src/uncomplicate/diamond/internal/cost.clj step by step, every vector
 * operation rounding to float as Neanderthal's float vectors do:
 *   kind 0 (:20-25)  a_y = a - y;  (nrm2 a_y)^2 / (2 n)
 *   kind 1 (:27-32)  a_y = a - y;  (asum a_y) / n
 *   kind 2 (:34-40)  asum( (y - 1) * log(1.0000001 - a) - y * log(a) ) / batch
 * d (may be NULL) receives a - y.  The sums are accumulated in double (the reference's nrm2/asum
 * are BLAS calls whose order is not specified); *truth gets the same quantity with every
 * elementwise step in double. */
int oracle_cost(int kind, int64_t n, int64_t batch, const float *a, const float *y, float *d,
                double *cost, double *truth) {
  double acc = 0, tacc = 0;
  for (int64_t i = 0; i < n; i++) {
    const float t = a[i] - y[i];
    if (d) d[i] = t;
    if (kind == 0) {
      acc += (double)t * (double)t;
      tacc += ((double)a[i] - (double)y[i]) * ((double)a[i] - (double)y[i]);
    } else if (kind == 1) {
      acc += fabs((double)t);
      tacc += fabs((double)a[i] - (double)y[i]);
    } else {
      const float lna = (float)log((double)a[i]);
      const float ylna = y[i] * lna;
      const float y1 = y[i] - 1.0f;
      const float om = 1.0000001f - a[i];
      const float l1 = (float)log((double)om);
      const float h = y1 * l1 - ylna;
      acc += fabs((double)h);
      tacc += fabs(((double)y[i] - 1.0) * log(1.0000001 - (double)a[i]) - (double)y[i] * log((double)a[i]));
    }
  }
  if (kind == 0) {
    /* the reference squares the float norm: (sqr (nrm2 a-y)) / (* 2 n) */
    *cost = acc / (2.0 * (double)n);
    if (truth) *truth = tacc / (2.0 * (double)n);
  } else if (kind == 1) {
    *cost = acc / (double)n;
    if (truth) *truth = tacc / (double)n;
  } else {
    *cost = acc / (double)batch;
    if (truth) *truth = tacc / (double)batch;
  }
  return 0;
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_num_threads(void) {
  int n = 1;
#ifdef _OPENMP
#pragma omp parallel
  {
#pragma omp master
    n = omp_get_num_threads();
  }
#endif
  return n;
}
