// Internal definitions shared by the kernels of libdd_b200.so (not part of the C ABI).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <type_traits>

#include <nvtx3/nvToolsExt.h>

#include "../../include/dd_b200.h"

// An NVTX range around one library call, named after the entry point, so that a timeline shows the
// calls of this library by name.  NVTX v3 is header-only: without a profiler attached (no injection
// library named in the environment) a push or pop is one test of a function pointer.
struct ddNvtxRange {
  explicit ddNvtxRange(const char *name) { nvtxRangePushA(name); }
  ~ddNvtxRange() { nvtxRangePop(); }
};
#define DD_RANGE(name) ddNvtxRange dd_nvtx_range_(name)

// ------------------------------------------------------------------ host-side objects --------

struct ddTensorStruct {
  ddDataType_t dtype;
  int nd;
  int64_t dims[DD_DIM_MAX];
  int64_t strides[DD_DIM_MAX];
  bool set;
};

struct ddActivationStruct {
  ddActivationMode_t mode;
  ddNanPropagation_t nan;
  double coef;
  double shift;
};

struct ddReduceTensorStruct {
  ddReduceTensorOp_t op;
  ddDataType_t comp;
  ddNanPropagation_t nan;
  double p = 2.0;    // the NORM_LP kinds: exponent and epsilon
  double eps = 0.0;
  int indices = 0;   // DD_REDUCE_TENSOR_FLATTENED_INDICES: positions of the min / max / amax are wanted
};

struct ddContext {
  int device;
  int smCount;
  cudaStream_t stream;
  void *scratch;        // DD_HANDLE_SCRATCH_BYTES of device memory, allocated once in ddCreate
  size_t scratchBytes;
  int64_t counterSlots;  // leading unsigned counters of `scratch` kept zero between launches (0: none)
  uint64_t launches;
  const char *lastKernel;
  // One int in mapped host memory that a kernel raises when one of its bounded waits ran out (the
  // copy engine never signalled a tile): the host reads it without a device round trip.  Null if
  // the allocation failed, and then no kernel that needs it is launched.
  int *faultWord;
  bool tmaAttr;  // the tile-tma kernel's shared-memory limit has been raised on this device
  int tileTma;   // 1: the 1-byte transposing reorder uses the TMA-loading kernel where it qualifies
  char msg[256];
};

#define DD_FAIL(h, st, ...)                                   \
  do {                                                        \
    if (h) snprintf((h)->msg, sizeof((h)->msg), __VA_ARGS__); \
    return (st);                                              \
  } while (0)

// Records a launch and turns a launch-time CUDA error into a status.
#define DD_LAUNCHED(h, name)                                                      \
  do {                                                                            \
    (h)->launches++;                                                              \
    (h)->lastKernel = (name);                                                     \
    cudaError_t e__ = cudaGetLastError();                                         \
    if (e__ != cudaSuccess)                                                       \
      DD_FAIL(h, DD_STATUS_EXECUTION_FAILED, "%s: %s", name, cudaGetErrorString(e__)); \
  } while (0)

// Programmatic dependent launch.  A kernel launched with dd_launch_pdl may be scheduled while the
// previous kernel of the stream is still draining, which takes the launch latency out of
// back-to-back calls.  Such a kernel MUST call dd_pdl_prologue() before its first access to global
// memory: it holds the thread until the previous kernel has completed and its writes are visible,
// then lets the NEXT kernel of the stream be scheduled early in turn.  Launched the ordinary way,
// the prologue returns at once.
__device__ __forceinline__ void dd_pdl_prologue() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename P>
static inline void dd_launch_pdl(void (*kernel)(P), unsigned grid, unsigned block, cudaStream_t stream,
                                 const P &params) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, params);  // a failure is picked up by DD_LAUNCHED's cudaGetLastError
}

// A launch whose CTAs form thread-block clusters of `cluster` along x (the grid is a multiple of it).
template <typename P>
static inline void dd_launch_cluster(void (*kernel)(P), unsigned grid, unsigned block, unsigned cluster,
                                     cudaStream_t stream, const P &params) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, params);  // a failure is picked up by DD_LAUNCHED's cudaGetLastError
}

// The same for kernels with two parameter blocks.
template <typename P, typename Q>
static inline void dd_launch_pdl2(void (*kernel)(P, Q), unsigned grid, unsigned block, cudaStream_t stream,
                                  const P &p, const Q &q) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, p, q);
}

// For kernels launched the ordinary way: lets a programmatically launched successor be scheduled
// while this grid runs (the successor still waits for this grid's completion before it reads).
__device__ __forceinline__ void dd_pdl_release_next() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Builds with -DDD_TUNE read launch-plan overrides (group sizes, split counts, grid sizes) from the
// environment, for parameter sweeps on a GPU; ordinary builds compile the look-ups away.
#ifdef DD_TUNE
#include <stdlib.h>
static inline int dd_tune(const char *name, int dflt) {
  const char *v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}
#else
static inline int dd_tune(const char *, int dflt) { return dflt; }
#endif

static inline int dd_type_size(ddDataType_t t) {
  switch (t) {
    case DD_DATA_FLOAT: return 4;
    case DD_DATA_DOUBLE: return 8;
    case DD_DATA_HALF: return 2;
    case DD_DATA_INT8: return 1;
    case DD_DATA_INT32: return 4;
    case DD_DATA_UINT8: return 1;
    case DD_DATA_BFLOAT16: return 2;
    case DD_DATA_INT64: return 8;
  }
  return 0;
}

static inline bool dd_type_is_float(ddDataType_t t) {
  return t == DD_DATA_FLOAT || t == DD_DATA_DOUBLE || t == DD_DATA_HALF || t == DD_DATA_BFLOAT16;
}

// Reads a host scalar whose C type follows the tensor data type (double for DD_DATA_DOUBLE,
// float otherwise).
static inline double dd_read_scalar(const void *p, ddDataType_t t) {
  return t == DD_DATA_DOUBLE ? *(const double *)p : (double)*(const float *)p;
}

// ------------------------------------------------------------------ iteration space ----------

#define DD_MAX_OPS 4

// A canonical iteration space over up to DD_MAX_OPS operands: size-1 dims dropped, dims ordered
// by the chosen operand's stride (largest first) and adjacent dims merged when every operand
// walks them as one run.  Broadcast operands carry stride 0.
struct ddCanon {
  int nd;
  int nops;
  int64_t dims[DD_DIM_MAX];
  int64_t st[DD_MAX_OPS][DD_DIM_MAX];
  int64_t total;  // product of dims
};

void dd_canonicalize(ddCanon *c, int nd, const int64_t *dims, int nops,
                     const int64_t (*strides)[DD_DIM_MAX], int orderBy);

// Largest element offset (inclusive) an operand touches.
static inline int64_t dd_canon_span(const ddCanon *c, int op) {
  int64_t s = 0;
  for (int i = 0; i < c->nd; i++) s += (c->dims[i] - 1) * c->st[op][i];
  return s;
}

ddStatus_t dd_check_desc(ddHandle_t h, const ddTensorStruct *d, const char *what);
bool dd_same_dims(const ddTensorStruct *a, const ddTensorStruct *b);

// Division of a 31-bit unsigned value by a fixed divisor as multiply-high + shift (round-up method
// of Granlund & Montgomery): q = (umulhi(x, m) + x) >> s with s = ceil(log2 d) and
// m = ceil(2^(32+s) / d) - 2^32.  Exact for 0 <= x < 2^31, 1 <= d < 2^31.
struct ddFastDiv {
  uint32_t d, m, s;
};

static inline ddFastDiv dd_fastdiv(uint32_t d) {
  ddFastDiv f;
  f.d = d;
  uint32_t s = 0;
  while (s < 32 && ((uint64_t)1 << s) < d) s++;
  f.s = s;
  unsigned __int128 one = 1;
  unsigned __int128 num = one << (32 + s);
  uint64_t m = (uint64_t)((num + d - 1) / d);
  f.m = (uint32_t)(m - ((uint64_t)1 << 32));
  return f;
}

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t dd_div(uint32_t x, const ddFastDiv &f) {
  return (__umulhi(x, f.m) + x) >> f.s;
}
__device__ __forceinline__ void dd_divmod(uint32_t x, const ddFastDiv &f, uint32_t &q, uint32_t &r) {
  q = dd_div(x, f);
  r = x - q * f.d;
}
#endif

// Kernel-side form of ddCanon for the generic strided kernels.
template <int NOPS>
struct ddStridedParams {
  int nd;
  int64_t total;
  int64_t dims[DD_DIM_MAX];
  int64_t st[NOPS][DD_DIM_MAX];
  ddFastDiv fd[DD_DIM_MAX];  // valid when total < 2^31 (the 32-bit index path)
};

template <int NOPS>
static inline ddStridedParams<NOPS> dd_strided_params(const ddCanon &c) {
  ddStridedParams<NOPS> p;
  memset(&p, 0, sizeof(p));
  p.nd = c.nd;
  p.total = c.total;
  for (int i = 0; i < c.nd; i++) {
    p.dims[i] = c.dims[i];
    if (c.total < 0x7fffffffLL) p.fd[i] = dd_fastdiv((uint32_t)c.dims[i]);
    for (int o = 0; o < NOPS; o++) p.st[o][i] = c.st[o][i];
  }
  return p;
}

// Per-launch grid size for flat streaming kernels: enough CTAs to fill the machine several times
// over, capped so the grid-stride loop does the rest.
static inline unsigned dd_flat_grid(const ddContext *h, int64_t work_items, int threads,
                                    int ctas_per_sm) {
  int64_t need = (work_items + threads - 1) / threads;
  int64_t cap = (int64_t)h->smCount * ctas_per_sm * dd_tune("DD_FLAT_MULT", 1);
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}

// ------------------------------------------------------------------ device helpers -----------

#ifdef __CUDACC__

template <ddDataType_t T> struct dd_ctype;
template <> struct dd_ctype<DD_DATA_FLOAT> { typedef float type; };
template <> struct dd_ctype<DD_DATA_DOUBLE> { typedef double type; };
template <> struct dd_ctype<DD_DATA_HALF> { typedef __half type; };
template <> struct dd_ctype<DD_DATA_INT8> { typedef int8_t type; };
template <> struct dd_ctype<DD_DATA_INT32> { typedef int32_t type; };
template <> struct dd_ctype<DD_DATA_UINT8> { typedef uint8_t type; };
template <> struct dd_ctype<DD_DATA_BFLOAT16> { typedef __nv_bfloat16 type; };
template <> struct dd_ctype<DD_DATA_INT64> { typedef int64_t type; };

// to compute type ------------------------------------------------------------
template <typename C, typename T> __device__ __forceinline__ C dd_load(T v) { return (C)v; }
template <> __device__ __forceinline__ float dd_load<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ double dd_load<double, __half>(__half v) { return (double)__half2float(v); }
template <> __device__ __forceinline__ float dd_load<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ double dd_load<double, __nv_bfloat16>(__nv_bfloat16 v) { return (double)__bfloat162float(v); }

// from compute type: round-to-nearest-even for floating destinations, saturate + RNE for
// integer destinations (NaN -> 0).
template <typename T, typename C> struct dd_store_t;
template <typename C> struct dd_store_t<float, C> { static __device__ __forceinline__ float f(C v) { return (float)v; } };
template <typename C> struct dd_store_t<double, C> { static __device__ __forceinline__ double f(C v) { return (double)v; } };
template <> struct dd_store_t<__half, float> { static __device__ __forceinline__ __half f(float v) { return __float2half_rn(v); } };
template <> struct dd_store_t<__half, double> { static __device__ __forceinline__ __half f(double v) { return __double2half(v); } };
template <> struct dd_store_t<__nv_bfloat16, float> { static __device__ __forceinline__ __nv_bfloat16 f(float v) { return __float2bfloat16_rn(v); } };
template <> struct dd_store_t<__nv_bfloat16, double> { static __device__ __forceinline__ __nv_bfloat16 f(double v) { return __double2bfloat16(v); } };
template <> struct dd_store_t<int8_t, float> {
  static __device__ __forceinline__ int8_t f(float v) {
    if (v != v) return 0;
    v = fminf(fmaxf(v, -128.f), 127.f);
    return (int8_t)__float2int_rn(v);
  }
};
template <> struct dd_store_t<int8_t, double> {
  static __device__ __forceinline__ int8_t f(double v) {
    if (v != v) return 0;
    v = fmin(fmax(v, -128.0), 127.0);
    return (int8_t)__double2int_rn(v);
  }
};
template <> struct dd_store_t<uint8_t, float> {
  static __device__ __forceinline__ uint8_t f(float v) {
    if (v != v) return 0;
    v = fminf(fmaxf(v, 0.f), 255.f);
    return (uint8_t)__float2int_rn(v);
  }
};
template <> struct dd_store_t<uint8_t, double> {
  static __device__ __forceinline__ uint8_t f(double v) {
    if (v != v) return 0;
    v = fmin(fmax(v, 0.0), 255.0);
    return (uint8_t)__double2int_rn(v);
  }
};
template <> struct dd_store_t<int32_t, float> {
  static __device__ __forceinline__ int32_t f(float v) {
    if (v != v) return 0;
    return __float2int_rn(v);  // saturates at the int32 range
  }
};
template <> struct dd_store_t<int32_t, double> {
  static __device__ __forceinline__ int32_t f(double v) {
    if (v != v) return 0;
    return __double2int_rn(v);
  }
};
template <> struct dd_store_t<int64_t, float> {
  static __device__ __forceinline__ int64_t f(float v) {
    if (v != v) return 0;
    return __float2ll_rn(v);
  }
};
template <> struct dd_store_t<int64_t, double> {
  static __device__ __forceinline__ int64_t f(double v) {
    if (v != v) return 0;
    return __double2ll_rn(v);
  }
};
template <typename T, typename C> __device__ __forceinline__ T dd_store(C v) { return dd_store_t<T, C>::f(v); }

// N consecutive results into their storage type (dst 4-byte aligned).  float -> bf16 / f16 goes two
// at a time through the packed conversion (cvt.rn.{bf16x2,f16x2}.f32: each half rounds exactly as the
// single conversion does), half the conversion instructions and no packing of 16-bit halves.
template <typename T, typename C, int N>
__device__ __forceinline__ void dd_store_n(T *dst, const C *v) {
  if constexpr (std::is_same<C, float>::value && N % 2 == 0 && std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
    for (int k = 0; k < N; k += 2) *(__nv_bfloat162 *)&dst[k] = __floats2bfloat162_rn(v[k], v[k + 1]);
  } else if constexpr (std::is_same<C, float>::value && N % 2 == 0 && std::is_same<T, __half>::value) {
#pragma unroll
    for (int k = 0; k < N; k += 2) *(__half2 *)&dst[k] = __floats2half2_rn(v[k], v[k + 1]);
  } else {
#pragma unroll
    for (int k = 0; k < N; k++) dst[k] = dd_store<T, C>(v[k]);
  }
}

// alpha*v + beta*old, each product and the sum rounded separately (no FMA contraction), a factor
// of exactly 1 skipped and beta == 0 not reading `old`.  The CPU oracle follows the same rule.
__device__ __forceinline__ float dd_mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double dd_mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float dd_add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double dd_add_rn(double a, double b) { return __dadd_rn(a, b); }

template <typename C>
__device__ __forceinline__ C dd_scale(C alpha, C v) { return alpha == (C)1 ? v : dd_mul_rn(alpha, v); }

// Decomposes a linear index over the canonical dims into per-operand element offsets.
// 32-bit indices (total < 2^31) divide by multiply-shift; 64-bit indices by plain division.
template <int NOPS>
__device__ __forceinline__ void dd_offsets32(const ddStridedParams<NOPS> &p, uint32_t idx, int64_t (&off)[NOPS]) {
#pragma unroll
  for (int o = 0; o < NOPS; o++) off[o] = 0;
  for (int d = p.nd - 1; d > 0; d--) {
    uint32_t q, r;
    dd_divmod(idx, p.fd[d], q, r);
#pragma unroll
    for (int o = 0; o < NOPS; o++) off[o] += (int64_t)r * p.st[o][d];
    idx = q;
  }
#pragma unroll
  for (int o = 0; o < NOPS; o++) off[o] += (int64_t)idx * p.st[o][0];
}

template <int NOPS, typename I>
__device__ __forceinline__ void dd_offsets(const ddStridedParams<NOPS> &p, I idx, int64_t (&off)[NOPS]) {
  if constexpr (sizeof(I) == 4) {
    dd_offsets32<NOPS>(p, (uint32_t)idx, off);
  } else {
    if (p.total < 0x7fffffffLL) {
      dd_offsets32<NOPS>(p, (uint32_t)idx, off);
      return;
    }
#pragma unroll
    for (int o = 0; o < NOPS; o++) off[o] = 0;
    for (int d = p.nd - 1; d > 0; d--) {
      I dim = (I)p.dims[d];
      I q = idx / dim;
      I r = idx - q * dim;
#pragma unroll
      for (int o = 0; o < NOPS; o++) off[o] += (int64_t)r * p.st[o][d];
      idx = q;
    }
#pragma unroll
    for (int o = 0; o < NOPS; o++) off[o] += (int64_t)idx * p.st[o][0];
  }
}

#endif  // __CUDACC__

// ------------------------------------------------------------------ per-op entry points ------
// Implemented one per .cu file; the C ABI functions in dd_api.cu validate and forward here.

ddStatus_t dd_transform_impl(ddHandle_t h, double alpha, const ddTensorStruct *xd, const void *x,
                             double beta, const ddTensorStruct *yd, void *y);
ddStatus_t dd_gather_transform_impl(ddHandle_t h, int count, const int64_t *srcOff,
                                    const int64_t *dstOff, const ddTensorStruct *xd, const void *x,
                                    const ddTensorStruct *yd, void *y);
ddStatus_t dd_equals_impl(ddHandle_t h, const ddTensorStruct *xd, const void *x,
                          const ddTensorStruct *yd, const void *y, int *flag);
ddStatus_t dd_activation_fwd_impl(ddHandle_t h, const ddActivationStruct *act, double alpha,
                                  const ddTensorStruct *xd, const void *x, double beta,
                                  const ddTensorStruct *yd, void *y);
ddStatus_t dd_activation_bwd_impl(ddHandle_t h, const ddActivationStruct *act, double alpha,
                                  const ddTensorStruct *dyd, const void *dy,
                                  const ddTensorStruct *xd, const void *x, double beta,
                                  const ddTensorStruct *dxd, void *dx);
ddStatus_t dd_set_impl(ddHandle_t h, const ddTensorStruct *yd, void *y, double value);
ddStatus_t dd_scale_impl(ddHandle_t h, const ddTensorStruct *yd, void *y, double alpha);
ddStatus_t dd_optensor_impl(ddHandle_t h, ddOpTensorOp_t op, double alpha1,
                            const ddTensorStruct *ad, const void *A, double alpha2,
                            const ddTensorStruct *bd, const void *B, double beta,
                            const ddTensorStruct *cd, void *C);
ddStatus_t dd_sum_impl(ddHandle_t h, int n, const float *scales, const ddTensorStruct *const *sd,
                       const void *const *srcs, const ddTensorStruct *dd, void *dst);

// Reduction.  `partialOnly` keeps the pre-finish value (sum, sum|x|, sum x^2, max ...) in fp32/fp64
// `partialOut` (one value per output element, dense) instead of finishing into y: the multi-GPU path
// all-reduces that buffer and then calls dd_reduce_finish_impl.
ddStatus_t dd_reduce_ws_size(ddHandle_t h, const ddReduceTensorStruct *red,
                             const ddTensorStruct *xd, const ddTensorStruct *yd, size_t *bytes);
ddStatus_t dd_reduce_impl(ddHandle_t h, const ddReduceTensorStruct *red, void *ws, size_t wsBytes,
                          double alpha, const ddTensorStruct *xd, const void *x, double beta,
                          const ddTensorStruct *yd, void *y, bool partialOnly, void *partialOut);
ddStatus_t dd_reduce_indices_impl(ddHandle_t h, const ddReduceTensorStruct *red, const ddTensorStruct *xd, const void *x,
                                  const ddTensorStruct *yd, unsigned *indices);
ddStatus_t dd_reduce_finish_impl(ddHandle_t h, const ddReduceTensorStruct *red, const void *partial,
                                 double count, double alpha, double beta, const ddTensorStruct *xd,
                                 const ddTensorStruct *yd, void *y);
// The same finish, fed by the cross-GPU exchange of dd_reduce_kernels.cuh instead of a local buffer.
struct ddPeerParams;
ddStatus_t dd_reduce_fused_exchange_impl(ddHandle_t h, const ddReduceTensorStruct *red, const ddPeerParams *peer,
                                         double count, double alpha, const ddTensorStruct *xd, const void *x,
                                         double beta, const ddTensorStruct *yd, void *y, void *partialOut,
                                         bool onlyDistributed, bool *fused);
ddStatus_t dd_reduce_exchange_impl(ddHandle_t h, const ddReduceTensorStruct *red, const ddPeerParams *peer,
                                   double count, double alpha, double beta, const ddTensorStruct *xd,
                                   const ddTensorStruct *yd, void *y);
