// Callers either side of the hot path, fused:
//
//  ddMultiTransform   up to 8 independent reorder/convert copies in ONE launch.  The reference's
//                     branch and concatenate layers run one transformer per sub-tensor
//                     (cudnn/directed.clj:1289-1549: `(doseq [ft fwd-trans] (ft))`); here the k
//                     sub-tensor copies of a forward (or backward) pass are one kernel.
//  ddCostDiff         d = a - y written out AND its cost (sum (a-y)^2 / 2n or sum |a-y| / n) reduced
//                     in the same pass.  The reference's cost glue is `axpy! -1` followed by `nrm2`
//                     / `asum` (cudnn/directed.clj:367-458, base/internal/cost.clj:20-34): two or
//                     three sweeps over the same data.
//
// Both are HBM-bound streams.  Algorithmic bytes per element: multi-transform sizeof(S)+sizeof(D);
// cost-diff 3*sizeof(T).
#include "dd_internal.cuh"
#include "dd_math_f32.cuh"

#define DD_MULTI_MAX 8

struct ddMultiParams {
  const void *x[DD_MULTI_MAX];
  void *y[DD_MULTI_MAX];
  ddStridedParams<2> sp[DD_MULTI_MAX];  // per item; innermost dim in units of `vec` elements when vec > 1
  int64_t start[DD_MULTI_MAX + 1];      // prefix sums of the items' work units
  int count;
  int vec;                              // elements moved per work unit (1, or 16 / sizeof(T) for bit copies)
};

// SAME: source and destination share the element type: a bit copy, `vec` elements (16 bytes) at a time
// when every item allows it.  Otherwise one converted element per work unit.
template <typename S, typename D, typename C, bool SAME>
__global__ void __launch_bounds__(256) dd_multi_kernel(const __grid_constant__ ddMultiParams p) {
  const int64_t total = p.start[p.count];
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nthreads) {
    int k = 0;
#pragma unroll
    for (int j = 1; j < DD_MULTI_MAX; j++)
      if (j < p.count && i >= p.start[j]) k = j;
    int64_t off[2];
    dd_offsets32<2>(p.sp[k], (uint32_t)(i - p.start[k]), off);
    if constexpr (SAME) {
      if (p.vec > 1) {
        *(uint4 *)((D *)p.y[k] + off[1]) = *(const uint4 *)((const S *)p.x[k] + off[0]);
      } else {
        ((D *)p.y[k])[off[1]] = (D)((const S *)p.x[k])[off[0]];
      }
    } else {
      ((D *)p.y[k])[off[1]] = dd_store<D, C>(dd_load<C, S>(((const S *)p.x[k])[off[0]]));
    }
  }
}

template <typename S, typename D, typename C, bool SAME>
static ddStatus_t multi_launch(ddHandle_t h, const ddMultiParams &p) {
  unsigned grid = dd_flat_grid(h, p.start[p.count], 256, 64);  // 16 -> 64: branch / concatenate +2.4-3.3 %
  dd_multi_kernel<S, D, C, SAME><<<grid, 256, 0, h->stream>>>(p);
  DD_LAUNCHED(h, p.vec > 1 ? "multi-transform/vec" : "multi-transform/scalar");
  return DD_STATUS_SUCCESS;
}

template <typename S>
static ddStatus_t multi_to(ddHandle_t h, ddDataType_t dt, const ddMultiParams &p) {
  switch (dt) {
    case DD_DATA_FLOAT: return multi_launch<S, float, float, false>(h, p);
    case DD_DATA_HALF: return multi_launch<S, __half, float, false>(h, p);
    case DD_DATA_BFLOAT16: return multi_launch<S, __nv_bfloat16, float, false>(h, p);
    case DD_DATA_INT8: return multi_launch<S, int8_t, float, false>(h, p);
    case DD_DATA_UINT8: return multi_launch<S, uint8_t, float, false>(h, p);
    default: break;
  }
  DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddMultiTransform: converting copies support float, half, bf16, int8, uint8");
}

extern "C" ddStatus_t ddMultiTransform(ddHandle_t h, int count, const ddTensorDescriptor_t *xDescs,
                                       const void *const *xs, const ddTensorDescriptor_t *yDescs,
                                       void *const *ys) {
  DD_RANGE("ddMultiTransform");
  if (!h) return DD_STATUS_BAD_PARAM;
  if (count < 1 || count > DD_MULTI_MAX) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddMultiTransform: count must be in 1..%d", DD_MULTI_MAX);
  if (!xDescs || !xs || !yDescs || !ys) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddMultiTransform: null pointer");
  static thread_local ddMultiParams p;  // 3 KB: kept off the stack, one per calling thread
  memset(&p, 0, sizeof(p));
  p.count = count;
  const ddDataType_t st = xDescs[0] ? xDescs[0]->dtype : DD_DATA_FLOAT, dt = yDescs[0] ? yDescs[0]->dtype : DD_DATA_FLOAT;
  const bool same = st == dt;
  const int V = 16 / dd_type_size(st);
  ddCanon canon[DD_MULTI_MAX];
  bool vec = same;
  for (int k = 0; k < count; k++) {
    ddStatus_t s1 = dd_check_desc(h, xDescs[k], "ddMultiTransform x"), s2 = dd_check_desc(h, yDescs[k], "ddMultiTransform y");
    if (s1 != DD_STATUS_SUCCESS) return s1;
    if (s2 != DD_STATUS_SUCCESS) return s2;
    if (!xs[k] || !ys[k]) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddMultiTransform: null buffer %d", k);
    if (!dd_same_dims(xDescs[k], yDescs[k])) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddMultiTransform: item %d: x and y dims differ", k);
    if (xDescs[k]->dtype != st || yDescs[k]->dtype != dt)
      DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddMultiTransform: all items must share one source and one destination data type");
    int64_t strides[2][DD_DIM_MAX];
    for (int i = 0; i < xDescs[k]->nd; i++) {
      strides[0][i] = xDescs[k]->strides[i];
      strides[1][i] = yDescs[k]->strides[i];
    }
    dd_canonicalize(&canon[k], xDescs[k]->nd, xDescs[k]->dims, 2, strides, 1);
    const ddCanon &c = canon[k];
    if (c.total >= 0x7fffffffLL) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddMultiTransform: item %d too large", k);
    // 16-byte path: unit innermost stride on both sides, extent and all other strides multiples of V
    const int L = c.nd - 1;
    if (c.st[0][L] != 1 || c.st[1][L] != 1 || c.dims[L] % V) vec = false;
    for (int i = 0; i < L; i++)
      if (c.st[0][i] % V || c.st[1][i] % V) vec = false;
    if ((((uintptr_t)xs[k]) | ((uintptr_t)ys[k])) & 15) vec = false;
  }
  p.vec = vec ? V : 1;
  for (int k = 0; k < count; k++) {
    ddCanon c = canon[k];
    if (vec) {
      const int L = c.nd - 1;
      c.dims[L] /= V;
      c.total /= V;
      c.st[0][L] = V;
      c.st[1][L] = V;
    }
    p.sp[k] = dd_strided_params<2>(c);
    p.x[k] = xs[k];
    p.y[k] = ys[k];
    p.start[k + 1] = p.start[k] + c.total;
  }
  if (same) {
    switch (dd_type_size(st)) {
      case 1: return multi_launch<uint8_t, uint8_t, float, true>(h, p);
      case 2: return multi_launch<uint16_t, uint16_t, float, true>(h, p);
      case 4: return multi_launch<uint32_t, uint32_t, float, true>(h, p);
      default: return multi_launch<uint64_t, uint64_t, float, true>(h, p);
    }
  }
  switch (st) {
    case DD_DATA_FLOAT: return multi_to<float>(h, dt, p);
    case DD_DATA_HALF: return multi_to<__half>(h, dt, p);
    case DD_DATA_BFLOAT16: return multi_to<__nv_bfloat16>(h, dt, p);
    case DD_DATA_INT8: return multi_to<int8_t>(h, dt, p);
    case DD_DATA_UINT8: return multi_to<uint8_t>(h, dt, p);
    default: break;
  }
  DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddMultiTransform: converting copies support float, half, bf16, int8, uint8");
}

// ------------------------------------------------------------------ cost -----------------------

struct ddCostParams {
  const void *a;
  const void *y;
  void *d;          // may be NULL: only the cost is wanted
  void *cost;       // one element of T
  double *part;     // per-CTA partial sums (handle scratch, after the counters)
  unsigned *counter;
  int64_t n;
  int64_t divisor;  // n for the mean absolute cost, the batch extent for the cross-entropy
  int vec;
};

// One element's contribution.  KIND 2 follows the reference's vector steps one rounding at a time:
// y*log(a), (y-1), log(1.0000001 - a), their product, the difference (cost.clj:34-38).
template <typename T, int KIND>
__device__ __forceinline__ T dd_cost_term(T a, T y, T t, T acc) {
  if constexpr (KIND == 0) {
    if constexpr (sizeof(T) == 4) return fmaf(t, t, acc);
    else return fma(t, t, acc);
  } else if constexpr (KIND == 1) {
    return dd_add_rn(acc, t < (T)0 ? -t : t);
  } else {
    if constexpr (sizeof(T) == 4) {
      const float2 lg = dd_log_pair(make_float2(a, __fadd_rn(1.0000001f, -a)));  // log(a), log(1.0000001 - a)
      const float ylna = __fmul_rn(y, lg.x);
      const float h = __fadd_rn(__fmul_rn(__fadd_rn(y, -1.0f), lg.y), -ylna);
      return __fadd_rn(acc, fabsf(h));
    } else {
      const double ylna = __dmul_rn(y, log(a));
      const double h = __dadd_rn(__dmul_rn(__dadd_rn(y, -1.0), log(__dadd_rn(1.0000001, -a))), -ylna);
      return __dadd_rn(acc, fabs(h));
    }
  }
}

template <typename T, int KIND>
__global__ void __launch_bounds__(256, 6) dd_cost_kernel(ddCostParams p) {
  constexpr int V = 16 / sizeof(T);
  const T *a = (const T *)p.a;
  const T *y = (const T *)p.y;
  T *d = (T *)p.d;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  T acc = (T)0;
  int64_t done = 0;
  if (p.vec) {
    const int64_t nv = p.n / V;
    for (int64_t i = tid; i < nv; i += nthreads) {
      uint4 av = *(const uint4 *)(a + i * V), yv = *(const uint4 *)(y + i * V), dv;
      const T *ap = (const T *)&av, *yp = (const T *)&yv;
      T *dp = (T *)&dv;
#pragma unroll
      for (int k = 0; k < V; k++) {
        T t = dd_add_rn(ap[k], -yp[k]);
        dp[k] = t;
        acc = dd_cost_term<T, KIND>(ap[k], yp[k], t, acc);
      }
      if (d) *(uint4 *)(d + i * V) = dv;
    }
    done = nv * V;
  }
  for (int64_t i = done + tid; i < p.n; i += nthreads) {
    const T av = a[i], yv = y[i];
    T t = dd_add_rn(av, -yv);
    if (d) d[i] = t;
    acc = dd_cost_term<T, KIND>(av, yv, t, acc);
  }
  // CTA tree in double, then the last CTA to arrive folds the per-CTA partials in index order
  __shared__ double smem[8];
  __shared__ int lastFlag;
  double s = (double)acc;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double b = 0;
    for (int w = 0; w < 8; w++) b += smem[w];
    p.part[blockIdx.x] = b;
    __threadfence();
    lastFlag = atomicAdd(p.counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!lastFlag) return;
  // the last CTA folds the per-CTA partials: every thread takes a strided share, then the same
  // fixed tree as above (the order depends only on the grid size, so results repeat run to run)
  __threadfence();
  double mine = 0;
  for (unsigned b = threadIdx.x; b < gridDim.x; b += blockDim.x) mine += __ldcg(p.part + b);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine += __shfl_down_sync(0xffffffffu, mine, o);
  __syncthreads();  // smem is reused
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tot = 0;
    for (int w = 0; w < 8; w++) tot += smem[w];
    tot = KIND == 0 ? tot / (2.0 * (double)p.n) : tot / (double)p.divisor;
    *(T *)p.cost = (T)tot;
    *p.counter = 0;
  }
}

extern "C" ddStatus_t ddCostDiff(ddHandle_t h, int kind, ddTensorDescriptor_t desc, const void *a,
                                 const void *y, void *d, void *cost) {
  DD_RANGE("ddCostDiff");
  if (!h) return DD_STATUS_BAD_PARAM;
  ddStatus_t st = dd_check_desc(h, desc, "ddCostDiff");
  if (st != DD_STATUS_SUCCESS) return st;
  if (!a || !y || !cost) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddCostDiff: null pointer");
  if (kind < 0 || kind > 2)
    DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddCostDiff: kind must be 0 (quadratic), 1 (mean absolute) or 2 (cross-entropy)");
  if (desc->dtype != DD_DATA_FLOAT && desc->dtype != DD_DATA_DOUBLE)
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddCostDiff: float and double only");
  int64_t strides[1][DD_DIM_MAX];
  for (int i = 0; i < desc->nd; i++) strides[0][i] = desc->strides[i];
  ddCanon c;
  dd_canonicalize(&c, desc->nd, desc->dims, 1, strides, 0);
  if (!(c.nd == 1 && c.st[0][0] == 1))
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddCostDiff: the three tensors must be dense (the reference's cost works on the vector view)");
  ddCostParams p;
  p.a = a;
  p.y = y;
  p.d = d;
  p.cost = cost;
  p.counter = (unsigned *)h->scratch + (h->counterSlots - 1);  // the last arrival counter is this kernel's
  p.part = (double *)((char *)h->scratch + h->counterSlots * sizeof(unsigned));
  p.n = c.total;
  p.divisor = kind == 2 ? desc->dims[0] : c.total;
  p.vec = ((((uintptr_t)a) | ((uintptr_t)y) | ((uintptr_t)d)) & 15) == 0;
  const int V = 16 / dd_type_size(desc->dtype);
  // four resident waves' worth (6 CTAs per SM resident): the cross-entropy measured 3978 GB/s with one wave,
  // 4284 / 4377 / 4406 with two / three / four; the quadratic cost 6174 / 6265 / 6254 / 6250
  unsigned grid = dd_flat_grid(h, (p.n + V - 1) / V, 256, 24);
  const bool f = desc->dtype == DD_DATA_FLOAT;
  if (kind == 0) {
    if (f) dd_cost_kernel<float, 0><<<grid, 256, 0, h->stream>>>(p);
    else dd_cost_kernel<double, 0><<<grid, 256, 0, h->stream>>>(p);
  } else if (kind == 1) {
    if (f) dd_cost_kernel<float, 1><<<grid, 256, 0, h->stream>>>(p);
    else dd_cost_kernel<double, 1><<<grid, 256, 0, h->stream>>>(p);
  } else {
    if (f) dd_cost_kernel<float, 2><<<grid, 256, 0, h->stream>>>(p);
    else dd_cost_kernel<double, 2><<<grid, 256, 0, h->stream>>>(p);
  }
  DD_LAUNCHED(h, "cost-diff/flat");
  return DD_STATUS_SUCCESS;
}
