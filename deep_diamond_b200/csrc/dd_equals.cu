// ddTensorEquals: any-mismatch test over two strided views of one data type.  Replaces the five
// rank-specific kernels of the reference (blas-plus.cu:9-101), which run one thread per (n,c,h)
// with serial inner loops; here every element gets a thread (16-byte vectors when both views are
// dense).  A warp that sees a mismatch raises the flag at once and stops; after every pass (four
// vectors of each operand) the others look at the flag and stop too, so tensors that differ cost a fraction of a full pass
// (equal tensors read everything: 2*sizeof(T) algorithmic bytes per element).  Comparison is the
// typed `!=` of the reference (NaN differs from everything, -0 equals +0).
#include "dd_internal.cuh"

struct ddEqParams {
  const void *x;
  const void *y;
  int *flag;
  ddStridedParams<2> sp;
  int flat;
};

template <typename T> __device__ __forceinline__ bool dd_ne(T a, T b) { return a != b; }
template <> __device__ __forceinline__ bool dd_ne<__half>(__half a, __half b) { return __half2float(a) != __half2float(b); }
template <> __device__ __forceinline__ bool dd_ne<__nv_bfloat16>(__nv_bfloat16 a, __nv_bfloat16 b) { return __bfloat162float(a) != __bfloat162float(b); }

template <typename T>
__global__ void __launch_bounds__(256) dd_equals_kernel(ddEqParams p) {
  const T *x = (const T *)p.x;
  const T *y = (const T *)p.y;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  bool diff = false;
  if (p.flat) {
    constexpr int V = 16 / sizeof(T);
    const int64_t n = p.sp.total;
    int64_t done = 0;
    if (((((uintptr_t)x) | ((uintptr_t)y)) & 15) == 0) {
      const int64_t nv = n / V;
      // four vectors of each operand per pass: the eight loads go out together (a vote after every
      // vector would hold each pass back until its own two loads had come in), then one vote and one
      // look at the flag
      constexpr int U = 4;
      for (int64_t i = tid; i < nv; i += U * nthreads) {
        uint4 a[U], b[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int64_t j = i + u * nthreads;
          if (j < nv) {
            a[u] = *(const uint4 *)(x + j * V);
            b[u] = *(const uint4 *)(y + j * V);
          }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
          if (i + u * nthreads < nv) {
            const T *av = (const T *)&a[u], *bv = (const T *)&b[u];
#pragma unroll
            for (int k = 0; k < V; k++) diff |= dd_ne<T>(av[k], bv[k]);
          }
        }
        // the lanes of a warp run this loop in step (trip counts differ by one at most)
        const unsigned found = __ballot_sync(__activemask(), diff);
        if (found) {
          if ((threadIdx.x & 31) == __ffs(found) - 1) atomicAdd(p.flag, 1);
          break;
        }
        if (*(volatile const int *)p.flag != 0) break;
      }
      done = nv * V;
    }
    for (int64_t i = done + tid; i < n; i += nthreads) diff |= dd_ne<T>(x[i], y[i]);
  } else {
    for (int64_t i = tid; i < p.sp.total; i += nthreads) {
      int64_t off[2];
      dd_offsets<2, int64_t>(p.sp, i, off);
      diff |= dd_ne<T>(x[off[0]], y[off[1]]);
    }
  }
  if (__syncthreads_or(diff) && threadIdx.x == 0) atomicAdd(p.flag, 1);
}

template <typename T>
static ddStatus_t equals_typed(ddHandle_t h, const ddEqParams &p, const ddCanon &c) {
  constexpr int V = 16 / sizeof(T);
  unsigned grid = dd_flat_grid(h, p.flat ? (c.total + V - 1) / V : c.total, 256, 48);  // 16 -> 48: +5 %
  dd_equals_kernel<T><<<grid, 256, 0, h->stream>>>(p);
  DD_LAUNCHED(h, p.flat ? "equals/flat" : "equals/strided");
  return DD_STATUS_SUCCESS;
}

ddStatus_t dd_equals_impl(ddHandle_t h, const ddTensorStruct *xd, const void *x,
                          const ddTensorStruct *yd, const void *y, int *flag) {
  int64_t st[2][DD_DIM_MAX];
  for (int i = 0; i < xd->nd; i++) {
    st[0][i] = xd->strides[i];
    st[1][i] = yd->strides[i];
  }
  ddCanon c;
  dd_canonicalize(&c, xd->nd, xd->dims, 2, st, 0);
  ddEqParams p;
  p.x = x;
  p.y = y;
  p.flag = flag;
  p.sp = dd_strided_params<2>(c);
  p.flat = c.nd == 1 && c.st[0][0] == 1 && c.st[1][0] == 1;
  switch (xd->dtype) {
    case DD_DATA_FLOAT: return equals_typed<float>(h, p, c);
    case DD_DATA_DOUBLE: return equals_typed<double>(h, p, c);
    case DD_DATA_HALF: return equals_typed<__half>(h, p, c);
    case DD_DATA_BFLOAT16: return equals_typed<__nv_bfloat16>(h, p, c);
    case DD_DATA_INT8: return equals_typed<int8_t>(h, p, c);
    case DD_DATA_UINT8: return equals_typed<uint8_t>(h, p, c);
    case DD_DATA_INT32: return equals_typed<int32_t>(h, p, c);
    case DD_DATA_INT64: return equals_typed<int64_t>(h, p, c);
  }
  DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddTensorEquals: unknown data type");
}
