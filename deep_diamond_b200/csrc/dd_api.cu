// C ABI of libdd_b200.so: handle and descriptor objects, argument validation, and forwarding to
// the per-op implementations.  Declarations and the reference bindings they replace are in
// include/dd_b200.h.
#include "dd_internal.cuh"

#include <algorithm>
#include <new>

// ------------------------------------------------------------------ shared helpers -----------

void dd_canonicalize(ddCanon *c, int nd, const int64_t *dims, int nops,
                     const int64_t (*strides)[DD_DIM_MAX], int orderBy) {
  int idx[DD_DIM_MAX];
  int n = 0;
  for (int i = 0; i < nd; i++)
    if (dims[i] != 1) idx[n++] = i;
  // stable order: largest stride of the ordering operand first
  std::stable_sort(idx, idx + n, [&](int a, int b) { return strides[orderBy][a] > strides[orderBy][b]; });
  c->nops = nops;
  c->nd = 0;
  c->total = 1;
  for (int k = 0; k < n; k++) {
    int i = idx[k];
    c->total *= dims[i];
    if (c->nd > 0) {
      int p = c->nd - 1;
      bool merge = true;
      for (int o = 0; o < nops; o++)
        if (c->st[o][p] != strides[o][i] * dims[i]) merge = false;
      if (merge) {
        c->dims[p] *= dims[i];
        for (int o = 0; o < nops; o++) c->st[o][p] = strides[o][i];
        continue;
      }
    }
    c->dims[c->nd] = dims[i];
    for (int o = 0; o < nops; o++) c->st[o][c->nd] = strides[o][i];
    c->nd++;
  }
  if (c->nd == 0) {  // a single element
    c->nd = 1;
    c->dims[0] = 1;
    for (int o = 0; o < nops; o++) c->st[o][0] = 1;
  }
}

ddStatus_t dd_check_desc(ddHandle_t h, const ddTensorStruct *d, const char *what) {
  if (!d) DD_FAIL(h, DD_STATUS_BAD_PARAM, "%s: null tensor descriptor", what);
  if (!d->set) DD_FAIL(h, DD_STATUS_BAD_PARAM, "%s: tensor descriptor was never set", what);
  return DD_STATUS_SUCCESS;
}

bool dd_same_dims(const ddTensorStruct *a, const ddTensorStruct *b) {
  if (a->nd != b->nd) return false;
  for (int i = 0; i < a->nd; i++)
    if (a->dims[i] != b->dims[i]) return false;
  return true;
}

static bool valid_dtype(int t) {
  switch (t) {
    case DD_DATA_FLOAT: case DD_DATA_DOUBLE: case DD_DATA_HALF: case DD_DATA_INT8:
    case DD_DATA_INT32: case DD_DATA_UINT8: case DD_DATA_BFLOAT16: case DD_DATA_INT64:
      return true;
  }
  return false;
}

// ------------------------------------------------------------------ handle -------------------

extern "C" {

size_t ddGetVersion(void) { return DD_B200_VERSION; }

const char *ddGetErrorString(ddStatus_t s) {
  switch (s) {
    case DD_STATUS_SUCCESS: return "DD_STATUS_SUCCESS";
    case DD_STATUS_NOT_INITIALIZED: return "DD_STATUS_NOT_INITIALIZED";
    case DD_STATUS_ALLOC_FAILED: return "DD_STATUS_ALLOC_FAILED";
    case DD_STATUS_BAD_PARAM: return "DD_STATUS_BAD_PARAM";
    case DD_STATUS_INTERNAL_ERROR: return "DD_STATUS_INTERNAL_ERROR";
    case DD_STATUS_INVALID_VALUE: return "DD_STATUS_INVALID_VALUE";
    case DD_STATUS_ARCH_MISMATCH: return "DD_STATUS_ARCH_MISMATCH";
    case DD_STATUS_MAPPING_ERROR: return "DD_STATUS_MAPPING_ERROR";
    case DD_STATUS_EXECUTION_FAILED: return "DD_STATUS_EXECUTION_FAILED";
    case DD_STATUS_NOT_SUPPORTED: return "DD_STATUS_NOT_SUPPORTED";
    case DD_STATUS_TIMEOUT: return "DD_STATUS_TIMEOUT";
    case DD_STATUS_COMM_FAILED: return "DD_STATUS_COMM_FAILED";
  }
  return "DD_STATUS_UNKNOWN";
}

ddStatus_t ddCreate(ddHandle_t *handle) {
  if (!handle) return DD_STATUS_BAD_PARAM;
  *handle = nullptr;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return DD_STATUS_NOT_INITIALIZED;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return DD_STATUS_NOT_INITIALIZED;
  if (prop.major != 10) return DD_STATUS_ARCH_MISMATCH;  // the kernels are built for sm_100a only
  ddContext *h = new (std::nothrow) ddContext();
  if (!h) return DD_STATUS_ALLOC_FAILED;
  memset(h, 0, sizeof(*h));
  h->device = dev;
  h->smCount = prop.multiProcessorCount;
  h->stream = nullptr;
  h->scratchBytes = DD_HANDLE_SCRATCH_BYTES;
  h->lastKernel = "";
  h->msg[0] = 0;
  if (cudaMalloc(&h->scratch, h->scratchBytes) != cudaSuccess) {
    cudaGetLastError();
    delete h;
    return DD_STATUS_ALLOC_FAILED;
  }
  // the first 64 KB are arrival counters of split reductions: zero now, kept zero by the kernels
  h->counterSlots = (64 << 10) / sizeof(unsigned);
  // (the memset runs on the legacy default stream; the handle may later be bound to a stream that
  // is not ordered after it, so it is finished before the handle is handed out)
  if (cudaMemset(h->scratch, 0, h->counterSlots * sizeof(unsigned)) != cudaSuccess ||
      cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    cudaFree(h->scratch);
    delete h;
    return DD_STATUS_ALLOC_FAILED;
  }
  if (cudaHostAlloc((void **)&h->faultWord, 64, cudaHostAllocMapped) == cudaSuccess)
    *h->faultWord = 0;
  else {
    cudaGetLastError();
    h->faultWord = nullptr;
  }
  // The TMA-loading form of the 1-byte transposing reorder measured within 2 % of the
  // register-staged kernel on tensors of 50 MB and 3 % behind it on larger ones, so it is not the
  // default; DD_B200_TILE_TMA=1 in the environment of ddCreate selects it for this handle.
  const char *tma = getenv("DD_B200_TILE_TMA");
  h->tileTma = (tma && tma[0] == '1') ? 1 : 0;
  *handle = h;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddGetDeviceFault(ddHandle_t h, int *word) {
  if (!h || !word) return DD_STATUS_BAD_PARAM;
  *word = h->faultWord ? *(volatile int *)h->faultWord : 0;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddResetCounters(ddHandle_t h) {
  if (!h) return DD_STATUS_BAD_PARAM;
  if (!h->scratch || h->counterSlots == 0) return DD_STATUS_SUCCESS;
  cudaError_t e = cudaMemsetAsync(h->scratch, 0, h->counterSlots * sizeof(unsigned), h->stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    DD_FAIL(h, DD_STATUS_EXECUTION_FAILED, "ddResetCounters: %s", cudaGetErrorString(e));
  }
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddDestroy(ddHandle_t h) {
  if (!h) return DD_STATUS_BAD_PARAM;
  if (h->scratch) cudaFree(h->scratch);
  if (h->faultWord) cudaFreeHost(h->faultWord);
  delete h;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddSetStream(ddHandle_t h, void *stream) {
  if (!h) return DD_STATUS_BAD_PARAM;
  h->stream = (cudaStream_t)stream;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddGetStream(ddHandle_t h, void **stream) {
  if (!h || !stream) return DD_STATUS_BAD_PARAM;
  *stream = (void *)h->stream;
  return DD_STATUS_SUCCESS;
}

const char *ddGetLastErrorMessage(ddHandle_t h) { return h ? h->msg : "null handle"; }

ddStatus_t ddGetLaunchCount(ddHandle_t h, uint64_t *count) {
  if (!h || !count) return DD_STATUS_BAD_PARAM;
  *count = h->launches;
  return DD_STATUS_SUCCESS;
}

const char *ddGetLastKernelName(ddHandle_t h) { return h ? h->lastKernel : ""; }

// ------------------------------------------------------------------ tensor descriptor --------

ddStatus_t ddCreateTensorDescriptor(ddTensorDescriptor_t *desc) {
  if (!desc) return DD_STATUS_BAD_PARAM;
  ddTensorStruct *d = new (std::nothrow) ddTensorStruct();
  if (!d) return DD_STATUS_ALLOC_FAILED;
  memset(d, 0, sizeof(*d));
  *desc = d;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddDestroyTensorDescriptor(ddTensorDescriptor_t desc) {
  if (!desc) return DD_STATUS_BAD_PARAM;
  delete desc;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddSetTensorNdDescriptor(ddTensorDescriptor_t d, ddDataType_t dt, int nd,
                                   const int64_t *dims, const int64_t *strides) {
  if (!d || !dims || !strides) return DD_STATUS_BAD_PARAM;
  if (nd < 1 || nd > DD_DIM_MAX) return DD_STATUS_NOT_SUPPORTED;
  if (!valid_dtype((int)dt)) return DD_STATUS_BAD_PARAM;
  for (int i = 0; i < nd; i++)
    if (dims[i] < 1 || strides[i] < 1) return DD_STATUS_BAD_PARAM;
  d->dtype = dt;
  d->nd = nd;
  for (int i = 0; i < nd; i++) {
    d->dims[i] = dims[i];
    d->strides[i] = strides[i];
  }
  d->set = true;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddSetTensorNdDescriptorEx(ddTensorDescriptor_t d, ddTensorFormat_t fmt, ddDataType_t dt,
                                     int nd, const int64_t *dims) {
  if (!d || !dims) return DD_STATUS_BAD_PARAM;
  if (nd < 1 || nd > DD_DIM_MAX) return DD_STATUS_NOT_SUPPORTED;
  int64_t st[DD_DIM_MAX];
  if (fmt == DD_TENSOR_NCHW) {
    int64_t s = 1;
    for (int i = nd - 1; i >= 0; i--) { st[i] = s; s *= dims[i] > 0 ? dims[i] : 1; }
  } else if (fmt == DD_TENSOR_NHWC) {
    if (nd < 3) return DD_STATUS_BAD_PARAM;
    // channels (dim 1) innermost, then the spatial dims, then the batch
    st[1] = 1;
    int64_t s = dims[1] > 0 ? dims[1] : 1;
    for (int i = nd - 1; i >= 2; i--) { st[i] = s; s *= dims[i] > 0 ? dims[i] : 1; }
    st[0] = s;
  } else {
    return DD_STATUS_BAD_PARAM;
  }
  return ddSetTensorNdDescriptor(d, dt, nd, dims, st);
}

ddStatus_t ddSetTensor4dDescriptor(ddTensorDescriptor_t d, ddTensorFormat_t fmt, ddDataType_t dt,
                                   int64_t n, int64_t c, int64_t h, int64_t w) {
  int64_t dims[4] = {n, c, h, w};
  return ddSetTensorNdDescriptorEx(d, fmt, dt, 4, dims);
}

ddStatus_t ddSetTensor4dDescriptorEx(ddTensorDescriptor_t d, ddDataType_t dt, int64_t n, int64_t c,
                                     int64_t h, int64_t w, int64_t ns, int64_t cs, int64_t hs,
                                     int64_t ws) {
  int64_t dims[4] = {n, c, h, w};
  int64_t st[4] = {ns, cs, hs, ws};
  return ddSetTensorNdDescriptor(d, dt, 4, dims, st);
}

ddStatus_t ddGetTensorNdDescriptor(ddTensorDescriptor_t d, int nbReq, ddDataType_t *dt, int *nd,
                                   int64_t *dims, int64_t *strides) {
  if (!d || !d->set) return DD_STATUS_BAD_PARAM;
  if (dt) *dt = d->dtype;
  if (nd) *nd = d->nd;
  int n = nbReq < d->nd ? nbReq : d->nd;
  for (int i = 0; i < n; i++) {
    if (dims) dims[i] = d->dims[i];
    if (strides) strides[i] = d->strides[i];
  }
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddGetTensorSizeInBytes(ddTensorDescriptor_t d, size_t *bytes) {
  if (!d || !d->set || !bytes) return DD_STATUS_BAD_PARAM;
  int64_t span = 1;
  for (int i = 0; i < d->nd; i++) span += (d->dims[i] - 1) * d->strides[i];
  *bytes = (size_t)span * dd_type_size(d->dtype);
  return DD_STATUS_SUCCESS;
}

// ------------------------------------------------------------------ activation descriptor ----

ddStatus_t ddCreateActivationDescriptor(ddActivationDescriptor_t *desc) {
  if (!desc) return DD_STATUS_BAD_PARAM;
  ddActivationStruct *a = new (std::nothrow) ddActivationStruct();
  if (!a) return DD_STATUS_ALLOC_FAILED;
  a->mode = DD_ACTIVATION_RELU;
  a->nan = DD_PROPAGATE_NAN;
  a->coef = 0.0;
  a->shift = 0.0;
  *desc = a;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddDestroyActivationDescriptor(ddActivationDescriptor_t desc) {
  if (!desc) return DD_STATUS_BAD_PARAM;
  delete desc;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddSetActivationDescriptorEx(ddActivationDescriptor_t a, ddActivationMode_t mode,
                                       ddNanPropagation_t nanOpt, double coef, double shift) {
  if (!a) return DD_STATUS_BAD_PARAM;
  if ((int)mode < 0 || (int)mode > DD_ACTIVATION_CLIP_V2_DST_BWD) return DD_STATUS_BAD_PARAM;
  a->mode = mode;
  a->nan = nanOpt;
  a->coef = coef;
  a->shift = shift;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddSetActivationDescriptor(ddActivationDescriptor_t a, ddActivationMode_t mode,
                                     ddNanPropagation_t nanOpt, double coef) {
  return ddSetActivationDescriptorEx(a, mode, nanOpt, coef, 0.0);
}

ddStatus_t ddGetActivationDescriptor(ddActivationDescriptor_t a, ddActivationMode_t *mode,
                                     ddNanPropagation_t *nanOpt, double *coef) {
  if (!a) return DD_STATUS_BAD_PARAM;
  if (mode) *mode = a->mode;
  if (nanOpt) *nanOpt = a->nan;
  if (coef) *coef = a->coef;
  return DD_STATUS_SUCCESS;
}

// ------------------------------------------------------------------ reduce descriptor --------

ddStatus_t ddCreateReduceTensorDescriptor(ddReduceTensorDescriptor_t *desc) {
  if (!desc) return DD_STATUS_BAD_PARAM;
  ddReduceTensorStruct *r = new (std::nothrow) ddReduceTensorStruct();
  if (!r) return DD_STATUS_ALLOC_FAILED;
  r->op = DD_REDUCE_TENSOR_ADD;
  r->comp = DD_DATA_FLOAT;
  r->nan = DD_PROPAGATE_NAN;
  *desc = r;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddDestroyReduceTensorDescriptor(ddReduceTensorDescriptor_t desc) {
  if (!desc) return DD_STATUS_BAD_PARAM;
  delete desc;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddSetReduceTensorDescriptor(ddReduceTensorDescriptor_t r, ddReduceTensorOp_t op,
                                       ddDataType_t comp, ddNanPropagation_t nanOpt) {
  if (!r) return DD_STATUS_BAD_PARAM;
  if ((int)op < 0 || (int)op > DD_REDUCE_TENSOR_NORM_LP_POWER_P_SUM) return DD_STATUS_BAD_PARAM;
  if (comp != DD_DATA_FLOAT && comp != DD_DATA_DOUBLE) return DD_STATUS_NOT_SUPPORTED;
  r->op = op;
  r->comp = comp;
  r->nan = nanOpt;
  r->p = 2.0;
  r->eps = 0.0;
  r->indices = 0;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddSetReduceTensorDescriptorLp(ddReduceTensorDescriptor_t r, ddReduceTensorOp_t op, ddDataType_t comp,
                                         ddNanPropagation_t nanOpt, double p, double eps) {
  if (!(p >= 1.0) || !(eps == eps)) return DD_STATUS_BAD_PARAM;  // oneDNN: p >= 1; NaN refused
  ddStatus_t st = ddSetReduceTensorDescriptor(r, op, comp, nanOpt);
  if (st != DD_STATUS_SUCCESS) return st;
  r->p = p;
  r->eps = eps;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddSetReduceTensorDescriptorIndices(ddReduceTensorDescriptor_t r, ddReduceTensorIndices_t indices) {
  if (!r || ((int)indices != DD_REDUCE_TENSOR_NO_INDICES && (int)indices != DD_REDUCE_TENSOR_FLATTENED_INDICES))
    return DD_STATUS_BAD_PARAM;
  r->indices = (int)indices;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddGetReduceTensorDescriptorLp(ddReduceTensorDescriptor_t r, double *p, double *eps) {
  if (!r) return DD_STATUS_BAD_PARAM;
  if (p) *p = r->p;
  if (eps) *eps = r->eps;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddGetReduceTensorDescriptor(ddReduceTensorDescriptor_t r, ddReduceTensorOp_t *op,
                                       ddDataType_t *comp, ddNanPropagation_t *nanOpt) {
  if (!r) return DD_STATUS_BAD_PARAM;
  if (op) *op = r->op;
  if (comp) *comp = r->comp;
  if (nanOpt) *nanOpt = r->nan;
  return DD_STATUS_SUCCESS;
}

// ------------------------------------------------------------------ compute calls ------------

#define DD_CHECK_HANDLE(h) \
  if (!(h)) return DD_STATUS_BAD_PARAM
#define DD_CHECK(expr)                       \
  do {                                       \
    ddStatus_t st__ = (expr);                \
    if (st__ != DD_STATUS_SUCCESS) return st__; \
  } while (0)

ddStatus_t ddSetTensor(ddHandle_t h, ddTensorDescriptor_t yd, void *y, const void *value) {
  DD_RANGE("ddSetTensor");
  DD_CHECK_HANDLE(h);
  DD_CHECK(dd_check_desc(h, yd, "ddSetTensor y"));
  if (!y || !value) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddSetTensor: null pointer");
  return dd_set_impl(h, yd, y, dd_read_scalar(value, yd->dtype));
}

ddStatus_t ddScaleTensor(ddHandle_t h, ddTensorDescriptor_t yd, void *y, const void *alpha) {
  DD_RANGE("ddScaleTensor");
  DD_CHECK_HANDLE(h);
  DD_CHECK(dd_check_desc(h, yd, "ddScaleTensor y"));
  if (!y || !alpha) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddScaleTensor: null pointer");
  return dd_scale_impl(h, yd, y, dd_read_scalar(alpha, yd->dtype));
}

ddStatus_t ddAddTensor(ddHandle_t h, const void *alpha, ddTensorDescriptor_t xd, const void *x,
                       const void *beta, ddTensorDescriptor_t yd, void *y) {
  DD_RANGE("ddAddTensor");
  DD_CHECK_HANDLE(h);
  DD_CHECK(dd_check_desc(h, xd, "ddAddTensor x"));
  DD_CHECK(dd_check_desc(h, yd, "ddAddTensor y"));
  if (!x || !y || !alpha || !beta) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddAddTensor: null pointer");
  // y = 1*(beta*y) (+) alpha*bcast(x): op-tensor ADD with A = C = y
  double a = dd_read_scalar(alpha, xd->dtype);
  double b = dd_read_scalar(beta, yd->dtype);
  return dd_optensor_impl(h, DD_OP_TENSOR_ADD, b, yd, y, a, xd, x, 0.0, yd, y);
}

ddStatus_t ddOpTensor(ddHandle_t h, ddOpTensorOp_t op, const void *alpha1, ddTensorDescriptor_t ad,
                      const void *A, const void *alpha2, ddTensorDescriptor_t bd, const void *B,
                      const void *beta, ddTensorDescriptor_t cd, void *C) {
  DD_RANGE("ddOpTensor");
  DD_CHECK_HANDLE(h);
  DD_CHECK(dd_check_desc(h, ad, "ddOpTensor A"));
  DD_CHECK(dd_check_desc(h, bd, "ddOpTensor B"));
  DD_CHECK(dd_check_desc(h, cd, "ddOpTensor C"));
  if (!A || !B || !C || !alpha1 || !alpha2 || !beta)
    DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddOpTensor: null pointer");
  if ((int)op < 0 || (int)op > DD_OP_TENSOR_NE) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddOpTensor: bad op");
  return dd_optensor_impl(h, op, dd_read_scalar(alpha1, ad->dtype), ad, A,
                          dd_read_scalar(alpha2, bd->dtype), bd, B, dd_read_scalar(beta, cd->dtype),
                          cd, C);
}

ddStatus_t ddSumTensors(ddHandle_t h, int n, const float *scales, const ddTensorDescriptor_t *sd,
                        const void *const *srcs, ddTensorDescriptor_t dd, void *dst) {
  DD_RANGE("ddSumTensors");
  DD_CHECK_HANDLE(h);
  if (n < 1 || n > 8) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddSumTensors: n must be in 1..8");
  if (!scales || !sd || !srcs || !dst) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddSumTensors: null pointer");
  DD_CHECK(dd_check_desc(h, dd, "ddSumTensors dst"));
  for (int i = 0; i < n; i++) {
    DD_CHECK(dd_check_desc(h, sd[i], "ddSumTensors src"));
    if (!srcs[i]) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddSumTensors: null source %d", i);
  }
  return dd_sum_impl(h, n, scales, (const ddTensorStruct *const *)sd, srcs, dd, dst);
}

ddStatus_t ddTransformTensor(ddHandle_t h, const void *alpha, ddTensorDescriptor_t xd,
                             const void *x, const void *beta, ddTensorDescriptor_t yd, void *y) {
  DD_RANGE("ddTransformTensor");
  DD_CHECK_HANDLE(h);
  DD_CHECK(dd_check_desc(h, xd, "ddTransformTensor x"));
  DD_CHECK(dd_check_desc(h, yd, "ddTransformTensor y"));
  if (!x || !y || !alpha || !beta) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddTransformTensor: null pointer");
  if (!dd_same_dims(xd, yd))
    DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddTransformTensor: x and y dims differ");
  return dd_transform_impl(h, dd_read_scalar(alpha, xd->dtype), xd, x,
                           dd_read_scalar(beta, yd->dtype), yd, y);
}

ddStatus_t ddGatherTransform(ddHandle_t h, int count, const int64_t *srcOff, const int64_t *dstOff,
                             ddTensorDescriptor_t xd, const void *x, ddTensorDescriptor_t yd,
                             void *y) {
  DD_RANGE("ddGatherTransform");
  DD_CHECK_HANDLE(h);
  DD_CHECK(dd_check_desc(h, xd, "ddGatherTransform x"));
  DD_CHECK(dd_check_desc(h, yd, "ddGatherTransform y"));
  if (!x || !y || !srcOff || !dstOff) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddGatherTransform: null pointer");
  if (count < 0 || count > 4096) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddGatherTransform: count must be in 0..4096");
  if (!dd_same_dims(xd, yd)) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddGatherTransform: x and y dims differ");
  for (int i = 0; i < count; i++)
    if (srcOff[i] < 0 || dstOff[i] < 0) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddGatherTransform: negative offset");
  if (count == 0) return DD_STATUS_SUCCESS;
  return dd_gather_transform_impl(h, count, srcOff, dstOff, xd, x, yd, y);
}

ddStatus_t ddTensorEquals(ddHandle_t h, ddTensorDescriptor_t xd, const void *x,
                          ddTensorDescriptor_t yd, const void *y, int *flag) {
  DD_RANGE("ddTensorEquals");
  DD_CHECK_HANDLE(h);
  DD_CHECK(dd_check_desc(h, xd, "ddTensorEquals x"));
  DD_CHECK(dd_check_desc(h, yd, "ddTensorEquals y"));
  if (!x || !y || !flag) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddTensorEquals: null pointer");
  if (!dd_same_dims(xd, yd)) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddTensorEquals: dims differ");
  if (xd->dtype != yd->dtype) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddTensorEquals: data types differ");
  return dd_equals_impl(h, xd, x, yd, y, flag);
}

ddStatus_t ddActivationForward(ddHandle_t h, ddActivationDescriptor_t act, const void *alpha,
                               ddTensorDescriptor_t xd, const void *x, const void *beta,
                               ddTensorDescriptor_t yd, void *y) {
  DD_RANGE("ddActivationForward");
  DD_CHECK_HANDLE(h);
  if (!act) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddActivationForward: null activation descriptor");
  DD_CHECK(dd_check_desc(h, xd, "ddActivationForward x"));
  DD_CHECK(dd_check_desc(h, yd, "ddActivationForward y"));
  if (!x || !y || !alpha || !beta) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddActivationForward: null pointer");
  if (!dd_same_dims(xd, yd)) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddActivationForward: x and y dims differ");
  if (xd->dtype != yd->dtype) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddActivationForward: x and y data types differ");
  if (!dd_type_is_float(xd->dtype)) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddActivationForward: data type must be floating point");
  return dd_activation_fwd_impl(h, act, dd_read_scalar(alpha, xd->dtype), xd, x,
                                dd_read_scalar(beta, yd->dtype), yd, y);
}

ddStatus_t ddActivationBackward(ddHandle_t h, ddActivationDescriptor_t act, const void *alpha,
                                ddTensorDescriptor_t yd, const void *y, ddTensorDescriptor_t dyd,
                                const void *dy, ddTensorDescriptor_t xd, const void *x,
                                const void *beta, ddTensorDescriptor_t dxd, void *dx) {
  DD_RANGE("ddActivationBackward");
  DD_CHECK_HANDLE(h);
  if (!act) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddActivationBackward: null activation descriptor");
  // the *-dst-bwd kinds differentiate from the forward result: y takes the place of x
  if (act->mode >= DD_ACTIVATION_RELU_DST_BWD && act->mode <= DD_ACTIVATION_CLIP_V2_DST_BWD) {
    xd = yd;
    x = y;
  }
  DD_CHECK(dd_check_desc(h, dyd, "ddActivationBackward dy"));
  DD_CHECK(dd_check_desc(h, xd, "ddActivationBackward x"));
  DD_CHECK(dd_check_desc(h, dxd, "ddActivationBackward dx"));
  if (!dy || !x || !dx || !alpha || !beta) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddActivationBackward: null pointer");
  if (!dd_same_dims(xd, dyd) || !dd_same_dims(xd, dxd))
    DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddActivationBackward: dims differ");
  if (xd->dtype != dyd->dtype || xd->dtype != dxd->dtype)
    DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddActivationBackward: data types differ");
  if (!dd_type_is_float(xd->dtype)) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddActivationBackward: data type must be floating point");
  return dd_activation_bwd_impl(h, act, dd_read_scalar(alpha, xd->dtype), dyd, dy, xd, x,
                                dd_read_scalar(beta, dxd->dtype), dxd, dx);
}

static bool dd_wants_indices(const ddReduceTensorStruct *red) {
  return red->indices == DD_REDUCE_TENSOR_FLATTENED_INDICES &&
         (red->op == DD_REDUCE_TENSOR_MIN || red->op == DD_REDUCE_TENSOR_MAX || red->op == DD_REDUCE_TENSOR_AMAX);
}

static ddStatus_t check_reduce_shapes(ddHandle_t h, const ddTensorStruct *xd, const ddTensorStruct *yd) {
  if (xd->nd != yd->nd) DD_FAIL(h, DD_STATUS_BAD_PARAM, "reduce: x and y ranks differ");
  for (int i = 0; i < xd->nd; i++)
    if (yd->dims[i] != xd->dims[i] && yd->dims[i] != 1)
      DD_FAIL(h, DD_STATUS_BAD_PARAM, "reduce: y dim %d must equal x's or be 1", i);
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddGetReductionIndicesSize(ddHandle_t h, ddReduceTensorDescriptor_t red,
                                     ddTensorDescriptor_t xd, ddTensorDescriptor_t yd, size_t *bytes) {
  DD_CHECK_HANDLE(h);
  if (!bytes) DD_FAIL(h, DD_STATUS_BAD_PARAM, "null pointer");
  *bytes = 0;
  if (red && dd_wants_indices(red)) {
    DD_CHECK(dd_check_desc(h, xd, "reduce x"));
    DD_CHECK(dd_check_desc(h, yd, "reduce y"));
    DD_CHECK(check_reduce_shapes(h, xd, yd));
    size_t nout = 1;
    for (int i = 0; i < yd->nd; i++) nout *= (size_t)yd->dims[i];
    *bytes = nout * sizeof(unsigned);
  }
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddGetReductionWorkspaceSize(ddHandle_t h, ddReduceTensorDescriptor_t red,
                                       ddTensorDescriptor_t xd, ddTensorDescriptor_t yd, size_t *bytes) {
  DD_CHECK_HANDLE(h);
  if (!red || !bytes) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddGetReductionWorkspaceSize: null pointer");
  DD_CHECK(dd_check_desc(h, xd, "reduce x"));
  DD_CHECK(dd_check_desc(h, yd, "reduce y"));
  DD_CHECK(check_reduce_shapes(h, xd, yd));
  return dd_reduce_ws_size(h, red, xd, yd, bytes);
}

ddStatus_t ddReduceTensor(ddHandle_t h, ddReduceTensorDescriptor_t red, void *indices,
                          size_t indicesBytes, void *ws, size_t wsBytes, const void *alpha,
                          ddTensorDescriptor_t xd, const void *x, const void *beta,
                          ddTensorDescriptor_t yd, void *y) {
  DD_RANGE("ddReduceTensor");
  DD_CHECK_HANDLE(h);
  if (!red) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddReduceTensor: null reduce descriptor");
  DD_CHECK(dd_check_desc(h, xd, "ddReduceTensor x"));
  DD_CHECK(dd_check_desc(h, yd, "ddReduceTensor y"));
  if (!x || !y || !alpha || !beta) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddReduceTensor: null pointer");
  DD_CHECK(check_reduce_shapes(h, xd, yd));
  if (!dd_type_is_float(xd->dtype) || !dd_type_is_float(yd->dtype))
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddReduceTensor: data types must be floating point");
  if (dd_wants_indices(red)) {
    size_t nout = 1;
    for (int i = 0; i < yd->nd; i++) nout *= (size_t)yd->dims[i];
    if (!indices || indicesBytes < nout * sizeof(unsigned))
      DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddReduceTensor: the indices buffer holds %zu bytes, %zu are needed",
              indices ? indicesBytes : (size_t)0, nout * sizeof(unsigned));
    if (x == y) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddReduceTensor: indices need x after y is written; x and y must differ");
  }
  // alpha and beta follow the compute type like cuDNN's: float unless the tensors are double
  DD_CHECK(dd_reduce_impl(h, red, ws, wsBytes, dd_read_scalar(alpha, xd->dtype), xd, x,
                          dd_read_scalar(beta, yd->dtype), yd, y, false, nullptr));
  if (dd_wants_indices(red)) return dd_reduce_indices_impl(h, red, xd, x, yd, (unsigned *)indices);
  return DD_STATUS_SUCCESS;
}

// db = alpha * sum of dy over every dim where db's extent is 1 (N, H, W for a [1,C,1,1] bias)
// + beta * db: the (N,H,W) sum of ddReduceTensor under the name the convolution layers call.
ddStatus_t ddConvolutionBackwardBias(ddHandle_t h, const void *alpha, ddTensorDescriptor_t dyd,
                                     const void *dy, const void *beta, ddTensorDescriptor_t dbd, void *db) {
  DD_RANGE("ddConvolutionBackwardBias");
  DD_CHECK_HANDLE(h);
  DD_CHECK(dd_check_desc(h, dyd, "ddConvolutionBackwardBias dy"));
  DD_CHECK(dd_check_desc(h, dbd, "ddConvolutionBackwardBias db"));
  if (!dy || !db || !alpha || !beta) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddConvolutionBackwardBias: null pointer");
  DD_CHECK(check_reduce_shapes(h, dyd, dbd));
  if (!dd_type_is_float(dyd->dtype) || !dd_type_is_float(dbd->dtype))
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddConvolutionBackwardBias: data types must be floating point");
  ddReduceTensorStruct red;
  red.op = DD_REDUCE_TENSOR_ADD;
  red.comp = dyd->dtype == DD_DATA_DOUBLE ? DD_DATA_DOUBLE : DD_DATA_FLOAT;
  red.nan = DD_PROPAGATE_NAN;
  return dd_reduce_impl(h, &red, nullptr, 0, dd_read_scalar(alpha, dyd->dtype), dyd, dy,
                        dd_read_scalar(beta, dbd->dtype), dbd, db, false, nullptr);
}

}  // extern "C"
