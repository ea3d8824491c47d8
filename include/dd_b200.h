/*
 * dd_b200.h -- C ABI of libdd_b200.so: hand-written sm_100a kernels for Deep Diamond's
 * data-parallel tensor hot path (layout reorder with dtype conversion, eltwise activation
 * forward/backward, broadcast op-tensor, reduce-tensor).
 *
 * The entry points are shaped after the cuDNN calls that Deep Diamond's cuDNN backend binds in
 *   deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/impl.clj
 * so that a Clojure `impl` namespace for this library translates one call to one call.  Each
 * declaration below cites the reference binding it replaces (file:line inside the reference
 * project).  Numeric parity target is the reference's DNNL (oneDNN) CPU backend,
 *   deep-diamond-dnnl/src/uncomplicate/diamond/internal/dnnl/{core,impl}.clj.
 *
 * Conventions
 *  - Every function returns a ddStatus_t; 0 is success.  Nothing aborts, throws or prints.
 *  - All device pointers are plain CUDA device addresses owned by the caller.
 *  - Every compute call enqueues work on the handle's stream and returns; no call synchronises
 *    the device or allocates device memory (the handle owns a fixed scratch buffer allocated once
 *    in ddCreate), except where a comment says otherwise.
 *  - alpha/beta/value scalars are HOST pointers to float, or to double when the tensor data type
 *    is DD_DATA_DOUBLE (same rule the reference follows with `cast-prim`,
 *    cudnn/tensor.clj:193-194).
 *  - With beta == 0 the destination is never read (NaN/Inf already there do not propagate).
 *  - A handle is used from one host thread at a time (the reference drives a factory from a
 *    single thread, cudnn/factory.clj:481-494).
 */
#ifndef DD_B200_H
#define DD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DD_B200_VERSION 100 /* 0.1.0 */
#if defined(__GNUC__)
#define DD_API __attribute__((visibility("default")))
#else
#define DD_API
#endif
#define DD_DIM_MAX 8

/* Status codes.  Values 0..9 keep the order of the cuDNN status keywords the reference decodes in
 * cudnn/constants.clj:16-33 so the Clojure side can reuse its keyword table. */
typedef enum {
  DD_STATUS_SUCCESS = 0,
  DD_STATUS_NOT_INITIALIZED = 1,
  DD_STATUS_ALLOC_FAILED = 2,
  DD_STATUS_BAD_PARAM = 3,
  DD_STATUS_INTERNAL_ERROR = 4,
  DD_STATUS_INVALID_VALUE = 5,
  DD_STATUS_ARCH_MISMATCH = 6,
  DD_STATUS_MAPPING_ERROR = 7,
  DD_STATUS_EXECUTION_FAILED = 8,
  DD_STATUS_NOT_SUPPORTED = 9,
  DD_STATUS_TIMEOUT = 10,       /* a bounded host-side wait ran out (multi-GPU set-up only) */
  DD_STATUS_COMM_FAILED = 11    /* the collective library reported an error */
} ddStatus_t;

/* Data types.  Codes 0,1,2,3,4,6 are the cuDNN codes decoded in cudnn/constants.clj:111-124
 * (:float :double :half :byte :int :uint8); 9 = bfloat16 and 15 = int64 follow cuDNN's numbering
 * for types the reference's table does not list yet. */
typedef enum {
  DD_DATA_FLOAT = 0,
  DD_DATA_DOUBLE = 1,
  DD_DATA_HALF = 2,
  DD_DATA_INT8 = 3,
  DD_DATA_INT32 = 4,
  DD_DATA_UINT8 = 6,
  DD_DATA_BFLOAT16 = 9,
  DD_DATA_INT64 = 15
} ddDataType_t;

/* Named layouts, cudnn/constants.clj:43-55. */
typedef enum { DD_TENSOR_NCHW = 0, DD_TENSOR_NHWC = 1 } ddTensorFormat_t;

/* Activation modes, cudnn/constants.clj:150-158 (+ ddnl names in dnnl/constants.clj:277-308). */
typedef enum {
  DD_ACTIVATION_SIGMOID = 0,      /* :logistic / :sigmoid   y = 1/(1+exp(-x))                    */
  DD_ACTIVATION_RELU = 1,         /* :relu                  y = x>0 ? x : coef*x  (coef: slope)  */
  DD_ACTIVATION_TANH = 2,         /* :tanh                                                       */
  DD_ACTIVATION_CLIPPED_RELU = 3, /* :clipped-relu          y = min(max(x,0),coef)               */
  DD_ACTIVATION_ELU = 4,          /* :elu                   y = x>0 ? x : coef*(exp(x)-1)        */
  DD_ACTIVATION_LINEAR = 5,       /* :linear / :identity    y = coef*x + shift                   */
  DD_ACTIVATION_ABS = 6,          /* :abs (dnnl only; dnnl-t/core_test.clj:183-200)             */
  /* The other kinds of the reference's oneDNN table (dnnl/constants.clj:277-308), which its DNNL
   * backend accepts in `activation`; a = coef, b = shift of ddSetActivationDescriptorEx, defined as
   * oneDNN documents them. */
  DD_ACTIVATION_SQUARE = 7,       /* :square      y = x^2                                        */
  DD_ACTIVATION_SQRT = 8,         /* :sqrt                                                       */
  DD_ACTIVATION_EXP = 9,          /* :exp                                                        */
  DD_ACTIVATION_LOG = 10,         /* :log                                                        */
  DD_ACTIVATION_SOFT_RELU = 11,   /* :soft-relu   y = log(1+exp(a*x))/a                          */
  DD_ACTIVATION_SWISH = 12,       /* :swish       y = x/(1+exp(-a*x))                            */
  DD_ACTIVATION_GELU_TANH = 13,   /* :gelu :gelu-tanh  y = 0.5x(1+tanh(sqrt(2/pi)(x+0.044715x^3))) */
  DD_ACTIVATION_GELU_ERF = 14,    /* :gelu-erf    y = 0.5x(1+erf(x/sqrt 2))                      */
  DD_ACTIVATION_HARDSWISH = 15,   /* :hardswish   y = x*max(0,min(1,a*x+b))                      */
  DD_ACTIVATION_CLIP = 16,        /* :clip        y = min(max(x,a),b); dx = dy where a < x <= b  */
  DD_ACTIVATION_CLIP_V2 = 17,     /* :clip-v2     the same;            dx = dy where a < x <  b  */
  DD_ACTIVATION_POW = 18,         /* :pow         y = a*x^b                                      */
  DD_ACTIVATION_MISH = 19,        /* :mish        y = x*tanh(log(1+exp(x)))                      */
  DD_ACTIVATION_ROUND = 20,       /* :round       to nearest, ties to even; forward only         */
  /* Same forward as the kind named; backward takes the derivative from the forward RESULT, which
   * ddActivationBackward then reads from its y argument (x may be NULL). */
  DD_ACTIVATION_RELU_DST_BWD = 21,
  DD_ACTIVATION_TANH_DST_BWD = 22,
  DD_ACTIVATION_ELU_DST_BWD = 23,
  DD_ACTIVATION_SQRT_DST_BWD = 24,
  DD_ACTIVATION_LOGISTIC_DST_BWD = 25,
  DD_ACTIVATION_EXP_DST_BWD = 26,
  DD_ACTIVATION_CLIP_V2_DST_BWD = 27
} ddActivationMode_t;

typedef enum { DD_NOT_PROPAGATE_NAN = 0, DD_PROPAGATE_NAN = 1 } ddNanPropagation_t;

/* Binary ops: cudnnOpTensor's set, plus the oneDNN binary kinds the reference names in
 * dnnl/constants.clj:359-371: the arithmetic ones and the comparisons (1 where the relation holds
 * between alpha1*A and alpha2*B, else 0, stored in the tensors' data type; a NaN compares false,
 * except under NE). */
typedef enum {
  DD_OP_TENSOR_ADD = 0,
  DD_OP_TENSOR_MUL = 1,
  DD_OP_TENSOR_MIN = 2,
  DD_OP_TENSOR_MAX = 3,
  DD_OP_TENSOR_SUB = 4,
  DD_OP_TENSOR_DIV = 5,
  DD_OP_TENSOR_GE = 6,
  DD_OP_TENSOR_GT = 7,
  DD_OP_TENSOR_LE = 8,
  DD_OP_TENSOR_LT = 9,
  DD_OP_TENSOR_EQ = 10,
  DD_OP_TENSOR_NE = 11
} ddOpTensorOp_t;

/* Reduce ops, cudnn/constants.clj:171-180; oneDNN's kinds (dnnl/constants.clj:393-402) map as
 * sum->ADD, mean->AVG, max, min, mul, norm-lp-sum p=1 -> NORM1, norm-lp-sum p=2 -> NORM2.
 * The four NORM_LP kinds are oneDNN's own, with the p and epsilon that the reference's `reduction`
 * passes (dnnl/core.clj:796-803); S = sum of |x|^p over the reduced dims:
 *   NORM_LP_MAX          max(S, eps)^(1/p)        NORM_LP_SUM          (S + eps)^(1/p)
 *   NORM_LP_POWER_P_MAX  max(S, eps)              NORM_LP_POWER_P_SUM  S + eps
 * p and eps are set with ddSetReduceTensorDescriptorLp (p = 2, eps = 0 otherwise). */
typedef enum {
  DD_REDUCE_TENSOR_ADD = 0,
  DD_REDUCE_TENSOR_MUL = 1,
  DD_REDUCE_TENSOR_MIN = 2,
  DD_REDUCE_TENSOR_MAX = 3,
  DD_REDUCE_TENSOR_AMAX = 4,
  DD_REDUCE_TENSOR_AVG = 5,
  DD_REDUCE_TENSOR_NORM1 = 6,
  DD_REDUCE_TENSOR_NORM2 = 7,
  DD_REDUCE_TENSOR_MUL_NO_ZEROS = 8,
  DD_REDUCE_TENSOR_NORM_LP_MAX = 9,
  DD_REDUCE_TENSOR_NORM_LP_SUM = 10,
  DD_REDUCE_TENSOR_NORM_LP_POWER_P_MAX = 11,
  DD_REDUCE_TENSOR_NORM_LP_POWER_P_SUM = 12
} ddReduceTensorOp_t;

/* cudnnReduceTensorIndices_t, cudnn/constants.clj:182-184 (:no-indices, :flattened). */
typedef enum { DD_REDUCE_TENSOR_NO_INDICES = 0, DD_REDUCE_TENSOR_FLATTENED_INDICES = 1 } ddReduceTensorIndices_t;

typedef struct ddContext *ddHandle_t;
typedef struct ddTensorStruct *ddTensorDescriptor_t;
typedef struct ddActivationStruct *ddActivationDescriptor_t;
typedef struct ddReduceTensorStruct *ddReduceTensorDescriptor_t;
typedef struct ddShardedStruct *ddShardedHandle_t;

/* ------------------------------------------------------------------ handle ------------------ */

/* Replaces cudnnCreate / cudnnDestroy (cudnn/impl.clj:56-71).  ddCreate binds the handle to the
 * calling thread's current CUDA device and allocates the handle's scratch buffer (the only
 * device allocation the library ever makes for single-GPU work). */
DD_API ddStatus_t ddCreate(ddHandle_t *handle);
DD_API ddStatus_t ddDestroy(ddHandle_t handle);
/* Replaces cudnnSetStream / cudnnGetStream (cudnn/impl.clj:73-83).  `stream` is a CUstream /
 * cudaStream_t; NULL is the legacy default stream. */
DD_API ddStatus_t ddSetStream(ddHandle_t handle, void *stream);
DD_API ddStatus_t ddGetStream(ddHandle_t handle, void **stream);
/* Replaces cudnnGetErrorString (cudnn/impl.clj:30-41 turns a status into ex-info). */
DD_API const char *ddGetErrorString(ddStatus_t status);
/* A human-readable reason for the last non-success status returned through this handle
 * (never NULL; valid until the next call on the handle). */
DD_API const char *ddGetLastErrorMessage(ddHandle_t handle);
DD_API size_t ddGetVersion(void);
/* Number of kernels this handle has launched since ddCreate (a harness counter). */
DD_API ddStatus_t ddGetLaunchCount(ddHandle_t handle, uint64_t *count);
/* Name of the kernel family chosen by the most recent compute call ("flat", "tile", "strided",
 * "rowreduce", ...): lets tests assert that the intended fast path ran. */
DD_API const char *ddGetLastKernelName(ddHandle_t handle);
/* No counterpart in the reference.  Split reductions and ddCostDiff count CTA arrivals in the first
 * 64 KB of the handle's scratch; every launch leaves those counters at zero when it completes.  A
 * launch that did NOT complete (a call that returned DD_STATUS_EXECUTION_FAILED, or a later CUDA
 * error that names one of this library's kernels) may leave some of them non-zero, and the next
 * split reduction through the same handle would then never see its last arrival and write no
 * result.  After such a failure either destroy the handle and create a new one, or call
 * ddResetCounters: it zeroes the counters on the handle's stream (ordered after everything already
 * enqueued there).  Nothing else in a handle depends on an earlier launch. */
DD_API ddStatus_t ddResetCounters(ddHandle_t handle);
/* No counterpart in the reference.  The transposing reorder of 1-byte elements has the GPU's copy
 * engine (TMA) bring its tiles into shared memory, and the kernel's waits for those copies are
 * bounded: a CTA whose tile never arrives raises a word in host-mapped memory, leaves its part of
 * the output unwritten and returns, so that the context stays usable.  *word is that word as of
 * now: 0 = no kernel of this handle ever gave up; read it after synchronising the handle's stream
 * to learn whether the launches so far completed.  Once it is non-zero every later
 * ddTransformTensor on the handle returns DD_STATUS_EXECUTION_FAILED; destroy the handle. */
DD_API ddStatus_t ddGetDeviceFault(ddHandle_t handle, int *word);

/* --------------------------------------------------------------- descriptors ---------------- */

/* Replace cudnnCreateTensorDescriptor / cudnnDestroyTensorDescriptor / cudnnSetTensor4dDescriptor /
 * cudnnSetTensor4dDescriptorEx / cudnnSetTensorNdDescriptor / cudnnSetTensorNdDescriptorEx /
 * cudnnGetTensorNdDescriptor / cudnnGetTensorSizeInBytes (cudnn/impl.clj:98-180), and oneDNN's
 * dnnl_memory_desc_create_with_{tag,strides} (dnnl/impl.clj:144-190).  Dims are positive,
 * strides positive (element units); rank 1..DD_DIM_MAX.  Unlike cuDNN, rank < 4 is accepted
 * without padding and dims/strides are 64-bit. */
DD_API ddStatus_t ddCreateTensorDescriptor(ddTensorDescriptor_t *desc);
DD_API ddStatus_t ddDestroyTensorDescriptor(ddTensorDescriptor_t desc);
DD_API ddStatus_t ddSetTensor4dDescriptor(ddTensorDescriptor_t desc, ddTensorFormat_t format,
                                   ddDataType_t dataType, int64_t n, int64_t c, int64_t h,
                                   int64_t w);
DD_API ddStatus_t ddSetTensor4dDescriptorEx(ddTensorDescriptor_t desc, ddDataType_t dataType, int64_t n,
                                     int64_t c, int64_t h, int64_t w, int64_t nStride,
                                     int64_t cStride, int64_t hStride, int64_t wStride);
DD_API ddStatus_t ddSetTensorNdDescriptor(ddTensorDescriptor_t desc, ddDataType_t dataType, int nbDims,
                                   const int64_t *dims, const int64_t *strides);
DD_API ddStatus_t ddSetTensorNdDescriptorEx(ddTensorDescriptor_t desc, ddTensorFormat_t format,
                                     ddDataType_t dataType, int nbDims, const int64_t *dims);
DD_API ddStatus_t ddGetTensorNdDescriptor(ddTensorDescriptor_t desc, int nbDimsRequested,
                                   ddDataType_t *dataType, int *nbDims, int64_t *dims,
                                   int64_t *strides);
/* Bytes spanned: (1 + sum (dim-1)*stride) * width, the rule of base/tensor.clj:172-183. */
DD_API ddStatus_t ddGetTensorSizeInBytes(ddTensorDescriptor_t desc, size_t *bytes);

/* ---------------------------------------------------------------- op-tensor ----------------- */

/* y[:] = *value.  Replaces cudnnSetTensor (cudnn/impl.clj:182-185; used by set-all and zero-init,
 * cudnn/factory.clj:191-193,362-366). */
DD_API ddStatus_t ddSetTensor(ddHandle_t handle, ddTensorDescriptor_t yDesc, void *y, const void *value);
/* y *= *alpha.  Replaces cudnnScaleTensor (cudnn/impl.clj:197-200; `scal`, cudnn/factory.clj:183-185). */
DD_API ddStatus_t ddScaleTensor(ddHandle_t handle, ddTensorDescriptor_t yDesc, void *y, const void *alpha);
/* y = alpha*bcast(x) + beta*y, every dim of x equal to y's or 1.  Replaces cudnnAddTensor
 * (cudnn/impl.clj:187-190; axpy/axpby cudnn/factory.clj:169-171,194-196; bias add
 * cudnn/directed.clj:508,579) and, for same-shape operands, oneDNN sum (dnnl/core.clj:392-426).
 * Arithmetic: fl(fl(alpha*x) + fl(beta*y)) in the compute type, a factor of exactly 1 skipped. */
DD_API ddStatus_t ddAddTensor(ddHandle_t handle, const void *alpha, ddTensorDescriptor_t xDesc,
                       const void *x, const void *beta, ddTensorDescriptor_t yDesc, void *y);
/* C = op(alpha1*A, alpha2*bcast(B)) + beta*C, every dim of B equal to A's or 1; A and C have equal
 * dims.  Replaces cudnnOpTensor and oneDNN binary (dnnl/core.clj:430-447, dnnl/impl.clj:363-368). */
DD_API ddStatus_t ddOpTensor(ddHandle_t handle, ddOpTensorOp_t op, const void *alpha1,
                      ddTensorDescriptor_t aDesc, const void *A, const void *alpha2,
                      ddTensorDescriptor_t bDesc, const void *B, const void *beta,
                      ddTensorDescriptor_t cDesc, void *C);
/* dst = sum_i scales[i]*src[i] over n same-shape sources in one pass; dst may alias src[0].
 * Replaces oneDNN sum with n sources (dnnl/core.clj:392-426, dnnl/impl.clj:345-359) and the
 * loop of n-1 axpy! passes in the cuDNN sum layer (cudnn/directed.clj:1762-1766).
 * `srcs` is a HOST array of n device pointers, `scales` a HOST array of n floats; n <= 8. */
DD_API ddStatus_t ddSumTensors(ddHandle_t handle, int n, const float *scales,
                        const ddTensorDescriptor_t *srcDescs, const void *const *srcs,
                        ddTensorDescriptor_t dstDesc, void *dst);

/* ---------------------------------------------------------------- reorder ------------------- */

/* y = alpha*convert(x) + beta*y for every logical index; x and y have equal dims, any strides,
 * any pair of data types.  Replaces cudnnTransformTensor (cudnn/impl.clj:192-195; the body of
 * CUDnnTransformer / CUDnnBatcher / copy, cudnn/tensor.clj:188-195,248-258, cudnn/factory.clj:166-168)
 * and oneDNN reorder (dnnl/impl.clj:372-376, dnnl/core.clj:523-529).
 * Conversion: to bf16/f16 round-to-nearest-even; to s8/u8/s32/s64 saturate then
 * round-to-nearest-even; NaN -> 0 for integer destinations. x and y must not overlap. */
DD_API ddStatus_t ddTransformTensor(ddHandle_t handle, const void *alpha, ddTensorDescriptor_t xDesc,
                             const void *x, const void *beta, ddTensorDescriptor_t yDesc, void *y);

/* One launch that copies `count` sub-tensors of shape subDesc from x to y: item i reads at element
 * offset srcOffsets[i] and writes at dstOffsets[i].  Replaces the mb-size separate
 * cudnnTransformTensor calls a shuffler issues per invocation (cudnn/tensor.clj:306-317).
 * srcOffsets/dstOffsets are HOST arrays (count <= 4096), copied into the launch. */
DD_API ddStatus_t ddGatherTransform(ddHandle_t handle, int count, const int64_t *srcOffsets,
                             const int64_t *dstOffsets, ddTensorDescriptor_t xSubDesc,
                             const void *x, ddTensorDescriptor_t ySubDesc, void *y);

/* *deviceFlag += (number of blocks that saw a mismatch) ; the caller zeroes the int before and
 * reads it after.  x and y have equal dims and data type, any strides.  Replaces the five
 * tensor_{1..5}d_equals kernels, deep-diamond-cuda/src/device/uncomplicate/diamond/internal/cuda/
 * blas-plus.cu:9-101 (launched from cudnn/factory.clj:58-133). */
DD_API ddStatus_t ddTensorEquals(ddHandle_t handle, ddTensorDescriptor_t xDesc, const void *x,
                          ddTensorDescriptor_t yDesc, const void *y, int *deviceFlag);

/* Up to 8 independent reorder/convert copies y_i = convert(x_i) in ONE launch (all items share one
 * source and one destination data type; each item has its own dims and strides).  Replaces the
 * per-sub-tensor transformer loops of the branch and concatenate layers,
 * `(doseq [ft fwd-trans] (ft))`, cudnn/directed.clj:1289-1549 (blueprints :1455-1549).
 * xDescs/xs/yDescs/ys are HOST arrays of `count` entries. */
DD_API ddStatus_t ddMultiTransform(ddHandle_t handle, int count, const ddTensorDescriptor_t *xDescs,
                                   const void *const *xs, const ddTensorDescriptor_t *yDescs,
                                   void *const *ys);

/* d = a - y and, in the same pass, cost[0] = sum (a-y)^2 / (2n) (kind 0, quadratic) or
 * sum |a-y| / n (kind 1, mean absolute) or sum |(y-1) log(1.0000001-a) - y log(a)| / dims[0]
 * (kind 2, cross-entropy; the divisor is the batch extent); a, y, d dense tensors of one
 * descriptor, d may be NULL or alias a.  `cost` is one DEVICE element of the tensor's data type
 * (float or double).  Replaces the cost glue `axpy! -1.0 y a-y` + `nrm2`/`asum`, and the six
 * vector-math passes of the cross-entropy (cudnn/directed.clj:367-458 with
 * deep-diamond-base/src/uncomplicate/diamond/internal/cost.clj:20-40). */
DD_API ddStatus_t ddCostDiff(ddHandle_t handle, int kind, ddTensorDescriptor_t desc, const void *a,
                             const void *y, void *d, void *cost);

/* ---------------------------------------------------------------- activation ---------------- */

/* Replace cudnnCreate/Set/Get/DestroyActivationDescriptor (cudnn/impl.clj:206-221,
 * cudnn/core.clj:148-164).  `coef` is the reference's alpha (relu slope, elu scale, clip ceiling,
 * linear scale); ddSetActivationDescriptorEx also carries oneDNN's `beta` (the shift of :linear,
 * dnnl/core.clj:345-362). */
DD_API ddStatus_t ddCreateActivationDescriptor(ddActivationDescriptor_t *desc);
DD_API ddStatus_t ddDestroyActivationDescriptor(ddActivationDescriptor_t desc);
DD_API ddStatus_t ddSetActivationDescriptor(ddActivationDescriptor_t desc, ddActivationMode_t mode,
                                     ddNanPropagation_t nanOpt, double coef);
DD_API ddStatus_t ddSetActivationDescriptorEx(ddActivationDescriptor_t desc, ddActivationMode_t mode,
                                       ddNanPropagation_t nanOpt, double coef, double shift);
DD_API ddStatus_t ddGetActivationDescriptor(ddActivationDescriptor_t desc, ddActivationMode_t *mode,
                                     ddNanPropagation_t *nanOpt, double *coef);
/* y = alpha*act(x) + beta*y; x and y have equal dims and data type; y may be x (in place,
 * the inference form, cudnn/directed.clj:70-75, dnnl/directed.clj:152-156).  Replaces
 * cudnnActivationForward (cudnn/impl.clj:223-226) / oneDNN eltwise forward (dnnl/impl.clj:324-331).
 * Unlike cuDNN, DD_ACTIVATION_LINEAR is computed, not rejected. */
DD_API ddStatus_t ddActivationForward(ddHandle_t handle, ddActivationDescriptor_t act, const void *alpha,
                               ddTensorDescriptor_t xDesc, const void *x, const void *beta,
                               ddTensorDescriptor_t yDesc, void *y);
/* dx = alpha*act'(x)*dy + beta*dx.  Argument order is cudnnActivationBackward's
 * (cudnn/impl.clj:228-235).  The derivative is taken from x (the forward SOURCE), which is what
 * the reference's DNNL backend does (eltwise-bwd-args SRC, DIFF_DST, DIFF_SRC,
 * dnnl/core.clj:382-388); y is accepted for signature compatibility, may be NULL and is not
 * read -- except by the *_DST_BWD kinds, which take the derivative from y (the forward result), as
 * oneDNN's *_use_dst_for_bwd algorithms do, and leave xDesc and x unread (they may be NULL).  dx may
 * alias dy or x.  DD_ACTIVATION_ROUND has no backward (NOT_SUPPORTED). */
DD_API ddStatus_t ddActivationBackward(ddHandle_t handle, ddActivationDescriptor_t act, const void *alpha,
                                ddTensorDescriptor_t yDesc, const void *y,
                                ddTensorDescriptor_t dyDesc, const void *dy,
                                ddTensorDescriptor_t xDesc, const void *x, const void *beta,
                                ddTensorDescriptor_t dxDesc, void *dx);

/* ---------------------------------------------------------------- reduce -------------------- */

/* Replace cudnnCreate/Set/DestroyReduceTensorDescriptor, cudnnGetReductionIndicesSize,
 * cudnnGetReductionWorkspaceSize, cudnnReduceTensor (cudnn/impl.clj:239-285,
 * cudnn/core.clj:188-231) and oneDNN reduction (dnnl/impl.clj:557-562, dnnl/core.clj:796-803).
 * Reduced dims are those where y's dim is 1 and x's is not.  Accumulation is fp32 (fp64 for
 * DD_DATA_DOUBLE) in a fixed tree order: results are run-to-run identical.
 * y = alpha*reduce(x) + beta*y.  Indices are produced only on request (ddSetReduceTensorDescriptorIndices).
 * Workspace: pass the size ddGetReductionWorkspaceSize returns, or workspace == NULL to use the
 * handle's own scratch (then the size needed must not exceed DD_HANDLE_SCRATCH_BYTES - 64 KB). */
#define DD_HANDLE_SCRATCH_BYTES (8u << 20)
DD_API ddStatus_t ddCreateReduceTensorDescriptor(ddReduceTensorDescriptor_t *desc);
DD_API ddStatus_t ddDestroyReduceTensorDescriptor(ddReduceTensorDescriptor_t desc);
DD_API ddStatus_t ddSetReduceTensorDescriptor(ddReduceTensorDescriptor_t desc, ddReduceTensorOp_t op,
                                       ddDataType_t compType, ddNanPropagation_t nanOpt);
DD_API ddStatus_t ddGetReduceTensorDescriptor(ddReduceTensorDescriptor_t desc, ddReduceTensorOp_t *op,
                                       ddDataType_t *compType, ddNanPropagation_t *nanOpt);
/* The descriptor of oneDNN's reduction with its two extra arguments (dnnl/impl.clj:557-562
 * `reduction*` alg p epsilon; dnnl/core.clj:796-803).  p >= 1 (1 and 2 run the NORM1 / NORM2
 * accumulation, any other p raises |x| to it element by element); p and eps are read by the four
 * NORM_LP kinds only.  ddGetReduceTensorDescriptorLp returns them. */
DD_API ddStatus_t ddSetReduceTensorDescriptorLp(ddReduceTensorDescriptor_t desc, ddReduceTensorOp_t op,
                                         ddDataType_t compType, ddNanPropagation_t nanOpt, double p,
                                         double eps);
DD_API ddStatus_t ddGetReduceTensorDescriptorLp(ddReduceTensorDescriptor_t desc, double *p, double *eps);
/* The `indices` argument of the reference's 4-argument reduce-tensor-descriptor (cudnn/core.clj:188-196).
 * With DD_REDUCE_TENSOR_FLATTENED_INDICES and op MIN, MAX or AMAX, ddReduceTensor also writes, for every
 * output, the position of the element that gave the result as a 32-bit unsigned offset into the
 * flattened (row-major, original dim order) block of the reduced dims: the FIRST such element; with NaN
 * propagation on, the first NaN if there is one.  The indices buffer holds one value per output in the
 * row-major order of y's dims; ddGetReductionIndicesSize gives its size (0 for every other op or
 * without this setting).  The positions come from a second launch that scans x again (a warp per
 * output, or a thread per output when the unit-stride dim is kept): there for completeness, not tuned. */
DD_API ddStatus_t ddSetReduceTensorDescriptorIndices(ddReduceTensorDescriptor_t desc, ddReduceTensorIndices_t indices);
DD_API ddStatus_t ddGetReductionIndicesSize(ddHandle_t handle, ddReduceTensorDescriptor_t red,
                                     ddTensorDescriptor_t xDesc, ddTensorDescriptor_t yDesc,
                                     size_t *bytes);
DD_API ddStatus_t ddGetReductionWorkspaceSize(ddHandle_t handle, ddReduceTensorDescriptor_t red,
                                       ddTensorDescriptor_t xDesc, ddTensorDescriptor_t yDesc,
                                       size_t *bytes);
DD_API ddStatus_t ddReduceTensor(ddHandle_t handle, ddReduceTensorDescriptor_t red, void *indices,
                          size_t indicesBytes, void *workspace, size_t workspaceBytes,
                          const void *alpha, ddTensorDescriptor_t xDesc, const void *x,
                          const void *beta, ddTensorDescriptor_t yDesc, void *y);

/* ---------------------------------------------------------------- no-allocation reduce ------- */

/* db = alpha * (sum of dy over the dims where db's extent is 1) + beta * db: the bias gradient of
 * the convolution and fully connected layers, here the (N,H,W) sum of ddReduceTensor under its
 * cuDNN name.  Replaces convolution-bwd-bias*, cudnn/impl.clj:470-475 (core.clj:344-350, called
 * from cudnn/directed.clj:591). */
DD_API ddStatus_t ddConvolutionBackwardBias(ddHandle_t handle, const void *alpha,
                                            ddTensorDescriptor_t dyDesc, const void *dy,
                                            const void *beta, ddTensorDescriptor_t dbDesc, void *db);

/* No counterpart in the reference.  ddReduceTensor for callers that cannot allocate device memory:
 * code running where cudaMalloc is off limits (inside a real-time or latency-critical loop, under a
 * memory pool that owns the whole device, in a plugin whose host forbids allocations after start-up).
 * Such callers cannot make a handle either (ddCreate allocates the handle's scratch), so this entry
 * point takes the stream directly and no handle.  It calls no cudaMalloc, cudaFree or allocating
 * library routine; the caller passes inputs and outputs as usual.
 *
 * The partial results of split reductions live in an array built into the library,
 * DD_NOALLOC_SCRATCH_BYTES per GPU, which every GPU that loads the library holds until the process
 * exits.  A reduction whose plan needs more is refused with DD_STATUS_NOT_SUPPORTED and the reason in
 * `errbuf` (use ddReduceTensor with your own workspace then).  Nothing in the array has to start at
 * zero: every slot that is read was written earlier in the same call.  But all calls share the one
 * array, so two calls whose kernels overlap on the GPU (different streams, no ordering) race on it:
 * keep these calls on one stream or order them with events.
 *
 * The first call made with a given device current looks up the array's device address and the SM
 * count of that device; make that first call outside any stream capture.
 * Results are identical to ddReduceTensor's (same plan, same kernels).
 * `errbuf` (may be NULL) receives a NUL-terminated reason when the status is not success. */
#define DD_NOALLOC_SCRATCH_BYTES (64u << 10)
DD_API ddStatus_t ddReduceTensorNoAlloc(void *stream, ddReduceTensorOp_t op, ddNanPropagation_t nanOpt,
                                        const void *alpha, ddTensorDescriptor_t xDesc, const void *x,
                                        const void *beta, ddTensorDescriptor_t yDesc, void *y,
                                        char *errbuf, size_t errbufLen);

/* ---------------------------------------------------------------- multi-GPU ----------------- */

/* No counterpart in the reference (it has no multi-device code).  One process per GPU; a tensor is
 * sharded along its batch dim, each rank holding `x` = its own slice.  A reduction that spans the
 * sharded dim runs the local partial reduce, then combines the (small) partial results across the
 * ranks and finishes (sqrt / divide / alpha-beta): by one ncclAllReduce on the handle's stream plus
 * a finishing kernel, or by the peer exchange below.  The NCCL library is located at run time
 * (libnccl.so.2); nothing else in this header needs it.
 *
 * ddShardedGetUniqueId fills a 128-byte id on one rank; the caller ships it to the other ranks by
 * any means; every rank then calls ddShardedCreate.  The call is collective and returns when all
 * ranks have joined.  The join is bounded: if it has not completed after the join limit (120 s
 * unless ddShardedSetJoinLimit changed it) the call returns DD_STATUS_TIMEOUT; the communicator is
 * then unusable and the process should exit (the library cannot cancel NCCL's own rendezvous, the
 * thread that runs it is left behind).  Host code that has a transport of its own should first check
 * over it that every rank has arrived (deep_diamond_b200/sharded.py does, with its own limit), so
 * that this limit is the second line only. */
#define DD_UNIQUE_ID_BYTES 128
DD_API ddStatus_t ddShardedGetUniqueId(void *id128);
DD_API ddStatus_t ddShardedSetJoinLimit(double seconds);
DD_API ddStatus_t ddShardedCreate(ddShardedHandle_t *sharded, ddHandle_t handle, int nRanks, int rank,
                           const void *id128);
/* Tear-down is COLLECTIVE when the peer exchange is attached, in three steps:
 *   1. every rank calls ddShardedPeerDetach: it waits for this rank's own work (stream
 *      synchronise) and closes this rank's mappings of the other ranks' buffers, so that this rank
 *      can no longer store into them;
 *   2. all ranks meet at a barrier of the caller's (any host transport);
 *   3. every rank calls ddShardedDestroy, which frees the buffer this rank exported.
 * Freeing an exported buffer while another process still has it mapped is undefined, and a late
 * store into it can fault that process's GPU: do not skip the barrier.  If a bounded wait ran out
 * (ddShardedPeerStatus reported DD_STATUS_TIMEOUT) a peer may still be running a kernel that
 * stores into this rank's buffer; ddShardedDestroy then does NOT free the exchange buffer (it stays
 * allocated until the process exits).  Without an attached exchange ddShardedDestroy alone is
 * enough. */
DD_API ddStatus_t ddShardedPeerDetach(ddShardedHandle_t sharded);
DD_API ddStatus_t ddShardedDestroy(ddShardedHandle_t sharded);
/* xDesc describes the LOCAL shard; yDesc the (replicated) result.  `spansShardedDim` != 0 says the
 * sharded dim is among the reduced ones, so partial results are combined across ranks; with 0 the
 * call is ddReduceTensor on the local shard.  AVG divides by `globalCount`, the number of elements
 * folded into one output over ALL ranks (for a batch of N images sharded unevenly: N * H * W for a
 * reduction over (N,H,W), whatever this rank's share of N is).  globalCount == 0 means equal
 * shards: nRanks times this rank's own count.  A globalCount smaller than the local count is
 * refused with DD_STATUS_BAD_PARAM.  The other ops do not use it.  A rank whose shard is empty
 * cannot describe it (extents are positive): it must sit the call out, which the peer exchange and
 * NCCL do not allow, so every rank needs at least one batch entry. */
DD_API ddStatus_t ddShardedReduceTensor(ddShardedHandle_t sharded, ddReduceTensorDescriptor_t red,
                                 int spansShardedDim, int64_t globalCount, const void *alpha,
                                 ddTensorDescriptor_t xDesc, const void *x, const void *beta,
                                 ddTensorDescriptor_t yDesc, void *y);
/* Peer exchange: the combine step as ONE kernel per rank over NVLink instead of the NCCL call
 * (no counterpart in the reference).  Every rank calls ddShardedPeerExport (allocates its
 * exchange buffer once and returns a DD_PEER_HANDLE_BYTES handle for other processes of the same
 * box), the caller gathers all ranks' handles in rank order by any transport, and every rank calls
 * ddShardedPeerAttach with the nRanks * DD_PEER_HANDLE_BYTES bytes; from then on
 * ddShardedReduceTensor uses the exchange.  Up to 8 ranks.  ddShardedCreate accepts a NULL id for
 * a handle that only ever uses the peer exchange (no NCCL needed).
 * Two forms.  FUSED: the reduce kernel itself pushes each result to the other ranks the moment it is
 * final, ONE kernel for reduce + exchange.  Where the whole grid of a row reduction is resident at
 * once, the thread that finished an output then also waits (bounded) for the other ranks' values of
 * that output and writes y, so all outputs are collected in parallel; otherwise (<= 4096 outputs)
 * the CTA that finishes last collects them one after the other.  SEPARATE: a small exchange kernel
 * after the local pass.
 * ddShardedPeerConfigure: usePeer 0 = NCCL; 1 = the peer exchange in the form the library prefers
 * (fused when each output is collected where it was finished, else separate; the default);
 * 2 = fused wherever the plan allows; 3 = always separate; -1 = leave as is; and
 * waitSeconds > 0 sets the limit of the kernel's bounded waits (default 2 s).
 * ddShardedPeerStatus synchronises the handle's stream and reports whether a wait ran out
 * (*status = 1 + the rank waited for, return DD_STATUS_TIMEOUT); the kernel that gave up wrote no
 * result, returned normally, and the CUDA context stays usable. */
#define DD_PEER_HANDLE_BYTES 64
DD_API ddStatus_t ddShardedPeerExport(ddShardedHandle_t sharded, void *handle64);
DD_API ddStatus_t ddShardedPeerAttach(ddShardedHandle_t sharded, const void *allHandles);
DD_API ddStatus_t ddShardedPeerConfigure(ddShardedHandle_t sharded, int usePeer, double waitSeconds);
DD_API ddStatus_t ddShardedPeerStatus(ddShardedHandle_t sharded, int *status);
/* Non-blocking health check of the communicator (wraps ncclCommGetAsyncError). */
DD_API ddStatus_t ddShardedCheck(ddShardedHandle_t sharded);

#ifdef __cplusplus
}
#endif
#endif /* DD_B200_H */
