// Multi-GPU reduce: one process per GPU, tensors sharded along the batch dim.  A reduction that
// spans the sharded dim = local partial reduce -> ncclAllReduce of the partial buffer on the
// handle's stream -> finishing kernel.  NCCL is looked up at run time so that single-GPU users of
// the library never need it.
#include "dd_internal.cuh"

#include <dlfcn.h>
#include <mutex>
#include <new>

// The handful of NCCL declarations used, spelled out so the build needs no NCCL header.  They
// follow NCCL's public C API (nccl.h): opaque communicator, 128-byte unique id, enum values of
// ncclDataType_t / ncclRedOp_t.
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { DD_NCCL_FLOAT32 = 7, DD_NCCL_FLOAT64 = 8 };
enum { DD_NCCL_SUM = 0, DD_NCCL_PROD = 1, DD_NCCL_MAX = 2, DD_NCCL_MIN = 3 };

struct ddNccl {
  void *lib;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *);
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*CommAbort)(ncclComm_t);
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *);
  ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t);
  const char *(*GetErrorString)(ncclResult_t);
};

static ddNccl g_nccl;
static std::mutex g_nccl_mu;

static bool load_nccl() {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (g_nccl.lib) return true;
  void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return false;
#define DD_SYM(field, name)                                   \
  *(void **)(&g_nccl.field) = dlsym(lib, name);               \
  if (!g_nccl.field) { dlclose(lib); return false; }
  DD_SYM(GetUniqueId, "ncclGetUniqueId")
  DD_SYM(CommInitRank, "ncclCommInitRank")
  DD_SYM(CommDestroy, "ncclCommDestroy")
  DD_SYM(CommAbort, "ncclCommAbort")
  DD_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
  DD_SYM(AllReduce, "ncclAllReduce")
  DD_SYM(GetErrorString, "ncclGetErrorString")
#undef DD_SYM
  g_nccl.lib = lib;
  return true;
}

#define DD_PARTIAL_BYTES (1u << 20)

struct ddShardedStruct {
  ddHandle_t h;
  ncclComm_t comm;
  int nRanks, rank;
  void *partial;  // DD_PARTIAL_BYTES of device memory for the all-reduced accumulators
};

extern "C" {

ddStatus_t ddShardedGetUniqueId(void *id128) {
  if (!id128) return DD_STATUS_BAD_PARAM;
  if (!load_nccl()) return DD_STATUS_NOT_INITIALIZED;
  ncclUniqueId id;
  if (g_nccl.GetUniqueId(&id) != 0) return DD_STATUS_COMM_FAILED;
  memcpy(id128, &id, sizeof(id));
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedCreate(ddShardedHandle_t *out, ddHandle_t h, int nRanks, int rank,
                           const void *id128) {
  if (!out || !h || !id128) return DD_STATUS_BAD_PARAM;
  *out = nullptr;
  if (nRanks < 1 || rank < 0 || rank >= nRanks) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddShardedCreate: bad rank %d of %d", rank, nRanks);
  if (!load_nccl()) DD_FAIL(h, DD_STATUS_NOT_INITIALIZED, "ddShardedCreate: libnccl.so.2 not found: %s", dlerror());
  ddShardedStruct *s = new (std::nothrow) ddShardedStruct();
  if (!s) return DD_STATUS_ALLOC_FAILED;
  s->h = h;
  s->nRanks = nRanks;
  s->rank = rank;
  s->comm = nullptr;
  s->partial = nullptr;
  if (cudaMalloc(&s->partial, DD_PARTIAL_BYTES) != cudaSuccess) {
    cudaGetLastError();
    delete s;
    DD_FAIL(h, DD_STATUS_ALLOC_FAILED, "ddShardedCreate: cudaMalloc failed");
  }
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  ncclResult_t r = g_nccl.CommInitRank(&s->comm, nRanks, id, rank);
  if (r != 0) {
    cudaFree(s->partial);
    delete s;
    DD_FAIL(h, DD_STATUS_COMM_FAILED, "ncclCommInitRank: %s", g_nccl.GetErrorString(r));
  }
  *out = s;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedDestroy(ddShardedHandle_t s) {
  if (!s) return DD_STATUS_BAD_PARAM;
  if (s->comm) g_nccl.CommDestroy(s->comm);
  if (s->partial) cudaFree(s->partial);
  delete s;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedCheck(ddShardedHandle_t s) {
  if (!s) return DD_STATUS_BAD_PARAM;
  ncclResult_t async = 0;
  ncclResult_t r = g_nccl.CommGetAsyncError(s->comm, &async);
  if (r != 0) DD_FAIL(s->h, DD_STATUS_COMM_FAILED, "ncclCommGetAsyncError: %s", g_nccl.GetErrorString(r));
  if (async != 0) DD_FAIL(s->h, DD_STATUS_COMM_FAILED, "communicator error: %s", g_nccl.GetErrorString(async));
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedReduceTensor(ddShardedHandle_t s, ddReduceTensorDescriptor_t red, int spans,
                                 const void *alpha, ddTensorDescriptor_t xd, const void *x,
                                 const void *beta, ddTensorDescriptor_t yd, void *y) {
  if (!s) return DD_STATUS_BAD_PARAM;
  ddHandle_t h = s->h;
  if (!spans || s->nRanks == 1)
    return ddReduceTensor(h, red, nullptr, 0, nullptr, 0, alpha, xd, x, beta, yd, y);
  if (!red || !xd || !yd || !x || !y || !alpha || !beta) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddShardedReduceTensor: null argument");
  if (!xd->set || !yd->set) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddShardedReduceTensor: descriptor not set");
  if (xd->nd != yd->nd) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddShardedReduceTensor: ranks differ");
  int64_t nout = 1, nredLocal = 1;
  for (int i = 0; i < xd->nd; i++) {
    if (yd->dims[i] != xd->dims[i] && yd->dims[i] != 1) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddShardedReduceTensor: bad y dim %d", i);
    if (yd->dims[i] == 1) nredLocal *= xd->dims[i];
    else nout *= xd->dims[i];
  }
  const bool dbl = xd->dtype == DD_DATA_DOUBLE;
  if ((size_t)nout * (dbl ? 8 : 4) > DD_PARTIAL_BYTES)
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddShardedReduceTensor: result too large (%lld elements)", (long long)nout);
  int ncclOp;
  switch (red->op) {
    case DD_REDUCE_TENSOR_ADD: case DD_REDUCE_TENSOR_AVG: case DD_REDUCE_TENSOR_NORM1: case DD_REDUCE_TENSOR_NORM2:
      ncclOp = DD_NCCL_SUM; break;
    case DD_REDUCE_TENSOR_MUL: case DD_REDUCE_TENSOR_MUL_NO_ZEROS: ncclOp = DD_NCCL_PROD; break;
    case DD_REDUCE_TENSOR_MIN: ncclOp = DD_NCCL_MIN; break;
    default: ncclOp = DD_NCCL_MAX; break;  // MAX, AMAX
  }
  double a = dd_read_scalar(alpha, xd->dtype), b = dd_read_scalar(beta, yd->dtype);
  ddStatus_t st = dd_reduce_impl(h, red, nullptr, 0, 1.0, xd, x, 0.0, yd, y, true, s->partial);
  if (st != DD_STATUS_SUCCESS) return st;
  ncclResult_t r = g_nccl.AllReduce(s->partial, s->partial, (size_t)nout, dbl ? DD_NCCL_FLOAT64 : DD_NCCL_FLOAT32,
                                    ncclOp, s->comm, h->stream);
  if (r != 0) DD_FAIL(h, DD_STATUS_COMM_FAILED, "ncclAllReduce: %s", g_nccl.GetErrorString(r));
  // equal shards: the global count is nRanks times the local one
  return dd_reduce_finish_impl(h, red, s->partial, (double)nredLocal * s->nRanks, a, b, xd, yd, y);
}

}  // extern "C"
