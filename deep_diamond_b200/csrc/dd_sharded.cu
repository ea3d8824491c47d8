// Multi-GPU reduce: one process per GPU, tensors sharded along the batch dim.  A reduction that
// spans the sharded dim = local partial reduce, then the partial results (a few KB) are combined
// across the ranks and finished.  Two ways to combine:
//
//   peer exchange   ONE kernel per rank that pushes its accumulators into every rank's exchange
//                   buffer over NVLink (CUDA IPC mappings) as tagged 8-byte cells, polls its own
//                   buffer for the others' and finishes (dd_reduce_exchange_kernel).  Needs ddShardedPeerExport/Attach; up to
//                   DD_PEER_MAX ranks of one box.
//   NCCL            ncclAllReduce of the partial buffer on the handle's stream, then the finishing
//                   kernel.  NCCL is looked up at run time so that single-GPU users of the library
//                   never need it.
#include "dd_internal.cuh"
#include "dd_reduce_kernels.cuh"

#include <dlfcn.h>
#include <chrono>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <new>
#include <thread>

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

// ncclCommInitRank blocks until every rank has joined and has no limit of its own that a caller
// could set per call.  It therefore runs on a helper thread; the calling thread waits for it with a
// limit.  When the limit passes the helper is left behind (it still owns the state it writes to)
// and the caller gets DD_STATUS_TIMEOUT.
static double g_join_limit_s = 120.0;

struct ddJoinState {
  std::mutex mu;
  std::condition_variable cv;
  bool done = false;
  ncclResult_t result = 0;
  ncclComm_t comm = nullptr;
};

static int bounded_comm_init(int device, int nRanks, int rank, const ncclUniqueId &id, ncclComm_t *comm,
                             ncclResult_t *result) {
  auto st = std::make_shared<ddJoinState>();
  std::thread([st, device, nRanks, rank, id]() {
    ncclComm_t c = nullptr;
    ncclResult_t r = cudaSetDevice(device) == cudaSuccess ? g_nccl.CommInitRank(&c, nRanks, id, rank) : 1;
    std::lock_guard<std::mutex> lock(st->mu);
    st->comm = c;
    st->result = r;
    st->done = true;
    st->cv.notify_all();
  }).detach();
  std::unique_lock<std::mutex> lock(st->mu);
  const bool joined = st->cv.wait_for(lock, std::chrono::duration<double>(g_join_limit_s), [&] { return st->done; });
  if (!joined) return 0;
  *comm = st->comm;
  *result = st->result;
  return 1;
}

struct ddShardedStruct {
  ddHandle_t h;
  ncclComm_t comm;  // NULL: created without an id, peer exchange only
  int nRanks, rank;
  void *partial;    // DD_PARTIAL_BYTES of device memory for the local (NCCL: all-reduced) accumulators
  unsigned char *xbuf;                   // this rank's exchange buffer (DD_PEER_BYTES), NULL until exported
  unsigned char *peerBase[DD_PEER_MAX];  // every rank's exchange buffer as mapped here
  bool peerOpened[DD_PEER_MAX];          // mapped with cudaIpcOpenMemHandle (to be closed)
  bool attached;
  int usePeer;                           // 1: combine over the peer exchange when attached
  int fuse;                              // reduce + exchange in one kernel: 0 never, 1 wherever the plan
                                         // allows, 2 (default) only in the distributed form (each output is
                                         // collected by the thread that finished it)
  unsigned long long waitNs;
};

static_assert(DD_PEER_SLOT_BYTES == 2 * DD_PARTIAL_BYTES, "one slot holds one partial buffer as 8-byte {word, tag} cells");
static_assert(sizeof(cudaIpcMemHandle_t) == DD_PEER_HANDLE_BYTES, "IPC handle size");

extern "C" {

ddStatus_t ddShardedGetUniqueId(void *id128) {
  if (!id128) return DD_STATUS_BAD_PARAM;
  if (!load_nccl()) return DD_STATUS_NOT_INITIALIZED;
  ncclUniqueId id;
  if (g_nccl.GetUniqueId(&id) != 0) return DD_STATUS_COMM_FAILED;
  memcpy(id128, &id, sizeof(id));
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedSetJoinLimit(double seconds) {
  if (!(seconds > 0.0)) return DD_STATUS_BAD_PARAM;
  g_join_limit_s = seconds;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedCreate(ddShardedHandle_t *out, ddHandle_t h, int nRanks, int rank,
                           const void *id128) {
  if (!out || !h) return DD_STATUS_BAD_PARAM;
  *out = nullptr;
  if (nRanks < 1 || rank < 0 || rank >= nRanks) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddShardedCreate: bad rank %d of %d", rank, nRanks);
  if (id128 && !load_nccl()) DD_FAIL(h, DD_STATUS_NOT_INITIALIZED, "ddShardedCreate: libnccl.so.2 not found: %s", dlerror());
  ddShardedStruct *s = new (std::nothrow) ddShardedStruct();
  if (!s) return DD_STATUS_ALLOC_FAILED;
  s->h = h;
  s->nRanks = nRanks;
  s->rank = rank;
  s->comm = nullptr;
  s->partial = nullptr;
  s->xbuf = nullptr;
  for (int i = 0; i < DD_PEER_MAX; i++) {
    s->peerBase[i] = nullptr;
    s->peerOpened[i] = false;
  }
  s->attached = false;
  s->usePeer = 1;
  s->fuse = 2;
  s->waitNs = 2000000000ull;  // 2 s
  if (cudaMalloc(&s->partial, DD_PARTIAL_BYTES) != cudaSuccess) {
    cudaGetLastError();
    delete s;
    DD_FAIL(h, DD_STATUS_ALLOC_FAILED, "ddShardedCreate: cudaMalloc failed");
  }
  if (id128) {
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclResult_t r = 0;
    if (!bounded_comm_init(h->device, nRanks, rank, id, &s->comm, &r)) {
      cudaFree(s->partial);
      delete s;
      DD_FAIL(h, DD_STATUS_TIMEOUT, "ddShardedCreate: not every one of the %d ranks joined within %.0f s", nRanks, g_join_limit_s);
    }
    if (r != 0) {
      cudaFree(s->partial);
      delete s;
      DD_FAIL(h, DD_STATUS_COMM_FAILED, "ncclCommInitRank: %s", g_nccl.GetErrorString(r));
    }
  }
  *out = s;
  return DD_STATUS_SUCCESS;
}

static void peer_detach(ddShardedStruct *s) {
  for (int i = 0; i < DD_PEER_MAX; i++) {
    if (s->peerOpened[i] && s->peerBase[i]) cudaIpcCloseMemHandle(s->peerBase[i]);
    s->peerBase[i] = nullptr;
    s->peerOpened[i] = false;
  }
  s->attached = false;
}

ddStatus_t ddShardedPeerDetach(ddShardedHandle_t s) {
  if (!s) return DD_STATUS_BAD_PARAM;
  if (s->h) cudaStreamSynchronize(s->h->stream);  // no exchange of this rank may still be in flight
  peer_detach(s);
  cudaGetLastError();
  return DD_STATUS_SUCCESS;
}

// Collective when the exchange is attached: every rank detaches, the ranks meet at a host barrier,
// then every rank destroys (see the header).  An exchange buffer whose status word says that a wait
// ran out is not freed: a late peer may still store into it.
ddStatus_t ddShardedDestroy(ddShardedHandle_t s) {
  if (!s) return DD_STATUS_BAD_PARAM;
  if (s->h) cudaStreamSynchronize(s->h->stream);
  peer_detach(s);
  if (s->comm) g_nccl.CommDestroy(s->comm);
  if (s->xbuf) {
    int status = 0;
    if (cudaMemcpy(&status, s->xbuf + 2 * sizeof(unsigned), sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) status = -1;
    if (status == 0) cudaFree(s->xbuf);
  }
  if (s->partial) cudaFree(s->partial);
  cudaGetLastError();
  delete s;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedPeerExport(ddShardedHandle_t s, void *handle64) {
  if (!s || !handle64) return DD_STATUS_BAD_PARAM;
  ddHandle_t h = s->h;
  if (s->nRanks > DD_PEER_MAX)
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddShardedPeerExport: the peer exchange covers up to %d ranks", DD_PEER_MAX);
  if (!s->xbuf) {
    void *p = nullptr;
    if (cudaMalloc(&p, DD_PEER_BYTES) != cudaSuccess) {
      cudaGetLastError();
      DD_FAIL(h, DD_STATUS_ALLOC_FAILED, "ddShardedPeerExport: cudaMalloc failed");
    }
    // control words and every cell's tag start at zero (no call has number 0); finished before
    // anyone can learn the handle
    if (cudaMemset(p, 0, DD_PEER_BYTES) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
      cudaGetLastError();
      cudaFree(p);
      DD_FAIL(h, DD_STATUS_EXECUTION_FAILED, "ddShardedPeerExport: clearing the exchange buffer failed");
    }
    s->xbuf = (unsigned char *)p;
  }
  cudaIpcMemHandle_t ipc;
  cudaError_t e = cudaIpcGetMemHandle(&ipc, s->xbuf);
  if (e != cudaSuccess) {
    cudaGetLastError();
    DD_FAIL(h, DD_STATUS_MAPPING_ERROR, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &ipc, sizeof(ipc));
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedPeerAttach(ddShardedHandle_t s, const void *handles) {
  if (!s || !handles) return DD_STATUS_BAD_PARAM;
  ddHandle_t h = s->h;
  if (!s->xbuf) DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddShardedPeerAttach: call ddShardedPeerExport first");
  if (s->attached) peer_detach(s);
  cudaIpcMemHandle_t own;
  if (cudaIpcGetMemHandle(&own, s->xbuf) != cudaSuccess) {
    cudaGetLastError();
    DD_FAIL(h, DD_STATUS_MAPPING_ERROR, "ddShardedPeerAttach: cudaIpcGetMemHandle failed");
  }
  for (int r = 0; r < s->nRanks; r++) {
    cudaIpcMemHandle_t ipc;
    memcpy(&ipc, (const char *)handles + (size_t)r * sizeof(ipc), sizeof(ipc));
    // an entry that names this rank's own buffer (its own position always does) needs no mapping
    if (r == s->rank || memcmp(&ipc, &own, sizeof(ipc)) == 0) {
      s->peerBase[r] = s->xbuf;
      continue;
    }
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, ipc, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      peer_detach(s);
      DD_FAIL(h, DD_STATUS_MAPPING_ERROR, "cudaIpcOpenMemHandle (rank %d): %s", r, cudaGetErrorString(e));
    }
    s->peerBase[r] = (unsigned char *)p;
    s->peerOpened[r] = true;
  }
  s->attached = true;
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedPeerConfigure(ddShardedHandle_t s, int usePeer, double waitSeconds) {
  if (!s) return DD_STATUS_BAD_PARAM;
  if (usePeer >= 0) {
    s->usePeer = usePeer ? 1 : 0;
    // 1: fused only in its distributed form, else the exchange kernel; 2: fused wherever the plan
    // allows; 3: never fused
    s->fuse = usePeer == 2 ? 1 : (usePeer == 3 ? 0 : 2);
  }
  if (waitSeconds > 0) s->waitNs = (unsigned long long)(waitSeconds * 1e9);
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedPeerStatus(ddShardedHandle_t s, int *status) {
  if (!s || !status) return DD_STATUS_BAD_PARAM;
  *status = 0;
  if (!s->xbuf) return DD_STATUS_SUCCESS;
  ddHandle_t h = s->h;
  cudaError_t e = cudaMemcpyAsync(status, s->xbuf + 2 * sizeof(unsigned), sizeof(int), cudaMemcpyDeviceToHost, h->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    DD_FAIL(h, DD_STATUS_EXECUTION_FAILED, "ddShardedPeerStatus: %s", cudaGetErrorString(e));
  }
  if (*status != 0)
    DD_FAIL(h, DD_STATUS_TIMEOUT, "peer exchange: the wait for rank %d ran out; the exchange buffers are out of step, create a new sharded handle", *status - 1);
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedCheck(ddShardedHandle_t s) {
  if (!s) return DD_STATUS_BAD_PARAM;
  if (!s->comm) return DD_STATUS_SUCCESS;
  ncclResult_t async = 0;
  ncclResult_t r = g_nccl.CommGetAsyncError(s->comm, &async);
  if (r != 0) DD_FAIL(s->h, DD_STATUS_COMM_FAILED, "ncclCommGetAsyncError: %s", g_nccl.GetErrorString(r));
  if (async != 0) DD_FAIL(s->h, DD_STATUS_COMM_FAILED, "communicator error: %s", g_nccl.GetErrorString(async));
  return DD_STATUS_SUCCESS;
}

ddStatus_t ddShardedReduceTensor(ddShardedHandle_t s, ddReduceTensorDescriptor_t red, int spans,
                                 int64_t globalCount, const void *alpha, ddTensorDescriptor_t xd, const void *x,
                                 const void *beta, ddTensorDescriptor_t yd, void *y) {
  DD_RANGE("ddShardedReduceTensor");
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
    case DD_REDUCE_TENSOR_NORM_LP_MAX: case DD_REDUCE_TENSOR_NORM_LP_SUM:
    case DD_REDUCE_TENSOR_NORM_LP_POWER_P_MAX: case DD_REDUCE_TENSOR_NORM_LP_POWER_P_SUM:
      ncclOp = DD_NCCL_SUM; break;
    case DD_REDUCE_TENSOR_MUL: case DD_REDUCE_TENSOR_MUL_NO_ZEROS: ncclOp = DD_NCCL_PROD; break;
    case DD_REDUCE_TENSOR_MIN: ncclOp = DD_NCCL_MIN; break;
    default: ncclOp = DD_NCCL_MAX; break;  // MAX, AMAX
  }
  double a = dd_read_scalar(alpha, xd->dtype), b = dd_read_scalar(beta, yd->dtype);
  if (globalCount < 0 || (globalCount > 0 && globalCount < nredLocal))
    DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddShardedReduceTensor: global count %lld is smaller than this rank's %lld",
            (long long)globalCount, (long long)nredLocal);
  // elements folded into one output over all ranks: given by the caller (uneven shards), or nRanks
  // times the local count (equal shards)
  const double count = globalCount > 0 ? (double)globalCount : (double)nredLocal * s->nRanks;
  const bool peer = s->attached && s->usePeer;
  if (!peer && !s->comm)
    DD_FAIL(h, DD_STATUS_NOT_INITIALIZED, "ddShardedReduceTensor: no NCCL communicator and no peer exchange attached");
  ddStatus_t st;
  if (peer) {
    ddPeerParams q;
    for (int i = 0; i < DD_PEER_MAX; i++) q.base[i] = s->peerBase[i];
    q.partial = s->partial;
    q.world = s->nRanks;
    q.rank = s->rank;
    q.waitNs = s->waitNs;
    if (s->fuse) {
      // fuse == 2 (the default): only the distributed form, which measured faster than the
      // two-kernel form; fuse == 1 (asked for): also the form whose last CTA collects
      bool fused = false;
      st = dd_reduce_fused_exchange_impl(h, red, &q, count, a, xd, x, b, yd, y, s->partial, s->fuse == 2, &fused);
      if (st != DD_STATUS_SUCCESS || fused) return st;
    }
    st = dd_reduce_impl(h, red, nullptr, 0, 1.0, xd, x, 0.0, yd, y, true, s->partial);
    if (st != DD_STATUS_SUCCESS) return st;
    return dd_reduce_exchange_impl(h, red, &q, count, a, b, xd, yd, y);
  }
  st = dd_reduce_impl(h, red, nullptr, 0, 1.0, xd, x, 0.0, yd, y, true, s->partial);
  if (st != DD_STATUS_SUCCESS) return st;
  ncclResult_t r = g_nccl.AllReduce(s->partial, s->partial, (size_t)nout, dbl ? DD_NCCL_FLOAT64 : DD_NCCL_FLOAT32,
                                    ncclOp, s->comm, h->stream);
  if (r != 0) DD_FAIL(h, DD_STATUS_COMM_FAILED, "ncclAllReduce: %s", g_nccl.GetErrorString(r));
  return dd_reduce_finish_impl(h, red, s->partial, count, a, b, xd, yd, y);
}

}  // extern "C"
