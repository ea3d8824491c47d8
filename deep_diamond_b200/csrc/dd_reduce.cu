// ddReduceTensor: host-side planning (which dims are reduced, kernel family, splits, workspace)
// and dispatch.  Kernels are in dd_reduce_kernels.cuh, instantiated per element type in
// dd_reduce_{f32,f64,f16,bf16}.cu.
#include "dd_reduce_kernels.cuh"

static int next_pow2(int64_t v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

ddStatus_t dd_reduce_plan(ddHandle_t h, const ddReduceTensorStruct *red, const ddTensorStruct *xd,
                          const void *x, const ddTensorStruct *yd, ddRedPlan *pl) {
  memset(pl, 0, sizeof(*pl));
  switch (red->op) {
    case DD_REDUCE_TENSOR_ADD: pl->opc = DD_OPC_SUM; pl->p.post = DD_POST_NONE; break;
    case DD_REDUCE_TENSOR_AVG: pl->opc = DD_OPC_SUM; pl->p.post = DD_POST_AVG; break;
    case DD_REDUCE_TENSOR_NORM1: pl->opc = DD_OPC_SUMABS; pl->p.post = DD_POST_NONE; break;
    case DD_REDUCE_TENSOR_NORM2: pl->opc = DD_OPC_SUMSQ; pl->p.post = DD_POST_SQRT; break;
    case DD_REDUCE_TENSOR_MUL: pl->opc = DD_OPC_PROD; pl->p.post = DD_POST_NONE; break;
    case DD_REDUCE_TENSOR_MUL_NO_ZEROS: pl->opc = DD_OPC_PRODNZ; pl->p.post = DD_POST_NONE; break;
    case DD_REDUCE_TENSOR_MIN: pl->opc = DD_OPC_MIN; pl->p.post = DD_POST_NONE; break;
    case DD_REDUCE_TENSOR_MAX: pl->opc = DD_OPC_MAX; pl->p.post = DD_POST_NONE; break;
    case DD_REDUCE_TENSOR_AMAX: pl->opc = DD_OPC_AMAX; pl->p.post = DD_POST_NONE; break;
    default: DD_FAIL(h, DD_STATUS_BAD_PARAM, "reduce: unknown op");
  }
  if (xd->dtype != yd->dtype) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: x and y must share one data type");
  const int esize = dd_type_size(xd->dtype);
  const int csize = xd->dtype == DD_DATA_DOUBLE ? 8 : 4;
  const int V = 16 / esize;

  int64_t st[2][DD_DIM_MAX];
  for (int i = 0; i < xd->nd; i++) {
    st[0][i] = xd->strides[i];
    st[1][i] = (yd->dims[i] == 1 && xd->dims[i] != 1) ? 0 : yd->strides[i];
  }
  ddCanon c;
  dd_canonicalize(&c, xd->nd, xd->dims, 2, st, 0);

  int64_t nout = 1, nred = 1;
  for (int i = 0; i < c.nd; i++) {
    if (c.st[1][i] != 0) nout *= c.dims[i];
    else nred *= c.dims[i];
  }
  if (c.nd == 1 && c.dims[0] == 1) { nout = 1; nred = 1; }
  pl->nout = nout;

  // match x[k1][r1][k2][r2] from the innermost dim outwards
  int slotDim[4] = {-1, -1, -1, -1};  // canonical dim index held by K1, R1, K2, R2
  bool fits = true;
  {
    int slot = 3;
    for (int i = c.nd - 1; i >= 0 && fits; i--) {
      const bool kept = c.st[1][i] != 0;
      // next free slot at or below `slot` of the right kind (odd slots reduce, even slots keep)
      while (slot >= 0 && ((slot & 1) == 1) == kept) slot--;
      if (slot < 0) { fits = false; break; }
      slotDim[slot] = i;
      slot--;
    }
  }
  ddRedParams &p = pl->p;
  auto ext = [&](int s) { return slotDim[s] < 0 ? (int64_t)1 : c.dims[slotDim[s]]; };
  auto sx = [&](int s) { return slotDim[s] < 0 ? (int64_t)0 : c.st[0][slotDim[s]]; };
  auto sy = [&](int s) { return slotDim[s] < 0 ? (int64_t)0 : c.st[1][slotDim[s]]; };
  if (c.nd == 1 && c.dims[0] == 1) { slotDim[0] = slotDim[1] = slotDim[2] = slotDim[3] = -1; fits = true; }
  p.x = x;
  p.K1 = ext(0); p.R1 = ext(1); p.K2 = ext(2); p.R2 = ext(3);
  p.sxK1 = sx(0); p.sxR1 = sx(1); p.sxK2 = sx(2); p.sxR2 = sx(3);
  p.syK1 = sy(0); p.syK2 = sy(2);
  p.count = (double)nred;
  p.nanProp = red->nan == DD_PROPAGATE_NAN;
  p.S = 1;

  const int64_t desired = (int64_t)h->smCount * 6;
  const bool aligned = (((uintptr_t)x) & 15) == 0;
  auto mult = [&](int64_t extent, int64_t stride) { return extent == 1 || stride % V == 0; };

  if (fits && p.R2 > 1 && p.sxR2 == 1 && nred > 32) {
    pl->kind = DD_RED_ROW;
    pl->vec = aligned && p.R2 % V == 0 && mult(p.K1, p.sxK1) && mult(p.R1, p.sxR1) && mult(p.K2, p.sxK2);
    const int v = pl->vec ? V : 1;
    // threads per output: enough lanes to cover one run of R2 in a single pass (so that no lane
    // idles on short runs), a whole CTA for long reductions, a warp for short ones
    // threads per output: the group size whose passes over a run of R2 leave the fewest lanes idle
    // (ties go to the larger group: fewer partials); a warp for short reductions
    {
      int best = 32;
      double bestUse = -1.0;
      for (int gsz = 32; gsz <= 256; gsz *= 2) {
        const int64_t ch = (int64_t)gsz * v;
        const double use = (double)p.R2 / (double)(((p.R2 + ch - 1) / ch) * ch);
        if (use >= bestUse - 1e-9) { bestUse = use > bestUse ? use : bestUse; best = gsz; }
      }
      p.G = nred <= 2048 ? 32 : best;
    }
    const int gpb = 256 / p.G;
    p.CH = (int64_t)p.G * v;
    p.cpr = (p.R2 + p.CH - 1) / p.CH;
    const int64_t want = desired * gpb;
    if (nout < want) {
      int64_t units = p.R1 * p.cpr;
      // once splitting, take the smallest split count whose CTAs fill whole waves of the
      // 4-CTA-per-SM residency (64 registers/thread) to 95 % or better; failing that, the best seen
      const int64_t slots = (int64_t)h->smCount * 4;
      int64_t smax = units / 4;
      if (smax > 64) smax = 64;
      int64_t S = 2;
      double bestEff = -1.0;
      for (int64_t cand = 2; cand <= smax; cand++) {
        const int64_t ctas = (nout * cand + gpb - 1) / gpb;
        if (ctas < slots * 9 / 10) continue;  // less than a wave: keep adding splits
        const double eff = (double)ctas / (double)(((ctas + slots - 1) / slots) * slots);
        if (eff > bestEff + 1e-9) { bestEff = eff; S = cand; }
        if (eff >= 0.95) break;
      }
      if (bestEff < 0.0) S = smax < 2 ? 2 : smax;  // cannot reach a wave at all: as many splits as allowed
      if (S > units / 4) S = units / 4;
      if (S > 1024) S = 1024;
      if (S > 1) {
        if (p.R1 >= S) {
          p.splitR1 = 1;
          int64_t per = (p.R1 + S - 1) / S;
          S = (p.R1 + per - 1) / per;
        } else {
          p.splitR1 = 0;
          if (S > p.cpr) S = p.cpr;
        }
      }
      p.S = S < 1 ? 1 : (int)S;
    }
    int64_t groups = nout * p.S;
    int64_t ctas = (groups + gpb - 1) / gpb;
    if (ctas > 0x7fffffffLL) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: too many outputs");
    pl->grid = (unsigned)ctas;
  } else if (fits && p.R2 == 1 && (p.K2 == 1 || p.sxK2 == 1)) {
    pl->kind = DD_RED_COL;
    pl->vec = aligned && p.K2 % V == 0 && mult(p.K1, p.sxK1) && mult(p.R1, p.sxR1);
    const int v = pl->vec ? V : 1;
    int tx = next_pow2((p.K2 + v - 1) / v);
    p.TX = tx > 32 ? 32 : tx;
    // narrower tiles (down to 8 lanes = 128 contiguous bytes) while that is what it takes to fill
    // the machine without splitting the reduced range
    auto tiles = [&](int t) { return (p.K2 + (int64_t)t * v - 1) / ((int64_t)t * v); };
    while (p.TX > 8 && p.K1 * tiles(p.TX) < desired) p.TX /= 2;
    const int TY = 256 / p.TX;
    p.tilesK2 = tiles(p.TX);
    int64_t ctas0 = p.K1 * p.tilesK2;
    if (ctas0 < desired) {
      int64_t S = (desired + ctas0 - 1) / ctas0;
      int64_t cap = p.R1 / ((int64_t)TY * 4);
      if (S > cap) S = cap;
      if (S > 1024) S = 1024;
      if (S > 1) {
        int64_t per = (p.R1 + S - 1) / S;
        S = (p.R1 + per - 1) / per;
      }
      p.S = S < 1 ? 1 : (int)S;
    }
    int64_t ctas = ctas0 * p.S;
    if (ctas > 0x7fffffffLL) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: too many outputs");
    pl->grid = (unsigned)ctas;
  } else {
    pl->kind = DD_RED_GENERIC;
    ddRedGenericParams &g = pl->g;
    g.x = x;
    g.nk = g.nr = 0;
    for (int i = 0; i < c.nd; i++) {
      if (c.nd == 1 && c.dims[0] == 1) break;
      if (c.st[1][i] != 0) {
        g.kd[g.nk] = c.dims[i]; g.kx[g.nk] = c.st[0][i]; g.ky[g.nk] = c.st[1][i]; g.nk++;
      } else {
        g.rd[g.nr] = c.dims[i]; g.rx[g.nr] = c.st[0][i]; g.nr++;
      }
    }
    g.nout = nout;
    g.nred = nred;
    g.count = (double)nred;
    g.post = p.post;
    g.nanProp = p.nanProp;
    pl->grid = dd_flat_grid(h, nout, 256, 16);
  }
  pl->wsBytes = p.S > 1 ? (size_t)nout * p.S * csize : 0;
  return DD_STATUS_SUCCESS;
}

ddStatus_t dd_reduce_ws_size(ddHandle_t h, const ddReduceTensorStruct *red,
                             const ddTensorStruct *xd, const ddTensorStruct *yd, size_t *bytes) {
  ddRedPlan pl;
  // alignment of x is unknown here: plan as if aligned (the split count does not depend on it
  // beyond the vector width, and an unaligned x only lowers the chunk size, never raises S*nout
  // above what the aligned plan needs ... so take the larger of both plans)
  ddStatus_t st = dd_reduce_plan(h, red, xd, (const void *)0, yd, &pl);
  if (st != DD_STATUS_SUCCESS) return st;
  size_t a = pl.wsBytes;
  st = dd_reduce_plan(h, red, xd, (const void *)4, yd, &pl);
  if (st != DD_STATUS_SUCCESS) return st;
  *bytes = a > pl.wsBytes ? a : pl.wsBytes;
  return DD_STATUS_SUCCESS;
}

static ddStatus_t launch_by_type(ddHandle_t h, ddDataType_t t, const ddRedPlan &pl) {
  switch (t) {
    case DD_DATA_FLOAT: return dd_reduce_launch<float, float>(h, pl);
    case DD_DATA_DOUBLE: return dd_reduce_launch<double, double>(h, pl);
    case DD_DATA_HALF: return dd_reduce_launch<__half, float>(h, pl);
    case DD_DATA_BFLOAT16: return dd_reduce_launch<__nv_bfloat16, float>(h, pl);
    default: break;
  }
  DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: data type must be floating point");
}

ddStatus_t dd_reduce_impl(ddHandle_t h, const ddReduceTensorStruct *red, void *ws, size_t wsBytes,
                          double alpha, const ddTensorStruct *xd, const void *x, double beta,
                          const ddTensorStruct *yd, void *y, bool partialOnly, void *partialOut) {
  ddRedPlan pl;
  ddStatus_t st = dd_reduce_plan(h, red, xd, x, yd, &pl);
  if (st != DD_STATUS_SUCCESS) return st;
  if (partialOnly && pl.kind == DD_RED_GENERIC)
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "sharded reduce: this dim pattern is not supported");
  unsigned *counters = nullptr;
  if (pl.wsBytes > 0) {
    // arrival counters live in the first DD_COUNTER_BYTES of the handle's own scratch (zeroed at
    // ddCreate, reset by the kernels); a context without them (counterSlots == 0) or a reduction with
    // more counters than fit falls back to the separate finishing kernel
    const int64_t nctr = pl.kind == DD_RED_ROW ? pl.nout : pl.p.K1 * pl.p.tilesK2;
    if (h->counterSlots > 0 && nctr < h->counterSlots) counters  /* the last slot belongs to ddCostDiff */ = (unsigned *)h->scratch;
    if (!ws) {
      ws = (char *)h->scratch + h->counterSlots * sizeof(unsigned);
      wsBytes = h->scratchBytes - h->counterSlots * sizeof(unsigned);
    }
    if (wsBytes < pl.wsBytes)
      DD_FAIL(h, DD_STATUS_BAD_PARAM, "reduce: workspace of %zu bytes needed, %zu given", pl.wsBytes, wsBytes);
    if (((uintptr_t)ws) & 7) DD_FAIL(h, DD_STATUS_BAD_PARAM, "reduce: workspace must be 8-byte aligned");
  }
  pl.p.y = y;
  pl.p.part = ws;
  pl.p.partOut = partialOut;
  pl.p.counters = counters;
  pl.p.alpha = alpha;
  pl.p.beta = beta;
  pl.p.partialOnly = partialOnly ? 1 : 0;
  for (int i = 0; i < DD_PEER_MAX; i++) pl.p.peerBase[i] = nullptr;
  pl.p.peerWorld = pl.p.peerRank = 0;
  pl.p.peerWaitNs = 0;
  pl.g.y = y;
  pl.g.partOut = partialOut;
  pl.g.alpha = alpha;
  pl.g.beta = beta;
  pl.g.partialOnly = partialOnly ? 1 : 0;
  return launch_by_type(h, xd->dtype, pl);
}

ddStatus_t dd_reduce_finish_impl(ddHandle_t h, const ddReduceTensorStruct *red, const void *partial,
                                 double count, double alpha, double beta, const ddTensorStruct *xd,
                                 const ddTensorStruct *yd, void *y) {
  ddRedPlan pl;
  ddStatus_t st = dd_reduce_plan(h, red, xd, (const void *)0, yd, &pl);
  if (st != DD_STATUS_SUCCESS) return st;
  if (pl.kind == DD_RED_GENERIC)
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "sharded reduce: this dim pattern is not supported");
  pl.p.y = y;
  pl.p.alpha = alpha;
  pl.p.beta = beta;
  pl.p.count = count;
  switch (xd->dtype) {
    case DD_DATA_FLOAT: return dd_reduce_finish_launch<float, float>(h, pl, partial);
    case DD_DATA_DOUBLE: return dd_reduce_finish_launch<double, double>(h, pl, partial);
    case DD_DATA_HALF: return dd_reduce_finish_launch<__half, float>(h, pl, partial);
    case DD_DATA_BFLOAT16: return dd_reduce_finish_launch<__nv_bfloat16, float>(h, pl, partial);
    default: break;
  }
  DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: data type must be floating point");
}

// Fused form: ONE kernel reduces the local shard, pushes each accumulator to the peers as soon as it
// is final and lets its last CTA collect and finish.  *fused = false (nothing launched) when the plan
// does not allow it: many outputs, or splits that a second kernel would have to combine.
#define DD_PEER_FUSED_MAX_OUT 4096
ddStatus_t dd_reduce_fused_exchange_impl(ddHandle_t h, const ddReduceTensorStruct *red, const ddPeerParams *peer,
                                         double count, double alpha, const ddTensorStruct *xd, const void *x,
                                         double beta, const ddTensorStruct *yd, void *y, void *partialOut,
                                         bool *fused) {
  *fused = false;
  ddRedPlan pl;
  ddStatus_t st = dd_reduce_plan(h, red, xd, x, yd, &pl);
  if (st != DD_STATUS_SUCCESS) return st;
  if (pl.kind == DD_RED_GENERIC || pl.nout > DD_PEER_FUSED_MAX_OUT) return DD_STATUS_SUCCESS;
  unsigned *counters = nullptr;
  void *ws = nullptr;
  if (pl.wsBytes > 0) {
    const int64_t nctr = pl.kind == DD_RED_ROW ? pl.nout : pl.p.K1 * pl.p.tilesK2;
    if (!(h->counterSlots > 0 && nctr < h->counterSlots)) return DD_STATUS_SUCCESS;
    counters = (unsigned *)h->scratch;
    ws = (char *)h->scratch + h->counterSlots * sizeof(unsigned);
    if (h->scratchBytes - h->counterSlots * sizeof(unsigned) < pl.wsBytes) return DD_STATUS_SUCCESS;
  }
  pl.p.y = y;
  pl.p.part = ws;
  pl.p.partOut = partialOut;
  pl.p.counters = counters;
  pl.p.alpha = alpha;
  pl.p.beta = beta;
  pl.p.count = count;
  pl.p.partialOnly = 2;
  for (int i = 0; i < DD_PEER_MAX; i++) pl.p.peerBase[i] = peer->base[i];
  pl.p.peerWorld = peer->world;
  pl.p.peerRank = peer->rank;
  pl.p.peerWaitNs = peer->waitNs;
  *fused = true;
  return launch_by_type(h, xd->dtype, pl);
}

ddStatus_t dd_reduce_exchange_impl(ddHandle_t h, const ddReduceTensorStruct *red, const ddPeerParams *peer,
                                   double count, double alpha, double beta, const ddTensorStruct *xd,
                                   const ddTensorStruct *yd, void *y) {
  ddRedPlan pl;
  ddStatus_t st = dd_reduce_plan(h, red, xd, (const void *)0, yd, &pl);
  if (st != DD_STATUS_SUCCESS) return st;
  if (pl.kind == DD_RED_GENERIC)
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "sharded reduce: this dim pattern is not supported");
  pl.p.y = y;
  pl.p.alpha = alpha;
  pl.p.beta = beta;
  pl.p.count = count;
  switch (xd->dtype) {
    case DD_DATA_FLOAT: return dd_reduce_exchange_launch<float, float>(h, pl, *peer);
    case DD_DATA_DOUBLE: return dd_reduce_exchange_launch<double, double>(h, pl, *peer);
    case DD_DATA_HALF: return dd_reduce_exchange_launch<__half, float>(h, pl, *peer);
    case DD_DATA_BFLOAT16: return dd_reduce_exchange_launch<__nv_bfloat16, float>(h, pl, *peer);
    default: break;
  }
  DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: data type must be floating point");
}

// ------------------------------------------------------------------ no-allocation entry ------
//
// ddReduceTensorNoAlloc: the same planning and the same kernels as ddReduceTensor, for callers
// that must not allocate device memory (no handle, hence no ddCreate and no cudaMalloc).  The
// partial-result workspace is this file-scope device array.  Its name is only a host-side
// stand-in here: the device address is looked up with cudaGetSymbolAddress once per device (with
// that device current) and handed to the kernels like any caller-owned workspace.

#include <mutex>

static __device__ __align__(256) unsigned char dd_static_scratch[DD_NOALLOC_SCRATCH_BYTES];

#define DD_NOALLOC_MAX_DEVICES 64
static std::mutex g_noalloc_mu;
static void *g_noalloc_ptr[DD_NOALLOC_MAX_DEVICES];
static int g_noalloc_sms[DD_NOALLOC_MAX_DEVICES];

static void noalloc_msg(char *buf, size_t len, const char *text) {
  if (buf && len) snprintf(buf, len, "%s", text);
}

extern "C" ddStatus_t ddReduceTensorNoAlloc(void *stream, ddReduceTensorOp_t op, ddNanPropagation_t nanOpt,
                                            const void *alpha, ddTensorDescriptor_t xd, const void *x,
                                            const void *beta, ddTensorDescriptor_t yd, void *y,
                                            char *errbuf, size_t errbufLen) {
  noalloc_msg(errbuf, errbufLen, "");
  if (!alpha || !beta || !x || !y || !xd || !yd || !xd->set || !yd->set) {
    noalloc_msg(errbuf, errbufLen, "ddReduceTensorNoAlloc: null pointer or unset descriptor");
    return DD_STATUS_BAD_PARAM;
  }
  if ((int)op < 0 || (int)op > DD_REDUCE_TENSOR_MUL_NO_ZEROS) {
    noalloc_msg(errbuf, errbufLen, "ddReduceTensorNoAlloc: unknown reduce op");
    return DD_STATUS_BAD_PARAM;
  }
  if (xd->nd != yd->nd) {
    noalloc_msg(errbuf, errbufLen, "ddReduceTensorNoAlloc: x and y ranks differ");
    return DD_STATUS_BAD_PARAM;
  }
  for (int i = 0; i < xd->nd; i++)
    if (yd->dims[i] != xd->dims[i] && yd->dims[i] != 1) {
      noalloc_msg(errbuf, errbufLen, "ddReduceTensorNoAlloc: each y dim must equal x's or be 1");
      return DD_STATUS_BAD_PARAM;
    }
  if (!dd_type_is_float(xd->dtype) || !dd_type_is_float(yd->dtype)) {
    noalloc_msg(errbuf, errbufLen, "ddReduceTensorNoAlloc: data types must be floating point");
    return DD_STATUS_NOT_SUPPORTED;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= DD_NOALLOC_MAX_DEVICES) {
    noalloc_msg(errbuf, errbufLen, "ddReduceTensorNoAlloc: no usable current CUDA device");
    return DD_STATUS_NOT_INITIALIZED;
  }
  void *scratch = nullptr;
  int sms = 0;
  {
    // per-device set-up on the first call made with that device current
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
      void *ptr = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&ptr, dd_static_scratch);
      if (e != cudaSuccess || !ptr) {
        cudaGetLastError();
        if (errbuf && errbufLen)
          snprintf(errbuf, errbufLen, "ddReduceTensorNoAlloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        return DD_STATUS_NOT_INITIALIZED;
      }
      int n = 0;
      e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess || n < 1) {
        cudaGetLastError();
        noalloc_msg(errbuf, errbufLen, "ddReduceTensorNoAlloc: cannot query the device");
        return DD_STATUS_NOT_INITIALIZED;
      }
      g_noalloc_sms[dev] = n;
      g_noalloc_ptr[dev] = ptr;
    }
    scratch = g_noalloc_ptr[dev];
    sms = g_noalloc_sms[dev];
  }
  // a handle-shaped context on the stack: nothing in it is allocated
  ddContext ctx;
  memset(&ctx, 0, sizeof(ctx));
  ctx.device = dev;
  ctx.smCount = sms;
  ctx.stream = (cudaStream_t)stream;
  ctx.scratch = scratch;
  ctx.scratchBytes = DD_NOALLOC_SCRATCH_BYTES;
  ctx.lastKernel = "";
  ddReduceTensorStruct red;
  red.op = op;
  red.comp = xd->dtype == DD_DATA_DOUBLE ? DD_DATA_DOUBLE : DD_DATA_FLOAT;
  red.nan = nanOpt;
  ddRedPlan pl;
  ddStatus_t st = dd_reduce_plan(&ctx, &red, xd, x, yd, &pl);
  if (st == DD_STATUS_SUCCESS && pl.wsBytes > DD_NOALLOC_SCRATCH_BYTES) {
    if (errbuf && errbufLen)
      snprintf(errbuf, errbufLen,
               "ddReduceTensorNoAlloc: this reduction needs %zu bytes of scratch, the built-in array holds %u; "
               "use ddReduceTensor with a caller-owned workspace",
               pl.wsBytes, (unsigned)DD_NOALLOC_SCRATCH_BYTES);
    return DD_STATUS_NOT_SUPPORTED;
  }
  if (st == DD_STATUS_SUCCESS)
    st = dd_reduce_impl(&ctx, &red, scratch, DD_NOALLOC_SCRATCH_BYTES, dd_read_scalar(alpha, xd->dtype), xd, x,
                        dd_read_scalar(beta, yd->dtype), yd, y, false, nullptr);
  if (st != DD_STATUS_SUCCESS) noalloc_msg(errbuf, errbufLen, ctx.msg);
  return st;
}
