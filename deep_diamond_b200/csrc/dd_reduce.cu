// ddReduceTensor: host-side planning (which dims are reduced, kernel family, splits, workspace)
// and dispatch.  Kernels are in dd_reduce_kernels.cuh, instantiated per element type in
// dd_reduce_{f32,f64,f16,bf16}.cu.
#include "dd_reduce_kernels.cuh"

static int next_pow2(int64_t v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

// flags: DD_PLAN_STRUCTURED: the caller needs the x[k1][r1][k2][r2] form (the sharded path addresses partial
// results by (k1, k2)), so short reductions, which otherwise run one thread per output, take the
// row kernel with warp-sized groups.  DD_PLAN_NO_CLUSTER: splits of the col kernel go through the
// counter protocol (the fused cross-GPU form pushes from the CTA that folds the partials).
ddStatus_t dd_reduce_plan(ddHandle_t h, const ddReduceTensorStruct *red, const ddTensorStruct *xd,
                          const void *x, const ddTensorStruct *yd, ddRedPlan *pl, int flags) {
  const bool structured = (flags & DD_PLAN_STRUCTURED) != 0;
  memset(pl, 0, sizeof(*pl));
  pl->bs = 256;
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
    case DD_REDUCE_TENSOR_NORM_LP_MAX: case DD_REDUCE_TENSOR_NORM_LP_SUM:
    case DD_REDUCE_TENSOR_NORM_LP_POWER_P_MAX: case DD_REDUCE_TENSOR_NORM_LP_POWER_P_SUM:
      // sum of |x|^p: p = 1 and p = 2 are the NORM1 / NORM2 accumulations, any other p goes through pow
      if (!(red->p >= 1.0)) DD_FAIL(h, DD_STATUS_BAD_PARAM, "reduce: the norm's p must be at least 1");
      pl->opc = red->p == 1.0 ? DD_OPC_SUMABS : (red->p == 2.0 ? DD_OPC_SUMSQ : DD_OPC_SUMPOW);
      pl->p.post = DD_POST_LP;
      pl->p.lpP = red->p;
      pl->p.lpEps = red->eps;
      pl->p.lpMax = red->op == DD_REDUCE_TENSOR_NORM_LP_MAX || red->op == DD_REDUCE_TENSOR_NORM_LP_POWER_P_MAX;
      pl->p.lpRoot = red->op == DD_REDUCE_TENSOR_NORM_LP_MAX || red->op == DD_REDUCE_TENSOR_NORM_LP_SUM;
      break;
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
  auto mult4 = [&](int64_t extent, int64_t stride) { return extent == 1 || stride % 4 == 0; };
  // the 8-byte form: 16-bit elements, base on an 8-byte boundary, innermost extent a multiple of 4;
  // not for the plans of the cross-GPU paths (their kernels are built for 16-byte or element loads)
  auto half8 = [&](int64_t inner) {
    return esize == 2 && !structured && (((uintptr_t)x) & 7) == 0 && inner % 4 == 0 && dd_tune("DD_RED_VEC8", 1);
  };

  if (fits && p.R2 > 1 && p.sxR2 == 1 && (nred > 32 || structured)) {
    pl->kind = DD_RED_ROW;
    // one long contiguous run per output (norm over (C,H,W) of an nchw tensor): read it as rows of
    // 256 16-byte vectors, so that splits take whole rows and the lean kernel applies
    if (dd_tune("DD_ROW_FOLD", 1) && p.R1 == 1 && aligned && p.R2 % (256 * V) == 0 && p.R2 / (256 * V) >= 8) {
      p.R1 = p.R2 / (256 * V);
      p.R2 = 256 * V;
      p.sxR1 = p.R2;
    }
    pl->vec = aligned && p.R2 % V == 0 && mult(p.K1, p.sxK1) && mult(p.R1, p.sxR1) && mult(p.K2, p.sxK2);
    // 16-bit types whose runs start on 8-byte boundaries only (196-long runs: 14 x 14 maps): 8-byte loads
    if (!pl->vec && half8(p.R2) && mult4(p.K1, p.sxK1) && mult4(p.R1, p.sxR1) && mult4(p.K2, p.sxK2)) pl->vec = 2;
    const int v = pl->vec == 1 ? V : (pl->vec == 2 ? 4 : 1);
    // Threads per output (G) and per CTA (bs).  A group passes over a run of R2 in chunks of G
    // 16-byte vectors; the lean kernel (8 loads in flight per thread) takes plans with at most 4
    // chunks per run.  Score = the share of lanes that a pass keeps busy, times 1.25 when the lean
    // kernel applies (it measured 8-25 % faster than the general walk at equal lane use); ties go to
    // the larger group (fewer groups, fewer partials).  One exception to the tie rule: when every
    // group of 128 fits one resident wave of 128-thread CTAs, groups of 256 would not, and a thread
    // of the smaller group still has at most 32 loads to do, the smaller group wins (the whole
    // reduction is then two to four round trips to memory with every CTA on the machine at once).
    {
      auto cprOf = [&](int gsz) { return (p.R2 + (int64_t)gsz * v - 1) / ((int64_t)gsz * v); };
      auto leanOk = [&](int gsz) { return pl->vec == 1 && cprOf(gsz) <= 4 && p.R1 < 0x7fffffffLL; };
      int best = 32;
      double bestScore = -1.0;
      for (int gsz = 256; gsz >= 32; gsz /= 2) {
        const int64_t ch = (int64_t)gsz * v;
        const double use = (double)p.R2 / (double)(cprOf(gsz) * ch);
        const double score = use * (leanOk(gsz) ? 1.25 : 1.0);
        if (score > bestScore + 1e-9) { bestScore = score; best = gsz; }
      }
      if (best == 256 && leanOk(128) && cprOf(128) == 2 * cprOf(256) &&
          nout <= (int64_t)h->smCount * 8 && nout > (int64_t)h->smCount * 4 && p.R1 * cprOf(128) <= 32)
        best = 128;
      // Too few outputs to fill the machine even with the best group size: splits are due anyway.
      // With 128 outputs or more the smallest group that ties on the score measured fastest (f32
      // 784-long runs, 256 outputs: 64 lanes 0.92 of the copy rate, 128 lanes 0.89, 256 lanes 0.75;
      // bf16: 32 lanes 0.77, 64 lanes 0.64); with fewer outputs (one output takes tens of splits)
      // the largest did (1024-long runs, 8 outputs: 256 lanes 10.5 us, 128 lanes 12.0, 64 lanes 13.8).
      if (nout * best < (int64_t)h->smCount * 1024 * 4 / 5 && nout >= 128) {
        const int lo = dd_tune("DD_ROW_GMIN", 32);
        for (int gsz = lo; gsz < best; gsz *= 2)
          if (leanOk(gsz) && cprOf(gsz) * gsz == cprOf(best) * best) { best = gsz; break; }
      }
      p.G = nred <= 2048 ? 32 : best;
    }
    p.G = dd_tune("DD_ROW_G", p.G);
    // 128-thread CTAs for groups of 128 or fewer lanes (finer grain: 8 resident CTAs per SM)
    pl->bs = dd_tune("DD_ROW_BS", (p.G <= 128 && nred > 2048) ? 128 : 256);
    if (pl->bs < p.G) pl->bs = p.G;
    const int gpb = pl->bs / p.G;
    p.CH = (int64_t)p.G * v;
    p.cpr = (p.R2 + p.CH - 1) / p.CH;
    // groups wanted before an output's range is split: 6 CTAs of 256 threads per SM, or, with
    // 128-thread CTAs, four fifths of one resident wave (1024 threads per SM at 64 registers): a split
    // costs a partial store, a fence, an atomic and a fold by the last arrival, about 3 us
    const int64_t want = pl->bs == 128 ? ((int64_t)h->smCount * 1024 * 4 / 5) / p.G : desired * gpb;
    if (nout < want || dd_tune("DD_ROW_S", 0) > 1) {
      int64_t units = p.R1 * p.cpr;
      const int64_t slots = (int64_t)h->smCount * (1024 / pl->bs);
      int64_t smax = units / 4;
      if (smax > 1024) smax = 1024;
      int64_t S = 0;
      // first choice: ONE resident wave, as full as the split count allows and at least four fifths
      // full (one wave of long-running threads measured faster than several waves of short ones, and
      // 1152 CTAs in 1184 slots faster than 1024)
      {
        int64_t cand = slots * gpb / (nout > 0 ? nout : 1);
        if (cand > smax) cand = smax;
        if (cand >= 1 && (nout * cand + gpb - 1) / gpb >= slots * 4 / 5) S = cand;
      }
      if (S == 0) {
        // none lands in one wave: the smallest split count whose CTAs fill whole waves to 95 % or
        // better, failing that the best seen
        double bestEff = -1.0;
        for (int64_t cand = 2; cand <= smax; cand++) {
          const int64_t ctas = (nout * cand + gpb - 1) / gpb;
          if (ctas < slots * 9 / 10) continue;
          const double eff = (double)ctas / (double)(((ctas + slots - 1) / slots) * slots);
          if (eff > bestEff + 1e-9) { bestEff = eff; S = cand; }
          if (eff >= 0.95) break;
        }
      }
      if (S == 0) S = smax < 2 ? 2 : smax;  // cannot reach a wave at all: as many splits as allowed
      if (S > units / 4) S = units / 4;
      if (S > 1024) S = 1024;
      S = dd_tune("DD_ROW_S", (int)S);
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
    // the lean kernel (8 loads in flight per thread) where the plan allows it
    if (dd_tune("DD_ROW_LEAN", 1) && pl->vec == 1 && (p.S == 1 || p.splitR1) && p.cpr <= 4 && p.R1 < 0x7fffffffLL)
      pl->lean = p.cpr == 3 ? 4 : (int)p.cpr;
    // A few hundred outputs whose splits fit one resident wave as clusters of 2, 4 or 8 CTAs (sum over
    // (N,H,W) of a [256,256,28,28] tensor: 256 outputs, clusters of 4): the splits of an output are the
    // gpb groups of each CTA of its cluster and are combined through distributed shared memory
    // instead of the counter protocol.
    // Measured on [N,256,28,28]: bf16 / f16 3-6 % faster than the counters at 51 and 103 MB, equal at
    // 205 MB; f32 equal to 6 % slower (its groups of 64 lanes make 8 splits where the counter plan
    // has 9, a less full wave), so 16-bit types only.
    if (pl->lean && p.S > 1 && p.splitR1 && pl->bs == 128 && !structured && !(flags & DD_PLAN_NO_CLUSTER) &&
        dd_tune("DD_ROW_CLUSTER", esize == 2 ? 1 : 0)) {
      const int64_t slots = (int64_t)h->smCount * 8;
      int cs = 0;
      for (int cand = 8; cand >= 2; cand /= 2)
        if (nout * cand <= slots) { cs = cand; break; }
      cs = dd_tune("DD_ROW_CS", cs);
      if (cs >= 2 && cs <= 8 && nout * cs >= slots * 3 / 5 && p.R1 / ((int64_t)gpb * cs) >= 4) {
        pl->cluster = 1;
        p.rowCluster = cs;
        p.S = gpb * cs;
      }
    }
    int64_t groups = nout * p.S;
    int64_t ctas = (groups + gpb - 1) / gpb;
    if (ctas > 0x7fffffffLL) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: too many outputs");
    pl->grid = (unsigned)ctas;
  } else if (fits && p.R2 == 1 && (p.K2 == 1 || p.sxK2 == 1)) {
    pl->kind = DD_RED_COL;
    pl->vec = aligned && p.K2 % V == 0 && mult(p.K1, p.sxK1) && mult(p.R1, p.sxR1);
    if (!pl->vec && half8(p.K2) && mult4(p.K1, p.sxK1) && mult4(p.R1, p.sxR1)) pl->vec = 2;
    const int v = pl->vec == 1 ? V : (pl->vec == 2 ? 4 : 1);
    int tx = next_pow2((p.K2 + v - 1) / v);
    p.TX = tx > 32 ? 32 : tx;
    const int txMin = dd_tune("DD_COL_TXMIN", 8);
    pl->pdl = dd_tune("DD_COL_PDL", 0);
    // narrower tiles (down to 8 lanes = 128 contiguous bytes) while that is what it takes to fill
    // the machine without splitting the reduced range
    auto tiles = [&](int t) { return (p.K2 + (int64_t)t * v - 1) / ((int64_t)t * v); };
    while (p.TX > txMin && p.K1 * tiles(p.TX) < desired) p.TX /= 2;
    // ... and narrower still while that cuts the padding of the last tile along k2 by a twentieth or
    // more of the lanes (784 elements: 32 lanes of 16 bytes leave a quarter of the bf16 lanes idle)
    if (dd_tune("DD_COL_PAD", esize >= 4 ? 1 : 0)) {  // (16-bit types measured slower with the narrower tiles)
      auto laneUse = [&](int t) { return (double)p.K2 / (double)(tiles(t) * t * v); };
      while (p.TX > txMin && laneUse(p.TX / 2) > laneUse(p.TX) + 0.05) p.TX /= 2;
    }
    p.TX = dd_tune("DD_COL_TX", p.TX);
    const int TY = 256 / p.TX;
    p.tilesK2 = tiles(p.TX);
    int64_t ctas0 = p.K1 * p.tilesK2;
    // Too few tiles to fill the machine: split r1 (when the range is long enough to be worth it).
    if (ctas0 < desired) {
      int64_t S = (desired + ctas0 - 1) / ctas0;
      int64_t cap = p.R1 / ((int64_t)TY * 4);
      if (S > cap) S = cap;
      if (S > 1024) S = 1024;
      S = dd_tune("DD_COL_S", (int)S);
      if (S > 1) {
        int64_t per = (p.R1 + S - 1) / S;
        S = (p.R1 + per - 1) / per;
      }
      p.S = S < 1 ? 1 : (int)S;
    }
    // Where a split is due and 2, 4 or 8 splits give at least a quarter of a resident wave of 128-thread
    // CTAs, the splits of a tile form a thread-block cluster and combine through distributed shared
    // memory (dd_reduce_colc_kernel): 256-byte runs along k2 (16 lanes), 8 row groups per CTA.  The
    // fused cross-GPU form keeps the counter protocol.
    if (p.S > 1 && pl->vec == 1 && !(flags & DD_PLAN_NO_CLUSTER) && dd_tune("DD_COL_CLUSTER", 1)) {
      int txc = next_pow2((p.K2 + v - 1) / v);
      if (txc > 16) txc = 16;
      const int tyc = DD_COLC_THREADS / txc;
      const int64_t tilesC = (p.K2 + (int64_t)txc * v - 1) / ((int64_t)txc * v);
      const int64_t base = p.K1 * tilesC;
      const int64_t wave = (int64_t)h->smCount * 8;
      int sc = 2;
      while (sc < 8 && base * sc < wave * 4 / 5) sc *= 2;
      while (sc > 1 && p.R1 / ((int64_t)sc * tyc) < 1) sc /= 2;
      sc = dd_tune("DD_COL_SC", sc);
      if (sc >= 2 && sc <= 8 && base * sc >= wave / 4 && base * sc <= 0x7fffffffLL) {
        pl->cluster = 1;
        p.TX = txc;
        p.tilesK2 = tilesC;
        p.S = sc;
        ctas0 = base;
      }
    }
    // 16-bit element types without a split: the same lean kernel, no cluster.  The general kernel
    // keeps 8 accumulators and 4 loads of 8 elements per thread in 64 registers at 4 CTAs per SM;
    // the lean one runs 8 CTAs of 128 threads with 8 loads each.  Lanes along k2: 8 to 16, the count
    // that pads the last tile least (784 elements = 98 vectors: 14 lanes, 7 tiles).
    if (p.S == 1 && !pl->cluster && pl->vec == 1 && esize == 2 && !(flags & DD_PLAN_NO_CLUSTER) &&
        dd_tune("DD_COL_LEAN16", 1)) {
      const int64_t vecs = p.K2 / v;
      int txc = 16;
      double bestUse = -1.0;
      for (int cand = 16; cand >= 8; cand--) {
        const double use = (double)vecs / (double)(((vecs + cand - 1) / cand) * cand);
        if (use > bestUse + 1e-9) { bestUse = use; txc = cand; }
      }
      if (vecs < 8) txc = (int)vecs;
      txc = dd_tune("DD_COL_TX16", txc);
      const int tyc = DD_COLC_THREADS / txc;
      const int64_t tilesC = (vecs + txc - 1) / txc;
      if (p.R1 / tyc >= 8 && p.K1 * tilesC >= (int64_t)h->smCount * 4 && p.K1 * tilesC <= 0x7fffffffLL) {
        pl->cluster = 1;
        p.TX = txc;
        p.tilesK2 = tilesC;
        ctas0 = p.K1 * tilesC;
      }
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
    g.lpP = p.lpP; g.lpEps = p.lpEps; g.lpMax = p.lpMax; g.lpRoot = p.lpRoot;
    g.nanProp = p.nanProp;
    pl->grid = dd_flat_grid(h, nout, 256, 16);
  }
  pl->wsBytes = (p.S > 1 && !pl->cluster) ? (size_t)nout * p.S * csize : 0;
  if (dd_tune("DD_PLAN_DEBUG", 0))
    fprintf(stderr, "[dd plan] kind %d vec %d lean %d cluster %d bs %d G %d S %d splitR1 %d cpr %lld TX %d tiles %lld grid %u | K1 %lld R1 %lld K2 %lld R2 %lld\n",
            pl->kind, pl->vec, pl->lean, pl->cluster, pl->bs, p.G, p.S, p.splitR1, (long long)p.cpr, p.TX,
            (long long)p.tilesK2, pl->grid, (long long)p.K1, (long long)p.R1, (long long)p.K2, (long long)p.R2);
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
  // ... and of the plans for a base that is 8-byte aligned only (8-byte loads for 16-bit types) and
  // for one that is not even that (element loads)
  st = dd_reduce_plan(h, red, xd, (const void *)8, yd, &pl);
  if (st != DD_STATUS_SUCCESS) return st;
  a = a > pl.wsBytes ? a : pl.wsBytes;
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

// Reductions over (outer dim, innermost runs) whose runs are NOT vector-aligned -- the per-channel
// sum of an nchw tensor with 7 x 7 or 13 x 13 maps, which is also the bias gradient of such a layer:
// x[r1][k2][r2] dense, r2 odd.  The row kernel would walk the runs with element loads (0.13-0.24 of
// the copy rate measured on [512,1024,7,7]).  The whole block of one r1 is contiguous and a whole
// number of 16-byte vectors though, so the work is done in two launches instead: a column reduce
// over r1 that treats (k2, r2) as one kept dim of k2 * r2 elements (16-byte loads, raw accumulators
// into the handle's scratch), then the finishing kernel folding the r2 accumulators of each k2 in
// index order and applying the post-operation, alpha and beta.  *done = false: not this case, nothing
// launched.
static ddStatus_t dd_reduce_two_stage(ddHandle_t h, const ddReduceTensorStruct *red, const ddRedPlan &pl,
                                      double alpha, const ddTensorStruct *xd, const void *x, double beta,
                                      void *y, bool *done) {
  *done = false;
  const ddRedParams &p = pl.p;
  // (a real handle only: the entry point without one has 64 KiB of scratch and keeps to one launch plan)
  if (!dd_tune("DD_RED_TWO_STAGE", 1) || pl.kind != DD_RED_ROW || pl.vec == 1 || !h->scratch || h->counterSlots == 0)
    return DD_STATUS_SUCCESS;
  const int esize = dd_type_size(xd->dtype);
  const int V = 16 / esize;
  const int csize = xd->dtype == DD_DATA_DOUBLE ? 8 : 4;
  const int64_t inner = p.K2 * p.R2;
  if (p.K1 != 1 || p.R1 < 8 || p.R2 < 2 || p.R2 > 4096 || p.sxR2 != 1 || (p.K2 > 1 && p.sxK2 != p.R2) ||
      p.sxR1 != inner || inner % V != 0 || (((uintptr_t)x) & 15) || inner >= (1LL << 31))
    return DD_STATUS_SUCCESS;
  // stage 1 as a reduction of the [R1, inner] matrix over its first dim
  ddTensorStruct x1 = *xd, y1 = *xd;
  x1.nd = y1.nd = 2;
  x1.dims[0] = p.R1; x1.dims[1] = inner; x1.strides[0] = inner; x1.strides[1] = 1;
  y1.dims[0] = 1; y1.dims[1] = inner; y1.strides[0] = inner; y1.strides[1] = 1;
  ddRedPlan p1;
  ddStatus_t st = dd_reduce_plan(h, red, &x1, x, &y1, &p1, DD_PLAN_STRUCTURED);
  if (st != DD_STATUS_SUCCESS || p1.kind != DD_RED_COL || p1.vec != 1) return DD_STATUS_SUCCESS;
  const size_t tempBytes = (((size_t)inner * csize) + 255) & ~(size_t)255;
  const size_t ctrBytes = h->counterSlots * sizeof(unsigned);
  if (h->scratchBytes < ctrBytes + p1.wsBytes + tempBytes + 256) return DD_STATUS_SUCCESS;
  void *temp = (char *)h->scratch + h->scratchBytes - tempBytes;  // stage 1's own partials sit at the front
  st = dd_reduce_impl(h, red, nullptr, 0, 1.0, &x1, x, 0.0, &y1, nullptr, /*partialOnly=*/true, temp);
  if (st != DD_STATUS_SUCCESS) return st;
  ddRedPlan p2 = pl;  // the outputs, post-operation and count of the whole reduction
  p2.foldS = (int)p.R2;
  p2.p.y = y;
  p2.p.alpha = alpha;
  p2.p.beta = beta;
  p2.p.partOut = nullptr;
  p2.p.counters = nullptr;
  p2.p.peerDistributed = 0;
  switch (xd->dtype) {
    case DD_DATA_FLOAT: st = dd_reduce_finish_launch<float, float>(h, p2, temp); break;
    case DD_DATA_DOUBLE: st = dd_reduce_finish_launch<double, double>(h, p2, temp); break;
    case DD_DATA_HALF: st = dd_reduce_finish_launch<__half, float>(h, p2, temp); break;
    case DD_DATA_BFLOAT16: st = dd_reduce_finish_launch<__nv_bfloat16, float>(h, p2, temp); break;
    default: DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: data type must be floating point");
  }
  *done = st == DD_STATUS_SUCCESS;
  return st;
}

static ddStatus_t finish_by_type(ddHandle_t h, ddDataType_t t, const ddRedPlan &pl, const void *part) {
  switch (t) {
    case DD_DATA_FLOAT: return dd_reduce_finish_launch<float, float>(h, pl, part);
    case DD_DATA_DOUBLE: return dd_reduce_finish_launch<double, double>(h, pl, part);
    case DD_DATA_HALF: return dd_reduce_finish_launch<__half, float>(h, pl, part);
    case DD_DATA_BFLOAT16: return dd_reduce_finish_launch<__nv_bfloat16, float>(h, pl, part);
    default: break;
  }
  DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: data type must be floating point");
}

// Column reductions (reduce across a strided dim, innermost kept: max over C of an nchw tensor) whose
// kept rows are NOT whole vectors (7 x 7 maps: 49 elements) but follow one another densely:
// x[k1][r1][k2], sxR1 == K2.  P = V / gcd(K2, V) consecutive rows together are a whole number of
// vectors, so the reduction runs over r1 / P with P * K2 kept elements (16-byte loads; element
// j * K2 + k2 of a kept row belongs to output k2 and to the rows r1 = j mod P), raw accumulators into
// the handle's scratch, and a second launch folds the P sets.  *done = false: not this case.
static ddStatus_t dd_reduce_col_periodic(ddHandle_t h, const ddReduceTensorStruct *red, const ddRedPlan &pl,
                                         double alpha, const ddTensorStruct *xd, const void *x, double beta,
                                         void *y, bool *done) {
  *done = false;
  const ddRedParams &p = pl.p;
  if (!dd_tune("DD_RED_PERIODIC", 1) || pl.kind != DD_RED_COL || pl.vec == 1 || !h->scratch || h->counterSlots == 0)
    return DD_STATUS_SUCCESS;
  const int esize = dd_type_size(xd->dtype);
  const int V = 16 / esize;
  const int csize = xd->dtype == DD_DATA_DOUBLE ? 8 : 4;
  int g = V;
  for (int64_t a = p.K2 % V; a;) { int64_t t = g % a; g = (int)a; a = t; }  // gcd(K2, V)
  const int P = V / g;
  if (P < 2 || p.K2 < 2 || p.sxK2 != 1 || p.sxR1 != p.K2 || p.R1 % P != 0 || p.R1 / P < 8 ||
      (p.K1 > 1 && p.sxK1 % V != 0) || (((uintptr_t)x) & 15) || p.K1 * P * p.K2 >= (1LL << 31))
    return DD_STATUS_SUCCESS;
  ddTensorStruct x1 = *xd, y1 = *xd;
  x1.nd = y1.nd = 3;
  x1.dims[0] = p.K1; x1.dims[1] = p.R1 / P; x1.dims[2] = P * p.K2;
  x1.strides[0] = p.K1 > 1 ? p.sxK1 : p.R1 * p.K2; x1.strides[1] = P * p.K2; x1.strides[2] = 1;
  y1.dims[0] = p.K1; y1.dims[1] = 1; y1.dims[2] = P * p.K2;
  y1.strides[0] = P * p.K2; y1.strides[1] = P * p.K2; y1.strides[2] = 1;
  ddRedPlan p1;
  ddStatus_t st = dd_reduce_plan(h, red, &x1, x, &y1, &p1, DD_PLAN_STRUCTURED);
  if (st != DD_STATUS_SUCCESS || p1.kind != DD_RED_COL || p1.vec != 1) return DD_STATUS_SUCCESS;
  const size_t tempBytes = (((size_t)(p.K1 * P * p.K2) * csize) + 255) & ~(size_t)255;
  const size_t ctrBytes = h->counterSlots * sizeof(unsigned);
  if (h->scratchBytes < ctrBytes + p1.wsBytes + tempBytes + 256) return DD_STATUS_SUCCESS;
  void *temp = (char *)h->scratch + h->scratchBytes - tempBytes;
  st = dd_reduce_impl(h, red, nullptr, 0, 1.0, &x1, x, 0.0, &y1, nullptr, /*partialOnly=*/true, temp);
  if (st != DD_STATUS_SUCCESS) return st;
  ddRedPlan p2 = pl;
  p2.foldS = -P;
  p2.p.y = y;
  p2.p.alpha = alpha;
  p2.p.beta = beta;
  p2.p.partOut = nullptr;
  p2.p.counters = nullptr;
  p2.p.peerDistributed = 0;
  st = finish_by_type(h, xd->dtype, p2, temp);
  *done = st == DD_STATUS_SUCCESS;
  return st;
}

ddStatus_t dd_reduce_impl(ddHandle_t h, const ddReduceTensorStruct *red, void *ws, size_t wsBytes,
                          double alpha, const ddTensorStruct *xd, const void *x, double beta,
                          const ddTensorStruct *yd, void *y, bool partialOnly, void *partialOut) {
  ddRedPlan pl;
  ddStatus_t st = dd_reduce_plan(h, red, xd, x, yd, &pl, partialOnly ? DD_PLAN_STRUCTURED : 0);
  if (st != DD_STATUS_SUCCESS) return st;
  if (partialOnly && pl.kind == DD_RED_GENERIC)
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "sharded reduce: this dim pattern is not supported");
  if (!partialOnly) {
    bool done = false;
    st = dd_reduce_two_stage(h, red, pl, alpha, xd, x, beta, y, &done);
    if (st != DD_STATUS_SUCCESS || done) return st;
    st = dd_reduce_col_periodic(h, red, pl, alpha, xd, x, beta, y, &done);
    if (st != DD_STATUS_SUCCESS || done) return st;
  }
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
  pl.p.peerDistributed = 0;
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
  ddStatus_t st = dd_reduce_plan(h, red, xd, (const void *)0, yd, &pl, DD_PLAN_STRUCTURED);
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

// Fused form: ONE kernel reduces the local shard and pushes each accumulator to the peers as soon as
// it is final.  Who collects depends on the plan.  Row kernels whose whole grid is resident at once:
// the thread that finished an output also waits for the other ranks' values of THAT output and
// writes y ("distributed": the waits of all outputs run in parallel, and every rank's CTAs push
// before they wait, so no wait depends on a CTA that is not running yet).  Otherwise the CTA that
// finishes last collects every output (at most DD_PEER_FUSED_MAX_OUT of them).
// *fused = false (nothing launched) when the plan does not allow the form asked for; `onlyDistributed`
// restricts it to the first kind.
#define DD_PEER_FUSED_MAX_OUT 4096
ddStatus_t dd_reduce_fused_exchange_impl(ddHandle_t h, const ddReduceTensorStruct *red, const ddPeerParams *peer,
                                         double count, double alpha, const ddTensorStruct *xd, const void *x,
                                         double beta, const ddTensorStruct *yd, void *y, void *partialOut,
                                         bool onlyDistributed, bool *fused) {
  *fused = false;
  ddRedPlan pl;
  ddStatus_t st = dd_reduce_plan(h, red, xd, x, yd, &pl, DD_PLAN_STRUCTURED | DD_PLAN_NO_CLUSTER);
  if (st != DD_STATUS_SUCCESS) return st;
  if (pl.kind == DD_RED_GENERIC) return DD_STATUS_SUCCESS;
  // resident CTAs per SM of the fused row kernels: 64 registers per thread (__launch_bounds__(256, 4))
  const bool distributed = pl.kind == DD_RED_ROW && (int64_t)pl.grid <= (int64_t)h->smCount * (1024 / pl.bs);
  if (!distributed && (onlyDistributed || pl.nout > DD_PEER_FUSED_MAX_OUT)) return DD_STATUS_SUCCESS;
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
  pl.p.peerDistributed = distributed ? 1 : 0;
  *fused = true;
  return launch_by_type(h, xd->dtype, pl);
}

ddStatus_t dd_reduce_exchange_impl(ddHandle_t h, const ddReduceTensorStruct *red, const ddPeerParams *peer,
                                   double count, double alpha, double beta, const ddTensorStruct *xd,
                                   const ddTensorStruct *yd, void *y) {
  ddRedPlan pl;
  ddStatus_t st = dd_reduce_plan(h, red, xd, (const void *)0, yd, &pl, DD_PLAN_STRUCTURED);
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
  DD_RANGE("ddReduceTensorNoAlloc");
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

// ---- positions of the min / max / amax (the reference's :flattened indices) --------------------
// One warp per output scans the reduced elements again in the flattened order of the ORIGINAL dims
// (not the canonical ones: the position is defined over the tensor as the caller described it) and
// keeps the first element that wins; lanes stride over the range, then a shuffle tree picks the
// winner with the smaller position among equals.  A second pass over x, not tuned: the option is
// there for completeness.
struct ddRedIndexParams {
  const void *x;
  unsigned *indices;
  int nk, nr;
  int64_t kd[DD_DIM_MAX], kx[DD_DIM_MAX];  // kept dims in original order: extent, x stride
  int64_t rd[DD_DIM_MAX], rx[DD_DIM_MAX];  // reduced dims in original order: extent, x stride
  int64_t nout, nred;
  int op, nanProp;
};

// does candidate (v, i) beat the holder (b, bi)?  NaN with propagation: the first NaN wins outright.
template <typename C>
__device__ __forceinline__ bool dd_index_beats(int op, bool nanProp, C v, unsigned i, C b, unsigned bi) {
  const bool vn = v != v, bn = b != b;
  if (vn || bn) {
    if (!nanProp) return bn && !vn;          // a number beats the NaN placeholder; NaN never beats a number
    if (vn && bn) return i < bi;
    return vn;
  }
  if (v == b) return i < bi;
  return op == DD_REDUCE_TENSOR_MIN ? v < b : v > b;
}

template <typename T, typename C>
__global__ void __launch_bounds__(256) dd_reduce_indices_kernel(ddRedIndexParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const bool nanProp = p.nanProp != 0;
  for (int64_t o = warp; o < p.nout; o += nwarps) {
    int64_t ox = 0, rem = o;
    for (int d = p.nk - 1; d >= 0; d--) {
      const int64_t q = rem / p.kd[d];
      ox += (rem - q * p.kd[d]) * p.kx[d];
      rem = q;
    }
    C best = (C)0;
    unsigned bi = 0xffffffffu;  // nothing held yet
    for (int64_t i = lane; i < p.nred; i += 32) {
      int64_t off = ox, rr = i;
      for (int d = p.nr - 1; d >= 0; d--) {
        const int64_t q = rr / p.rd[d];
        off += (rr - q * p.rd[d]) * p.rx[d];
        rr = q;
      }
      C v = dd_load<C, T>(((const T *)p.x)[off]);
      if (p.op == DD_REDUCE_TENSOR_AMAX) v = v < (C)0 ? -v : v;
      if (bi == 0xffffffffu || dd_index_beats<C>(p.op, nanProp, v, (unsigned)i, best, bi)) {
        best = v;
        bi = (unsigned)i;
      }
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
      const C ob = __shfl_xor_sync(0xffffffffu, best, d);
      const unsigned obi = __shfl_xor_sync(0xffffffffu, bi, d);
      if (obi != 0xffffffffu && (bi == 0xffffffffu || dd_index_beats<C>(p.op, nanProp, ob, obi, best, bi))) {
        best = ob;
        bi = obi;
      }
    }
    if (lane == 0) p.indices[o] = bi == 0xffffffffu ? 0u : bi;
  }
}

// The same scan with one THREAD per output, for reductions across a strided dim with the unit-stride
// dim kept (max over C of nchw): consecutive threads then read consecutive addresses.
template <typename T, typename C>
__global__ void __launch_bounds__(256) dd_reduce_indices_thread_kernel(ddRedIndexParams p) {
  const bool nanProp = p.nanProp != 0;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < p.nout; o += nthreads) {
    int64_t ox = 0, rem = o;
    for (int d = p.nk - 1; d >= 0; d--) {
      const int64_t q = rem / p.kd[d];
      ox += (rem - q * p.kd[d]) * p.kx[d];
      rem = q;
    }
    C best = (C)0;
    unsigned bi = 0xffffffffu;
    for (int64_t i = 0; i < p.nred; i++) {
      int64_t off = ox, rr = i;
      for (int d = p.nr - 1; d >= 0; d--) {
        const int64_t q = rr / p.rd[d];
        off += (rr - q * p.rd[d]) * p.rx[d];
        rr = q;
      }
      C v = dd_load<C, T>(((const T *)p.x)[off]);
      if (p.op == DD_REDUCE_TENSOR_AMAX) v = v < (C)0 ? -v : v;
      if (bi == 0xffffffffu || dd_index_beats<C>(p.op, nanProp, v, (unsigned)i, best, bi)) {
        best = v;
        bi = (unsigned)i;
      }
    }
    p.indices[o] = bi == 0xffffffffu ? 0u : bi;
  }
}

ddStatus_t dd_reduce_indices_impl(ddHandle_t h, const ddReduceTensorStruct *red, const ddTensorStruct *xd, const void *x,
                                  const ddTensorStruct *yd, unsigned *indices) {
  ddRedIndexParams p;
  memset(&p, 0, sizeof(p));
  p.x = x;
  p.indices = indices;
  p.op = (int)red->op;
  p.nanProp = red->nan == DD_PROPAGATE_NAN;
  p.nout = p.nred = 1;
  for (int i = 0; i < xd->nd; i++) {
    if (yd->dims[i] == 1 && xd->dims[i] != 1) {
      p.rd[p.nr] = xd->dims[i]; p.rx[p.nr] = xd->strides[i]; p.nr++;
      p.nred *= xd->dims[i];
    } else {
      p.kd[p.nk] = xd->dims[i]; p.kx[p.nk] = xd->strides[i]; p.nk++;
      p.nout *= xd->dims[i];
    }
  }
  if (p.nred > 0xfffffffeLL) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: 32-bit positions cannot address %lld reduced elements", (long long)p.nred);
  // the unit-stride dim of x kept and at least a few thousand outputs: a thread per output reads
  // coalesced; otherwise a warp per output, its lanes along the reduced range
  bool unitKept = false;
  for (int d = 0; d < p.nk; d++)
    if (p.kx[d] == 1 && p.kd[d] > 1) unitKept = true;
  const bool perThread = unitKept && p.nout >= 4096;
  const int64_t cap = (int64_t)h->smCount * 16;
  int64_t ctas = perThread ? (p.nout + 255) / 256 : (p.nout + 7) / 8;
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
#define DD_LAUNCH_POSITIONS(T, C)                                                                          \
  do {                                                                                                     \
    if (perThread) dd_reduce_indices_thread_kernel<T, C><<<(unsigned)ctas, 256, 0, h->stream>>>(p);       \
    else dd_reduce_indices_kernel<T, C><<<(unsigned)ctas, 256, 0, h->stream>>>(p);                         \
  } while (0)
  switch (xd->dtype) {
    case DD_DATA_FLOAT: DD_LAUNCH_POSITIONS(float, float); break;
    case DD_DATA_DOUBLE: DD_LAUNCH_POSITIONS(double, double); break;
    case DD_DATA_HALF: DD_LAUNCH_POSITIONS(__half, float); break;
    case DD_DATA_BFLOAT16: DD_LAUNCH_POSITIONS(__nv_bfloat16, float); break;
    default: DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "reduce: data types must be floating point");
  }
#undef DD_LAUNCH_POSITIONS
  DD_LAUNCHED(h, "reduce/positions");
  return DD_STATUS_SUCCESS;
}
