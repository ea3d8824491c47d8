// Reduce-tensor kernels: y = alpha*post(reduce(pre(x))) + beta*y over the dims where y's extent is 1.
//
// The canonical iteration space (dims ordered by x stride, merged) is matched against the form
//     x[k1][r1][k2][r2]      k* kept, r* reduced, any of the four may have extent 1
// which covers nchw/nhwc reductions over any subset of (N, C, spatial).  Two kernel families:
//
//   row   r2 > 1 and contiguous in x (reduce over the innermost run; e.g. nchw sum over (N,H,W)
//         or norm over (C,H,W)).  A group of 32 to 256 threads owns one (output, split): 16-byte
//         loads along r2, register accumulation, warp shuffle tree, shared-memory tree across warps.
//         dd_reduce_rowl_kernel (lean: 8 loads in flight, aligned runs of at most 4 chunks per
//         thread) takes the plans it can, dd_reduce_row_kernel (general walk, 4 loads) the rest.
//   col   r2 == 1 and k2 contiguous in x (reduce across a strided dim; e.g. nchw max over C).
//         Lanes run along k2 with 16-byte loads, warps stride over r1, shared-memory combine:
//         dd_reduce_col_kernel; dd_reduce_colc_kernel (lean, 128 threads) when the reduced range
//         is split over a thread-block cluster, and for 16-bit element types.
//
// When an output's reduce range is split over several CTAs (few outputs, long ranges) the splits
// are combined one of two ways.  Column reductions with 2, 4 or 8 splits: the splits form a cluster
// and the first CTA reads the others' results from their shared memory.  Everything else: each
// split writes one partial to the workspace and bumps an arrival counter; the split that arrives
// last folds all partials in a fixed order and finishes (one launch, nobody waits, results are
// run-to-run identical).  Without counters (the entry point that has no handle, whose memory
// nobody has zeroed) dd_reduce_finish_kernel does the fold instead.  Anything that does not fit the
// 4-level form runs one thread per output (generic).  All are HBM-bound: algorithmic bytes = input
// bytes + output bytes.
#pragma once
#include "dd_internal.cuh"
#include <cooperative_groups.h>

enum { DD_OPC_SUM = 0, DD_OPC_SUMABS, DD_OPC_SUMSQ, DD_OPC_PROD, DD_OPC_PRODNZ, DD_OPC_MIN, DD_OPC_MAX, DD_OPC_AMAX, DD_OPC_SUMPOW, DD_OPC_COUNT };
enum { DD_POST_NONE = 0, DD_POST_AVG = 1, DD_POST_SQRT = 2, DD_POST_LP = 3 };

template <typename C> __device__ __forceinline__ C dd_inf();
template <> __device__ __forceinline__ float dd_inf<float>() { return __int_as_float(0x7f800000); }
template <> __device__ __forceinline__ double dd_inf<double>() { return __longlong_as_double(0x7ff0000000000000LL); }
__device__ __forceinline__ float dd_abs(float v) { return fabsf(v); }
__device__ __forceinline__ double dd_abs(double v) { return fabs(v); }
__device__ __forceinline__ float dd_fma(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double dd_fma(double a, double b, double c) { return fma(a, b, c); }
__device__ __forceinline__ float dd_fmax(float a, float b) { return fmaxf(a, b); }
__device__ __forceinline__ double dd_fmax(double a, double b) { return fmax(a, b); }
__device__ __forceinline__ float dd_fmin(float a, float b) { return fminf(a, b); }
__device__ __forceinline__ double dd_fmin(double a, double b) { return fmin(a, b); }
__device__ __forceinline__ float dd_fmax_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float dd_fmin_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float dd_sqrt(float v) { return __fsqrt_rn(v); }
__device__ __forceinline__ double dd_sqrt(double v) { return __dsqrt_rn(v); }
__device__ __forceinline__ float dd_div(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ double dd_div(double a, double b) { return __ddiv_rn(a, b); }
__device__ __forceinline__ float dd_pow(float a, float b) { return powf(a, b); }
__device__ __forceinline__ double dd_pow(double a, double b) { return pow(a, b); }

template <typename C, int OPC>
struct dd_red {
  static __device__ __forceinline__ C identity() {
    if (OPC == DD_OPC_PROD || OPC == DD_OPC_PRODNZ) return (C)1;
    if (OPC == DD_OPC_MIN) return dd_inf<C>();
    if (OPC == DD_OPC_MAX) return -dd_inf<C>();
    return (C)0;
  }
  // acc (+)= pre(v); pw: the exponent of the general Lp sum, unused by every other kind
  static __device__ __forceinline__ C accum(C acc, C v, bool nanProp, C pw) {
    if (OPC == DD_OPC_SUMPOW) {  // p = 3 and p = 4 by multiplication, any other p through pow
      const C a = dd_abs(v), a2 = dd_mul_rn(a, a);
      if (pw == (C)3) return dd_fma(a2, a, acc);
      if (pw == (C)4) return dd_fma(a2, a2, acc);
      return dd_add_rn(acc, dd_pow(a, pw));
    }
    if (OPC == DD_OPC_SUM) return dd_add_rn(acc, v);
    if (OPC == DD_OPC_SUMABS) return dd_add_rn(acc, dd_abs(v));
    if (OPC == DD_OPC_SUMSQ) return dd_fma(v, v, acc);
    if (OPC == DD_OPC_PROD) return dd_mul_rn(acc, v);
    if (OPC == DD_OPC_PRODNZ) return v == (C)0 ? acc : dd_mul_rn(acc, v);
    if (OPC == DD_OPC_AMAX) return comb(acc, dd_abs(v), nanProp);
    return comb(acc, v, nanProp);
  }
  // combines two accumulators
  static __device__ __forceinline__ C comb(C a, C b, bool nanProp) {
    if (OPC == DD_OPC_SUM || OPC == DD_OPC_SUMABS || OPC == DD_OPC_SUMSQ || OPC == DD_OPC_SUMPOW) return dd_add_rn(a, b);
    if (OPC == DD_OPC_PROD || OPC == DD_OPC_PRODNZ) return dd_mul_rn(a, b);
    // propagate: a NaN on either side wins (b beats a only when it compares so or is NaN; a NaN in a
    // survives because every comparison with it is false).  Otherwise IEEE maxNum/minNum: the number wins.
    if (nanProp) {
      if constexpr (sizeof(C) == 4) {  // one instruction: the NaN-propagating forms of min / max
        if (OPC == DD_OPC_MIN) return dd_fmin_nan(a, b);
        return dd_fmax_nan(a, b);
      } else {
        if (OPC == DD_OPC_MIN) return (b < a || b != b) ? b : a;
        return (b > a || b != b) ? b : a;
      }
    }
    if (OPC == DD_OPC_MIN) return dd_fmin(a, b);
    return dd_fmax(a, b);
  }
};

template <int OPC> struct dd_is_minmax { static constexpr bool value = OPC == DD_OPC_MIN || OPC == DD_OPC_MAX || OPC == DD_OPC_AMAX; };

// acc[k] (+)= wv[k] for the V elements of one 16-byte load.  For min / max / amax the NaN mode, which
// is the same for the whole grid, is branched on once per vector so that each element is ONE
// instruction (max / max.NaN) instead of both forms and a select.
template <typename T, typename C, int OPC, int V>
__device__ __forceinline__ void dd_accum_vec(C (&acc)[V], const T *wv, bool nanProp, C pw) {
  if constexpr (dd_is_minmax<OPC>::value) {
    if (nanProp) {
#pragma unroll
      for (int k = 0; k < V; k++) acc[k] = dd_red<C, OPC>::accum(acc[k], dd_load<C, T>(wv[k]), true, pw);
    } else {
#pragma unroll
      for (int k = 0; k < V; k++) acc[k] = dd_red<C, OPC>::accum(acc[k], dd_load<C, T>(wv[k]), false, pw);
    }
  } else {
#pragma unroll
    for (int k = 0; k < V; k++) acc[k] = dd_red<C, OPC>::accum(acc[k], dd_load<C, T>(wv[k]), nanProp, pw);
  }
}

// min / max / amax of 16-bit element types in their own packed form (max.{NaN.}bf16x2 / f16x2: two
// elements per instruction, no conversion; the result is one of the inputs, so nothing is rounded).
template <typename T> struct dd_pack2;
template <> struct dd_pack2<__nv_bfloat16> { typedef __nv_bfloat162 P; static constexpr unsigned NEG_INF2 = 0xFF80FF80u, POS_INF2 = 0x7F807F80u; };
template <> struct dd_pack2<__half> { typedef __half2 P; static constexpr unsigned NEG_INF2 = 0xFC00FC00u, POS_INF2 = 0x7C007C00u; };

template <typename T, int OPC>
__device__ __forceinline__ unsigned dd_minmax2_identity() {
  return OPC == DD_OPC_MIN ? dd_pack2<T>::POS_INF2 : (OPC == DD_OPC_MAX ? dd_pack2<T>::NEG_INF2 : 0u);
}

template <typename T, int OPC, bool NANPROP>
__device__ __forceinline__ unsigned dd_minmax2(unsigned a, unsigned b) {
  typedef typename dd_pack2<T>::P P;
  P pa = *(const P *)&a, pb = *(const P *)&b, r;
  if (OPC == DD_OPC_AMAX) pb = __habs2(pb);
  if (OPC == DD_OPC_MIN) r = NANPROP ? __hmin2_nan(pa, pb) : __hmin2(pa, pb);
  else r = NANPROP ? __hmax2_nan(pa, pb) : __hmax2(pa, pb);
  return *(const unsigned *)&r;
}

// pacc = min/max(pacc, v) over the four packed pairs of a 16-byte vector
template <typename T, int OPC>
__device__ __forceinline__ void dd_minmax_packed(uint4 &pacc, const uint4 &v, bool nanProp) {
  if (nanProp) {
    pacc.x = dd_minmax2<T, OPC, true>(pacc.x, v.x); pacc.y = dd_minmax2<T, OPC, true>(pacc.y, v.y);
    pacc.z = dd_minmax2<T, OPC, true>(pacc.z, v.z); pacc.w = dd_minmax2<T, OPC, true>(pacc.w, v.w);
  } else {
    pacc.x = dd_minmax2<T, OPC, false>(pacc.x, v.x); pacc.y = dd_minmax2<T, OPC, false>(pacc.y, v.y);
    pacc.z = dd_minmax2<T, OPC, false>(pacc.z, v.z); pacc.w = dd_minmax2<T, OPC, false>(pacc.w, v.w);
  }
}

// acc (+)= every element of one 16-byte load (the row kernels' scalar accumulator)
template <typename T, typename C, int OPC, int V>
__device__ __forceinline__ C dd_accum_run(C acc, const T *wv, bool nanProp, C pw) {
  if constexpr (dd_is_minmax<OPC>::value && sizeof(T) == 2 && V == 8) {
    // fold the vector's four pairs in packed form, then the two survivors in float
    const uint4 v = *(const uint4 *)wv;
    unsigned m;
    if (nanProp) {
      const unsigned lo = OPC == DD_OPC_AMAX ? dd_minmax2<T, OPC, true>(0u, v.x) : v.x;  // |.| of the first operand too
      m = dd_minmax2<T, OPC, true>(dd_minmax2<T, OPC, true>(lo, v.y), v.z);
      m = dd_minmax2<T, OPC, true>(m, v.w);
    } else {
      const unsigned lo = OPC == DD_OPC_AMAX ? dd_minmax2<T, OPC, false>(0u, v.x) : v.x;
      m = dd_minmax2<T, OPC, false>(dd_minmax2<T, OPC, false>(lo, v.y), v.z);
      m = dd_minmax2<T, OPC, false>(m, v.w);
    }
    const T *mv = (const T *)&m;
    // the pair is already |.| for amax, so the plain max finishes it
    constexpr int FIN = OPC == DD_OPC_MIN ? DD_OPC_MIN : DD_OPC_MAX;
    if (nanProp) {
      acc = dd_red<C, FIN>::comb(acc, dd_load<C, T>(mv[0]), true);
      acc = dd_red<C, FIN>::comb(acc, dd_load<C, T>(mv[1]), true);
    } else {
      acc = dd_red<C, FIN>::comb(acc, dd_load<C, T>(mv[0]), false);
      acc = dd_red<C, FIN>::comb(acc, dd_load<C, T>(mv[1]), false);
    }
    return acc;
  } else if constexpr (dd_is_minmax<OPC>::value) {
    if (nanProp) {
#pragma unroll
      for (int k = 0; k < V; k++) acc = dd_red<C, OPC>::accum(acc, dd_load<C, T>(wv[k]), true, pw);
    } else {
#pragma unroll
      for (int k = 0; k < V; k++) acc = dd_red<C, OPC>::accum(acc, dd_load<C, T>(wv[k]), false, pw);
    }
    return acc;
  } else {
#pragma unroll
    for (int k = 0; k < V; k++) acc = dd_red<C, OPC>::accum(acc, dd_load<C, T>(wv[k]), nanProp, pw);
    return acc;
  }
}

// ---- cross-GPU exchange: constants and cell helpers (the protocol is described further down) ----
#define DD_PEER_MAX 8
#define DD_PEER_GRID_MAX 128
#define DD_PEER_SLOT_BYTES (2u << 20)
#define DD_PEER_SLOTS_OFF 8192u
#define DD_PEER_BYTES (DD_PEER_SLOTS_OFF + 2u * DD_PEER_MAX * DD_PEER_SLOT_BYTES)

struct ddPeerParams {
  unsigned char *base[DD_PEER_MAX];  // every rank's exchange buffer as mapped here; base[rank] is the own one
  const void *partial;               // this rank's accumulators
  int world, rank;
  unsigned long long waitNs;         // wall-clock limit of one wait
};

__device__ __forceinline__ void dd_st_cell(uint2 *p, unsigned word, unsigned tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(word), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 dd_ld_cell(const uint2 *p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long dd_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <typename C> struct dd_words;
template <> struct dd_words<float> {
  static constexpr int N = 1;
  static __device__ __forceinline__ void split(float v, unsigned *w) { w[0] = __float_as_uint(v); }
  static __device__ __forceinline__ float join(const unsigned *w) { return __uint_as_float(w[0]); }
};
template <> struct dd_words<double> {
  static constexpr int N = 2;
  static __device__ __forceinline__ void split(double v, unsigned *w) {
    w[0] = (unsigned)__double2loint(v);
    w[1] = (unsigned)__double2hiint(v);
  }
  static __device__ __forceinline__ double join(const unsigned *w) { return __hiloint2double((int)w[1], (int)w[0]); }
};

struct ddRedParams {
  const void *x;
  void *y;
  void *part;     // workspace: [out][split] accumulators of the compute type (used when S > 1)
  void *partOut;  // partialOnly: [out] raw accumulators (no post/alpha/beta) instead of y
  int rowCluster;      // row, lean: the splits of an output are the groups of this many consecutive CTAs, one cluster (0: none)
  unsigned *counters;  // S > 1: per-output (row) / per-tile (col) arrival counters, zero between launches;
                       // the last split to arrive combines all partials and finishes.  NULL: a separate
                       // finishing kernel does it.
  int64_t K1, R1, K2, R2;
  int64_t sxK1, sxR1, sxK2, sxR2;
  int64_t syK1, syK2;
  int S;             // CTAs (groups) per output
  int G;             // row: threads per group (32 or 256)
  int64_t CH;        // row: elements of r2 covered per group iteration (G * V)
  int64_t cpr;       // row: chunks per r2 run
  int splitR1;       // row: 1 = splits partition r1, 0 = splits interleave the chunks of r2
  int TX;            // col: lanes along k2
  int64_t tilesK2;   // col: tiles along k2
  double alpha, beta, count;
  int post;
  double lpP, lpEps;   // DD_POST_LP (oneDNN's norm_lp kinds): exponent and epsilon,
  int lpMax, lpRoot;   //   max(S, eps) instead of S + eps; the 1/p power taken or not
  int nanProp;
  int partialOnly;   // 1: store the raw accumulator into partOut[out] and leave y alone
                     // 2: the same, and push it to the other ranks; the last CTA of the grid then
                     //    combines the world's accumulators and finishes into y (fused exchange)
  unsigned char *peerBase[DD_PEER_MAX];  // partialOnly == 2: every rank's exchange buffer
  int peerWorld, peerRank;
  int peerDistributed;  // partialOnly == 2: the thread that finishes an output also collects the other
                        // ranks' values for it and writes y (row kernels whose grid is resident at
                        // once); 0: the CTA that finishes last collects every output
  unsigned long long peerWaitNs;
};

// what follows the fold of an output: mean's division, the norms' root, epsilon
template <typename C, typename P>
__device__ __forceinline__ C dd_red_post(const P &p, C v) {
  if (p.post == DD_POST_AVG) v = dd_div(v, (C)p.count);
  if (p.post == DD_POST_SQRT) v = dd_sqrt(v);
  if (p.post == DD_POST_LP) {
    v = p.lpMax ? dd_fmax(v, (C)p.lpEps) : dd_add_rn(v, (C)p.lpEps);
    if (p.lpRoot) v = p.lpP == 2.0 ? dd_sqrt(v) : (p.lpP == 1.0 ? v : dd_pow(v, (C)(1.0 / p.lpP)));
  }
  return v;
}

// post-processing + alpha/beta + store of one finished output
template <typename T, typename C>
__device__ __forceinline__ void dd_red_output(const ddRedParams &p, int64_t k1, int64_t k2, C acc) {
  C v = dd_red_post(p, acc);
  v = dd_scale((C)p.alpha, v);
  T *yp = (T *)p.y + k1 * p.syK1 + k2 * p.syK2;
  if (p.beta != 0.0) v = dd_add_rn(v, dd_mul_rn((C)p.beta, dd_load<C, T>(*yp)));
  *yp = dd_store<T, C>(v);
}

// partialOnly == 2: this rank's accumulator of output o goes to the other ranks as tagged cells
// `call`: this call's number when the caller has read it already, else 0 (read here).
template <typename C>
__device__ __forceinline__ unsigned dd_peer_push(const ddRedParams &p, int64_t o, C acc, unsigned call = 0) {
  constexpr int NW = dd_words<C>::N;
  if (call == 0) call = __ldcg((const unsigned *)p.peerBase[p.peerRank]) + 1u;
  const size_t off = DD_PEER_SLOTS_OFF + ((size_t)(call & 1u) * DD_PEER_MAX + p.peerRank) * DD_PEER_SLOT_BYTES;
  unsigned w[NW];
  dd_words<C>::split(acc, w);
  for (int r = 0; r < p.peerWorld; r++) {
    if (r == p.peerRank) continue;
    uint2 *cell = (uint2 *)(p.peerBase[r] + off) + o * NW;
#pragma unroll
    for (int k = 0; k < NW; k++) dd_st_cell(cell + k, w[k], call);
  }
  return call;
}

template <typename T, typename C, int OPC>
__device__ __forceinline__ bool dd_peer_collect(const ddRedParams &p, unsigned char *mine, unsigned call,
                                                int W, int rank, unsigned long long t0,
                                                unsigned long long waitNs, int64_t o, C mineVal);

// OPC: only the distributed fused exchange needs it (the combine across ranks); -1 elsewhere.
template <typename T, typename C, bool PEER = false, int OPC = -1>
__device__ __forceinline__ void dd_red_finish(const ddRedParams &p, int64_t k1, int64_t k2, C acc,
                                              unsigned peerCall = 0) {
  if (p.partialOnly) {
    const int64_t o = k1 * p.K2 + k2;
    ((C *)p.partOut)[o] = acc;
    if constexpr (PEER) {
      const unsigned call = dd_peer_push<C>(p, o, acc, peerCall);
      if constexpr (OPC >= 0) {
        // this rank's value is on its way; now wait (bounded) for the other ranks' values of the
        // same output, which their CTAs push at about the same time, and finish it here
        if (p.peerDistributed)
          dd_peer_collect<T, C, OPC>(p, p.peerBase[p.peerRank], call, p.peerWorld, p.peerRank, dd_globaltimer(),
                                     p.peerWaitNs, o, acc);
      }
    }
    return;
  }
  dd_red_output<T, C>(p, k1, k2, acc);
}

// Polls this rank's own exchange buffer for the other ranks' accumulators of output o (bounded),
// combines the world's values in rank order (own value `mineVal`) and finishes into y.  Returns
// false when the wait ran out (status word set, output skipped).
template <typename T, typename C, int OPC>
__device__ __forceinline__ bool dd_peer_collect(const ddRedParams &p, unsigned char *mine, unsigned call,
                                                int W, int rank, unsigned long long t0,
                                                unsigned long long waitNs, int64_t o, C mineVal) {
  constexpr int NW = dd_words<C>::N;
  const bool nanProp = p.nanProp != 0;
  const size_t parOff = DD_PEER_SLOTS_OFF + (size_t)(call & 1u) * DD_PEER_MAX * DD_PEER_SLOT_BYTES;
  uint2 v[DD_PEER_MAX][NW];
  unsigned spins = 0;
  int late = -1;
  for (;;) {
    late = -1;
#pragma unroll
    for (int r = 0; r < DD_PEER_MAX; r++) {
      if (r < W && r != rank) {
        const uint2 *cell = (const uint2 *)(mine + parOff + (size_t)r * DD_PEER_SLOT_BYTES) + o * NW;
#pragma unroll
        for (int k = 0; k < NW; k++) v[r][k] = dd_ld_cell(cell + k);
      }
    }
#pragma unroll
    for (int r = 0; r < DD_PEER_MAX; r++) {
      if (r < W && r != rank) {
#pragma unroll
        for (int k = 0; k < NW; k++)
          if (v[r][k].y != call) late = r;
      }
    }
    if (late < 0) break;
    if (++spins > (1u << 24) || ((spins & 63u) == 0 && dd_globaltimer() - t0 > waitNs)) break;
  }
  if (late >= 0) {
    atomicExch((int *)mine + 2, 1 + late);
    return false;
  }
  C acc = (C)0;
#pragma unroll
  for (int r = 0; r < DD_PEER_MAX; r++) {
    if (r < W) {
      C val;
      if (r == rank) {
        val = mineVal;
      } else {
        unsigned w[NW];
#pragma unroll
        for (int k = 0; k < NW; k++) w[k] = v[r][k].x;
        val = dd_words<C>::join(w);
      }
      acc = r == 0 ? val : dd_red<C, OPC>::comb(acc, val, nanProp);
    }
  }
  const int64_t k1 = o / p.K2;
  dd_red_output<T, C>(p, k1, o - k1 * p.K2, acc);
  return true;
}

// partialOnly == 2, called by every thread at the end of a reduce kernel: the CTA that arrives last
// (all local accumulators are in partOut and on their way to the peers by then) collects the other
// ranks' values for every output and finishes; it then publishes the call number.  Only this one
// CTA ever waits, and only on other GPUs.
template <typename T, typename C, int OPC>
__device__ __forceinline__ void dd_peer_tail(const ddRedParams &p) {
  __shared__ int lastFlag;
  unsigned char *mine = p.peerBase[p.peerRank];
  unsigned *ctl = (unsigned *)mine;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) lastFlag = atomicAdd(ctl + 1, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!lastFlag) return;
  __threadfence();
  const unsigned call = __ldcg(ctl) + 1u;
  if (!p.peerDistributed) {
    const int64_t nout = p.K1 * p.K2;
    const unsigned long long t0 = dd_globaltimer();
    for (int64_t o = threadIdx.x; o < nout; o += blockDim.x)
      dd_peer_collect<T, C, OPC>(p, mine, call, p.peerWorld, p.peerRank, t0, p.peerWaitNs, o,
                                 __ldcg((const C *)p.partOut + o));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    ctl[1] = 0;
    __stcg(ctl, call);
  }
}

// Tree over the G threads of a group (G = 32: one warp; G = 256: the CTA).  Result valid in lane 0
// of the group.
template <typename C, int OPC>
__device__ __forceinline__ C dd_group_reduce(C acc, int G, bool nanProp, C *smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    C other = __shfl_down_sync(0xffffffffu, acc, o);
    acc = dd_red<C, OPC>::comb(acc, other, nanProp);
  }
  if (G == 32) return acc;
  // G = 64, 128 or 256: the group's G/32 warps leave their values in shared memory and the first
  // lane of the group folds them in warp order
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = acc;
  __syncthreads();
  if (G == 256) {  // the whole CTA is one group: warp 0 folds the eight values with shuffles
    if (warp == 0) {
      acc = lane < 8 ? smem[lane] : dd_red<C, OPC>::identity();
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        C other = __shfl_down_sync(0xffffffffu, acc, o);
        acc = dd_red<C, OPC>::comb(acc, other, nanProp);
      }
    }
    return acc;
  }
  if ((threadIdx.x % G) == 0) {
    const int gw = G >> 5;
    acc = smem[warp];
    for (int w = 1; w < gw; w++) acc = dd_red<C, OPC>::comb(acc, smem[warp + w], nanProp);
  }
  return acc;
}

// Distributed fused exchange, first thing in the kernel (every thread of the CTA calls it): reads
// this call's number and counts the CTA's arrival.  The CTA that arrives last publishes the number
// for the next launch right away: every CTA has read the old one by then, nothing else depends on
// it during this launch, and the publication is off the critical path of the outputs.  Returns 0 in
// the other fused form (dd_peer_tail publishes then).
__device__ __forceinline__ unsigned dd_peer_begin(const ddRedParams &p) {
  if (!p.peerDistributed) return 0;
  __shared__ unsigned callShared;
  unsigned *ctl = (unsigned *)p.peerBase[p.peerRank];
  if (threadIdx.x == 0) {
    // one thread reads the number and hands it to the CTA through shared memory, so that the value
    // is in hand before this CTA's arrival counts
    const unsigned call = __ldcg(ctl) + 1u;
    callShared = call;
    if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1) {
      ctl[1] = 0;
      __stcg(ctl, call);
    }
  }
  __syncthreads();
  return callShared;
}

// Folds the S partials of one output.  Called by all 32 lanes of a warp; the result is valid in
// lane 0.  Up to 32 partials: lane 0 folds them in index order.  More: lane l folds partials l,
// l + 32, ... in index order and the lanes combine in a shuffle tree.  The order is fixed either
// way, and the in-kernel fold (last arrival) and dd_reduce_finish_kernel both come here, so the two
// give the same bits.
template <typename C, int OPC>
__device__ __forceinline__ C dd_fold_partials(const C *part, int S, bool nanProp, int lane) {
  if (S <= 32) {
    C a = dd_red<C, OPC>::identity();
    if (lane == 0) {
      a = __ldcg(part);
      for (int i = 1; i < S; i++) a = dd_red<C, OPC>::comb(a, __ldcg(part + i), nanProp);
    }
    return a;
  }
  C a = __ldcg(part + lane);
  for (int i = lane + 32; i < S; i += 32) a = dd_red<C, OPC>::comb(a, __ldcg(part + i), nanProp);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    C other = __shfl_down_sync(0xffffffffu, a, o);
    a = dd_red<C, OPC>::comb(a, other, nanProp);
  }
  return a;
}

// What follows a thread's own accumulation in the row kernels: the group's tree, then either the
// finished output or this split's partial (the split that arrives last folds them all).
template <typename T, typename C, int OPC, bool PEER>
__device__ __forceinline__ void dd_row_epilogue(const ddRedParams &p, C acc, C *smem, unsigned peerCall) {
  const bool nanProp = p.nanProp != 0;
  acc = dd_group_reduce<C, OPC>(acc, p.G, nanProp, smem);
  if constexpr (!PEER) {
    if (p.rowCluster) {
      // The S splits of an output are the groups of rowCluster consecutive CTAs, launched as one
      // thread-block cluster: each group leaves its value in its CTA's shared memory and the
      // cluster's first CTA folds them in split order, reading the other CTAs' values through
      // distributed shared memory.  Two cluster barriers instead of the partial store, fence, atomic
      // and re-read through global memory.
      namespace cg = cooperative_groups;
      cg::cluster_group cluster = cg::this_cluster();
      __shared__ C cpart[8];
      if (threadIdx.x % p.G == 0) cpart[threadIdx.x / p.G] = acc;
      cluster.sync();
      if (cluster.block_rank() == 0 && threadIdx.x == 0) {
        const int gpb = blockDim.x / p.G;
        C a = cpart[0];
        for (int w = 1; w < gpb; w++) a = dd_red<C, OPC>::comb(a, cpart[w], nanProp);
        for (int r = 1; r < p.rowCluster; r++) {
          const C *rp = cluster.map_shared_rank(cpart, r);
          for (int w = 0; w < gpb; w++) a = dd_red<C, OPC>::comb(a, rp[w], nanProp);
        }
        const int64_t out = blockIdx.x / p.rowCluster;
        const int64_t k1 = out / p.K2;
        dd_red_finish<T, C, false, -1>(p, k1, out - k1 * p.K2, a, 0u);
      }
      cluster.sync();  // nobody leaves while its shared memory may still be read
      return;
    }
  }
  // which group this is and which output and split it works on: worked out again here rather than
  // kept in registers across the kernel's main loop (which has none to spare)
  const int lane = threadIdx.x % p.G;
  const int64_t g = (int64_t)blockIdx.x * (blockDim.x / p.G) + threadIdx.x / p.G;
  const bool live = g < p.K1 * p.K2 * p.S;
  int64_t out = 0, k1 = 0, k2 = 0;
  int s = 0;
  if (live && lane < 32) {
    out = g / p.S;
    s = (int)(g - out * p.S);
    k1 = out / p.K2;
    k2 = out - k1 * p.K2;
  }
  if (p.S == 1) {
    if (live && lane == 0) dd_red_finish<T, C, PEER, PEER ? OPC : -1>(p, k1, k2, acc, peerCall);
  } else if (lane < 32) {
    // the first warp of the group: lane 0 leaves this split's partial and counts its arrival; the
    // split that arrives last folds all S partials with the whole warp (a fixed order, so the result
    // does not depend on which split came last).  No waiting anywhere.
    C *part = (C *)p.part + out * p.S;
    int last = 0;
    if (live && lane == 0) {
      part[s] = acc;
      if (p.counters) {
        __threadfence();
        last = atomicAdd(p.counters + out, 1u) == (unsigned)(p.S - 1);
      }
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      __threadfence();
      const C a = dd_fold_partials<C, OPC>(part, p.S, nanProp, lane);
      if (lane == 0) {
        dd_red_finish<T, C, PEER, PEER ? OPC : -1>(p, k1, k2, a, peerCall);
        p.counters[out] = 0;
      }
    }
  }
  if constexpr (PEER) {
    if (!p.peerDistributed) dd_peer_tail<T, C, OPC>(p);
  }
}

// PEER: the fused exchange (partialOnly == 2), its own instantiation so that the plain kernels keep
// their register budget.
// The CTA has 128 or 256 threads (blockDim.x), a whole number of groups.
template <typename T, typename C, int OPC, int VEC, bool PEER>
__global__ void __launch_bounds__(256, PEER ? 4 : 0) dd_reduce_row_kernel(ddRedParams p) {
  // VEC: 1 = 16-byte loads, 2 = 8-byte loads (16-bit types whose runs are only 8-byte aligned), 0 = one element
  constexpr int V = VEC == 1 ? 16 / sizeof(T) : (VEC == 2 ? 8 / sizeof(T) : 1);
  // independent loads in flight per thread: four of 16 bytes, eight of 8 bytes; element loads (runs
  // that are not vector-aligned: 7 x 7 and 13 x 13 maps) 16 of a 16-bit type, 8 of a 32-bit one
  constexpr int U = VEC == 2 ? 8 : (VEC == 0 ? (sizeof(T) == 2 ? 16 : (sizeof(T) == 4 ? 8 : 4)) : 4);
  __shared__ C smem[8];
  dd_pdl_prologue();
  unsigned peerCall = 0;
  if constexpr (PEER) peerCall = dd_peer_begin(p);
  const bool nanProp = p.nanProp != 0;
  const int G = p.G;
  const int gpb = blockDim.x / G;  // groups per CTA
  const int64_t g = (int64_t)blockIdx.x * gpb + threadIdx.x / G;
  const int lane = threadIdx.x % G;
  const int64_t nout = p.K1 * p.K2;
  C acc = dd_red<C, OPC>::identity();
  const bool live = g < nout * p.S;  // G == 32 only: trailing groups of the last CTA idle
  if (live) {
    const int64_t out = g / p.S;
    const int s = (int)(g - out * p.S);
    const int64_t k1 = out / p.K2;
    const int64_t k2 = out - k1 * p.K2;
    // splits either partition r1 (each takes whole runs) or interleave the chunks of every run
    // (split s takes chunks s, s + S, ...): concurrently running splits of one output then read
    // neighbouring 16-byte-vector rows, like one flat stream
    int64_t r1lo = 0, r1hi = p.R1, jlo = 0, jstep = 1;
    if (p.S > 1) {
      if (p.splitR1) {
        int64_t per = (p.R1 + p.S - 1) / p.S;
        r1lo = s * per;
        r1hi = r1lo + per < p.R1 ? r1lo + per : p.R1;
      } else {
        jlo = s;
        jstep = p.S;
      }
    }
    const T *xb = (const T *)p.x + k1 * p.sxK1 + k2 * p.sxK2;
    const int64_t nj = jlo < p.cpr ? (p.cpr - jlo + jstep - 1) / jstep : 0;
    const int64_t iters = (r1hi > r1lo && nj > 0) ? (r1hi - r1lo) * nj : 0;
    // the walk is kept in increments (no multiplication per load): `row` points at run r1, `e` is
    // this lane's element offset inside it, `j` the chunk number
    const T *row = xb + r1lo * p.sxR1;
    const int64_t eFirst = jlo * p.CH + (int64_t)lane * V, eStep = jstep * p.CH;
    int64_t e = eFirst, j = jlo, left = iters;
    for (int64_t it = 0; it < iters; it += U) {
      // U loads in flight, kept as loaded (16 bytes each) and converted only while accumulating
      uint4 raw[U];
      bool ok[U];
#pragma unroll
      for (int q = 0; q < U; q++) {
        ok[q] = (left > 0) && (e < p.R2);
        if (ok[q]) {
          if (VEC == 1) raw[q] = *(const uint4 *)(row + e);
          else if (VEC == 2) *(uint2 *)&raw[q] = *(const uint2 *)(row + e);
          else *(T *)&raw[q] = row[e];
        }
        left--;
        j += jstep;
        e += eStep;
        if (j >= p.cpr) { j = jlo; e = eFirst; row += p.sxR1; }
      }
#pragma unroll
      for (int q = 0; q < U; q++) {
        if (ok[q]) {
          const T *wv = (const T *)&raw[q];
          acc = dd_accum_run<T, C, OPC, V>(acc, wv, nanProp, (C)p.lpP);
        }
      }
    }
  }
  dd_row_epilogue<T, C, OPC, PEER>(p, acc, smem, peerCall);
}

// Lean form of the row kernel for small inputs, where the whole reduction is two or three round
// trips to memory and what counts is how many bytes are in flight: EIGHT 16-byte loads per thread
// and nothing else in the loop but one pointer.  Plans that qualify: 16-byte aligned runs, a
// thread's share of a run at most CPR chunks (CPR = 1, 2 or 4; a row batch is 8 / CPR runs), and
// splits, if any, that partition r1.  Same accumulation order as the general kernel.
template <typename T, typename C, int OPC, int CPR, bool PEER>
__global__ void __launch_bounds__(256, 4) dd_reduce_rowl_kernel(ddRedParams p) {
  constexpr int V = 16 / sizeof(T);
  constexpr int U = 8, RB = U / CPR;
  __shared__ C smem[8];
  dd_pdl_prologue();
  unsigned peerCall = 0;
  if constexpr (PEER) peerCall = dd_peer_begin(p);
  const bool nanProp = p.nanProp != 0;
  const int G = p.G;
  const int gpb = blockDim.x / G;
  const int64_t g = (int64_t)blockIdx.x * gpb + threadIdx.x / G;
  const int lane = threadIdx.x % G;
  const int64_t nout = p.K1 * p.K2;
  C acc = dd_red<C, OPC>::identity();
  const bool live = g < nout * p.S;
  if (live) {
    const int64_t out = g / p.S;
    const int s = (int)(g - out * p.S);
    const int64_t k1 = out / p.K2;
    const int64_t k2 = out - k1 * p.K2;
    int64_t r1lo = 0, r1hi = p.R1;
    if (p.S > 1) {
      int64_t per = (p.R1 + p.S - 1) / p.S;
      r1lo = s * per;
      r1hi = r1lo + per < p.R1 ? r1lo + per : p.R1;
    }
    const T *ptr = (const T *)p.x + k1 * p.sxK1 + k2 * p.sxK2 + r1lo * p.sxR1 + (int64_t)lane * V;
    const int nrows = r1hi > r1lo ? (int)(r1hi - r1lo) : 0;
    const int ch = (int)p.CH;  // at most 256 vectors of V elements
    bool okc[CPR];
#pragma unroll
    for (int c = 0; c < CPR; c++) okc[c] = (int64_t)lane * V + c * ch < p.R2;
    if constexpr (!PEER) {
      // batches of RB runs; the loads of a batch go out together, those of the last, partial batch
      // too (a run at a time they would be up to RB - 1 more round trips to memory)
      for (int left = nrows; left > 0; left -= RB) {
        uint4 raw[U];
#pragma unroll
        for (int q = 0; q < RB; q++)
#pragma unroll
          for (int c = 0; c < CPR; c++)
            if (q < left && okc[c]) raw[q * CPR + c] = *(const uint4 *)(ptr + q * p.sxR1 + c * ch);
        ptr += RB * p.sxR1;
#pragma unroll
        for (int q = 0; q < RB; q++)
#pragma unroll
          for (int c = 0; c < CPR; c++)
            if (q < left && okc[c]) {
              const T *wv = (const T *)&raw[q * CPR + c];
              acc = dd_accum_run<T, C, OPC, V>(acc, wv, nanProp, (C)p.lpP);
            }
      }
    } else {
      // the fused exchange keeps more values live across the loop (the call number, the exchange
      // buffers): whole batches without the predicate, then the remaining runs one at a time
      int r = 0;
      for (; r + RB <= nrows; r += RB) {
        uint4 raw[U];
#pragma unroll
        for (int q = 0; q < RB; q++)
#pragma unroll
          for (int c = 0; c < CPR; c++)
            if (okc[c]) raw[q * CPR + c] = *(const uint4 *)(ptr + q * p.sxR1 + c * ch);
        ptr += RB * p.sxR1;
#pragma unroll
        for (int q = 0; q < RB; q++)
#pragma unroll
          for (int c = 0; c < CPR; c++)
            if (okc[c]) {
              const T *wv = (const T *)&raw[q * CPR + c];
              acc = dd_accum_run<T, C, OPC, V>(acc, wv, nanProp, (C)p.lpP);
            }
      }
      for (; r < nrows; r++) {
        uint4 raw[CPR];
#pragma unroll
        for (int c = 0; c < CPR; c++)
          if (okc[c]) raw[c] = *(const uint4 *)(ptr + c * ch);
        ptr += p.sxR1;
#pragma unroll
        for (int c = 0; c < CPR; c++)
          if (okc[c]) {
            const T *wv = (const T *)&raw[c];
            acc = dd_accum_run<T, C, OPC, V>(acc, wv, nanProp, (C)p.lpP);
          }
      }
    }
  }
  dd_row_epilogue<T, C, OPC, PEER>(p, acc, smem, peerCall);
}

// col: CTA = TX lanes along k2 (V elements each, TX a power of two <= 256) x TY = 256/TX row
// groups striding over r1.
template <typename T, typename C, int OPC, int VEC, bool PEER>
__global__ void __launch_bounds__(256, (PEER || sizeof(T) == 2) ? 4 : 8) dd_reduce_col_kernel(ddRedParams p) {
  constexpr int V = VEC == 1 ? 16 / sizeof(T) : (VEC == 2 ? 8 / sizeof(T) : 1);  // as in the row kernel
  constexpr int U = VEC == 2 ? 8 : (VEC == 0 ? (sizeof(T) == 2 ? 16 : (sizeof(T) == 4 ? 8 : 4)) : 4);
  __shared__ C smem[256 * V];
  // Large inputs launch this kernel the ordinary way (the programmatic launch measured 4 % slower on
  // a 268 MB tensor), small ones programmatically; the wait returns at once in the first case.
  dd_pdl_prologue();
  const bool nanProp = p.nanProp != 0;
  const int TX = p.TX, TY = 256 / TX;
  const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
  int64_t id = blockIdx.x;
  const int s = (int)(id % p.S);
  id /= p.S;
  const int64_t tk = id % p.tilesK2;
  const int64_t k1 = id / p.tilesK2;
  const int64_t k2 = (tk * TX + tx) * V;
  int64_t lo = 0, hi = p.R1;
  if (p.S > 1) {
    int64_t per = (p.R1 + p.S - 1) / p.S;
    lo = s * per;
    hi = lo + per < p.R1 ? lo + per : p.R1;
  }
  C acc[V];
#pragma unroll
  for (int k = 0; k < V; k++) acc[k] = dd_red<C, OPC>::identity();
  if (k2 < p.K2) {
    const T *xb = (const T *)p.x + k1 * p.sxK1 + k2 * p.sxK2;
    for (int64_t r0 = lo + ty; r0 < hi; r0 += (int64_t)TY * U) {
      uint4 raw[U];  // kept as loaded, converted while accumulating
      bool ok[U];
#pragma unroll
      for (int q = 0; q < U; q++) {
        const int64_t r1 = r0 + (int64_t)q * TY;
        ok[q] = r1 < hi;
        if (ok[q]) {
          const T *ptr = xb + r1 * p.sxR1;
          if (VEC == 1) raw[q] = *(const uint4 *)ptr;
          else if (VEC == 2) *(uint2 *)&raw[q] = *(const uint2 *)ptr;
          else *(T *)&raw[q] = *ptr;
        }
      }
#pragma unroll
      for (int q = 0; q < U; q++) {
        if (ok[q]) {
          const T *wv = (const T *)&raw[q];
          dd_accum_vec<T, C, OPC, V>(acc, wv, nanProp, (C)p.lpP);
        }
      }
    }
  }
  // combine the TY row groups: smem[ty][tx*V + k], then the first TX*V threads fold TY values in
  // a fixed order
#pragma unroll
  for (int k = 0; k < V; k++) smem[ty * (TX * V) + tx * V + k] = acc[k];
  __syncthreads();
  for (int col = threadIdx.x; col < TX * V; col += 256) {
    C a = smem[col];
    for (int r = 1; r < TY; r++) a = dd_red<C, OPC>::comb(a, smem[r * (TX * V) + col], nanProp);
    const int64_t kk = tk * TX * V + col;
    if (kk < p.K2) {
      if (p.S == 1) dd_red_finish<T, C, PEER>(p, k1, kk, a);
      else ((C *)p.part)[(k1 * p.K2 + kk) * p.S + s] = a;
    }
  }
  if (p.S > 1 && p.counters) {
    // one counter per (k1, tile): the last split's CTA folds the partials of the whole tile
    __shared__ int lastFlag;
    __threadfence();
    __syncthreads();
    unsigned *ctr = p.counters + (k1 * p.tilesK2 + tk);
    if (threadIdx.x == 0) lastFlag = atomicAdd(ctr, 1u) == (unsigned)(p.S - 1);
    __syncthreads();
    if (lastFlag) {
      __threadfence();
      for (int col = threadIdx.x; col < TX * V; col += 256) {
        const int64_t kk = tk * TX * V + col;
        if (kk < p.K2) {
          const C *pp = (const C *)p.part + (k1 * p.K2 + kk) * p.S;
          C a = __ldcg(pp);
          for (int i = 1; i < p.S; i++) a = dd_red<C, OPC>::comb(a, __ldcg(pp + i), nanProp);
          dd_red_finish<T, C, PEER>(p, k1, kk, a);
        }
      }
      if (threadIdx.x == 0) *ctr = 0;
    }
  }
  if constexpr (PEER) dd_peer_tail<T, C, OPC>(p);
}

// col, split over a thread-block cluster: the S = 2, 4 or 8 CTAs that share a tile of outputs are
// one cluster, each reduces its share of r1 (eight 16-byte loads in flight per thread, nothing in
// the loop but one pointer), folds its row groups in shared memory, and the cluster's first CTA
// reads the other CTAs' folded values straight from THEIR shared memory (distributed shared
// memory) and finishes, in rank order.  Two cluster barriers replace the partial store, fence,
// atomic counter and re-read through global memory of the counter protocol (about 3 us on a 10 us
// kernel).  CTA = 128 threads: TX lanes along k2 (any number up to 32) by TY = 128 / TX row groups;
// threads beyond TX * TY idle.  With S = 1 (launched without a cluster) it is the column reduce for
// 16-bit element types: eight loads in flight where the general kernel, at twice the registers per
// accumulator set, keeps four.
#define DD_COLC_THREADS 128
template <typename T, typename C, int OPC>
__global__ void __launch_bounds__(DD_COLC_THREADS, 8) dd_reduce_colc_kernel(ddRedParams p) {
  constexpr int V = 16 / sizeof(T);
  constexpr int U = 8;
  constexpr int BS = DD_COLC_THREADS;
  __shared__ C smem[BS * V];
  __shared__ C folded[32 * V];
  dd_pdl_prologue();
  const bool nanProp = p.nanProp != 0;
  const int TX = p.TX, TY = BS / TX;
  const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;  // ty == TY: a thread left over, idle
  int64_t id = blockIdx.x;
  const int s = (int)(id % p.S);  // = this CTA's rank in its cluster (1-D grid, cluster of S along x)
  id /= p.S;
  const int64_t tk = id % p.tilesK2;
  const int64_t k1 = id / p.tilesK2;
  const int64_t k2 = (tk * TX + tx) * V;
  const int64_t per = (p.R1 + p.S - 1) / p.S;
  const int64_t lo = s * per;
  const int64_t hi = lo + per < p.R1 ? lo + per : p.R1;
  C acc[V];
#pragma unroll
  for (int k = 0; k < V; k++) acc[k] = dd_red<C, OPC>::identity();
  // min / max / amax of a 16-bit type: the running value stays in the packed 16-bit form (four
  // instructions per 16-byte load) and is widened once, after the last row
  constexpr bool PACKED = sizeof(T) == 2 && dd_is_minmax<OPC>::value;
  uint4 pacc;
  if constexpr (PACKED) pacc.x = pacc.y = pacc.z = pacc.w = dd_minmax2_identity<T, OPC>();
  if (k2 < p.K2 && ty < TY && lo + ty < hi) {
    const T *ptr = (const T *)p.x + k1 * p.sxK1 + k2 * p.sxK2 + (lo + ty) * p.sxR1;
    const int64_t step = (int64_t)TY * p.sxR1;
    const int n = (int)((hi - lo - ty + TY - 1) / TY);  // rows of this thread
    // batches of U rows; the loads of a batch go out together, those of the last, partial batch too
    // (one at a time they would be up to seven more round trips to memory)
    for (int left = n; left > 0; left -= U) {
      uint4 raw[U];
#pragma unroll
      for (int q = 0; q < U; q++)
        if (q < left) raw[q] = *(const uint4 *)(ptr + q * step);
      ptr += U * step;
#pragma unroll
      for (int q = 0; q < U; q++)
        if (q < left) {
          if constexpr (PACKED) {
            dd_minmax_packed<T, OPC>(pacc, raw[q], nanProp);
          } else {
            const T *wv = (const T *)&raw[q];
            dd_accum_vec<T, C, OPC, V>(acc, wv, nanProp, (C)p.lpP);
          }
        }
    }
    if constexpr (PACKED) {  // the packed accumulators become the float ones the combine below works on
      const T *pv = (const T *)&pacc;
#pragma unroll
      for (int k = 0; k < V; k++) acc[k] = dd_load<C, T>(pv[k]);
    }
  }
  if (ty < TY) {
#pragma unroll
    for (int k = 0; k < V; k++) smem[ty * (TX * V) + tx * V + k] = acc[k];
  }
  __syncthreads();
  for (int col = threadIdx.x; col < TX * V; col += BS) {
    C a = smem[col];
    for (int r = 1; r < TY; r++) a = dd_red<C, OPC>::comb(a, smem[r * (TX * V) + col], nanProp);
    if (p.S == 1) {
      const int64_t kk = tk * TX * V + col;
      if (kk < p.K2) dd_red_finish<T, C>(p, k1, kk, a);
    } else {
      folded[col] = a;
    }
  }
  if (p.S == 1) return;  // no cluster: every thread of the grid takes this branch
  cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
  cluster.sync();  // every CTA's folded values are in its shared memory
  if (s == 0) {
    for (int col = threadIdx.x; col < TX * V; col += BS) {
      const int64_t kk = tk * TX * V + col;
      if (kk < p.K2) {
        C a = folded[col];
        for (int r = 1; r < p.S; r++) a = dd_red<C, OPC>::comb(a, *cluster.map_shared_rank(&folded[col], r), nanProp);
        dd_red_finish<T, C>(p, k1, kk, a);
      }
    }
  }
  cluster.sync();  // nobody leaves while its shared memory may still be read
}

// Combines the S partials of each output in index order and finishes.  `part` may be an
// all-reduced buffer (S == 1) on the multi-GPU path.
template <typename T, typename C, int OPC>
__global__ void __launch_bounds__(256) dd_reduce_finish_kernel(ddRedParams p, const void *part) {
  const bool nanProp = p.nanProp != 0;
  const int64_t nout = p.K1 * p.K2;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (p.S > 32) {  // a warp per output, the fold of dd_fold_partials
    const int lane = threadIdx.x & 31;
    for (int64_t o = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; o < nout; o += nthreads >> 5) {
      const C acc = dd_fold_partials<C, OPC>((const C *)part + o * p.S, p.S, nanProp, lane);
      if (lane == 0) {
        const int64_t k1 = o / p.K2;
        dd_red_finish<T, C>(p, k1, o - k1 * p.K2, acc);
      }
    }
    return;
  }
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < nout; o += nthreads) {
    const C *pp = (const C *)part + o * p.S;
    C acc = pp[0];
    for (int s = 1; s < p.S; s++) acc = dd_red<C, OPC>::comb(acc, pp[s], nanProp);
    const int64_t k1 = o / p.K2;
    dd_red_finish<T, C>(p, k1, o - k1 * p.K2, acc);
  }
}

// Second launch of the column reduce over rows that are not whole vectors (dd_reduce_col_periodic in
// dd_reduce.cu): `part` holds, per k1, P interleaved sets of K2 raw accumulators (set j covers the
// rows r1 = j mod P); output (k1, k2) is their fold in set order.
template <typename T, typename C, int OPC>
__global__ void __launch_bounds__(256) dd_reduce_fold_sets_kernel(ddRedParams p, const void *part, int P) {
  const bool nanProp = p.nanProp != 0;
  const int64_t nout = p.K1 * p.K2;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < nout; o += nthreads) {
    const int64_t k1 = o / p.K2, k2 = o - k1 * p.K2;
    const C *pp = (const C *)part + k1 * (P * p.K2) + k2;
    C acc = pp[0];
    for (int j = 1; j < P; j++) acc = dd_red<C, OPC>::comb(acc, pp[(int64_t)j * p.K2], nanProp);
    dd_red_finish<T, C>(p, k1, k2, acc);
  }
}

// ------------------------------------------------------------------ cross-GPU exchange --------
//
// One process per GPU, every rank holding the raw accumulators of its own shard (nout values of C).
// Each rank owns an exchange buffer that all ranks of the box have mapped (CUDA IPC over NVLink):
//
//   [0, 256)                  control words, touched by the owner only:
//                             [0] number of the last finished call, [1] CTA arrivals, [2] status
//   [DD_PEER_SLOTS_OFF, ...)  slots[parity][sender][DD_PEER_SLOT_BYTES]: 8-byte cells, each one
//                             32-bit word of an accumulator paired with the number of the call that
//                             wrote it
//
// A call is one kernel per rank.  Every thread PUSHES the words of its outputs' accumulators into
// slot [parity][own rank] of every other rank, each as ONE 8-byte store {word, call number} to peer
// memory.  An aligned 8-byte store arrives whole, so a cell whose tag equals this call's number
// holds this call's word: no fence and no separate flag are needed, and a value crosses NVLink once.
// The thread then polls its outputs' cells in its OWN memory until every sender's tag matches,
// combines the world's values in rank order (its own straight from the local buffer; every rank
// computes bit-identical results) and finishes (divide / sqrt / alpha / beta) into y.
// Two parities alternate between calls: a rank can be at most one call ahead of the slowest one,
// because finishing call k+1 needs every rank's cells for k+1, which they send only after call k.
// The call number lives in the buffer (read at the start, advanced by the last CTA to finish), so
// a captured launch can be replayed.
//
// Every wait is bounded (wall-clock limit and an iteration cap): when it runs out the thread
// records 1 + the rank it waited for in the status word, skips its output and returns.  No thread
// waits on another thread of the same GPU.
//
// Two forms.  FUSED (few outputs): the reduce kernel itself pushes each output's accumulator the
// moment it is final (dd_peer_push from dd_red_finish), so the transfers overlap the rest of the
// local pass, and the CTA that finishes last collects and finishes (dd_peer_tail): one kernel for
// reduce + exchange.  SEPARATE (many outputs, or a plan whose splits are combined by a second
// kernel): the local pass writes its accumulators to a buffer and dd_reduce_exchange_kernel below
// does push + collect with all its CTAs.
template <typename T, typename C, int OPC>
__global__ void __launch_bounds__(256) dd_reduce_exchange_kernel(ddRedParams p, ddPeerParams q) {
  constexpr int NW = dd_words<C>::N;
  dd_pdl_prologue();  // scheduled while the local pass drains; nothing is read before it has completed
  const int64_t nout = p.K1 * p.K2;
  unsigned char *mine = q.base[q.rank];
  unsigned *ctl = (unsigned *)mine;
  const unsigned call = __ldcg(ctl) + 1u;  // published by the previous launch's last CTA
  const unsigned par = call & 1u;
  const int W = q.world;
  const C *part = (const C *)q.partial;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t parOff = DD_PEER_SLOTS_OFF + (size_t)par * DD_PEER_MAX * DD_PEER_SLOT_BYTES;

  for (int64_t o = first; o < nout; o += nthreads) {
    unsigned w[NW];
    dd_words<C>::split(part[o], w);
    for (int r = 0; r < W; r++) {
      if (r == q.rank) continue;
      uint2 *cell = (uint2 *)(q.base[r] + parOff + (size_t)q.rank * DD_PEER_SLOT_BYTES) + o * NW;
#pragma unroll
      for (int k = 0; k < NW; k++) dd_st_cell(cell + k, w[k], call);
    }
  }

  const unsigned long long t0 = dd_globaltimer();
  for (int64_t o = first; o < nout; o += nthreads)
    dd_peer_collect<T, C, OPC>(p, mine, call, W, q.rank, t0, q.waitNs, o, part[o]);

  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1) {
      ctl[1] = 0;
      __stcg(ctl, call);
    }
  }
}

// generic: one thread per output, serial walk over the reduced dims.
struct ddRedGenericParams {
  const void *x;
  void *y;
  void *partOut;
  int nk, nr;
  int64_t kd[DD_DIM_MAX], kx[DD_DIM_MAX], ky[DD_DIM_MAX];  // kept dims: extent, x stride, y stride
  int64_t rd[DD_DIM_MAX], rx[DD_DIM_MAX];                  // reduced dims: extent, x stride
  int64_t nout, nred;
  double alpha, beta, count;
  double lpP, lpEps;
  int lpMax, lpRoot;
  int post, nanProp, partialOnly;
};

template <typename T, typename C, int OPC>
__global__ void __launch_bounds__(256) dd_reduce_generic_kernel(ddRedGenericParams p) {
  const bool nanProp = p.nanProp != 0;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < p.nout; o += nthreads) {
    int64_t ox = 0, oy = 0, rem = o;
    for (int d = p.nk - 1; d >= 0; d--) {
      int64_t q = rem / p.kd[d], r = rem - q * p.kd[d];
      ox += r * p.kx[d];
      oy += r * p.ky[d];
      rem = q;
    }
    C acc = dd_red<C, OPC>::identity();
    for (int64_t i = 0; i < p.nred; i++) {
      int64_t off = ox, rr = i;
      for (int d = p.nr - 1; d >= 0; d--) {
        int64_t q = rr / p.rd[d];
        off += (rr - q * p.rd[d]) * p.rx[d];
        rr = q;
      }
      acc = dd_red<C, OPC>::accum(acc, dd_load<C, T>(((const T *)p.x)[off]), nanProp, (C)p.lpP);
    }
    if (p.partialOnly) {
      ((C *)p.partOut)[o] = acc;
    } else {
      C v = dd_red_post(p, acc);
      v = dd_scale((C)p.alpha, v);
      T *yp = (T *)p.y + oy;
      if (p.beta != 0.0) v = dd_add_rn(v, dd_mul_rn((C)p.beta, dd_load<C, T>(*yp)));
      *yp = dd_store<T, C>(v);
    }
  }
}

// ------------------------------------------------------------------ host plan ----------------

enum { DD_RED_ROW = 0, DD_RED_COL = 1, DD_RED_GENERIC = 2 };
enum { DD_PLAN_STRUCTURED = 1, DD_PLAN_NO_CLUSTER = 2 };

struct ddRedPlan {
  int kind;
  int vec;  // 0: element loads; 1: 16-byte loads; 2: 8-byte loads (16-bit types, rows only 8-byte aligned)
  int opc;
  int bs;   // row: threads per CTA (128 or 256)
  int lean; // row: 0 = the general kernel, else the lean kernel with this many chunks per run (1, 2, 4)
  int pdl;  // col: launched programmatically (small inputs) or the ordinary way
  int cluster;  // col: dd_reduce_colc_kernel (S > 1: the S splits of a tile form one thread-block cluster;
                // S == 1: the same kernel without a cluster, for 16-bit element types);
                // row: the lean kernel launched in clusters of p.rowCluster CTAs
  ddRedParams p;
  ddRedGenericParams g;
  int64_t nout;
  size_t wsBytes;  // workspace needed (0 when every output has a single split)
  unsigned grid;
  int foldS;       // finishing launch only: values of `part` folded per output (0: one, the all-reduced form;
                   // negative: -foldS interleaved sets, dd_reduce_fold_sets_kernel)
};

ddStatus_t dd_reduce_plan(ddHandle_t h, const ddReduceTensorStruct *red, const ddTensorStruct *xd,
                          const void *x, const ddTensorStruct *yd, ddRedPlan *pl, int flags = 0);

template <typename T, typename C>
ddStatus_t dd_reduce_launch(ddHandle_t h, const ddRedPlan &pl);
template <typename T, typename C>
ddStatus_t dd_reduce_finish_launch(ddHandle_t h, const ddRedPlan &pl, const void *part);
template <typename T, typename C>
ddStatus_t dd_reduce_exchange_launch(ddHandle_t h, const ddRedPlan &pl, const ddPeerParams &q);
#define DD_REDUCE_DECLARE(T, C)                                                   \
  template <> ddStatus_t dd_reduce_launch<T, C>(ddHandle_t, const ddRedPlan &);   \
  template <> ddStatus_t dd_reduce_finish_launch<T, C>(ddHandle_t, const ddRedPlan &, const void *); \
  template <> ddStatus_t dd_reduce_exchange_launch<T, C>(ddHandle_t, const ddRedPlan &, const ddPeerParams &);
DD_REDUCE_DECLARE(float, float)
DD_REDUCE_DECLARE(double, double)
DD_REDUCE_DECLARE(__half, float)
DD_REDUCE_DECLARE(__nv_bfloat16, float)

#define DD_REDUCE_DEFINE(T, C)                                                                     \
  template <int OPC>                                                                               \
  static ddStatus_t launch_opc_##T(ddHandle_t h, const ddRedPlan &pl) {                            \
    if (pl.p.partialOnly == 2) { /* fused exchange: row or col only, no second kernel */           \
      if (pl.kind == DD_RED_ROW && pl.lean) {                                                      \
        if (pl.lean == 1) dd_launch_pdl(dd_reduce_rowl_kernel<T, C, OPC, 1, true>, pl.grid, (unsigned)pl.bs, h->stream, pl.p);  \
        else if (pl.lean == 2) dd_launch_pdl(dd_reduce_rowl_kernel<T, C, OPC, 2, true>, pl.grid, (unsigned)pl.bs, h->stream, pl.p);  \
        else dd_launch_pdl(dd_reduce_rowl_kernel<T, C, OPC, 4, true>, pl.grid, (unsigned)pl.bs, h->stream, pl.p);  \
        DD_LAUNCHED(h, "reduce/row+peer-exchange");                                                \
      } else if (pl.kind == DD_RED_ROW) {                                                          \
        if (pl.vec == 1) dd_launch_pdl(dd_reduce_row_kernel<T, C, OPC, 1, true>, pl.grid, (unsigned)pl.bs, h->stream, pl.p);  \
        else dd_launch_pdl(dd_reduce_row_kernel<T, C, OPC, 0, true>, pl.grid, (unsigned)pl.bs, h->stream, pl.p);   \
        DD_LAUNCHED(h, "reduce/row+peer-exchange");                                                \
      } else {                                                                                     \
        if (pl.vec == 1) dd_reduce_col_kernel<T, C, OPC, 1, true><<<pl.grid, 256, 0, h->stream>>>(pl.p);  \
        else dd_reduce_col_kernel<T, C, OPC, 0, true><<<pl.grid, 256, 0, h->stream>>>(pl.p);   \
        DD_LAUNCHED(h, "reduce/col+peer-exchange");                                                \
      }                                                                                            \
      return DD_STATUS_SUCCESS;                                                                    \
    }                                                                                              \
    if (pl.kind == DD_RED_ROW && pl.lean && pl.cluster) {                                          \
      const unsigned cs = (unsigned)pl.p.rowCluster;                                               \
      if (pl.lean == 1) dd_launch_cluster(dd_reduce_rowl_kernel<T, C, OPC, 1, false>, pl.grid, (unsigned)pl.bs, cs, h->stream, pl.p);   \
      else if (pl.lean == 2) dd_launch_cluster(dd_reduce_rowl_kernel<T, C, OPC, 2, false>, pl.grid, (unsigned)pl.bs, cs, h->stream, pl.p);   \
      else dd_launch_cluster(dd_reduce_rowl_kernel<T, C, OPC, 4, false>, pl.grid, (unsigned)pl.bs, cs, h->stream, pl.p);   \
      DD_LAUNCHED(h, "reduce/row-cluster");                                                        \
      return DD_STATUS_SUCCESS;                                                                    \
    }                                                                                              \
    if (pl.kind == DD_RED_ROW) {                                                                   \
      if (pl.lean == 1) dd_launch_pdl(dd_reduce_rowl_kernel<T, C, OPC, 1, false>, pl.grid, (unsigned)pl.bs, h->stream, pl.p);   \
      else if (pl.lean == 2) dd_launch_pdl(dd_reduce_rowl_kernel<T, C, OPC, 2, false>, pl.grid, (unsigned)pl.bs, h->stream, pl.p);   \
      else if (pl.lean == 4) dd_launch_pdl(dd_reduce_rowl_kernel<T, C, OPC, 4, false>, pl.grid, (unsigned)pl.bs, h->stream, pl.p);   \
      else if (pl.vec == 1) dd_launch_pdl(dd_reduce_row_kernel<T, C, OPC, 1, false>, pl.grid, (unsigned)pl.bs, h->stream, pl.p);   \
      else if (pl.vec == 2) { if constexpr (sizeof(T) == 2 && OPC >= 0) dd_launch_pdl(dd_reduce_row_kernel<T, C, OPC, 2, false>, pl.grid, (unsigned)pl.bs, h->stream, pl.p); }  \
      else dd_launch_pdl(dd_reduce_row_kernel<T, C, OPC, 0, false>, pl.grid, (unsigned)pl.bs, h->stream, pl.p);    \
      DD_LAUNCHED(h, pl.lean ? "reduce/row-lean" : (pl.vec == 2 ? "reduce/row-v8" : "reduce/row"));  \
    } else if (pl.kind == DD_RED_COL && pl.cluster && pl.p.S == 1) {                               \
      dd_reduce_colc_kernel<T, C, OPC><<<pl.grid, DD_COLC_THREADS, 0, h->stream>>>(pl.p);          \
      DD_LAUNCHED(h, "reduce/col-lean");                                                           \
      return DD_STATUS_SUCCESS;                                                                    \
    } else if (pl.kind == DD_RED_COL && pl.cluster) {                                              \
      dd_launch_cluster(dd_reduce_colc_kernel<T, C, OPC>, pl.grid, (unsigned)DD_COLC_THREADS, (unsigned)pl.p.S, h->stream, pl.p);  \
      DD_LAUNCHED(h, "reduce/col-cluster");                                                        \
      return DD_STATUS_SUCCESS;                                                                    \
    } else if (pl.kind == DD_RED_COL) {                                                            \
      if (pl.pdl) {                                                                                \
        if (pl.vec == 1) dd_launch_pdl(dd_reduce_col_kernel<T, C, OPC, 1, false>, pl.grid, 256u, h->stream, pl.p);   \
        else if (pl.vec == 2) { if constexpr (sizeof(T) == 2 && OPC >= 0) dd_launch_pdl(dd_reduce_col_kernel<T, C, OPC, 2, false>, pl.grid, 256u, h->stream, pl.p); }  \
        else dd_launch_pdl(dd_reduce_col_kernel<T, C, OPC, 0, false>, pl.grid, 256u, h->stream, pl.p);    \
      } else {                                                                                     \
        if (pl.vec == 1) dd_reduce_col_kernel<T, C, OPC, 1, false><<<pl.grid, 256, 0, h->stream>>>(pl.p);   \
        else if (pl.vec == 2) { if constexpr (sizeof(T) == 2 && OPC >= 0) dd_reduce_col_kernel<T, C, OPC, 2, false><<<pl.grid, 256, 0, h->stream>>>(pl.p); }  \
        else dd_reduce_col_kernel<T, C, OPC, 0, false><<<pl.grid, 256, 0, h->stream>>>(pl.p);    \
      }                                                                                            \
      DD_LAUNCHED(h, pl.vec == 2 ? "reduce/col-v8" : "reduce/col");                                \
    } else {                                                                                       \
      dd_reduce_generic_kernel<T, C, OPC><<<pl.grid, 256, 0, h->stream>>>(pl.g);                   \
      DD_LAUNCHED(h, "reduce/generic");                                                            \
      return DD_STATUS_SUCCESS;                                                                    \
    }                                                                                              \
    if (pl.p.S > 1 && pl.p.counters == nullptr) {                                                  \
      unsigned fg = dd_flat_grid(h, pl.p.S > 32 ? pl.nout * 32 : pl.nout, 256, 8);                 \
      dd_reduce_finish_kernel<T, C, OPC><<<fg, 256, 0, h->stream>>>(pl.p, pl.p.part);              \
      DD_LAUNCHED(h, pl.kind == DD_RED_ROW ? "reduce/row+finish" : "reduce/col+finish");           \
    }                                                                                              \
    return DD_STATUS_SUCCESS;                                                                      \
  }                                                                                                \
  template <int OPC>                                                                               \
  static ddStatus_t finish_opc_##T(ddHandle_t h, const ddRedPlan &pl, const void *part) {          \
    ddRedParams p = pl.p;                                                                          \
    p.S = pl.foldS > 0 ? pl.foldS : 1;                                                             \
    p.partialOnly = 0;                                                                             \
    if (pl.foldS < 0) {                                                                            \
      unsigned fs = dd_flat_grid(h, pl.nout, 256, 8);                                              \
      dd_reduce_fold_sets_kernel<T, C, OPC><<<fs, 256, 0, h->stream>>>(p, part, -pl.foldS);        \
      DD_LAUNCHED(h, "reduce/col+fold-sets");                                                      \
      return DD_STATUS_SUCCESS;                                                                    \
    }                                                                                              \
    unsigned fg = dd_flat_grid(h, p.S > 32 ? pl.nout * 32 : pl.nout, 256, 8);                      \
    dd_reduce_finish_kernel<T, C, OPC><<<fg, 256, 0, h->stream>>>(p, part);                        \
    DD_LAUNCHED(h, pl.foldS > 0 ? "reduce/col+fold-runs" : "reduce/finish");                       \
    return DD_STATUS_SUCCESS;                                                                      \
  }                                                                                                \
  template <int OPC>                                                                               \
  static ddStatus_t exchange_opc_##T(ddHandle_t h, const ddRedPlan &pl, const ddPeerParams &q) {   \
    ddRedParams p = pl.p;                                                                          \
    p.S = 1;                                                                                       \
    p.partialOnly = 0;                                                                             \
    int64_t g = (pl.nout + 255) / 256;                                                             \
    unsigned grid = (unsigned)(g < 1 ? 1 : (g > DD_PEER_GRID_MAX ? DD_PEER_GRID_MAX : g));         \
    dd_launch_pdl2(dd_reduce_exchange_kernel<T, C, OPC>, grid, 256u, h->stream, p, q);             \
    DD_LAUNCHED(h, "reduce/peer-exchange");                                                        \
    return DD_STATUS_SUCCESS;                                                                      \
  }                                                                                                \
  template <>                                                                                      \
  ddStatus_t dd_reduce_exchange_launch<T, C>(ddHandle_t h, const ddRedPlan &pl, const ddPeerParams &q) { \
    switch (pl.opc) {                                                                              \
      case DD_OPC_SUM: return exchange_opc_##T<DD_OPC_SUM>(h, pl, q);                              \
      case DD_OPC_SUMABS: return exchange_opc_##T<DD_OPC_SUMABS>(h, pl, q);                        \
      case DD_OPC_SUMSQ: return exchange_opc_##T<DD_OPC_SUMSQ>(h, pl, q);                          \
      case DD_OPC_PROD: return exchange_opc_##T<DD_OPC_PROD>(h, pl, q);                            \
      case DD_OPC_PRODNZ: return exchange_opc_##T<DD_OPC_PRODNZ>(h, pl, q);                        \
      case DD_OPC_MIN: return exchange_opc_##T<DD_OPC_MIN>(h, pl, q);                              \
      case DD_OPC_MAX: return exchange_opc_##T<DD_OPC_MAX>(h, pl, q);                              \
      case DD_OPC_AMAX: return exchange_opc_##T<DD_OPC_AMAX>(h, pl, q);                            \
      case DD_OPC_SUMPOW: return exchange_opc_##T<DD_OPC_SUM>(h, pl, q);  /* accumulators add */   \
    }                                                                                              \
    return DD_STATUS_INTERNAL_ERROR;                                                               \
  }                                                                                                \
  template <>                                                                                      \
  ddStatus_t dd_reduce_launch<T, C>(ddHandle_t h, const ddRedPlan &pl) {                           \
    switch (pl.opc) {                                                                              \
      case DD_OPC_SUM: return launch_opc_##T<DD_OPC_SUM>(h, pl);                                   \
      case DD_OPC_SUMABS: return launch_opc_##T<DD_OPC_SUMABS>(h, pl);                             \
      case DD_OPC_SUMSQ: return launch_opc_##T<DD_OPC_SUMSQ>(h, pl);                               \
      case DD_OPC_PROD: return launch_opc_##T<DD_OPC_PROD>(h, pl);                                 \
      case DD_OPC_PRODNZ: return launch_opc_##T<DD_OPC_PRODNZ>(h, pl);                             \
      case DD_OPC_MIN: return launch_opc_##T<DD_OPC_MIN>(h, pl);                                   \
      case DD_OPC_MAX: return launch_opc_##T<DD_OPC_MAX>(h, pl);                                   \
      case DD_OPC_AMAX: return launch_opc_##T<DD_OPC_AMAX>(h, pl);                                 \
      case DD_OPC_SUMPOW: return launch_opc_##T<DD_OPC_SUMPOW>(h, pl);                             \
    }                                                                                              \
    return DD_STATUS_INTERNAL_ERROR;                                                               \
  }                                                                                                \
  template <>                                                                                      \
  ddStatus_t dd_reduce_finish_launch<T, C>(ddHandle_t h, const ddRedPlan &pl, const void *part) {  \
    switch (pl.opc) {                                                                              \
      case DD_OPC_SUM: return finish_opc_##T<DD_OPC_SUM>(h, pl, part);                             \
      case DD_OPC_SUMABS: return finish_opc_##T<DD_OPC_SUMABS>(h, pl, part);                       \
      case DD_OPC_SUMSQ: return finish_opc_##T<DD_OPC_SUMSQ>(h, pl, part);                         \
      case DD_OPC_PROD: return finish_opc_##T<DD_OPC_PROD>(h, pl, part);                           \
      case DD_OPC_PRODNZ: return finish_opc_##T<DD_OPC_PRODNZ>(h, pl, part);                       \
      case DD_OPC_MIN: return finish_opc_##T<DD_OPC_MIN>(h, pl, part);                             \
      case DD_OPC_MAX: return finish_opc_##T<DD_OPC_MAX>(h, pl, part);                             \
      case DD_OPC_AMAX: return finish_opc_##T<DD_OPC_AMAX>(h, pl, part);                           \
      case DD_OPC_SUMPOW: return finish_opc_##T<DD_OPC_SUM>(h, pl, part);  /* accumulators add */  \
    }                                                                                              \
    return DD_STATUS_INTERNAL_ERROR;                                                               \
  }
