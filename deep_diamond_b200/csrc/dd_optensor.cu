// Op-tensor family: fill, scale, broadcast binary ops and the n-ary scaled sum (the bodies of
// ddSetTensor, ddScaleTensor, ddAddTensor, ddOpTensor, ddSumTensors).
//
//   C = op(alpha1*A, alpha2*bcast(B)) + beta*C
//
// Fast path ("flat"): A and C dense with identical strides, B either dense like A or indexed by one
// middle dim only (the bias / per-channel-scale case: dims collapse to [outer, channel, inner] with
// B varying along `channel`).  One 16-byte vector of A in, one of C out per thread-iteration; B comes
// from L1/L2 (a few KB).  Algorithmic bytes/element: 2*sizeof(T) (+ the tiny B).  Everything else
// runs through the strided kernel.  Each product and the final sums round separately (no FMA
// contraction), a factor of exactly 1 is skipped and a zero factor means "operand not read".
#include "dd_internal.cuh"

template <typename C>
__device__ __forceinline__ C dd_binop(int op, C a, C b) {
  switch (op) {
    case DD_OP_TENSOR_ADD: return dd_add_rn(a, b);
    case DD_OP_TENSOR_MUL: return dd_mul_rn(a, b);
    case DD_OP_TENSOR_MIN: return a < b ? a : b;
    case DD_OP_TENSOR_MAX: return a > b ? a : b;
    case DD_OP_TENSOR_SUB: return dd_add_rn(a, -b);
    case DD_OP_TENSOR_GE: return a >= b ? (C)1 : (C)0;
    case DD_OP_TENSOR_GT: return a > b ? (C)1 : (C)0;
    case DD_OP_TENSOR_LE: return a <= b ? (C)1 : (C)0;
    case DD_OP_TENSOR_LT: return a < b ? (C)1 : (C)0;
    case DD_OP_TENSOR_EQ: return a == b ? (C)1 : (C)0;
    case DD_OP_TENSOR_NE: return a != b ? (C)1 : (C)0;
    default: return a / b;  // DIV (IEEE round-to-nearest division)
  }
}

// Multiplying by a factor of exactly 1 is exact, so the hot loops multiply unconditionally
// (one instruction) instead of testing the factor per element; the result is the same bits as
// "a factor of exactly 1 is skipped".
template <typename C>
__device__ __forceinline__ C dd_times(C alpha, C v) { return dd_mul_rn(alpha, v); }

struct ddOpFlatParams {
  const void *A;
  const void *B;
  void *C;
  int64_t n;         // elements of A / C
  int64_t inner;     // bmode 1: run length over which B is constant
  int64_t channels;  // bmode 1: extent of the dim B varies along
  int64_t sB;        // bmode 1: B's stride along that dim
  int bmode;         // 0: B dense like A; 1: B indexed by channel
  int op;
  int readA;         // 0: alpha1 == 0, A is not read (its term is +0)
  int vec;
  int fast;          // n < 2^31: channel index by multiply-shift division
  ddFastDiv fdInner, fdChannels;
  double alpha1, alpha2, beta;
};

__device__ __forceinline__ int64_t dd_channel_of(const ddOpFlatParams &p, int64_t e) {
  if (p.fast) {
    uint32_t q = dd_div((uint32_t)e, p.fdInner), c, r;
    dd_divmod(q, p.fdChannels, c, r);
    return r;
  }
  return (e / p.inner) % p.channels;
}

// OP < 0: the op comes from p.op at run time (the less common ops share one instantiation).
template <typename T, typename C, int OP, int BMODE>
__global__ void __launch_bounds__(256, 8) dd_op_flat_kernel(ddOpFlatParams p) {
  dd_pdl_prologue();
  constexpr int V = 16 / sizeof(T);
  const T *A = (const T *)p.A;
  const T *B = (const T *)p.B;
  T *Cp = (T *)p.C;
  const C a1 = (C)p.alpha1, a2 = (C)p.alpha2, beta = (C)p.beta;
  const bool useOld = p.beta != 0.0, readA = p.readA != 0;
  const int op = OP < 0 ? p.op : OP;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  int64_t done = 0;
  if (p.vec) {
    const int64_t nv = p.n / V;
    for (int64_t i = tid; i < nv; i += nthreads) {
      const int64_t e0 = i * V;
      uint4 ain = make_uint4(0, 0, 0, 0), oin = make_uint4(0, 0, 0, 0), bin = make_uint4(0, 0, 0, 0);
      if (readA) ain = *(const uint4 *)(A + e0);
      if (useOld) oin = *(const uint4 *)(Cp + e0);
      C bs = (C)0;
      if (BMODE == 0) {
        bin = *(const uint4 *)(B + e0);
      } else if (BMODE == 1) {  // inner % V == 0: the whole vector shares one channel
        const int64_t ch = dd_channel_of(p, e0);
        bs = dd_times(a2, dd_load<C, T>(__ldg(B + ch * p.sB)));
      }
      // BMODE 2, 3, 4: runs of B's value that are not whole vectors, the accesses to A and C staying 16
      // bytes wide.  3: a run is at least a vector long (7 x 7 maps: 49 elements), so at most one run ends
      // inside a vector.  4: runs of one element and a whole vector inside one pixel (nhwc bias): B's
      // values are one aligned 16-byte load.  2: anything else, each element stepping the position
      int64_t ch2 = 0, pos2 = 0;
      if (BMODE == 4) {
        // nhwc: consecutive elements are consecutive channels and a whole vector lies inside one pixel
        int64_t ch0;
        if (p.fast) {
          uint32_t q, r;
          dd_divmod((uint32_t)e0, p.fdChannels, q, r);
          ch0 = r;
        } else {
          ch0 = e0 % p.channels;
        }
        bin = __ldg((const uint4 *)(B + ch0));
      } else if (BMODE == 2 || BMODE == 3) {
        if (p.fast) {
          uint32_t q, r, c;
          dd_divmod((uint32_t)e0, p.fdInner, q, r);
          dd_divmod(q, p.fdChannels, c, q);
          ch2 = q;
          pos2 = r;
        } else {
          const int64_t q = e0 / p.inner;
          pos2 = e0 - q * p.inner;
          ch2 = q % p.channels;
        }
        bs = dd_times(a2, dd_load<C, T>(__ldg(B + ch2 * p.sB)));
      }
      uint4 res;
      const T *av = (const T *)&ain, *bv = (const T *)&bin, *ov = (const T *)&oin;
      T *rv = (T *)&res;
      C rs[V];
      if (BMODE == 4) {
#pragma unroll
        for (int k = 0; k < V; k++) {
          C a = dd_times(a1, dd_load<C, T>(av[k]));
          C r = dd_binop<C>(op, a, dd_times(a2, dd_load<C, T>(bv[k])));
          if (useOld) r = dd_add_rn(r, dd_mul_rn(beta, dd_load<C, T>(ov[k])));
          rs[k] = r;
        }
      } else if (BMODE == 3) {
        // a run is at least a vector long, so at most ONE run ends inside this vector: both channels'
        // values are fetched up front and each element selects (no per-element position counter, no
        // load in the middle of the loop)
        const int64_t leftInRun = p.inner - pos2;
        const int kb = leftInRun < V ? (int)leftInRun : V;  // elements from kb on belong to the next channel
        C bs1 = bs;
        if (kb < V) {
          const int64_t chn = ch2 + 1 == p.channels ? 0 : ch2 + 1;
          bs1 = dd_times(a2, dd_load<C, T>(__ldg(B + chn * p.sB)));
        }
#pragma unroll
        for (int k = 0; k < V; k++) {
          C a = dd_times(a1, dd_load<C, T>(av[k]));
          C r = dd_binop<C>(op, a, k < kb ? bs : bs1);
          if (useOld) r = dd_add_rn(r, dd_mul_rn(beta, dd_load<C, T>(ov[k])));
          rs[k] = r;
        }
      } else {
#pragma unroll
        for (int k = 0; k < V; k++) {
          C a = dd_times(a1, dd_load<C, T>(av[k]));  // readA == 0: a1 == 0 and av == 0, the term is +0
          C b = BMODE == 0 ? dd_times(a2, dd_load<C, T>(bv[k])) : bs;
          C r = dd_binop<C>(op, a, b);
          if (useOld) r = dd_add_rn(r, dd_mul_rn(beta, dd_load<C, T>(ov[k])));
          rs[k] = r;
          if (BMODE == 2 && ++pos2 == p.inner) {  // the next element starts the next channel's run
            pos2 = 0;
            if (++ch2 == p.channels) ch2 = 0;
            bs = dd_times(a2, dd_load<C, T>(__ldg(B + ch2 * p.sB)));
          }
        }
      }
      dd_store_n<T, C, V>(rv, rs);
      *(uint4 *)(Cp + e0) = res;
    }
    done = nv * V;
  }
  for (int64_t i = done + tid; i < p.n; i += nthreads) {
    C a = readA ? dd_scale(a1, dd_load<C, T>(A[i])) : (C)0;
    C b = BMODE == 0 ? dd_load<C, T>(B[i]) : dd_load<C, T>(B[dd_channel_of(p, i) * p.sB]);
    C r = dd_binop<C>(op, a, dd_scale(a2, b));
    if (useOld) r = dd_add_rn(r, dd_mul_rn(beta, dd_load<C, T>(Cp[i])));
    Cp[i] = dd_store<T, C>(r);
  }
}

// Bias / per-channel scale (B constant over a run that is a whole number of vectors), no blend with
// the old C: TWO vectors per thread-iteration.  The operation is usually in place (C == A), so the
// compiler cannot start the next iteration's load before this one's store; here both loads (and both
// channel look-ups) go out before the first store.
template <typename T, typename C, int OP>
__global__ void __launch_bounds__(256, 8) dd_op_bcast2_kernel(ddOpFlatParams p) {
  dd_pdl_prologue();
  constexpr int V = 16 / sizeof(T);
  const T *A = (const T *)p.A;
  const T *B = (const T *)p.B;
  T *Cp = (T *)p.C;
  const C a1 = (C)p.alpha1, a2 = (C)p.alpha2;
  const uint32_t nv = (uint32_t)(p.n / V), nthreads = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += 2 * nthreads) {
    const uint32_t i2 = i + nthreads;
    const bool two = i2 < nv;
    const uint4 x0 = *(const uint4 *)(A + (size_t)i * V);
    uint4 x1 = make_uint4(0, 0, 0, 0);
    if (two) x1 = *(const uint4 *)(A + (size_t)i2 * V);
    uint32_t q, c0, c1, r;
    q = dd_div(i * V, p.fdInner);
    dd_divmod(q, p.fdChannels, r, c0);
    q = dd_div((two ? i2 : i) * V, p.fdInner);
    dd_divmod(q, p.fdChannels, r, c1);
    const C b0 = dd_times(a2, dd_load<C, T>(__ldg(B + (int64_t)c0 * p.sB)));
    const C b1 = dd_times(a2, dd_load<C, T>(__ldg(B + (int64_t)c1 * p.sB)));
    uint4 y0, y1;
    C r0[V], r1[V];
    const T *v0 = (const T *)&x0, *v1 = (const T *)&x1;
#pragma unroll
    for (int k = 0; k < V; k++) {
      r0[k] = dd_binop<C>(OP, dd_times(a1, dd_load<C, T>(v0[k])), b0);
      r1[k] = dd_binop<C>(OP, dd_times(a1, dd_load<C, T>(v1[k])), b1);
    }
    dd_store_n<T, C, V>((T *)&y0, r0);
    dd_store_n<T, C, V>((T *)&y1, r1);
    *(uint4 *)(Cp + (size_t)i * V) = y0;
    if (two) *(uint4 *)(Cp + (size_t)i2 * V) = y1;
  }
}

struct ddOpStridedParams {
  const void *A;
  const void *B;
  void *C;
  ddStridedParams<3> sp;  // operands 0 = A, 1 = B (stride 0 where broadcast), 2 = C
  int op;
  int readA;
  double alpha1, alpha2, beta;
};

template <typename T, typename C>
__global__ void __launch_bounds__(256) dd_op_strided_kernel(ddOpStridedParams p) {
  const T *A = (const T *)p.A;
  const T *B = (const T *)p.B;
  T *Cp = (T *)p.C;
  const C a1 = (C)p.alpha1, a2 = (C)p.alpha2, beta = (C)p.beta;
  const bool useOld = p.beta != 0.0, readA = p.readA != 0;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.sp.total; i += nthreads) {
    int64_t off[3];
    dd_offsets<3, int64_t>(p.sp, i, off);
    C a = readA ? dd_scale(a1, dd_load<C, T>(A[off[0]])) : (C)0;
    C b = dd_scale(a2, dd_load<C, T>(B[off[1]]));
    C r = dd_binop<C>(p.op, a, b);
    if (useOld) r = dd_add_rn(r, dd_mul_rn(beta, dd_load<C, T>(Cp[off[2]])));
    Cp[off[2]] = dd_store<T, C>(r);
  }
}

// Rows: A and C contiguous along the innermost dim (any outer strides), B contiguous or constant
// along it: the strided walk over 16-byte vectors.  `sp` counts the innermost dim in vectors of V
// elements; bInner is B's stride along it (0 or 1).
template <typename T, typename C>
__global__ void __launch_bounds__(256) dd_op_rows_kernel(ddOpStridedParams p, int bInner) {
  constexpr int V = 16 / sizeof(T);
  const T *A = (const T *)p.A;
  const T *B = (const T *)p.B;
  T *Cp = (T *)p.C;
  const C a1 = (C)p.alpha1, a2 = (C)p.alpha2, beta = (C)p.beta;
  const bool useOld = p.beta != 0.0, readA = p.readA != 0;
  const uint32_t total = (uint32_t)p.sp.total, nthreads = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nthreads) {
    int64_t off[3];
    dd_offsets32<3>(p.sp, i, off);
    uint4 ain = make_uint4(0, 0, 0, 0), oin = make_uint4(0, 0, 0, 0), bin = make_uint4(0, 0, 0, 0);
    if (readA) ain = *(const uint4 *)(A + off[0]);
    if (useOld) oin = *(const uint4 *)(Cp + off[2]);
    C bs = (C)0;
    if (bInner) bin = *(const uint4 *)(B + off[1]);
    else bs = dd_times(a2, dd_load<C, T>(__ldg(B + off[1])));
    uint4 res;
    const T *av = (const T *)&ain, *bv = (const T *)&bin, *ov = (const T *)&oin;
    T *rv = (T *)&res;
    C rs[V];
#pragma unroll
    for (int k = 0; k < V; k++) {
      C a = dd_times(a1, dd_load<C, T>(av[k]));
      C b = bInner ? dd_times(a2, dd_load<C, T>(bv[k])) : bs;
      C r = dd_binop<C>(p.op, a, b);
      if (useOld) r = dd_add_rn(r, dd_mul_rn(beta, dd_load<C, T>(ov[k])));
      rs[k] = r;
    }
    dd_store_n<T, C, V>(rv, rs);
    *(uint4 *)(Cp + off[2]) = res;
  }
}

template <typename T>
static bool dd_op_rows_ok(const ddCanon &c, const void *A, const void *B, const void *Cp, int readA) {
  constexpr int V = 16 / (int)sizeof(T);
  const int last = c.nd - 1;
  if (c.nd < 2 || c.dims[last] % V != 0 || c.total / V >= 0x7fffffffLL) return false;
  if (c.st[0][last] != 1 || c.st[2][last] != 1 || (c.st[1][last] != 0 && c.st[1][last] != 1)) return false;
  uintptr_t bits = (uintptr_t)Cp | (readA ? (uintptr_t)A : 0) | (c.st[1][last] == 1 ? (uintptr_t)B : 0);
  if (bits & 15) return false;
  for (int i = 0; i < last; i++) {
    if ((c.st[0][i] * (int64_t)sizeof(T)) % 16 != 0 || (c.st[2][i] * (int64_t)sizeof(T)) % 16 != 0) return false;
    if (c.st[1][last] == 1 && (c.st[1][i] * (int64_t)sizeof(T)) % 16 != 0) return false;
  }
  return true;
}

template <typename T, typename C>
static ddStatus_t optensor_typed(ddHandle_t h, ddOpTensorOp_t op, double alpha1,
                                 const ddTensorStruct *ad, const void *A, double alpha2,
                                 const ddTensorStruct *bd, const void *B, double beta,
                                 const ddTensorStruct *cd, void *Cp) {
  int64_t st[3][DD_DIM_MAX];
  for (int i = 0; i < cd->nd; i++) {
    st[0][i] = ad->strides[i];
    st[1][i] = bd->dims[i] == 1 && cd->dims[i] != 1 ? 0 : bd->strides[i];
    st[2][i] = cd->strides[i];
  }
  ddCanon c;
  dd_canonicalize(&c, cd->nd, cd->dims, 3, st, 2);
  // for ADD a zero factor on A means "A is not read" (beta == 0 semantics of ddAddTensor)
  const int readA = !(alpha1 == 0.0 && op == DD_OP_TENSOR_ADD);
  constexpr int V = 16 / sizeof(T);

  // dense A and C?  After canonicalisation they are dense iff, walking from the innermost dim,
  // each stride equals the product of the inner extents.
  bool dense = true;
  int64_t run = 1;
  for (int i = c.nd - 1; i >= 0; i--) {
    if (c.st[0][i] != run || c.st[2][i] != run) dense = false;
    run *= c.dims[i];
  }
  int bmode = -1;
  int64_t inner = 1, channels = 1, sB = 0;
  if (dense) {
    if (c.nd == 1 && c.st[1][0] == 1) {
      bmode = 0;
    } else {
      // B must vary along exactly one dim
      int vary = -1, nvary = 0;
      for (int i = 0; i < c.nd; i++)
        if (c.st[1][i] != 0) { vary = i; nvary++; }
      if (nvary == 1) {
        bmode = 1;
        channels = c.dims[vary];
        sB = c.st[1][vary];
        for (int i = vary + 1; i < c.nd; i++) inner *= c.dims[i];
      } else if (nvary == 0) {  // B is a single element
        bmode = 1;
        channels = 1;
        sB = 0;
        inner = c.total;
      }
    }
  }
  if (bmode >= 0) {
    ddOpFlatParams p;
    p.A = A;
    p.B = B;
    p.C = Cp;
    p.n = c.total;
    p.inner = inner;
    p.channels = channels;
    p.sB = sB;
    p.bmode = bmode;
    p.op = (int)op;
    p.readA = readA;
    p.alpha1 = alpha1;
    p.alpha2 = alpha2;
    p.beta = beta;
    uintptr_t bits = (uintptr_t)A | (uintptr_t)Cp | (bmode == 0 ? (uintptr_t)B : 0);
    p.vec = (bits & 15) == 0;
    if (bmode == 1 && inner % V != 0) bmode = dd_tune("DD_OP_MIXED", 1) ? 2 : (p.vec = 0, 1);
    p.bmode = bmode;
    if (bmode == 2) {
      if (inner == 1 && sB == 1 && channels % V == 0 && ((uintptr_t)B & 15) == 0) bmode = 4;
      else if (inner >= V) bmode = 3;
    }
    p.fast = c.total < 0x7fffffffLL;
    if (p.fast) {
      p.fdInner = dd_fastdiv((uint32_t)inner);
      p.fdChannels = dd_fastdiv((uint32_t)channels);
    }
    unsigned grid = dd_flat_grid(h, (p.n + V - 1) / V, 256, dd_tune("DD_OPFLAT_CPS", 32));
    // add and mul (bias, per-channel scale, axpy, sum) get their own instantiations
    if (bmode >= 2) {
      // add and mul in the two forms layers meet (bias and per-channel scale on nchw maps that are not
      // whole vectors, and on nhwc); every other combination shares the run-time-op instantiation
      if (op == DD_OP_TENSOR_ADD && bmode == 3) dd_launch_pdl(dd_op_flat_kernel<T, C, DD_OP_TENSOR_ADD, 3>, grid, 256, h->stream, p);
      else if (op == DD_OP_TENSOR_MUL && bmode == 3) dd_launch_pdl(dd_op_flat_kernel<T, C, DD_OP_TENSOR_MUL, 3>, grid, 256, h->stream, p);
      else if (op == DD_OP_TENSOR_ADD && bmode == 4) dd_launch_pdl(dd_op_flat_kernel<T, C, DD_OP_TENSOR_ADD, 4>, grid, 256, h->stream, p);
      else if (op == DD_OP_TENSOR_MUL && bmode == 4) dd_launch_pdl(dd_op_flat_kernel<T, C, DD_OP_TENSOR_MUL, 4>, grid, 256, h->stream, p);
      else if (bmode == 3) dd_launch_pdl(dd_op_flat_kernel<T, C, -1, 3>, grid, 256, h->stream, p);
      else if (bmode == 4) dd_launch_pdl(dd_op_flat_kernel<T, C, -1, 4>, grid, 256, h->stream, p);
      else dd_launch_pdl(dd_op_flat_kernel<T, C, -1, 2>, grid, 256, h->stream, p);
      DD_LAUNCHED(h, bmode == 4 ? "optensor/flat-bcast-vector" : "optensor/flat-bcast-mixed");
      return DD_STATUS_SUCCESS;
    }
    if (bmode == 1 && (op == DD_OP_TENSOR_ADD || op == DD_OP_TENSOR_MUL) && beta == 0.0 && readA && p.vec && p.fast &&
        p.n % V == 0 && p.n / V <= (int64_t)h->smCount * 8 * 256 * 16 && dd_tune("DD_OP_BCAST2", 1)) {
      // small tensors only (at most 16 vectors per thread of a resident grid): [128,512,14,14] f32 19.07 -> 18.38 us;
      // on 205 MB tensors the one-vector kernel measured 3 % faster
      unsigned g2 = dd_flat_grid(h, (p.n / V + 1) / 2, 256, dd_tune("DD_OPFLAT_CPS", 32));
      if (op == DD_OP_TENSOR_ADD) dd_launch_pdl(dd_op_bcast2_kernel<T, C, DD_OP_TENSOR_ADD>, g2, 256, h->stream, p);
      else dd_launch_pdl(dd_op_bcast2_kernel<T, C, DD_OP_TENSOR_MUL>, g2, 256, h->stream, p);
      DD_LAUNCHED(h, "optensor/flat-bcast");
      return DD_STATUS_SUCCESS;
    }
    if (op == DD_OP_TENSOR_ADD && bmode == 0) dd_launch_pdl(dd_op_flat_kernel<T, C, DD_OP_TENSOR_ADD, 0>, grid, 256, h->stream, p);
    else if (op == DD_OP_TENSOR_ADD) dd_launch_pdl(dd_op_flat_kernel<T, C, DD_OP_TENSOR_ADD, 1>, grid, 256, h->stream, p);
    else if (op == DD_OP_TENSOR_MUL && bmode == 0) dd_launch_pdl(dd_op_flat_kernel<T, C, DD_OP_TENSOR_MUL, 0>, grid, 256, h->stream, p);
    else if (op == DD_OP_TENSOR_MUL) dd_launch_pdl(dd_op_flat_kernel<T, C, DD_OP_TENSOR_MUL, 1>, grid, 256, h->stream, p);
    else if (bmode == 0) dd_launch_pdl(dd_op_flat_kernel<T, C, -1, 0>, grid, 256, h->stream, p);
    else dd_launch_pdl(dd_op_flat_kernel<T, C, -1, 1>, grid, 256, h->stream, p);
    DD_LAUNCHED(h, bmode == 0 ? "optensor/flat" : "optensor/flat-bcast");
    return DD_STATUS_SUCCESS;
  }
  ddOpStridedParams p;
  p.A = A;
  p.B = B;
  p.C = Cp;
  p.op = (int)op;
  p.readA = readA;
  p.alpha1 = alpha1;
  p.alpha2 = alpha2;
  p.beta = beta;
  if (dd_op_rows_ok<T>(c, A, B, Cp, readA)) {
    const int last = c.nd - 1;
    const int bInner = c.st[1][last] == 1;
    ddCanon v = c;
    v.dims[last] = c.dims[last] / V;
    v.st[0][last] = V;
    v.st[1][last] = bInner ? V : 0;
    v.st[2][last] = V;
    v.total = c.total / V;
    p.sp = dd_strided_params<3>(v);
    unsigned grid = dd_flat_grid(h, v.total, 256, 16);
    dd_op_rows_kernel<T, C><<<grid, 256, 0, h->stream>>>(p, bInner);
    DD_LAUNCHED(h, "optensor/rows");
    return DD_STATUS_SUCCESS;
  }
  p.sp = dd_strided_params<3>(c);
  unsigned grid = dd_flat_grid(h, c.total, 256, 16);
  dd_op_strided_kernel<T, C><<<grid, 256, 0, h->stream>>>(p);
  DD_LAUNCHED(h, "optensor/strided");
  return DD_STATUS_SUCCESS;
}

ddStatus_t dd_optensor_impl(ddHandle_t h, ddOpTensorOp_t op, double alpha1,
                            const ddTensorStruct *ad, const void *A, double alpha2,
                            const ddTensorStruct *bd, const void *B, double beta,
                            const ddTensorStruct *cd, void *C) {
  if (!dd_same_dims(ad, cd)) DD_FAIL(h, DD_STATUS_BAD_PARAM, "op-tensor: A and C dims differ");
  if (bd->nd != cd->nd) DD_FAIL(h, DD_STATUS_BAD_PARAM, "op-tensor: operand ranks differ");
  for (int i = 0; i < cd->nd; i++)
    if (bd->dims[i] != cd->dims[i] && bd->dims[i] != 1)
      DD_FAIL(h, DD_STATUS_BAD_PARAM, "op-tensor: dim %d of the broadcast operand must equal the destination's or be 1", i);
  if (ad->dtype != cd->dtype || bd->dtype != cd->dtype)
    DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "op-tensor: operands must share one data type");
  switch (cd->dtype) {
    case DD_DATA_FLOAT: return optensor_typed<float, float>(h, op, alpha1, ad, A, alpha2, bd, B, beta, cd, C);
    case DD_DATA_DOUBLE: return optensor_typed<double, double>(h, op, alpha1, ad, A, alpha2, bd, B, beta, cd, C);
    case DD_DATA_HALF: return optensor_typed<__half, float>(h, op, alpha1, ad, A, alpha2, bd, B, beta, cd, C);
    case DD_DATA_BFLOAT16: return optensor_typed<__nv_bfloat16, float>(h, op, alpha1, ad, A, alpha2, bd, B, beta, cd, C);
    case DD_DATA_INT8: return optensor_typed<int8_t, float>(h, op, alpha1, ad, A, alpha2, bd, B, beta, cd, C);
    case DD_DATA_UINT8: return optensor_typed<uint8_t, float>(h, op, alpha1, ad, A, alpha2, bd, B, beta, cd, C);
    case DD_DATA_INT32: return optensor_typed<int32_t, double>(h, op, alpha1, ad, A, alpha2, bd, B, beta, cd, C);
    default: break;
  }
  DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "op-tensor: unsupported data type");
}

// ------------------------------------------------------------------ set / scale --------------

struct ddFillParams {
  void *y;
  ddStridedParams<1> sp;
  double value;
  int scale;  // 0: y = value, 1: y *= value
  int flat;
};

template <typename T, typename C>
__global__ void __launch_bounds__(256) dd_fill_kernel(ddFillParams p) {
  T *y = (T *)p.y;
  const C v = (C)p.value;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (p.flat) {
    constexpr int V = 16 / sizeof(T);
    const int64_t n = p.sp.total;
    int64_t done = 0;
    if ((((uintptr_t)y) & 15) == 0) {
      const int64_t nv = n / V;
      for (int64_t i = tid; i < nv; i += nthreads) {
        uint4 w;
        T *wv = (T *)&w;
        if (p.scale) {
          w = *(const uint4 *)(y + i * V);
#pragma unroll
          for (int k = 0; k < V; k++) wv[k] = dd_store<T, C>(dd_mul_rn(v, dd_load<C, T>(wv[k])));
        } else {
#pragma unroll
          for (int k = 0; k < V; k++) wv[k] = dd_store<T, C>(v);
        }
        *(uint4 *)(y + i * V) = w;
      }
      done = nv * V;
    }
    for (int64_t i = done + tid; i < n; i += nthreads)
      y[i] = p.scale ? dd_store<T, C>(dd_mul_rn(v, dd_load<C, T>(y[i]))) : dd_store<T, C>(v);
  } else {
    for (int64_t i = tid; i < p.sp.total; i += nthreads) {
      int64_t off[1];
      dd_offsets<1, int64_t>(p.sp, i, off);
      y[off[0]] = p.scale ? dd_store<T, C>(dd_mul_rn(v, dd_load<C, T>(y[off[0]]))) : dd_store<T, C>(v);
    }
  }
}

template <typename T, typename C>
static ddStatus_t fill_typed(ddHandle_t h, const ddTensorStruct *yd, void *y, double value, int scale) {
  int64_t st[1][DD_DIM_MAX];
  for (int i = 0; i < yd->nd; i++) st[0][i] = yd->strides[i];
  ddCanon c;
  dd_canonicalize(&c, yd->nd, yd->dims, 1, st, 0);
  ddFillParams p;
  p.y = y;
  p.sp = dd_strided_params<1>(c);
  p.value = value;
  p.scale = scale;
  p.flat = c.nd == 1 && c.st[0][0] == 1;
  constexpr int V = 16 / sizeof(T);
  unsigned grid = dd_flat_grid(h, p.flat ? (c.total + V - 1) / V : c.total, 256, 48);  // 16 -> 48: fill +6.7 %, scale +1.8 %
  dd_fill_kernel<T, C><<<grid, 256, 0, h->stream>>>(p);
  DD_LAUNCHED(h, scale ? (p.flat ? "scale/flat" : "scale/strided") : (p.flat ? "set/flat" : "set/strided"));
  return DD_STATUS_SUCCESS;
}

static ddStatus_t fill_dispatch(ddHandle_t h, const ddTensorStruct *yd, void *y, double v, int scale) {
  switch (yd->dtype) {
    case DD_DATA_FLOAT: return fill_typed<float, float>(h, yd, y, v, scale);
    case DD_DATA_DOUBLE: return fill_typed<double, double>(h, yd, y, v, scale);
    case DD_DATA_HALF: return fill_typed<__half, float>(h, yd, y, v, scale);
    case DD_DATA_BFLOAT16: return fill_typed<__nv_bfloat16, float>(h, yd, y, v, scale);
    case DD_DATA_INT8: return fill_typed<int8_t, float>(h, yd, y, v, scale);
    case DD_DATA_UINT8: return fill_typed<uint8_t, float>(h, yd, y, v, scale);
    case DD_DATA_INT32: return fill_typed<int32_t, double>(h, yd, y, v, scale);
    case DD_DATA_INT64: return fill_typed<int64_t, double>(h, yd, y, v, scale);
  }
  DD_FAIL(h, DD_STATUS_BAD_PARAM, "unknown data type");
}

ddStatus_t dd_set_impl(ddHandle_t h, const ddTensorStruct *yd, void *y, double value) {
  return fill_dispatch(h, yd, y, value, 0);
}
ddStatus_t dd_scale_impl(ddHandle_t h, const ddTensorStruct *yd, void *y, double alpha) {
  return fill_dispatch(h, yd, y, alpha, 1);
}

// ------------------------------------------------------------------ n-ary sum ----------------

#define DD_SUM_MAX 8
struct ddSumParams {
  const void *src[DD_SUM_MAX];
  float scale[DD_SUM_MAX];
  void *dst;
  int n;
  int64_t total;
  int vec;
};

// dst = (((s0*x0) + s1*x1) + s2*x2) ... : one pass over n dense same-layout sources.
// Algorithmic bytes/element: (n + 1)*sizeof(T).
template <typename T, typename C>
__global__ void __launch_bounds__(256) dd_sum_kernel(ddSumParams p) {
  constexpr int V = 16 / sizeof(T);
  T *dst = (T *)p.dst;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  int64_t done = 0;
  if (p.vec) {
    const int64_t nv = p.total / V;
    for (int64_t i = tid; i < nv; i += nthreads) {
      C acc[V];
#pragma unroll
      for (int s = 0; s < DD_SUM_MAX; s++) {
        if (s < p.n) {
          uint4 in = *(const uint4 *)((const T *)p.src[s] + i * V);
          const T *iv = (const T *)&in;
          const C sc = (C)p.scale[s];
#pragma unroll
          for (int k = 0; k < V; k++) {
            C t = dd_scale(sc, dd_load<C, T>(iv[k]));
            acc[k] = s == 0 ? t : dd_add_rn(acc[k], t);
          }
        }
      }
      uint4 res;
      T *rv = (T *)&res;
      dd_store_n<T, C, V>(rv, acc);
      *(uint4 *)(dst + i * V) = res;
    }
    done = nv * V;
  }
  for (int64_t i = done + tid; i < p.total; i += nthreads) {
    C acc = (C)0;
    for (int s = 0; s < p.n; s++) {
      C t = dd_scale((C)p.scale[s], dd_load<C, T>(((const T *)p.src[s])[i]));
      acc = s == 0 ? t : dd_add_rn(acc, t);
    }
    dst[i] = dd_store<T, C>(acc);
  }
}

template <typename T, typename C>
static ddStatus_t sum_typed(ddHandle_t h, const ddSumParams &p) {
  constexpr int V = 16 / sizeof(T);
  // one resident wave: with three sources and a destination streaming side by side, 8 CTAs per SM measured
  // 6377-6387 GB/s on [256,256,28,28], 6: 6238, 12: 5848, 16: 5978, 4: 5518
  unsigned grid = dd_flat_grid(h, (p.total + V - 1) / V, 256, dd_tune("DD_SUM_CPS", 8));
  dd_sum_kernel<T, C><<<grid, 256, 0, h->stream>>>(p);
  DD_LAUNCHED(h, "sum/flat");
  return DD_STATUS_SUCCESS;
}

ddStatus_t dd_sum_impl(ddHandle_t h, int n, const float *scales, const ddTensorStruct *const *sd,
                       const void *const *srcs, const ddTensorStruct *dd, void *dst) {
  // one-pass kernel when every operand is dense with the destination's strides
  bool same = true;
  for (int s = 0; s < n; s++) {
    if (!dd_same_dims(sd[s], dd) || sd[s]->dtype != dd->dtype)
      DD_FAIL(h, DD_STATUS_BAD_PARAM, "ddSumTensors: source %d differs from dst in dims or data type", s);
    for (int i = 0; i < dd->nd; i++)
      if (dd->dims[i] != 1 && sd[s]->strides[i] != dd->strides[i]) same = false;
  }
  int64_t st[1][DD_DIM_MAX];
  for (int i = 0; i < dd->nd; i++) st[0][i] = dd->strides[i];
  ddCanon c;
  dd_canonicalize(&c, dd->nd, dd->dims, 1, st, 0);
  const bool flat = same && c.nd == 1 && c.st[0][0] == 1;
  if (flat) {
    ddSumParams p;
    memset(&p, 0, sizeof(p));
    p.n = n;
    p.total = c.total;
    p.dst = dst;
    uintptr_t bits = (uintptr_t)dst;
    for (int s = 0; s < n; s++) {
      p.src[s] = srcs[s];
      p.scale[s] = scales[s];
      bits |= (uintptr_t)srcs[s];
    }
    p.vec = (bits & 15) == 0;
    switch (dd->dtype) {
      case DD_DATA_FLOAT: return sum_typed<float, float>(h, p);
      case DD_DATA_DOUBLE: return sum_typed<double, double>(h, p);
      case DD_DATA_HALF: return sum_typed<__half, float>(h, p);
      case DD_DATA_BFLOAT16: return sum_typed<__nv_bfloat16, float>(h, p);
      default: DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "ddSumTensors: data type must be floating point");
    }
  }
  // general layouts: dst = s0*src0 (a transform), then dst += si*srci, one pass each
  ddStatus_t st0 = dd_transform_impl(h, (double)scales[0], sd[0], srcs[0], 0.0, dd, dst);
  if (st0 != DD_STATUS_SUCCESS) return st0;
  for (int s = 1; s < n; s++) {
    ddStatus_t r = dd_optensor_impl(h, DD_OP_TENSOR_ADD, 1.0, dd, dst, (double)scales[s], sd[s], srcs[s], 0.0, dd, dst);
    if (r != DD_STATUS_SUCCESS) return r;
  }
  return DD_STATUS_SUCCESS;
}
