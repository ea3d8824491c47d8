// Reorder + data type conversion kernels: y = alpha*convert(x) + beta*y over equal dims and any
// strides (the body of ddTransformTensor / ddGatherTransform).  Three kernel families:
//
//   flat     both tensors walk memory as one dense run (same layout): 16-byte vector stream.
//   tile     the x-contiguous dim (A) and the y-contiguous dim (B) differ (nchw <-> nhwc and every
//            other stride permutation whose rows are 16-byte aligned): a CTA moves a TA x TB tile;
//            each thread loads 16-byte vectors along A, converts, transposes its VS x VD micro
//            block in registers, parks 16-byte vectors along B in XOR-swizzled shared memory, and
//            the CTA writes them back as contiguous 16-byte vectors along B.  Global traffic is
//            16-byte on both sides, shared-memory traffic is conflict-free 16-byte on both sides.
//   strided  anything else: one element per thread, index decomposition over <= 8 dims.
//
// All three are HBM-bound: algorithmic bytes per element = sizeof(S) + sizeof(D).
#pragma once
#include "dd_internal.cuh"
#include <type_traits>

// ------------------------------------------------------------------ conversion ---------------

template <typename S, typename D, typename C, bool RAW>
struct dd_cvt {
  static __device__ __forceinline__ D f(S v, C alpha) {
    return dd_store<D, C>(dd_scale(alpha, dd_load<C, S>(v)));
  }
  static __device__ __forceinline__ D blend(S v, C alpha, C beta, D old) {
    C t = dd_scale(alpha, dd_load<C, S>(v));
    C u = dd_scale(beta, dd_load<C, D>(old));
    return dd_store<D, C>(dd_add_rn(t, u));
  }
};
// RAW: S == D (as an unsigned integer of the same width), alpha == 1, beta == 0: a bit copy.
template <typename S, typename C>
struct dd_cvt<S, S, C, true> {
  static __device__ __forceinline__ S f(S v, C) { return v; }
  static __device__ __forceinline__ S blend(S v, C, C, S) { return v; }
};

// The non-blending conversion of V consecutive elements: float -> bf16 / f16 in packed pairs
// (dd_store_n), anything else element by element.
template <typename S, typename D, typename C, bool RAW, int V>
__device__ __forceinline__ void dd_cvt_n(const S *sv, D *dv, C alpha) {
  if constexpr (!RAW && std::is_same<S, float>::value && std::is_same<C, float>::value && sizeof(D) == 2 &&
                (std::is_same<D, __nv_bfloat16>::value || std::is_same<D, __half>::value)) {
    float t[V];
#pragma unroll
    for (int k = 0; k < V; k++) t[k] = dd_scale(alpha, sv[k]);
    dd_store_n<D, float, V>(dv, t);
  } else {
#pragma unroll
    for (int k = 0; k < V; k++) dv[k] = dd_cvt<S, D, C, RAW>::f(sv[k], alpha);
  }
}

// ------------------------------------------------------------------ flat ---------------------

// BYTES of payload moved with the widest legal accesses (16-byte units above 16 bytes).
template <int BYTES> struct dd_vec_unit { typedef uint4 U; };
template <> struct dd_vec_unit<8> { typedef uint2 U; };
template <> struct dd_vec_unit<4> { typedef uint32_t U; };
template <> struct dd_vec_unit<2> { typedef uint16_t U; };
template <> struct dd_vec_unit<1> { typedef uint8_t U; };

template <int BYTES>
struct dd_vec {
  typedef typename dd_vec_unit<BYTES> ::U U;
  static constexpr int N = BYTES <= 16 ? 1 : BYTES / 16;
  U v[N];
};

template <int BYTES>
__device__ __forceinline__ dd_vec<BYTES> dd_vload(const void *p) {
  dd_vec<BYTES> r;
  typedef typename dd_vec<BYTES>::U U;
#pragma unroll
  for (int i = 0; i < dd_vec<BYTES>::N; i++) r.v[i] = ((const U *)p)[i];
  return r;
}
template <int BYTES>
__device__ __forceinline__ void dd_vstore(void *p, const dd_vec<BYTES> &r) {
  typedef typename dd_vec<BYTES>::U U;
#pragma unroll
  for (int i = 0; i < dd_vec<BYTES>::N; i++) ((U *)p)[i] = r.v[i];
}

struct ddFlatParams {
  const void *x;
  void *y;
  int64_t n;     // elements
  double alpha, beta;
  int vec;       // 1: both pointers 16-byte aligned, vector main loop + scalar tail
};

// V = elements per thread-iteration so that the narrower side still moves 16 bytes.
template <typename S, typename D, typename C, bool RAW>
__global__ void __launch_bounds__(256) dd_flat_kernel(ddFlatParams p) {
  constexpr int MINW = sizeof(S) < sizeof(D) ? sizeof(S) : sizeof(D);
  constexpr int V = 16 / MINW;
  const S *x = (const S *)p.x;
  D *y = (D *)p.y;
  const C alpha = (C)p.alpha, beta = (C)p.beta;
  const bool blend = p.beta != 0.0;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  int64_t done = 0;
  if (p.vec) {
    const int64_t nv = p.n / V;
    for (int64_t i = tid; i < nv; i += nthreads) {
      dd_vec<V * sizeof(S)> in = dd_vload<V * sizeof(S)>(x + i * V);
      dd_vec<V * sizeof(D)> out;
      const S *sv = (const S *)&in;
      D *dv = (D *)&out;
      if (blend) {
        dd_vec<V * sizeof(D)> old = dd_vload<V * sizeof(D)>(y + i * V);
        const D *ov = (const D *)&old;
#pragma unroll
        for (int k = 0; k < V; k++) dv[k] = dd_cvt<S, D, C, RAW>::blend(sv[k], alpha, beta, ov[k]);
      } else {
        dd_cvt_n<S, D, C, RAW, V>(sv, dv, alpha);
      }
      dd_vstore<V * sizeof(D)>(y + i * V, out);
    }
    done = nv * V;
  }
  for (int64_t i = done + tid; i < p.n; i += nthreads) {
    y[i] = blend ? dd_cvt<S, D, C, RAW>::blend(x[i], alpha, beta, y[i])
                 : dd_cvt<S, D, C, RAW>::f(x[i], alpha);
  }
}

// ------------------------------------------------------------------ tile ---------------------

#define DD_TILE_BATCH_DIMS 6

struct ddTileParams {
  const void *x;
  void *y;
  int64_t LA, LB;    // extents of dim A (stride 1 in x) and dim B (stride 1 in y)
  int64_t sxB, syA;  // x stride along B, y stride along A (elements)
  int nb;            // number of batch dims
  int64_t bdims[DD_TILE_BATCH_DIMS], bsx[DD_TILE_BATCH_DIMS], bsy[DD_TILE_BATCH_DIMS];
  int64_t tilesA, tilesB;
  ddFastDiv fdA, fdB, fdBatch[DD_TILE_BATCH_DIMS];  // divisors tilesA, tilesB, bdims[] (tile count < 2^31)
  uint32_t ntiles;   // all tiles; a CTA takes tiles blockIdx.x, blockIdx.x + gridDim.x, ...
  int na, nbLog2;    // vector tile kernel: CTA of na x (1 << nbLog2) threads
  ddFastDiv fdNA;
  double alpha;
};

template <typename S, typename D>
struct dd_tile_geom {
  static constexpr int VS = 16 / sizeof(S);  // elements per 16-byte load along A
  static constexpr int VD = 16 / sizeof(D);  // elements per 16-byte store along B
  static constexpr int NA = 16;              // threads along A, at most
  static constexpr int NB = (VS >= 16) ? 8 : 16;  // threads along B when NA > 8 (keeps the tile <= 32 KB)
  static constexpr int NT = NA * NB;         // threads per CTA, at most
  static constexpr int SMEM = NA * VS * NB * 16;
  // resident CTAs per SM the bit-copy kernels are held to: 8 CTAs of 256 threads (32 registers per
  // thread) for 4- and 8-byte elements; narrower elements keep more 16-byte loads in flight per
  // thread (8 or 16) and take the registers that needs
  static constexpr int MINB_RAW = VS <= 4 ? 8 : 0;
};

// The CTA is na x nb threads (ddTileParams): na <= 16 lanes along A, chosen on the host by the
// padding the edge tiles would carry (784 bytes of int8 are 49 vectors: 4 tiles of 13 lanes, where
// 16 lanes would leave the fourth tile 6 % full), and nb = NB lanes along B, 2 NB when na <= 8.
// The tile is TA = na * VS elements along A by TB = nb * VD along B.  A CTA walks the tiles
// blockIdx.x, blockIdx.x + gridDim.x, ...: the grid is either one CTA per tile or, for the
// converting kernels, one resident wave.
template <typename S, typename D, typename C, bool RAW>
__global__ void __launch_bounds__((dd_tile_geom<S, D>::NT), (RAW ? dd_tile_geom<S, D>::MINB_RAW : 0)) dd_tile_kernel(ddTileParams p) {
  typedef dd_tile_geom<S, D> G;
  constexpr int VS = G::VS, VD = G::VD;
  __shared__ uint4 tile[G::SMEM / 16];
  dd_pdl_prologue();
  const int NA = p.na, NB = 1 << p.nbLog2;
  const int TA = NA * VS, TB = NB * VD;
  const int SWZ = NB >= 8 ? 7 : NB - 1;  // the swizzle stays inside a row of NB chunks
  const int t = threadIdx.x;
  const C alpha = (C)p.alpha;

  for (uint32_t tileId = blockIdx.x; tileId < p.ntiles; tileId += gridDim.x) {
    // tile id -> (batch index, tile along B, tile along A); A varies fastest
    uint32_t id = tileId, ta, tb;
    dd_divmod(id, p.fdA, id, ta);
    dd_divmod(id, p.fdB, id, tb);
    int64_t offx = 0, offy = 0;
    for (int d = p.nb - 1; d >= 0; d--) {
      uint32_t r;
      dd_divmod(id, p.fdBatch[d], id, r);
      offx += (int64_t)r * p.bsx[d];
      offy += (int64_t)r * p.bsy[d];
    }
    const S *xb = (const S *)p.x + offx;
    D *yb = (D *)p.y + offy;
    const int64_t a0 = (int64_t)ta * TA, b0 = (int64_t)tb * TB;

    {  // load 16-byte vectors along A for VD consecutive rows of B, convert, transpose in registers
      uint32_t mbU, maU;
      dd_divmod((uint32_t)t, p.fdNA, mbU, maU);
      const int ma = (int)maU, mb = (int)mbU;  // lanes run along A first
      const int64_t a = a0 + ma * VS;
      // one 64-bit multiplication per thread: the rows follow at a fixed step, and what is left of
      // the tensor below this thread's first row fits an int
      const int64_t bFirst = b0 + mb * VD;
      const int64_t left = p.LB - bFirst;
      const int rows = a < p.LA ? (left < VD ? (left > 0 ? (int)left : 0) : VD) : 0;
      const S *src = xb + bFirst * p.sxB + a;
      uint4 in[VD];
#pragma unroll
      for (int j = 0; j < VD; j++) {
        in[j] = j < rows ? *(const uint4 *)src : make_uint4(0, 0, 0, 0);
        src += p.sxB;
      }
      __align__(16) D reg[VS][VD];
      if constexpr (RAW && sizeof(S) == 1 && sizeof(D) == 1) {
        // 16 x 16 bytes as sixteen 4 x 4 byte blocks, each transposed with 8 byte permutes: word w of
        // rows 4jj..4jj+3 becomes word jj of columns 4w..4w+3
        uint4 *outv = (uint4 *)&reg[0][0];
#pragma unroll
        for (int w = 0; w < 4; w++) {
          uint32_t c[4][4];
#pragma unroll
          for (int jj = 0; jj < 4; jj++) {
            const uint32_t r0 = (&in[4 * jj + 0].x)[w], r1 = (&in[4 * jj + 1].x)[w];
            const uint32_t r2 = (&in[4 * jj + 2].x)[w], r3 = (&in[4 * jj + 3].x)[w];
            const uint32_t t0 = __byte_perm(r0, r1, 0x5140), t1 = __byte_perm(r0, r1, 0x7362);
            const uint32_t t2 = __byte_perm(r2, r3, 0x5140), t3 = __byte_perm(r2, r3, 0x7362);
            c[0][jj] = __byte_perm(t0, t2, 0x5410);
            c[1][jj] = __byte_perm(t0, t2, 0x7632);
            c[2][jj] = __byte_perm(t1, t3, 0x5410);
            c[3][jj] = __byte_perm(t1, t3, 0x7632);
          }
#pragma unroll
          for (int k = 0; k < 4; k++) outv[4 * w + k] = make_uint4(c[k][0], c[k][1], c[k][2], c[k][3]);
        }
      } else if constexpr (std::is_same<S, float>::value && std::is_same<C, float>::value &&
                           (std::is_same<D, __nv_bfloat16>::value || std::is_same<D, __half>::value)) {
        // two rows at a time: one packed conversion (cvt.rn.{bf16x2,f16x2}.f32) makes the adjacent pair
        // reg[i][j], reg[i][j+1]; each half is the same rounding as the single conversion
#pragma unroll
        for (int j = 0; j < VD; j += 2) {
          const float *s0 = (const float *)&in[j], *s1 = (const float *)&in[j + 1];
#pragma unroll
          for (int i = 0; i < VS; i++) {
            const float lo = dd_scale(alpha, s0[i]), hi = dd_scale(alpha, s1[i]);
            if constexpr (std::is_same<D, __nv_bfloat16>::value) *(__nv_bfloat162 *)&reg[i][j] = __floats2bfloat162_rn(lo, hi);
            else *(__half2 *)&reg[i][j] = __floats2half2_rn(lo, hi);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < VD; j++) {
          const S *sv = (const S *)&in[j];
#pragma unroll
          for (int i = 0; i < VS; i++) reg[i][j] = dd_cvt<S, D, C, RAW>::f(sv[i], alpha);
        }
      }
      // row = index along A inside the tile; 16-byte chunk index along B swizzled by the row's
      // micro-block number so that the 8 lanes of a quarter warp hit 8 different bank groups
      uint4 *dstRow = tile + (((ma * VS) << p.nbLog2) + (mb ^ (ma & SWZ)));
#pragma unroll
      for (int i = 0; i < VS; i++) dstRow[i << p.nbLog2] = *(const uint4 *)reg[i];
    }
    __syncthreads();
    {  // write rows of the tile: NB consecutive lanes cover one contiguous run along B
      const int rb = t & (NB - 1), ra = t >> p.nbLog2;  // lanes run along B first
      const int64_t b = b0 + rb * VD;
      const int64_t leftA = p.LA - a0;
      const int rowsA = b < p.LB ? (leftA < TA ? (int)leftA : TA) : 0;  // rows of this tile inside the tensor
      D *dst = yb + (a0 + ra) * p.syA + b;
      const int64_t step = (int64_t)NA * p.syA;
#pragma unroll
      for (int k = 0; k < VS; k++) {
        const int row = ra + k * NA;
        if (row < rowsA) {
          uint4 v = tile[(row << p.nbLog2) + (rb ^ ((row / VS) & SWZ))];
          *(uint4 *)dst = v;
        }
        dst += step;
      }
    }
    if (tileId + gridDim.x < p.ntiles) __syncthreads();  // the next tile reuses the shared-memory stage
  }
}

// Scalar tile: the same A/B transposition for tensors whose rows are not 16-byte aligned (odd
// spatial sizes, odd channel counts, unaligned bases).  32 x 32 elements per CTA through a padded
// shared-memory tile: warps read 32 consecutive elements along A and write 32 consecutive elements
// along B, so both global sides stay coalesced (at element, not 16-byte, granularity).
template <typename S, typename D, typename C, bool RAW>
__global__ void __launch_bounds__(256) dd_tile_scalar_kernel(ddTileParams p) {
  __shared__ D tile[32][33];
  uint32_t id = blockIdx.x, ta, tb;
  dd_divmod(id, p.fdA, id, ta);
  dd_divmod(id, p.fdB, id, tb);
  int64_t offx = 0, offy = 0;
  for (int d = p.nb - 1; d >= 0; d--) {
    uint32_t r;
    dd_divmod(id, p.fdBatch[d], id, r);
    offx += (int64_t)r * p.bsx[d];
    offy += (int64_t)r * p.bsy[d];
  }
  const S *xb = (const S *)p.x + offx;
  D *yb = (D *)p.y + offy;
  const int64_t a0 = (int64_t)ta * 32, b0 = (int64_t)tb * 32;
  const C alpha = (C)p.alpha;
  const int lx = threadIdx.x & 31, ly = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const int64_t b = b0 + ly + 8 * k, a = a0 + lx;
    if (a < p.LA && b < p.LB) tile[ly + 8 * k][lx] = dd_cvt<S, D, C, RAW>::f(xb[b * p.sxB + a], alpha);
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const int64_t a = a0 + ly + 8 * k, b = b0 + lx;
    if (a < p.LA && b < p.LB) yb[a * p.syA + b] = tile[lx][ly + 8 * k];
  }
}

// ------------------------------------------------------------------ tile, short odd rows ------
// The same A/B transposition when the rows on ONE side are short and not 16-byte aligned (7 x 7,
// 13 x 13, 14 x 14 maps of an nchw tensor: rows of 49, 169, 196 elements) while the block those rows
// form is contiguous and starts on a 16-byte boundary.  That side is then moved as a FLAT stream of
// aligned 16-byte vectors that pays no attention to where rows begin, the other side with 16-byte
// vectors along its own rows, and shared memory (element accesses, which are cheap there) does the
// re-indexing between the two.  Against dd_tile_scalar_kernel, whose global accesses are single
// elements: 16-byte global accesses on both sides for every element width.
//
//   flat-in   x[batch][b][a] with rows of LA elements back to back (sxB == LA): a CTA copies `rows`
//             rows of B (a contiguous chunk of x) into shared memory as it lies, then writes, for
//             every a, 16-byte vectors along b gathered from the chunk.
//   flat-out  y[batch][a][b] with rows of LB elements back to back (syA == LB): a CTA reads `rows`
//             elements of A for every b (16-byte vectors along a) into a pitched shared-memory
//             matrix, then writes its chunk of y as flat 16-byte vectors gathered from it.
struct ddTileFlatParams {
  const void *x;
  void *y;
  int64_t LA, LB;
  int64_t sxB, syA;          // flat-in: sxB == LA; flat-out: syA == LB
  int nb;
  int64_t bdims[DD_TILE_BATCH_DIMS], bsx[DD_TILE_BATCH_DIMS], bsy[DD_TILE_BATCH_DIMS];
  ddFastDiv fdBatch[DD_TILE_BATCH_DIMS];
  int rows;                  // rows of B (flat-in) or of A (flat-out) per CTA, a multiple of 16
  uint32_t chunks;           // CTAs per batch entry
  ddFastDiv fdChunks;
  ddFastDiv fdInner;         // flat-in: 2 * LA (output items run a-fastest in pairs along b); flat-out: LB
  ddFastDiv fdVPR;           // flat-out: 16-byte vectors per full row of the chunk (rows / VS, at most 256)
  int pitch;                 // flat-out: elements of S between rows of the shared-memory matrix
  unsigned smemBytes;
  double alpha;
};

template <typename S>
__device__ __forceinline__ void dd_tile_flat_batch(const ddTileFlatParams &p, uint32_t id, int64_t &offx, int64_t &offy) {
  offx = 0;
  offy = 0;
  for (int d = p.nb - 1; d >= 0; d--) {
    uint32_t r;
    dd_divmod(id, p.fdBatch[d], id, r);
    offx += (int64_t)r * p.bsx[d];
    offy += (int64_t)r * p.bsy[d];
  }
}

template <typename S, typename D, typename C, bool RAW>
__global__ void __launch_bounds__(256) dd_tile_flatin_kernel(ddTileFlatParams p) {
  constexpr int VS = 16 / sizeof(S), VD = 16 / sizeof(D);
  extern __shared__ __align__(16) unsigned char dd_flat_smem[];
  S *chunk = (S *)dd_flat_smem;
  dd_pdl_prologue();
  uint32_t batch, ck;
  dd_divmod(blockIdx.x, p.fdChunks, batch, ck);
  int64_t offx, offy;
  dd_tile_flat_batch<S>(p, batch, offx, offy);
  const int64_t b0 = (int64_t)ck * p.rows;
  const int rb = (int)(p.LB - b0 < p.rows ? p.LB - b0 : p.rows);  // rows of B in this chunk (a multiple of VD)
  const int LA = (int)p.LA;
  const S *xc = (const S *)p.x + offx + b0 * LA;                  // 16-byte aligned: b0 is a multiple of 16
  const int n = rb * LA;
  const C alpha = (C)p.alpha;
  {  // the chunk as it lies: 16-byte vectors, then the few elements that do not fill one
    const int nv = n / VS;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) ((uint4 *)chunk)[i] = ((const uint4 *)xc)[i];
    for (int i = nv * VS + threadIdx.x; i < n; i += blockDim.x) chunk[i] = xc[i];
  }
  __syncthreads();
  // output items: (pair of 16-byte vectors along b) x (a), lanes running over the two vectors of a
  // pair first (one 32-byte sector) and over a next
  D *yc = (D *)p.y + offy + b0;
  const int nvb = rb / VD;
  const uint32_t items = (uint32_t)(((nvb + 1) / 2) * 2 * LA);
  for (uint32_t i = threadIdx.x; i < items; i += blockDim.x) {
    uint32_t pr, rem;
    dd_divmod(i, p.fdInner, pr, rem);
    const int a = (int)(rem >> 1), bv = (int)(pr * 2 + (rem & 1u));
    if (bv >= nvb) continue;
    const S *src = chunk + (size_t)(bv * VD) * LA + a;
    __align__(16) D out[VD];
#pragma unroll
    for (int j = 0; j < VD; j++) out[j] = dd_cvt<S, D, C, RAW>::f(src[(size_t)j * LA], alpha);
    *(uint4 *)(yc + (int64_t)a * p.syA + bv * VD) = *(const uint4 *)out;
  }
}

template <typename S, typename D, typename C, bool RAW>
__global__ void __launch_bounds__(256) dd_tile_flatout_kernel(ddTileFlatParams p) {
  constexpr int VS = 16 / sizeof(S), VD = 16 / sizeof(D);
  extern __shared__ __align__(16) unsigned char dd_flat_smem[];
  S *mat = (S *)dd_flat_smem;  // [LB][pitch]; the pitch is an odd number of 32-bit words (of 64-bit ones for 8-byte S)
  dd_pdl_prologue();
  uint32_t batch, ck;
  dd_divmod(blockIdx.x, p.fdChunks, batch, ck);
  int64_t offx, offy;
  dd_tile_flat_batch<S>(p, batch, offx, offy);
  const int64_t a0 = (int64_t)ck * p.rows;
  const int ra = (int)(p.LA - a0 < p.rows ? p.LA - a0 : p.rows);  // elements of A in this chunk (a multiple of VS)
  const int LB = (int)p.LB;
  const S *xc = (const S *)p.x + offx + a0;
  const C alpha = (C)p.alpha;
  {  // rows of x (16-byte vectors along a) into the matrix, 32 bits at a time (the pitch is not a
     // multiple of 16 bytes); threads run over the vectors of a row first
    const int nva = ra / VS;
    uint32_t tb, tv;
    dd_divmod(threadIdx.x, p.fdVPR, tb, tv);
    const int step = (int)(blockDim.x / p.fdVPR.d);
    if ((int)tv < nva)
      for (int b = (int)tb; b < LB; b += step) {
        const uint4 in = *(const uint4 *)(xc + (int64_t)b * p.sxB + tv * VS);
        uint32_t *dst = (uint32_t *)(mat + (size_t)b * p.pitch + tv * VS);
        dst[0] = in.x; dst[1] = in.y; dst[2] = in.z; dst[3] = in.w;
      }
  }
  __syncthreads();
  // the chunk of y, a0 * LB elements into the batch entry's block, as flat 16-byte vectors
  D *yc = (D *)p.y + offy + a0 * LB;
  const int n = ra * LB;
  const int nv = n / VD;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    uint32_t ar, b;
    dd_divmod((uint32_t)(i * VD), p.fdInner, ar, b);
    __align__(16) D out[VD];
#pragma unroll
    for (int j = 0; j < VD; j++) {
      out[j] = dd_cvt<S, D, C, RAW>::f(mat[(size_t)b * p.pitch + ar], alpha);
      if (++b == (uint32_t)LB) { b = 0; ar++; }
    }
    *(uint4 *)(yc + (int64_t)i * VD) = *(const uint4 *)out;
  }
  for (int f = nv * VD + threadIdx.x; f < n; f += blockDim.x) {
    uint32_t ar, b;
    dd_divmod((uint32_t)f, p.fdInner, ar, b);
    yc[f] = dd_cvt<S, D, C, RAW>::f(mat[(size_t)b * p.pitch + ar], alpha);
  }
}

// ------------------------------------------------------------------ strided ------------------

struct ddStridedXformParams {
  const void *x;
  void *y;
  ddStridedParams<2> sp;  // operand 0 = x, operand 1 = y
  double alpha, beta;
};

template <typename S, typename D, typename C, bool RAW, typename I>
__global__ void __launch_bounds__(256) dd_strided_kernel(ddStridedXformParams p) {
  const S *x = (const S *)p.x;
  D *y = (D *)p.y;
  const C alpha = (C)p.alpha, beta = (C)p.beta;
  const bool blend = p.beta != 0.0;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.sp.total; i += nthreads) {
    int64_t off[2];
    dd_offsets<2, I>(p.sp, (I)i, off);
    S v = x[off[0]];
    y[off[1]] = blend ? dd_cvt<S, D, C, RAW>::blend(v, alpha, beta, y[off[1]])
                      : dd_cvt<S, D, C, RAW>::f(v, alpha);
  }
}

// Rows: the innermost dim has stride 1 on both sides (sub-tensor windows, swapped outer dims,
// padded outer strides), so the walk is the strided one over 16-byte vectors instead of elements.
// `sp` counts the innermost dim in vectors of V elements (extent / V, stride V).
template <typename S, typename D, typename C, bool RAW>
__global__ void __launch_bounds__(256) dd_rows_kernel(ddStridedXformParams p) {
  constexpr int MINW = sizeof(S) < sizeof(D) ? sizeof(S) : sizeof(D);
  constexpr int V = 16 / MINW;
  const S *x = (const S *)p.x;
  D *y = (D *)p.y;
  const C alpha = (C)p.alpha, beta = (C)p.beta;
  const bool blend = p.beta != 0.0;
  const uint32_t total = (uint32_t)p.sp.total, nthreads = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nthreads) {
    int64_t off[2];
    dd_offsets<2, uint32_t>(p.sp, i, off);
    dd_vec<V * sizeof(S)> in = dd_vload<V * sizeof(S)>(x + off[0]);
    dd_vec<V * sizeof(D)> out;
    const S *sv = (const S *)&in;
    D *dv = (D *)&out;
    if (blend) {
      dd_vec<V * sizeof(D)> old = dd_vload<V * sizeof(D)>(y + off[1]);
      const D *ov = (const D *)&old;
#pragma unroll
      for (int k = 0; k < V; k++) dv[k] = dd_cvt<S, D, C, RAW>::blend(sv[k], alpha, beta, ov[k]);
    } else {
      dd_cvt_n<S, D, C, RAW, V>(sv, dv, alpha);
    }
    dd_vstore<V * sizeof(D)>(y + off[1], out);
  }
}

// Gather form: `count` items, item k starts at element offsets so[k] / do_[k]; inside an item the
// walk is the strided one.  Offsets travel in the kernel parameters (no device scratch).
#define DD_GATHER_CHUNK 1024
struct ddGatherParams {
  const void *x;
  void *y;
  ddStridedParams<2> sp;  // one item
  int count;
  int64_t so[DD_GATHER_CHUNK], do_[DD_GATHER_CHUNK];
};

template <typename S, typename D, typename C, bool RAW>
__global__ void __launch_bounds__(256) dd_gather_kernel(const __grid_constant__ ddGatherParams p) {
  const S *x = (const S *)p.x;
  D *y = (D *)p.y;
  const int64_t per = p.sp.total;
  const int64_t total = per * p.count;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nthreads) {
    const int64_t k = i / per;
    const int64_t r = i - k * per;
    int64_t off[2];
    dd_offsets<2, int64_t>(p.sp, r, off);
    y[p.do_[k] + off[1]] = dd_cvt<S, D, C, RAW>::f(x[p.so[k] + off[0]], (C)1);
  }
}

// Dense gather: every item is one contiguous run on both sides, the destinations follow one
// another at a fixed step (what a shuffler or batcher produces), and the source offsets are
// multiples of one unit.  Up to 4096 items then fit the parameters of ONE launch as 32-bit indices,
// and the copy runs as a flat stream: a multiply-shift division finds the item of each 16-byte
// vector, consecutive threads copy consecutive vectors.
#define DD_GATHER_SEQ_MAX 4096
struct ddGatherSeqParams {
  const void *x;
  void *y;
  uint32_t total;    // count * vpi
  uint32_t vpi;      // accesses (16-byte vectors or single elements) per item
  ddFastDiv fdVpi;
  int64_t unit;      // source offset of item k: so[k] * unit elements
  int64_t d0, dstep; // destination offset of item k: d0 + k * dstep elements
  uint32_t so[DD_GATHER_SEQ_MAX];
};

template <typename S, typename D, typename C, bool RAW, bool VEC>
__global__ void __launch_bounds__(256) dd_gather_dense_kernel(const __grid_constant__ ddGatherSeqParams p) {
  static_assert(!VEC || sizeof(S) == sizeof(D), "the vector form copies equal-width elements");
  constexpr int V = VEC ? 16 / (int)sizeof(S) : 1;
  const S *x = (const S *)p.x;
  D *y = (D *)p.y;
  const uint32_t nthreads = gridDim.x * blockDim.x;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += nthreads) {
    uint32_t k, r;
    dd_divmod(i, p.fdVpi, k, r);
    const S *src = x + (int64_t)p.so[k] * p.unit + (int64_t)r * V;
    D *dst = y + p.d0 + (int64_t)k * p.dstep + (int64_t)r * V;
    if (VEC) {
      uint4 v = *(const uint4 *)src;
      if (!RAW) {
        uint4 o;
        const S *sv = (const S *)&v;
        D *dv = (D *)&o;
#pragma unroll
        for (int e = 0; e < V; e++) dv[e] = dd_cvt<S, D, C, RAW>::f(sv[e], (C)1);
        v = o;
      }
      *(uint4 *)dst = v;
    } else {
      *dst = dd_cvt<S, D, C, RAW>::f(*src, (C)1);
    }
  }
}

// ------------------------------------------------------------------ launchers ----------------

struct ddXformPlan {
  ddCanon canon;  // ordered by y strides
  double alpha, beta;
  const void *x;
  void *y;
};

template <typename S, typename D, typename C, bool RAW>
static ddStatus_t dd_launch_flat(ddHandle_t h, const ddXformPlan &pl) {
  ddFlatParams p;
  p.x = pl.x;
  p.y = pl.y;
  p.n = pl.canon.total;
  p.alpha = pl.alpha;
  p.beta = pl.beta;
  p.vec = (((uintptr_t)pl.x | (uintptr_t)pl.y) & 15) == 0;
  constexpr int MINW = sizeof(S) < sizeof(D) ? sizeof(S) : sizeof(D);
  constexpr int V = 16 / MINW;
  unsigned grid = dd_flat_grid(h, (p.n + V - 1) / V, 256, 64);  // 16 -> 64: same-layout f32 -> bf16 +3.5 %
  dd_flat_kernel<S, D, C, RAW><<<grid, 256, 0, h->stream>>>(p);
  DD_LAUNCHED(h, "transform/flat");
  return DD_STATUS_SUCCESS;
}

// Fills tile parameters if the canonical space fits a tile kernel; returns 0 if not, 1 for the
// 16-byte vector tile kernel, 2 for the scalar tile kernel (rows not 16-byte aligned), -1 for a
// transposition whose A or B is too thin for either (3 or 4 channels of an image: the parameters are
// filled for the short-rows forms, which take it if they can).
template <typename S, typename D>
static int dd_tile_plan(const ddXformPlan &pl, ddTileParams *tp) {
  typedef dd_tile_geom<S, D> G;
  const ddCanon &c = pl.canon;
  if (pl.beta != 0.0 || c.nd < 2) return 0;
  const int B = c.nd - 1;
  if (c.st[1][B] != 1) return 0;
  int A = -1;
  for (int i = 0; i < c.nd - 1; i++)
    if (c.st[0][i] == 1) A = i;
  if (A < 0) return 0;
  if (c.nd - 2 > DD_TILE_BATCH_DIMS) return 0;
  bool vec = ((((uintptr_t)pl.x) | ((uintptr_t)pl.y)) & 15) == 0;
  if (c.dims[A] % G::VS || c.dims[B] % G::VD) vec = false;
  for (int i = 0; i < c.nd; i++) {
    if (i != A && (c.st[0][i] % G::VS)) vec = false;
    if (i != B && (c.st[1][i] % G::VD)) vec = false;
  }
  // a tile that is mostly padding wastes the machine: leave short dims to the other kernels
  if (c.dims[A] < G::VS * 2 || c.dims[B] < G::VD * 2) vec = false;
  const bool thin = !vec && (c.dims[A] < 8 || c.dims[B] < 8);  // too thin to be worth a tile
  // CTA shape of the vector kernel: na lanes along A (5..16) by nb lanes along B (NB, or 2 NB when
  // na <= 8), chosen by the padding the edge tiles would carry
  int na = G::NA, nbLog2 = 0;
  while ((1 << nbLog2) < G::NB) nbLog2++;
  if (vec) {
    const int64_t vecsA = c.dims[A] / G::VS, vecsB = c.dims[B] / G::VD;
    // A short B (the 8 or 16 channels of a blocked layout: 2 or 4 vectors of f32) gets as few lanes
    // along B as cover it, and up to 64 lanes along A in their place: with the usual 16 lanes along B
    // three quarters or more of the CTA would sit out the load phase (nchw -> nChw16c of
    // [256,256,28,28] f32 measured 0.47 of the copy rate, nChw8c 0.24)
    int nbShort = 0;
    if (vecsB < G::NB && dd_tune("DD_TILE_SHORT_B", 1)) {
      nbShort = 2;
      while (nbShort < vecsB) nbShort *= 2;
    }
    const int naCap = nbShort ? (G::NT / nbShort < 64 ? G::NT / nbShort : 64) : G::NA;
    const int naLo = dd_tune("DD_TILE_NA_LO", vecsA < 5 ? (int)vecsA : 5), naHi = dd_tune("DD_TILE_NA_HI", naCap);
    auto eff = [&](int cand) {
      const int nbc = nbShort ? nbShort : (cand <= 8 ? 2 * G::NB : G::NB);
      const double effA = (double)vecsA / (double)(((vecsA + cand - 1) / cand) * cand);
      const double effB = (double)vecsB / (double)(((vecsB + nbc - 1) / nbc) * nbc);
      return effA * effB;
    };
    double best = -1.0;
    for (int cand = naHi; cand >= naLo; cand--) best = eff(cand) > best ? eff(cand) : best;
    // the widest CTA within a tenth of the best: longer contiguous runs along A measured faster
    // than the last few per cent of padding (49 vectors: 13 lanes beat 7 and 10; 196: 16 beat 14)
    for (int cand = naHi; cand >= naLo; cand--)
      if (eff(cand) >= best - 0.1) {
        na = cand;
        break;
      }
    nbLog2 = 0;
    while ((1 << nbLog2) < (nbShort ? nbShort : (na <= 8 ? 2 * G::NB : G::NB))) nbLog2++;
  }
  const int TAe = vec ? na * G::VS : 32, TBe = vec ? (1 << nbLog2) * G::VD : 32;
  tp->na = na;
  tp->nbLog2 = nbLog2;
  tp->fdNA = dd_fastdiv((uint32_t)na);
  tp->x = pl.x;
  tp->y = pl.y;
  tp->LA = c.dims[A];
  tp->LB = c.dims[B];
  tp->sxB = c.st[0][B];
  tp->syA = c.st[1][A];
  tp->nb = 0;
  for (int i = 0; i < c.nd - 1; i++) {
    if (i == A) continue;
    tp->bdims[tp->nb] = c.dims[i];
    tp->bsx[tp->nb] = c.st[0][i];
    tp->bsy[tp->nb] = c.st[1][i];
    tp->nb++;
  }
  tp->tilesA = (tp->LA + TAe - 1) / TAe;
  tp->tilesB = (tp->LB + TBe - 1) / TBe;
  int64_t tiles = tp->tilesA * tp->tilesB;
  for (int i = 0; i < tp->nb; i++) tiles *= tp->bdims[i];
  if (tiles >= 0x7fffffffLL) return 0;
  tp->fdA = dd_fastdiv((uint32_t)tp->tilesA);
  tp->fdB = dd_fastdiv((uint32_t)tp->tilesB);
  for (int i = 0; i < tp->nb; i++) tp->fdBatch[i] = dd_fastdiv((uint32_t)tp->bdims[i]);
  tp->alpha = pl.alpha;
  return thin ? -1 : (vec ? 1 : 2);
}

// The 1-byte bit copy with tile loads by the tensor memory accelerator (dd_tile_tma.cu); false when
// the reorder does not qualify, and then nothing was launched.
bool dd_launch_tile_tma(ddHandle_t h, const ddTileParams &tp);

template <typename S, typename D, typename C, bool RAW>
static ddStatus_t dd_launch_tile(ddHandle_t h, const ddTileParams &tp, int kind) {
  typedef dd_tile_geom<S, D> G;
  int64_t tiles = tp.tilesA * tp.tilesB;
  for (int i = 0; i < tp.nb; i++) tiles *= tp.bdims[i];
  if (tiles > 0x7fffffffLL) DD_FAIL(h, DD_STATUS_NOT_SUPPORTED, "transform/tile: too many tiles");
  if (kind == 1) {
    ddTileParams tq = tp;
    tq.ntiles = (uint32_t)tiles;
    // Converting kernels (48 registers, 5 resident CTAs of 256 threads per SM) run as one resident
    // wave whose CTAs walk the tiles: measured 6 % faster on f32 -> bf16 than a CTA per tile.  The
    // bit-copy kernels measured the same or slower that way and keep a CTA per tile.
    const int cps = dd_tune("DD_TILE_CPS", RAW ? 0 : 5);
    int64_t grid = tiles;
    if (cps > 0 && grid > (int64_t)h->smCount * cps) grid = (int64_t)h->smCount * cps;
    dd_launch_pdl(dd_tile_kernel<S, D, C, RAW>, (unsigned)grid, (unsigned)(tq.na << tq.nbLog2), h->stream, tq);
    DD_LAUNCHED(h, "transform/tile");
  } else {
    dd_tile_scalar_kernel<S, D, C, RAW><<<(unsigned)tiles, 256, 0, h->stream>>>(tp);
    DD_LAUNCHED(h, "transform/tile-scalar");
  }
  return DD_STATUS_SUCCESS;
}

// The short-odd-rows forms for a transposition that dd_tile_plan left to the scalar tile: returns 0
// (neither applies), 3 (flat-in) or 4 (flat-out) and fills `fp`.
template <typename S, typename D>
static int dd_tile_flat_plan(const ddTileParams &tp, ddTileFlatParams *fp) {
  constexpr int VS = 16 / (int)sizeof(S), VD = 16 / (int)sizeof(D);
  if (!dd_tune("DD_TILE_FLAT", 1)) return 0;
  // shared memory per CTA: 16 KB measured best over 8, 16, 24 and 32 on 7 x 7 and 14 x 14 maps of f32 and
  // int8 tensors, both directions (more resident CTAs against longer contiguous chunks)
  const int64_t SMEM = (int64_t)dd_tune("DD_TILE_FLAT_KB", 16) << 10;
  if ((((uintptr_t)tp.x) | ((uintptr_t)tp.y)) & 15) return 0;
  if (tp.LA >= (1 << 20) || tp.LB >= (1 << 20)) return 0;
  int64_t batches = 1;
  for (int i = 0; i < tp.nb; i++) batches *= tp.bdims[i];
  auto all = [&](const int64_t *st, int64_t m) {
    for (int i = 0; i < tp.nb; i++)
      if (tp.bdims[i] > 1 && st[i] % m) return false;
    return true;
  };
  int kind = 0, rows = 0;
  // (rows too long for sixteen of them in that much get twice as much)
  for (int64_t room = SMEM; !kind && room <= 2 * SMEM; room *= 2) {
    if (tp.sxB == tp.LA && tp.LB % VD == 0 && tp.syA % VD == 0 && all(tp.bsx, VS) && all(tp.bsy, VD)) {
      rows = (int)((room / (tp.LA * (int64_t)sizeof(S))) / 16 * 16);
      if (rows >= 16) kind = 3;
    }
    if (!kind && tp.syA == tp.LB && tp.LA % VS == 0 && tp.sxB % VS == 0 && all(tp.bsx, VS) && all(tp.bsy, VD)) {
      // rows of A per CTA: LB * (rows + pad) elements of S in shared memory, at most 256 vectors per row
      const int pad = sizeof(S) >= 4 ? 1 : 4 / (int)sizeof(S);
      rows = (int)((room / (tp.LB * (int64_t)sizeof(S)) - pad) / 16 * 16);
      if (rows > 256 * VS) rows = 256 * VS;
      if (rows >= 16) kind = 4;
    }
  }
  if (!kind) return 0;
  const int64_t extent = kind == 3 ? tp.LB : tp.LA;
  if (rows > (extent + 15) / 16 * 16) rows = (int)((extent + 15) / 16 * 16);
  const int64_t chunks = (extent + rows - 1) / rows;
  if (batches * chunks >= 0x7fffffffLL) return 0;
  fp->x = tp.x;
  fp->y = tp.y;
  fp->LA = tp.LA;
  fp->LB = tp.LB;
  fp->sxB = tp.sxB;
  fp->syA = tp.syA;
  fp->nb = tp.nb;
  for (int i = 0; i < tp.nb; i++) {
    fp->bdims[i] = tp.bdims[i];
    fp->bsx[i] = tp.bsx[i];
    fp->bsy[i] = tp.bsy[i];
    fp->fdBatch[i] = tp.fdBatch[i];
  }
  fp->rows = rows;
  fp->chunks = (uint32_t)chunks;
  fp->fdChunks = dd_fastdiv((uint32_t)chunks);
  fp->alpha = tp.alpha;
  if (kind == 3) {
    fp->fdInner = dd_fastdiv((uint32_t)(2 * tp.LA));
    fp->fdVPR = dd_fastdiv(1);
    fp->pitch = 0;
    fp->smemBytes = (unsigned)(rows * tp.LA * (int64_t)sizeof(S) + 16);
  } else {
    const int pad = sizeof(S) >= 4 ? 1 : 4 / (int)sizeof(S);
    fp->fdInner = dd_fastdiv((uint32_t)tp.LB);
    fp->fdVPR = dd_fastdiv((uint32_t)(rows / VS));
    fp->pitch = rows + pad;
    fp->smemBytes = (unsigned)(tp.LB * (int64_t)fp->pitch * (int64_t)sizeof(S) + 16);
  }
  return kind;
}

template <typename S, typename D, typename C, bool RAW>
static ddStatus_t dd_launch_tile_flat(ddHandle_t h, const ddTileFlatParams &fp, int kind) {
  int64_t batches = 1;
  for (int i = 0; i < fp.nb; i++) batches *= fp.bdims[i];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(batches * fp.chunks), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = fp.smemBytes;
  cfg.stream = h->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (kind == 3) {
    cudaLaunchKernelEx(&cfg, dd_tile_flatin_kernel<S, D, C, RAW>, fp);
    DD_LAUNCHED(h, "transform/tile-flat-in");
  } else {
    cudaLaunchKernelEx(&cfg, dd_tile_flatout_kernel<S, D, C, RAW>, fp);
    DD_LAUNCHED(h, "transform/tile-flat-out");
  }
  return DD_STATUS_SUCCESS;
}

template <typename S, typename D, typename C, bool RAW>
static ddStatus_t dd_launch_strided(ddHandle_t h, const ddXformPlan &pl) {
  ddStridedXformParams p;
  p.x = pl.x;
  p.y = pl.y;
  p.sp = dd_strided_params<2>(pl.canon);
  p.alpha = pl.alpha;
  p.beta = pl.beta;
  unsigned grid = dd_flat_grid(h, pl.canon.total, 256, 16);
  if (pl.canon.total < 0x7fffffffLL)
    dd_strided_kernel<S, D, C, RAW, uint32_t><<<grid, 256, 0, h->stream>>>(p);
  else
    dd_strided_kernel<S, D, C, RAW, int64_t><<<grid, 256, 0, h->stream>>>(p);
  DD_LAUNCHED(h, "transform/strided");
  return DD_STATUS_SUCCESS;
}

// Rows form: innermost dim contiguous on both sides, every vector start 16-byte aligned.
template <typename S, typename D, typename C, bool RAW>
static bool dd_launch_rows(ddHandle_t h, const ddXformPlan &pl) {
  constexpr int MINW = sizeof(S) < sizeof(D) ? sizeof(S) : sizeof(D);
  constexpr int V = 16 / MINW;
  const ddCanon &c = pl.canon;
  const int last = c.nd - 1;
  if (c.nd < 2 || c.st[0][last] != 1 || c.st[1][last] != 1 || c.dims[last] % V != 0) return false;
  if ((((uintptr_t)pl.x | (uintptr_t)pl.y) & 15) != 0 || c.total / V >= 0x7fffffffLL) return false;
  for (int i = 0; i < last; i++)
    if ((c.st[0][i] * (int64_t)sizeof(S)) % 16 != 0 || (c.st[1][i] * (int64_t)sizeof(D)) % 16 != 0) return false;
  ddCanon v = c;
  v.dims[last] = c.dims[last] / V;
  v.st[0][last] = V;
  v.st[1][last] = V;
  v.total = c.total / V;
  ddStridedXformParams p;
  p.x = pl.x;
  p.y = pl.y;
  p.sp = dd_strided_params<2>(v);
  p.alpha = pl.alpha;
  p.beta = pl.beta;
  unsigned grid = dd_flat_grid(h, v.total, 256, 64);  // 16 -> 64: sub-tensor copy +2.5 %
  dd_rows_kernel<S, D, C, RAW><<<grid, 256, 0, h->stream>>>(p);
  h->launches++;
  h->lastKernel = "transform/rows";
  return true;
}

template <typename S, typename D, typename C, bool RAW>
static ddStatus_t dd_xform_typed(ddHandle_t h, const ddXformPlan &pl) {
  const ddCanon &c = pl.canon;
  if (c.nd == 1 && c.st[0][0] == 1 && c.st[1][0] == 1) return dd_launch_flat<S, D, C, RAW>(h, pl);
  ddTileParams tp;
  if (int kind = dd_tile_plan<S, D>(pl, &tp)) {
    if constexpr (RAW && sizeof(S) == 1)
      if (kind == 1 && dd_launch_tile_tma(h, tp)) return DD_STATUS_SUCCESS;
    if (kind == 2 || kind == -1) {
      ddTileFlatParams fp;
      if (int fk = dd_tile_flat_plan<S, D>(tp, &fp)) return dd_launch_tile_flat<S, D, C, RAW>(h, fp, fk);
    }
    if (kind > 0) return dd_launch_tile<S, D, C, RAW>(h, tp, kind);
  }
  if (dd_launch_rows<S, D, C, RAW>(h, pl)) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) DD_FAIL(h, DD_STATUS_EXECUTION_FAILED, "transform/rows: %s", cudaGetErrorString(e));
    return DD_STATUS_SUCCESS;
  }
  return dd_launch_strided<S, D, C, RAW>(h, pl);
}

struct ddGatherPlan {
  ddCanon canon;  // one item, ordered by y strides
  const void *x;
  void *y;
  int count;
  const int64_t *so, *do_;
};

static inline int64_t dd_gcd64(int64_t a, int64_t b) {
  while (b) {
    int64_t t = a % b;
    a = b;
    b = t;
  }
  return a;
}

// Tries the dense single-launch form; returns false (nothing launched) when the items are not
// dense runs, the destinations are not evenly spaced or the indices do not fit 32 bits.
template <typename S, typename D, typename C, bool RAW>
static bool dd_gather_dense(ddHandle_t h, const ddGatherPlan &pl) {
  const ddCanon &c = pl.canon;
  if (!(c.nd == 1 && c.st[0][0] == 1 && c.st[1][0] == 1) || pl.count > DD_GATHER_SEQ_MAX) return false;
  const int64_t per = c.total;
  const int64_t d0 = pl.do_[0], dstep = pl.count > 1 ? pl.do_[1] - pl.do_[0] : 0;
  int64_t unit = 0;
  for (int k = 0; k < pl.count; k++) {
    if (pl.do_[k] != d0 + (int64_t)k * dstep) return false;
    unit = dd_gcd64(unit, pl.so[k]);
  }
  if (unit == 0) unit = 1;  // every source offset is 0
  for (int k = 0; k < pl.count; k++)
    if (pl.so[k] / unit > 0xffffffffLL) return false;
  constexpr int V = sizeof(S) == sizeof(D) ? 16 / (int)sizeof(S) : 1;
  bool vec = false;
  if (sizeof(S) == sizeof(D)) {
    const uintptr_t bytes = (uintptr_t)pl.x | (uintptr_t)pl.y | (uintptr_t)(unit * (int64_t)sizeof(S)) |
                            (uintptr_t)(d0 * (int64_t)sizeof(D)) | (uintptr_t)(dstep * (int64_t)sizeof(D)) |
                            (uintptr_t)(per * (int64_t)sizeof(S));
    vec = (bytes & 15) == 0;
  }
  const int64_t vpi = vec ? per / V : per;
  if (vpi <= 0 || vpi * pl.count >= 0x7fffffffLL) return false;
  static thread_local ddGatherSeqParams p;  // 16 KB: kept off the stack, one per calling thread
  p.x = pl.x;
  p.y = pl.y;
  p.total = (uint32_t)(vpi * pl.count);
  p.vpi = (uint32_t)vpi;
  p.fdVpi = dd_fastdiv((uint32_t)vpi);
  p.unit = unit;
  p.d0 = d0;
  p.dstep = dstep;
  for (int k = 0; k < pl.count; k++) p.so[k] = (uint32_t)(pl.so[k] / unit);
  unsigned grid = dd_flat_grid(h, p.total, 256, 64);  // 16 -> 64: shuffler +2.5 %
  if (vec) {
    if constexpr (sizeof(S) == sizeof(D)) dd_gather_dense_kernel<S, D, C, RAW, true><<<grid, 256, 0, h->stream>>>(p);
    h->launches++;
    h->lastKernel = "transform/gather-dense-vec";
  } else {
    dd_gather_dense_kernel<S, D, C, RAW, false><<<grid, 256, 0, h->stream>>>(p);
    h->launches++;
    h->lastKernel = "transform/gather-dense";
  }
  return true;
}

template <typename S, typename D, typename C, bool RAW>
static ddStatus_t dd_gather_typed(ddHandle_t h, const ddGatherPlan &pl) {
  if (dd_gather_dense<S, D, C, RAW>(h, pl)) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) DD_FAIL(h, DD_STATUS_EXECUTION_FAILED, "transform/gather-dense: %s", cudaGetErrorString(e));
    return DD_STATUS_SUCCESS;
  }
  static thread_local ddGatherParams p;  // 16 KB: kept off the stack, one per calling thread
  for (int base = 0; base < pl.count; base += DD_GATHER_CHUNK) {
    int n = pl.count - base < DD_GATHER_CHUNK ? pl.count - base : DD_GATHER_CHUNK;
    p.x = pl.x;
    p.y = pl.y;
    p.sp = dd_strided_params<2>(pl.canon);
    p.count = n;
    for (int i = 0; i < n; i++) {
      p.so[i] = pl.so[base + i];
      p.do_[i] = pl.do_[base + i];
    }
    unsigned grid = dd_flat_grid(h, pl.canon.total * n, 256, 16);
    dd_gather_kernel<S, D, C, RAW><<<grid, 256, 0, h->stream>>>(p);
    DD_LAUNCHED(h, "transform/gather");
  }
  return DD_STATUS_SUCCESS;
}

// Compute type: double when a 64-bit or 32-bit-integer type is involved on the source side or a
// 64-bit type on the destination side (so every conversion rounds once); float otherwise.
template <typename S, typename D>
struct dd_compute_type {
  static constexpr bool dbl = sizeof(S) == 8 || sizeof(D) == 8 || (sizeof(S) == 4 && !std::is_same<S, float>::value);
  typedef typename std::conditional<dbl, double, float>::type type;
};

// One translation unit per source type instantiates these for every destination type.
template <typename S>
ddStatus_t dd_xform_from(ddHandle_t h, ddDataType_t dstType, const ddXformPlan &pl);
template <typename S>
ddStatus_t dd_gather_from(ddHandle_t h, ddDataType_t dstType, const ddGatherPlan &pl);
ddStatus_t dd_xform_raw(ddHandle_t h, int width, const ddXformPlan &pl);
ddStatus_t dd_gather_raw(ddHandle_t h, int width, const ddGatherPlan &pl);

#define DD_XFORM_DECLARE_FROM(S)                                                          \
  template <> ddStatus_t dd_xform_from<S>(ddHandle_t, ddDataType_t, const ddXformPlan &); \
  template <> ddStatus_t dd_gather_from<S>(ddHandle_t, ddDataType_t, const ddGatherPlan &);
DD_XFORM_DECLARE_FROM(float)
DD_XFORM_DECLARE_FROM(double)
DD_XFORM_DECLARE_FROM(__half)
DD_XFORM_DECLARE_FROM(int8_t)
DD_XFORM_DECLARE_FROM(int32_t)
DD_XFORM_DECLARE_FROM(uint8_t)
DD_XFORM_DECLARE_FROM(__nv_bfloat16)
DD_XFORM_DECLARE_FROM(int64_t)

#define DD_XFORM_DEFINE_FROM(S)                                                              \
  template <>                                                                                \
  ddStatus_t dd_xform_from<S>(ddHandle_t h, ddDataType_t dt, const ddXformPlan &pl) {        \
    switch (dt) {                                                                            \
      case DD_DATA_FLOAT: return dd_xform_typed<S, float, dd_compute_type<S, float>::type, false>(h, pl); \
      case DD_DATA_DOUBLE: return dd_xform_typed<S, double, dd_compute_type<S, double>::type, false>(h, pl); \
      case DD_DATA_HALF: return dd_xform_typed<S, __half, dd_compute_type<S, __half>::type, false>(h, pl); \
      case DD_DATA_INT8: return dd_xform_typed<S, int8_t, dd_compute_type<S, int8_t>::type, false>(h, pl); \
      case DD_DATA_INT32: return dd_xform_typed<S, int32_t, dd_compute_type<S, int32_t>::type, false>(h, pl); \
      case DD_DATA_UINT8: return dd_xform_typed<S, uint8_t, dd_compute_type<S, uint8_t>::type, false>(h, pl); \
      case DD_DATA_BFLOAT16: return dd_xform_typed<S, __nv_bfloat16, dd_compute_type<S, __nv_bfloat16>::type, false>(h, pl); \
      case DD_DATA_INT64: return dd_xform_typed<S, int64_t, dd_compute_type<S, int64_t>::type, false>(h, pl); \
    }                                                                                        \
    return DD_STATUS_BAD_PARAM;                                                              \
  }                                                                                          \
  template <>                                                                                \
  ddStatus_t dd_gather_from<S>(ddHandle_t h, ddDataType_t dt, const ddGatherPlan &pl) {      \
    switch (dt) {                                                                            \
      case DD_DATA_FLOAT: return dd_gather_typed<S, float, dd_compute_type<S, float>::type, false>(h, pl); \
      case DD_DATA_DOUBLE: return dd_gather_typed<S, double, dd_compute_type<S, double>::type, false>(h, pl); \
      case DD_DATA_HALF: return dd_gather_typed<S, __half, dd_compute_type<S, __half>::type, false>(h, pl); \
      case DD_DATA_INT8: return dd_gather_typed<S, int8_t, dd_compute_type<S, int8_t>::type, false>(h, pl); \
      case DD_DATA_INT32: return dd_gather_typed<S, int32_t, dd_compute_type<S, int32_t>::type, false>(h, pl); \
      case DD_DATA_UINT8: return dd_gather_typed<S, uint8_t, dd_compute_type<S, uint8_t>::type, false>(h, pl); \
      case DD_DATA_BFLOAT16: return dd_gather_typed<S, __nv_bfloat16, dd_compute_type<S, __nv_bfloat16>::type, false>(h, pl); \
      case DD_DATA_INT64: return dd_gather_typed<S, int64_t, dd_compute_type<S, int64_t>::type, false>(h, pl); \
    }                                                                                        \
    return DD_STATUS_BAD_PARAM;                                                              \
  }
