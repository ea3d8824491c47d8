// Transposing reorder of 1-byte elements (int8 / uint8 bit copies, nchw <-> nhwc and the like) with
// the tile LOADS done by the tensor memory accelerator.
//
// The register-staged kernel (dd_tile_kernel) keeps sixteen 16-byte loads in flight per thread for
// this element width, and their 64 registers plus the 16 x 16 byte transpose leave four CTAs of about
// a hundred threads per SM: too few warps to hide the load latency on tensors of tens of megabytes.
// Here a persistent CTA has one thread issue `cp.async.bulk.tensor.3d` for tile i + 1 into the other
// half of a two-stage shared-memory ring while all threads transpose tile i out of the first: bytes in
// flight cost no registers, and a tile's load overlaps the previous tile's transpose and stores.
// The tensor map covers THIS GPU's memory only and the copy is plain (no multicast, no cluster).
//
// Shared memory per CTA: two input stages of TB rows x TA bytes as the copy engine lays them out
// (dense, row pitch TA), the XOR-swizzled output stage of dd_tile_kernel, two mbarriers.
// Every wait on an mbarrier is bounded; a wait that runs out raises the handle's fault word, and the
// CTA returns without touching the tile.
#include "dd_transform_kernels.cuh"

#include <cuda.h>

struct ddTileTmaParams {
  ddTileParams t;     // geometry, strides and the destination, as for dd_tile_kernel (nb <= 1, 8 lanes along B)
  int *fault;         // word in mapped host memory, raised when a bounded wait ran out
  int stages;         // input stages in shared memory
};

__device__ __forceinline__ uint32_t dd_smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void dd_mbar_init(uint64_t *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(dd_smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void dd_mbar_expect_tx(uint64_t *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(dd_smem_addr(bar)), "r"(bytes) : "memory");
}
// One try: may suspend the thread for up to about `hintNs` nanoseconds before it answers.
__device__ __forceinline__ bool dd_mbar_try_wait(uint64_t *bar, unsigned parity, unsigned hintNs) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(dd_smem_addr(bar)), "r"(parity), "r"(hintNs)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t dd_globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// One tile of the tensor map into shared memory; completion (in bytes) is counted on `bar`.
__device__ __forceinline__ void dd_tma_load_3d(void *dst, const CUtensorMap *map, int x, int y, int z, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dd_smem_addr(dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(z), "r"(dd_smem_addr(bar))
      : "memory");
}

#define DD_TMA_TB 128           // rows of B per tile (= 8 thread groups of 16 rows)
#define DD_TMA_MAX_STAGES 4
#define DD_TMA_WAIT_NS 1000000000ull   // one second per wait
#define DD_TMA_WAIT_TRIES (1u << 24)

// false when the phase did not complete within the limit: DD_TMA_WAIT_NS of wall time, and a cap on
// the tries as well in case the timer does not advance
__device__ __forceinline__ bool dd_mbar_wait_bounded(uint64_t *bar, unsigned parity) {
  if (dd_mbar_try_wait(bar, parity, 2000u)) return true;
  const uint64_t t0 = dd_globaltimer_ns();
  for (unsigned tries = 0; tries < DD_TMA_WAIT_TRIES; tries++) {
    if (dd_mbar_try_wait(bar, parity, 2000u)) return true;
    if (dd_globaltimer_ns() - t0 > DD_TMA_WAIT_NS) return false;
  }
  return false;
}

// CTA = na x 8 threads (na <= 16 lanes of 16 bytes along A), tile = TA = na * 16 bytes along A by 128
// rows along B.  x coordinates are multiples of TA, hence of 16 bytes.  `nst` input stages (2..4):
// the loads of the next nst - 1 tiles of this CTA are in flight while one tile is transposed.
__global__ void __launch_bounds__(128) dd_tile_tma_kernel(const __grid_constant__ CUtensorMap map, ddTileTmaParams q) {
  extern __shared__ __align__(128) unsigned char smem[];
  const ddTileParams &p = q.t;
  const int NA = p.na;
  const int TA = NA * 16;
  const int nst = q.stages;
  const unsigned stageBytes = (unsigned)TA * DD_TMA_TB;
  uint4 *tile = (uint4 *)(smem + (size_t)nst * stageBytes);            // [TA rows][8 chunks of 16 bytes]
  uint64_t *bars = (uint64_t *)(smem + (size_t)(nst + 1) * stageBytes);
  const int t = threadIdx.x;
  if (t == 0) {
    for (int k = 0; k < nst; k++) dd_mbar_init(&bars[k], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  dd_pdl_prologue();

  uint32_t mbU, maU;
  dd_divmod((uint32_t)t, p.fdNA, mbU, maU);
  const int ma = (int)maU, mb = (int)mbU;

  auto coords = [&](uint32_t tileId, int &x, int &y, int &z) {
    uint32_t id = tileId, ta, tb;
    dd_divmod(id, p.fdA, id, ta);
    dd_divmod(id, p.fdB, id, tb);
    x = (int)ta * TA;
    y = (int)tb * DD_TMA_TB;
    z = (int)id;  // index along the one batch dim (0 when there is none)
  };
  auto issue = [&](uint32_t tileId, unsigned stage) {
    int x, y, z;
    coords(tileId, x, y, z);
    dd_mbar_expect_tx(&bars[stage], stageBytes);
    dd_tma_load_3d(smem + (size_t)stage * stageBytes, &map, x, y, z, &bars[stage]);
  };

  if (t == 0)
    for (int k = 0; k < nst - 1; k++) {
      const uint64_t id = (uint64_t)blockIdx.x + (uint64_t)k * gridDim.x;
      if (id < p.ntiles) issue((uint32_t)id, (unsigned)k);
    }
  unsigned s = 0, parity = 0;  // stage and phase parity of tile `it`
  for (uint64_t tileId = blockIdx.x; tileId < p.ntiles; tileId += gridDim.x) {
    // the load of the tile nst - 1 ahead goes into the stage the previous iteration read out (every
    // thread passed a CTA barrier after those reads)
    if (t == 0) {
      const uint64_t ahead = tileId + (uint64_t)(nst - 1) * gridDim.x;
      if (ahead < p.ntiles) issue((uint32_t)ahead, s == 0 ? (unsigned)nst - 1 : s - 1);
    }
    const bool arrived = dd_mbar_wait_bounded(&bars[s], parity);
    // one decision for the whole CTA; the barrier also orders the previous tile's reads of the output
    // stage before this tile's writes to it
    if (__syncthreads_or(!arrived)) {
      if (t == 0) {
        *(volatile int *)q.fault = 1;
        // what this CTA still has in flight lands in its shared memory: give it the same limit again
        unsigned ks = s, kp = parity;
        uint64_t id = tileId;
        for (int k = 0; k < nst && id < p.ntiles; k++, id += gridDim.x) {
          dd_mbar_wait_bounded(&bars[ks], kp);
          if (++ks == (unsigned)nst) ks = 0, kp ^= 1u;
        }
      }
      __syncthreads();
      return;
    }
    int x0, y0, z0;
    coords((uint32_t)tileId, x0, y0, z0);
    const int64_t a0 = x0, b0 = y0;
    uint8_t *yb = (uint8_t *)p.y + (p.nb > 0 ? (int64_t)z0 * p.bsy[0] : 0);
    {  // sixteen rows of B x 16 bytes of A out of the stage, transposed in registers (4 x 4 byte blocks)
      uint4 in[16];
      const unsigned char *src = smem + (size_t)s * stageBytes + (size_t)(mb * 16) * TA + ma * 16;
#pragma unroll
      for (int j = 0; j < 16; j++) in[j] = *(const uint4 *)(src + (size_t)j * TA);
      uint4 outv[16];
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
      uint4 *dstRow = tile + ((ma * 16) * 8 + (mb ^ (ma & 7)));
#pragma unroll
      for (int i = 0; i < 16; i++) dstRow[i * 8] = outv[i];
    }
    __syncthreads();
    {  // rows of the output stage to global memory: 8 consecutive lanes cover 128 contiguous bytes along B
      const int rb = t & 7, ra = t >> 3;
      const int64_t b = b0 + rb * 16;
      const int64_t leftA = p.LA - a0;
      const int rowsA = b < p.LB ? (leftA < TA ? (int)leftA : TA) : 0;
      uint8_t *dst = yb + (a0 + ra) * p.syA + b;
      const int64_t step = (int64_t)NA * p.syA;
#pragma unroll
      for (int k = 0; k < 16; k++) {
        const int row = ra + k * NA;
        if (row < rowsA) *(uint4 *)dst = tile[row * 8 + (rb ^ ((row >> 4) & 7))];
        dst += step;
      }
    }
    if (++s == (unsigned)nst) s = 0, parity ^= 1u;
  }
}

typedef CUresult (*ddEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static ddEncodeTiledFn dd_encode_tiled() {
  static const ddEncodeTiledFn fn = []() -> ddEncodeTiledFn {
    void *f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return (ddEncodeTiledFn)f;
    cudaGetLastError();
    return nullptr;
  }();
  return fn;
}

// Launches the TMA form if the reorder qualifies; returns false (nothing launched, no error state)
// if it does not.  `tp` is a vector tile plan of 1-byte elements (bases 16-byte aligned, extents and
// the strides of x multiples of 16 bytes); on top of that the form wants at most one batch dim and
// extents that fit the 32-bit coordinates of a tensor map.
bool dd_launch_tile_tma(ddHandle_t h, const ddTileParams &tp) {
  if (!dd_tune("DD_TILE_TMA", h->tileTma) || !h->faultWord) return false;
  if (tp.nb > 1 || tp.na < 1) return false;
  const int na = tp.na > 16 ? 16 : tp.na;  // (the register-staged kernel may have chosen a wider CTA for a short B)
  if ((((uintptr_t)tp.x) & 15) || (tp.sxB & 15) || (tp.LA & 15) || (tp.LB & 15)) return false;
  if (tp.nb == 1 && (tp.bsx[0] & 15)) return false;
  const int64_t batch = tp.nb == 1 ? tp.bdims[0] : 1;
  if (tp.LA >= (1LL << 31) || tp.LB >= (1LL << 31) || batch >= (1LL << 31)) return false;
  const int64_t strideB = tp.sxB, strideBatch = tp.nb == 1 ? tp.bsx[0] : tp.sxB * tp.LB;
  if (strideB <= 0 || strideBatch <= 0 || strideB >= (1LL << 40) || strideBatch >= (1LL << 40)) return false;
  ddEncodeTiledFn encode = dd_encode_tiled();
  if (!encode) return false;

  ddTileTmaParams q;
  q.t = tp;
  q.t.nbLog2 = 3;
  const int TA = na * 16;
  q.t.na = na;
  q.t.fdNA = dd_fastdiv((uint32_t)na);
  q.t.tilesA = (tp.LA + TA - 1) / TA;
  q.t.tilesB = (tp.LB + DD_TMA_TB - 1) / DD_TMA_TB;
  const int64_t tiles = q.t.tilesA * q.t.tilesB * batch;
  if (tiles >= 0x7fffffffLL) return false;
  // with fewer than a few tiles per SM nothing is left to overlap, and the register-staged kernel's
  // one CTA per tile starts sooner
  if (tiles < (int64_t)h->smCount * dd_tune("DD_TILE_TMA_MIN", 4)) return false;
  q.t.ntiles = (uint32_t)tiles;
  q.t.fdA = dd_fastdiv((uint32_t)q.t.tilesA);
  q.t.fdB = dd_fastdiv((uint32_t)q.t.tilesB);
  q.fault = h->faultWord;
  // two input stages and two CTAs per SM measured best on [256,256,28,28] and [64,1024,32,32]
  // (three and four stages, and one, three or four CTAs, were 3 to 30 % slower)
  int stages = dd_tune("DD_TILE_TMA_STAGES", 2);
  stages = stages < 2 ? 2 : (stages > DD_TMA_MAX_STAGES ? DD_TMA_MAX_STAGES : stages);
  q.stages = stages;

  CUtensorMap map;
  cuuint64_t gdim[3] = {(cuuint64_t)tp.LA, (cuuint64_t)tp.LB, (cuuint64_t)batch};
  cuuint64_t gstride[2] = {(cuuint64_t)strideB, (cuuint64_t)strideBatch};
  cuuint32_t box[3] = {(cuuint32_t)TA, DD_TMA_TB, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(tp.x), gdim, gstride, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;

  const size_t maxSmem = (size_t)(DD_TMA_MAX_STAGES + 1) * 256 * DD_TMA_TB + 64;
  if (!h->tmaAttr) {
    if (cudaFuncSetAttribute(dd_tile_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)maxSmem) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    h->tmaAttr = true;
  }
  const size_t smemBytes = (size_t)(stages + 1) * TA * DD_TMA_TB + 64;
  // resident CTAs per SM by shared memory (227 KB usable, 1 KB reserved per CTA)
  int fit = (int)((227u << 10) / (smemBytes + 1024));
  fit = fit < 1 ? 1 : fit;
  const int cps = dd_tune("DD_TILE_TMA_CPS", fit);
  int64_t grid = tiles < (int64_t)h->smCount * cps ? tiles : (int64_t)h->smCount * cps;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3((unsigned)(na * 8), 1, 1);
  cfg.dynamicSmemBytes = smemBytes;
  cfg.stream = h->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, dd_tile_tma_kernel, map, q) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  h->launches++;
  h->lastKernel = "transform/tile-tma";
  return true;
}
