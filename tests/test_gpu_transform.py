"""GPU parity: ddTransformTensor (reorder + data type conversion) against the CPU oracle, bit for bit.

Covers the reference's reorder tests at the C level (dnnl core_test "Reordering memory" blocks,
deep-diamond-dnnl/test/uncomplicate/diamond/internal/dnnl/core_test.clj:260-361) and the stride /
data type space around them: every kernel family (flat, tile, strided, gather) and edge shapes.
"""
import numpy as np
import pytest

from deep_diamond_b200 import core

pytestmark = pytest.mark.gpu

NP = {"float": np.float32, "double": np.float64, "half": np.float16, "byte": np.int8,
      "int": np.int32, "uint8": np.uint8, "bf16": np.uint16, "long": np.int64}
TAG = {"float": "f32", "double": "f64", "half": "f16", "byte": "s8", "int": "s32", "uint8": "u8",
       "bf16": "bf16", "long": "s64"}


def make_values(rng, n, dt):
    """Source storage for data type `dt` with values that exercise rounding and saturation."""
    if dt in ("float", "double"):
        v = rng.standard_normal(n) * 100.0
        v[::7] = np.rint(v[::7]) + 0.5  # ties for round-to-nearest-even
        v[::13] *= 1e3                   # saturation for narrow integer destinations
        return v.astype(NP[dt])
    if dt == "half":
        return (rng.standard_normal(n) * 50.0).astype(np.float16)
    if dt == "bf16":
        f = (rng.standard_normal(n) * 50.0).astype(np.float32).view(np.uint32)
        return (f >> 16).astype(np.uint16)
    if dt == "byte":
        return rng.integers(-128, 128, n).astype(np.int8)
    if dt == "uint8":
        return rng.integers(0, 256, n).astype(np.uint8)
    if dt == "int":
        return rng.integers(-70000, 70000, n).astype(np.int32)
    return rng.integers(-70000, 70000, n).astype(np.int64)


def run_case(fact, dev, oracle, shape, sx, sy, sdt, ddt, alpha=1.0, beta=0.0, seed=0, expect=None):
    rng = np.random.default_rng(seed)
    nx, ny = oracle.span(shape, sx), oracle.span(shape, sy)
    xs = make_values(rng, nx, sdt)
    y0 = make_values(rng, ny, ddt) if beta != 0.0 else np.full(ny, 0, dtype=NP[ddt])
    if beta == 0.0:
        y0 = y0.view(np.uint8).copy()
        y0[:] = 0xCD  # canary: untouched padding must survive
        y0 = y0.view(NP[ddt])
    want = y0.copy()
    oracle.reorder(oracle.as_layout(xs, shape, sx), oracle.as_layout(want, shape, sy),
                   TAG[sdt], TAG[ddt], alpha, beta)
    dx, dy = dev.put(xs), dev.put(y0)
    xd = core.tensor_descriptor(shape, sdt, sx)
    yd = core.tensor_descriptor(shape, ddt, sy)
    core.transform_tensor(fact.handle, alpha, xd, dx, beta, yd, dy)
    got = dev.get(dy, NP[ddt])
    if expect:
        assert fact.handle.last_kernel() in ((expect,) if isinstance(expect, str) else expect), fact.handle.last_kernel()
    same = got.view(np.uint8) == want.view(np.uint8)
    if not same.all() and ddt in ("half", "bf16", "float", "double"):
        # NaN payloads may differ between the CPU and GPU converters; everything else is exact
        g = got.astype(np.float64) if ddt != "bf16" else (got.astype(np.uint32) << 16).view(np.float32)
        w = want.astype(np.float64) if ddt != "bf16" else (want.astype(np.uint32) << 16).view(np.float32)
        same = (got == want) | (np.isnan(g) & np.isnan(w))
    assert same.all(), "mismatch at %s" % np.flatnonzero(~same.reshape(-1))[:8]


def nchw(shape):
    import oracle
    return oracle.default_strides(shape)


def nhwc(shape):
    import oracle
    return oracle.nhwc_strides(shape)


def perm_strides(shape, order):
    """Dense strides whose physical order of dims (outermost first) is `order`."""
    st, run = [0] * len(shape), 1
    for d in reversed(order):
        st[d] = run
        run *= shape[d]
    return st


ALL = ["float", "double", "half", "byte", "int", "uint8", "bf16", "long"]


@pytest.mark.parametrize("sdt", ALL)
@pytest.mark.parametrize("ddt", ALL)
def test_every_type_pair_flat_tile_strided(fact, dev, oracle, sdt, ddt):
    # flat (same layout), tile (aligned nchw -> nhwc) and strided (odd shape) for each pair
    run_case(fact, dev, oracle, [3, 5, 7, 9], nchw([3, 5, 7, 9]), nchw([3, 5, 7, 9]), sdt, ddt, seed=1,
             expect="transform/flat")
    run_case(fact, dev, oracle, [2, 32, 8, 16], nchw([2, 32, 8, 16]), nhwc([2, 32, 8, 16]), sdt, ddt, seed=2,
             expect="transform/tile")
    run_case(fact, dev, oracle, [2, 3, 5, 7], nchw([2, 3, 5, 7]), nhwc([2, 3, 5, 7]), sdt, ddt, seed=3,
             expect="transform/strided")


@pytest.mark.parametrize("sdt,ddt", [("float", "float"), ("float", "bf16"), ("half", "float"), ("byte", "byte"),
                                     ("double", "float"), ("byte", "double"), ("int", "float")])
def test_rows_kernel(fact, dev, oracle, sdt, ddt):
    """Innermost dim contiguous on both sides but not one flat run: a channel window of a wider
    tensor, swapped outer dims, padded outer strides -- 16-byte vectors through the strided walk."""
    shape = [4, 6, 8, 16]
    window = [10 * 128, 128, 16, 1]                       # channels 0..5 of a [4,10,8,16] parent
    run_case(fact, dev, oracle, shape, window, nchw(shape), sdt, ddt, seed=41, expect="transform/rows")
    run_case(fact, dev, oracle, shape, nchw(shape), window, sdt, ddt, seed=42, expect="transform/rows")
    cnhw = [8 * 16, 4 * 8 * 16, 16, 1]                    # N and C swapped
    run_case(fact, dev, oracle, shape, nchw(shape), cnhw, sdt, ddt, seed=43, expect="transform/rows")
    padded = [6 * 8 * 32 + 64, 8 * 32, 32, 1]             # rows of 16 in a pitch of 32
    run_case(fact, dev, oracle, shape, padded, nchw(shape), sdt, ddt, seed=44, expect="transform/rows")
    if sdt == "float":
        run_case(fact, dev, oracle, shape, window, cnhw, sdt, ddt, alpha=2.0, beta=0.5, seed=45, expect="transform/rows")
    # a row length that is not a whole number of vectors stays with the element-wise walk
    odd = [4, 5, 7, 15]
    run_case(fact, dev, oracle, odd, [10 * 105, 105, 15, 1], nchw(odd), sdt, ddt, seed=46, expect="transform/strided")


@pytest.mark.parametrize("shape", [[2, 2, 3, 2], [1, 64, 56, 56], [4, 64, 8, 8], [2, 256, 28, 28],
                                   [3, 48, 4, 20], [2, 96, 1, 132], [5, 16, 3, 24], [1, 512, 2, 2]])
@pytest.mark.parametrize("pair", [("float", "float"), ("float", "bf16"), ("byte", "byte"),
                                  ("float", "byte"), ("half", "float")])
def test_nchw_nhwc_both_ways(fact, dev, oracle, shape, pair):
    sdt, ddt = pair
    run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), sdt, ddt, seed=4)
    run_case(fact, dev, oracle, shape, nhwc(shape), nchw(shape), sdt, ddt, seed=5)


ODD_TILE = ("transform/tile-scalar", "transform/tile-flat-in", "transform/tile-flat-out")


def test_unaligned_transposes_use_the_scalar_tile(fact, dev, oracle):
    # rows not 16-byte aligned: odd spatial sizes (7x7, 13x13), odd channel counts, every type width.
    # Where the short side's block is contiguous and the long side is vector-aligned the flat forms
    # run (asserted exactly in test_short_odd_rows_go_through_the_flat_tile), else the scalar tile.
    for shape in ([3, 24, 7, 7], [2, 33, 13, 13], [5, 9, 3, 11], [1, 100, 1, 37]):
        for sdt, ddt in (("float", "float"), ("float", "bf16"), ("byte", "byte"), ("half", "float"), ("double", "float")):
            run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), sdt, ddt, seed=31, expect=ODD_TILE)
            run_case(fact, dev, oracle, shape, nhwc(shape), nchw(shape), sdt, ddt, seed=32, expect=ODD_TILE)
    for shape in ([2, 33, 13, 13], [5, 9, 3, 11]):  # odd channel counts: neither side is vector-aligned
        run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), "float", "float", seed=31, expect="transform/tile-scalar")
    # an unaligned base pointer demotes an otherwise aligned reorder to the scalar tile
    shape = [2, 32, 8, 16]
    xs = make_values(np.random.default_rng(33), 1 + int(np.prod(shape)), "float")
    want = np.zeros(int(np.prod(shape)), np.float32)
    oracle.reorder(oracle.as_layout(xs, shape, nchw(shape), offset=1), oracle.as_layout(want, shape, nhwc(shape)))
    tx, ty = dev.put(xs), dev.put(np.zeros_like(want))
    core.transform_tensor(fact.handle, 1.0, core.tensor_descriptor(shape, "float", nchw(shape)), tx.data_ptr() + 4,
                          0.0, core.tensor_descriptor(shape, "float", nhwc(shape)), ty)
    assert fact.handle.last_kernel() == "transform/tile-scalar"
    assert np.array_equal(dev.get(ty, np.float32), want)


def test_tile_ragged_edges(fact, dev, oracle):
    # extents that are vector-aligned but not tile-aligned, in both tiled dims, with batch dims
    for shape in ([3, 72, 5, 12], [2, 200, 3, 28], [7, 8, 2, 68]):
        run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), "float", "float", seed=6,
                 expect="transform/tile")
    run_case(fact, dev, oracle, [2, 144, 4, 40], nchw([2, 144, 4, 40]), nhwc([2, 144, 4, 40]), "byte", "byte",
             seed=7, expect="transform/tile")
    run_case(fact, dev, oracle, [2, 144, 4, 40], nchw([2, 144, 4, 40]), nhwc([2, 144, 4, 40]), "float", "bf16",
             seed=8, expect="transform/tile")


@pytest.mark.parametrize("pair", [("float", "float"), ("byte", "byte"), ("float", "bf16"), ("bf16", "float"),
                                  ("half", "half"), ("double", "double"), ("float", "byte"), ("byte", "float"),
                                  ("uint8", "uint8"), ("int", "float"), ("long", "long")])
@pytest.mark.parametrize("shape", [[3, 64, 7, 7], [2, 48, 13, 13], [5, 32, 14, 14], [2, 256, 7, 7], [1, 16, 3, 5],
                                   [2, 400, 5, 5], [7, 16, 9, 9]])
def test_short_odd_rows_go_through_the_flat_tile(fact, dev, oracle, shape, pair):
    """nchw <-> nhwc with maps of 49, 169, 196, 15, 25, 81 elements and channel counts that are whole
    vectors: the nchw side moves as a flat stream of aligned 16-byte vectors (flat-in when it is the
    source, flat-out when it is the destination).  Bit for bit against the oracle; the canary in
    run_case checks that nothing is written outside the tensor."""
    sdt, ddt = pair
    n, c, hgt, w = shape
    vs, vd = 16 // np.dtype(NP[sdt]).itemsize, 16 // np.dtype(NP[ddt]).itemsize
    hw = hgt * w
    aligned_in = (c * hw) % vs == 0 or n == 1     # every batch entry's nchw block starts on a 16-byte boundary
    aligned_out = (c * hw) % vd == 0 or n == 1
    ok_in = aligned_in and c % vd == 0 and hw % vs != 0 and 16 * hw * np.dtype(NP[sdt]).itemsize <= 32768
    ok_out = aligned_out and c % vs == 0 and hw % vd != 0
    run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), sdt, ddt, seed=61,
             expect="transform/tile-flat-in" if ok_in else ODD_TILE + ("transform/tile", "transform/strided"))
    run_case(fact, dev, oracle, shape, nhwc(shape), nchw(shape), sdt, ddt, seed=62,
             expect="transform/tile-flat-out" if ok_out else ODD_TILE + ("transform/tile", "transform/strided"))


def test_flat_tile_many_chunks_and_batches(fact, dev, oracle):
    # more rows than one CTA's chunk holds (2048 channels of 49 bytes: 7 chunks; 2000 of 169 floats: 125 chunks),
    # a partial last chunk, and two batch dims that do not merge
    run_case(fact, dev, oracle, [3, 2048, 7, 7], nchw([3, 2048, 7, 7]), nhwc([3, 2048, 7, 7]), "byte", "byte", seed=63,
             expect="transform/tile-flat-in")
    run_case(fact, dev, oracle, [3, 2048, 7, 7], nhwc([3, 2048, 7, 7]), nchw([3, 2048, 7, 7]), "byte", "byte", seed=64,
             expect="transform/tile-flat-out")
    shape = [2, 2000, 13, 13]
    run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), "float", "bf16", seed=65, expect="transform/tile-flat-in")
    run_case(fact, dev, oracle, shape, nhwc(shape), nchw(shape), "bf16", "float", seed=66, expect="transform/tile-flat-out")
    run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), "byte", "byte", seed=67, expect="transform/tile-flat-in")
    run_case(fact, dev, oracle, shape, nhwc(shape), nchw(shape), "byte", "byte", seed=68, expect="transform/tile-flat-out")


@pytest.mark.parametrize("pair", [("float", "float"), ("uint8", "uint8"), ("uint8", "float"), ("float", "uint8"),
                                  ("byte", "byte"), ("half", "float"), ("float", "bf16")])
@pytest.mark.parametrize("shape", [[4, 3, 32, 48], [2, 4, 64, 64], [3, 1, 16, 80], [5, 2, 8, 24], [1, 3, 224, 224]])
def test_images_with_a_few_channels(fact, dev, oracle, shape, pair):
    """nchw <-> nhwc with 1 to 4 channels (a batch of images): the channel dim is too thin for a tile,
    so the interleaved side moves as a flat vector stream (the short-rows forms with rows of 3 or 4
    elements).  One channel is the same layout both ways: a flat copy."""
    sdt, ddt = pair
    n, c, hgt, w = shape
    to_nhwc = "transform/flat" if c == 1 else "transform/tile-flat-out"
    to_nchw = "transform/flat" if c == 1 else "transform/tile-flat-in"
    run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), sdt, ddt, seed=81, expect=to_nhwc)
    run_case(fact, dev, oracle, shape, nhwc(shape), nchw(shape), sdt, ddt, seed=82, expect=to_nchw)


@pytest.mark.parametrize("pair", [("float", "float"), ("float", "bf16"), ("byte", "byte"), ("half", "half"), ("double", "double")])
@pytest.mark.parametrize("n,c,hgt,w,blk", [(3, 64, 12, 20, 16), (2, 48, 28, 28, 8), (5, 64, 8, 16, 32), (1, 32, 6, 40, 4)])
def test_blocked_channel_layouts(fact, dev, oracle, n, c, hgt, w, blk, pair):
    """nchw <-> nChw{blk}c (oneDNN's blocked formats, written as rank-5 strides: the channel dim split
    into c / blk blocks and blk channels innermost).  A transposition whose B is only blk elements:
    the tile kernel runs it with as few lanes along B as cover blk (or the flat / strided forms where
    blk is less than two vectors).  Bit for bit against the oracle, both ways."""
    sdt, ddt = pair
    shape5 = [n, c // blk, blk, hgt, w]
    plain = [c * hgt * w, blk * hgt * w, hgt * w, w, 1]
    blocked = [c * hgt * w, blk * hgt * w, 1, blk * w, blk]
    run_case(fact, dev, oracle, shape5, plain, blocked, sdt, ddt, seed=91)
    run_case(fact, dev, oracle, shape5, blocked, plain, sdt, ddt, seed=92)
    vd = 16 // np.dtype(NP[ddt]).itemsize
    vs = 16 // np.dtype(NP[sdt]).itemsize
    if blk >= 2 * vd and (hgt * w) % vs == 0 and hgt * w >= 2 * vs:
        run_case(fact, dev, oracle, shape5, plain, blocked, sdt, ddt, seed=93, expect="transform/tile")


def test_padded_strides_round_trip(fact, dev, oracle):
    # core_test.clj:301-340: [2 2 3 2] through strides [48 100 8 3]; tensor_test.clj:171-194
    run_case(fact, dev, oracle, [2, 2, 3, 2], nchw([2, 2, 3, 2]), [48, 100, 8, 3], "float", "float", seed=9)
    run_case(fact, dev, oracle, [2, 2, 3, 2], [48, 100, 8, 3], nhwc([2, 2, 3, 2]), "float", "float", seed=10)
    run_case(fact, dev, oracle, [2, 3, 2, 1], [48, 16, 5, 2], [48, 13, 4, 2], "float", "float", seed=11)
    run_case(fact, dev, oracle, [2, 3, 2, 1], [48, 12, 4, 2], [48, 14, 4, 2], "float", "float", seed=12)


def test_alpha_beta_blend(fact, dev, oracle):
    for shape, sy in (([3, 5, 7, 9], nchw([3, 5, 7, 9])), ([2, 32, 8, 16], nhwc([2, 32, 8, 16]))):
        run_case(fact, dev, oracle, shape, nchw(shape), sy, "float", "float", alpha=3.0, beta=2.0, seed=13)
        run_case(fact, dev, oracle, shape, nchw(shape), sy, "float", "half", alpha=0.5, beta=0.0, seed=14)
        run_case(fact, dev, oracle, shape, nchw(shape), sy, "byte", "float", alpha=1.0, beta=1.0, seed=15)
        run_case(fact, dev, oracle, shape, nchw(shape), sy, "double", "double", alpha=2.0, beta=-1.0, seed=16)


def test_ranks_1_to_6_and_size_one_dims(fact, dev, oracle):
    run_case(fact, dev, oracle, [17], [1], [3], "float", "float", seed=17)
    run_case(fact, dev, oracle, [4, 6], [6, 1], [1, 4], "float", "float", seed=18)
    run_case(fact, dev, oracle, [2, 7, 1], [7, 1, 1], [1, 2, 1], "float", "float", seed=19)
    run_case(fact, dev, oracle, [1, 1, 1, 1], [1, 1, 1, 1], [1, 1, 1, 1], "float", "double", seed=20)
    run_case(fact, dev, oracle, [2, 3, 4, 5, 6], nchw([2, 3, 4, 5, 6]), nhwc([2, 3, 4, 5, 6]), "float", "float", seed=21)
    shape6 = [2, 3, 2, 3, 2, 4]
    run_case(fact, dev, oracle, shape6, nchw(shape6), perm_strides(shape6, [3, 0, 5, 1, 4, 2]), "float", "float", seed=22)
    run_case(fact, dev, oracle, shape6, perm_strides(shape6, [5, 4, 3, 2, 1, 0]), nchw(shape6), "byte", "float", seed=23)


def test_gather_matches_separate_transforms(fact, dev, oracle):
    # a shuffler invocation: rows [0 2 1] of a [6 2 1 1] source into a [3 2 1 1] destination with
    # another layout (tensor_test.clj:263-275), plus a typed case with larger items
    rng = np.random.default_rng(23)
    for (n_src, item, sdt, ddt) in ((6, [1, 2, 1, 1], "float", "float"), (9, [1, 16, 4, 8], "float", "half")):
        shape_src = [n_src] + item[1:]
        cols = [0, 2, 1, 5, 2]
        shape_dst = [len(cols)] + item[1:]
        sx, sy = nchw(shape_src), nhwc(shape_dst)
        xs = make_values(rng, oracle.span(shape_src, sx), sdt)
        want = np.zeros(oracle.span(shape_dst, sy), dtype=NP[ddt])
        for d, c in enumerate(cols):
            oracle.reorder(oracle.as_layout(xs, item, sx, offset=c * sx[0]),
                           oracle.as_layout(want, item, sy, offset=d * sy[0]), TAG[sdt], TAG[ddt])
        dx, dy = dev.put(xs), dev.put(np.zeros_like(want))
        xd = core.tensor_descriptor(item, sdt, sx)
        yd = core.tensor_descriptor(item, ddt, sy)
        core.gather_transform(fact.handle, [c * sx[0] for c in cols], [d * sy[0] for d in range(len(cols))],
                              xd, dx, yd, dy)
        got = dev.get(dy, NP[ddt])
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8))
        assert fact.handle.last_kernel().startswith("transform/gather")


def test_dense_gather_single_launch(fact, dev, oracle):
    """Shuffler-shaped gathers (contiguous rows, destinations one after another) take the dense
    single-launch kernel: 16-byte vectors when everything is aligned, single elements when not,
    with or without a conversion; scattered destinations fall back to the general kernel.  Checked
    against numpy row indexing (a row copy has no arithmetic) and the oracle's conversions."""
    rng = np.random.default_rng(31)
    cases = [  # rows in source, row length, picked rows, source type, destination type, expected kernel
        (5000, 64, 4096, "float", "float", "transform/gather-dense-vec"),
        (300, 7, 200, "float", "float", "transform/gather-dense"),
        (300, 48, 257, "byte", "byte", "transform/gather-dense-vec"),
        (100, 32, 60, "float", "int", "transform/gather-dense-vec"),
        (100, 32, 60, "float", "half", "transform/gather-dense"),
        (64, 33, 64, "half", "half", "transform/gather-dense"),
    ]
    for n_src, row, n_pick, sdt, ddt, kernel in cases:
        xs = make_values(rng, n_src * row, sdt)
        pick = rng.integers(0, n_src, n_pick)
        want = np.zeros(n_pick * row, dtype=NP[ddt])
        src_rows = xs.reshape(n_src, row)[pick]
        oracle.reorder(np.ascontiguousarray(src_rows), want.reshape(n_pick, row), TAG[sdt], TAG[ddt])
        dx, dy = dev.put(xs), dev.put(np.zeros_like(want))
        sub_x = core.tensor_descriptor([1, row], sdt, "nc")
        sub_y = core.tensor_descriptor([1, row], ddt, "nc")
        n0 = fact.handle.launch_count()
        core.gather_transform(fact.handle, [int(r) * row for r in pick], [d * row for d in range(n_pick)],
                              sub_x, dx, sub_y, dy)
        assert fact.handle.launch_count() - n0 == 1 and fact.handle.last_kernel() == kernel, (row, sdt, ddt)
        assert np.array_equal(dev.get(dy, NP[ddt]).view(np.uint8), want.view(np.uint8)), (row, sdt, ddt)
    # destinations in scattered order: the general kernel, 1500 items = two launches
    n_src, row, n_pick = 2000, 16, 1500
    xs = make_values(rng, n_src * row, "float")
    pick, place = rng.integers(0, n_src, n_pick), rng.permutation(n_pick)
    want = np.zeros(n_pick * row, np.float32)
    want.reshape(n_pick, row)[place] = xs.reshape(n_src, row)[pick]
    dx, dy = dev.put(xs), dev.put(np.zeros_like(want))
    sub = core.tensor_descriptor([1, row], "float", "nc")
    n0 = fact.handle.launch_count()
    core.gather_transform(fact.handle, [int(r) * row for r in pick], [int(d) * row for d in place], sub, dx, sub, dy)
    assert fact.handle.launch_count() - n0 == 2 and fact.handle.last_kernel() == "transform/gather"
    assert np.array_equal(dev.get(dy, np.float32), want)


def test_bad_arguments_are_reported_not_executed(fact, dev):
    import ctypes
    from deep_diamond_b200._lib import DiamondError
    x = dev.empty(1024)
    a = core.tensor_descriptor([2, 3, 4, 5], "float", "nchw")
    b = core.tensor_descriptor([2, 3, 4, 4], "float", "nchw")
    with pytest.raises(DiamondError) as e:
        core.transform_tensor(fact.handle, 1.0, a, x, 0.0, b, x)
    assert e.value.data["type"] == "bad-param"
    with pytest.raises(DiamondError):
        core.tensor_descriptor([2, 0, 4, 5], "float", "nchw")
    with pytest.raises(DiamondError):
        core.tensor_descriptor([2, 3], "f128", [3, 1])
