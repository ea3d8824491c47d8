"""GPU parity: ddReduceTensor against the CPU oracle.

Bars: max/min/amax bit-exact; sums, means and norms within 1e-5 relative of the fp32 oracle and of the
long-double truth, the denominator conditioned as max(|truth|, eps * sum|x|) so that cancelling sums
are judged against what fp32 summation can deliver.  Reference vectors:
deep-diamond-dnnl/test/.../dnnl/core_test.clj:888-943, deep-diamond-cuda/test/.../cudnn/core_test.clj:149-178.
"""
import numpy as np
import pytest

from deep_diamond_b200 import core

pytestmark = pytest.mark.gpu

EXACT = {"max", "min", "amax"}


def run_reduce(fact, dev, oracle, op, shape, yshape, sx=None, sy=None, alpha=1.0, beta=0.0, seed=0,
               dtype="float", expect=None, data=None):
    np_t = {"float": np.float32, "double": np.float64}[dtype]
    sx = sx or oracle.default_strides(shape)
    sy = sy or oracle.default_strides(yshape)
    rng = np.random.default_rng(seed)
    nx, ny = oracle.span(shape, sx), oracle.span(yshape, sy)
    if data is None:
        data = (np.exp(rng.standard_normal(nx)) * np.where(rng.random(nx) < 0.5, -1, 1)).astype(np_t)
        if op in ("mul", "mul-no-zeros"):
            data = (1.0 + 0.01 * rng.standard_normal(nx)).astype(np_t)
    y0 = rng.standard_normal(ny).astype(np_t)
    want = y0.copy()
    _, truth = oracle.reduce(op, oracle.as_layout(data, shape, sx), oracle.as_layout(want, yshape, sy),
                             alpha=alpha, beta=beta, want_truth=True)
    tx, ty = dev.put(data), dev.put(y0)
    xd, yd = core.tensor_descriptor(shape, dtype, sx), core.tensor_descriptor(yshape, dtype, sy)
    rtd = core.reduce_tensor_descriptor(op, dtype)
    core.reduce_tensor(fact.handle, rtd, alpha, xd, tx, beta, yd, ty)
    got = dev.get(ty, np_t)
    if expect:
        assert fact.handle.last_kernel().startswith(expect), fact.handle.last_kernel()
    if op in EXACT and beta == 0.0:
        assert np.array_equal(got, want)
        return got
    # Error bar: 1e-5 relative to the result, or -- where the terms cancel and the result is small
    # against sum|x| -- the error bound of pairwise fp32 summation, log2(n) * u * sum|x| (u = eps/2).
    # Against the fp32 oracle both sides carry that error, so the floor doubles.
    absx = np.abs(oracle.as_layout(data, shape, sx).astype(np.float64))
    axes = tuple(i for i in range(len(shape)) if yshape[i] == 1 and shape[i] != 1)
    nred = int(np.prod([shape[i] for i in axes])) if axes else 1
    if op in ("add", "avg"):
        scale = absx.sum(axis=axes, keepdims=True)
        if op == "avg":
            scale = scale / nred
    else:
        scale = np.abs(truth)
    gv = oracle.as_layout(got, yshape, sy).astype(np.float64)
    wv = oracle.as_layout(want, yshape, sy).astype(np.float64)
    y0v = oracle.as_layout(y0, yshape, sy).astype(np.float64)
    tv = alpha * truth + beta * y0v
    u = np.finfo(np_t).eps / 2
    floor = abs(alpha) * max(1.0, np.ceil(np.log2(max(nred, 2)))) * u * scale.reshape(tv.shape)
    rel = 1e-5 if dtype == "float" else 1e-13
    assert (np.abs(gv - tv) <= np.maximum(rel * np.abs(tv), floor)).all()
    assert (np.abs(gv - wv) <= np.maximum(rel * np.abs(wv), 2 * floor)).all()
    return got


OPS = ["add", "avg", "max", "min", "amax", "norm1", "norm2", "mul"]


@pytest.mark.parametrize("op", OPS)
def test_nchw_patterns(fact, dev, oracle, op):
    shape = [6, 20, 12, 16]
    run_reduce(fact, dev, oracle, op, shape, [1, 20, 1, 1], seed=1, expect="reduce/row")      # keep C
    run_reduce(fact, dev, oracle, op, shape, [6, 1, 12, 16], seed=2, expect="reduce/col")     # over C
    run_reduce(fact, dev, oracle, op, shape, [6, 1, 1, 1], seed=3, expect="reduce/row")       # keep N
    run_reduce(fact, dev, oracle, op, shape, [1, 1, 1, 1], seed=4, expect="reduce/row")       # everything
    run_reduce(fact, dev, oracle, op, shape, [6, 20, 12, 1], seed=5)                          # over W
    run_reduce(fact, dev, oracle, op, shape, [6, 20, 1, 1], seed=6)                           # over H, W
    run_reduce(fact, dev, oracle, op, shape, [1, 1, 12, 16], seed=7, expect="reduce/col")     # over N, C
    run_reduce(fact, dev, oracle, op, shape, [6, 20, 12, 16], seed=8)                         # nothing reduced


@pytest.mark.parametrize("op", ["add", "max", "norm2"])
def test_nhwc_and_odd_shapes(fact, dev, oracle, op):
    shape = [3, 24, 5, 7]
    sx = oracle.nhwc_strides(shape)
    run_reduce(fact, dev, oracle, op, shape, [1, 24, 1, 1], sx=sx, seed=9, expect="reduce/col")
    run_reduce(fact, dev, oracle, op, shape, [3, 1, 5, 7], sx=sx, seed=10)
    run_reduce(fact, dev, oracle, op, [5, 3, 7, 11], [1, 3, 1, 1], seed=11)   # unaligned rows: scalar loads
    run_reduce(fact, dev, oracle, op, [5, 3, 7, 11], [5, 1, 7, 11], seed=12)
    run_reduce(fact, dev, oracle, op, [2, 2, 3, 2], [2, 1, 3, 1], sx=[48, 100, 8, 3], seed=13,
               expect="reduce/generic")


@pytest.mark.parametrize("op", ["add", "avg", "max", "norm2"])
def test_split_ranges_use_the_workspace(fact, dev, oracle, op):
    # few outputs with long reduce ranges: several CTAs per output + the finishing kernel
    run_reduce(fact, dev, oracle, op, [4, 64, 32, 32], [4, 1, 1, 1], seed=14, expect="reduce/row")
    run_reduce(fact, dev, oracle, op, [1, 1, 1, 1 << 20], [1, 1, 1, 1], seed=15, expect="reduce/row")
    run_reduce(fact, dev, oracle, op, [2048, 8, 1, 16], [1, 8, 1, 16], seed=16, expect="reduce/col")
    run_reduce(fact, dev, oracle, op, [64, 16, 32, 32], [1, 16, 1, 1], seed=17, expect="reduce/row")


def test_alpha_beta_and_double(fact, dev, oracle):
    run_reduce(fact, dev, oracle, "add", [6, 20, 12, 16], [1, 20, 1, 1], alpha=3.0, beta=2.0, seed=18)
    run_reduce(fact, dev, oracle, "max", [6, 20, 12, 16], [6, 1, 12, 16], alpha=2.5, beta=0.0, seed=19)
    run_reduce(fact, dev, oracle, "add", [6, 20, 12, 16], [1, 20, 1, 1], dtype="double", seed=20)
    run_reduce(fact, dev, oracle, "norm2", [6, 20, 12, 16], [6, 1, 1, 1], dtype="double", seed=21)
    run_reduce(fact, dev, oracle, "max", [6, 20, 12, 16], [6, 1, 12, 16], dtype="double", seed=22)


def test_reference_vectors(fact, dev, oracle):
    x = np.arange(120, dtype=np.float32)
    # core_test.clj:888-905 sum over W
    got = run_reduce(fact, dev, oracle, "add", [2, 3, 4, 5], [2, 3, 4, 1], data=x)
    assert got[:3].tolist() == [10.0, 35.0, 60.0]
    # :907-924 max over (N,H,W)
    got = run_reduce(fact, dev, oracle, "max", [2, 3, 4, 5], [1, 3, 1, 1], data=x)
    assert got.tolist() == [79.0, 99.0, 119.0]
    # :926-943 L2 over W
    got = run_reduce(fact, dev, oracle, "norm2", [2, 3, 4, 5], [2, 3, 4, 1], data=x)
    want = [np.float32(np.sqrt(sum(i * i for i in range(a, a + 5)))) for a in (0, 5, 10)]
    assert np.allclose(got[:3], want, rtol=1e-6)
    # cudnn core_test.clj:149-178: 3*sum + 2*y, 2.5*max, 1.5*prod over [2 3 1 1] -> [1 1 1 1]
    v = np.array([1, 2, 3, 4, 5, 6], dtype=np.float32)
    d_x = core.tensor_descriptor([2, 3, 1, 1], "float", "nchw")
    d_y = core.tensor_descriptor([1, 1, 1, 1], "float", "nchw")
    tx, ty = dev.put(v), dev.put(np.zeros(1, np.float32))
    core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor("add", "float"), 3.0, d_x, tx, 2.0, d_y, ty)
    assert dev.get(ty, np.float32)[0] == 63.0
    core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor("max", "float"), 2.5, d_x, tx, 0.0, d_y, ty)
    assert dev.get(ty, np.float32)[0] == 15.0
    core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor("mul", "float"), 1.5, d_x, tx, 0.0, d_y, ty)
    assert dev.get(ty, np.float32)[0] == 1080.0


def test_caller_workspace_and_run_to_run_identity(fact, dev, oracle):
    import torch
    shape, yshape = [4, 64, 32, 32], [4, 1, 1, 1]
    x = np.random.default_rng(30).standard_normal(int(np.prod(shape))).astype(np.float32)
    xd = core.tensor_descriptor(shape, "float", "nchw")
    yd = core.tensor_descriptor(yshape, "float", "nchw")
    rtd = core.reduce_tensor_descriptor("add", "float")
    need = core.reduction_workspace_size(fact.handle, rtd, xd, yd)
    assert need > 0 and core.reduction_indices_size(fact.handle, rtd, xd, yd) == 0
    ws = torch.empty(need, dtype=torch.uint8, device=fact.device)
    tx = dev.put(x)
    outs = []
    for _ in range(3):
        ty = dev.put(np.zeros(4, np.float32))
        core.reduce_tensor(fact.handle, rtd, None, ws, 1.0, xd, tx, 0.0, yd, ty)
        outs.append(dev.get(ty, np.float32))
    ty = dev.put(np.zeros(4, np.float32))
    core.reduce_tensor(fact.handle, rtd, 1.0, xd, tx, 0.0, yd, ty)   # handle-owned scratch
    outs.append(dev.get(ty, np.float32))
    for o in outs[1:]:
        assert np.array_equal(o.view(np.uint32), outs[0].view(np.uint32))
    from deep_diamond_b200._lib import DiamondError
    small = torch.empty(8, dtype=torch.uint8, device=fact.device)
    with pytest.raises(DiamondError):
        core.reduce_tensor(fact.handle, rtd, None, small, 1.0, xd, tx, 0.0, yd, ty)


def test_nan_propagation(fact, dev):
    v = np.array([1, np.nan, 3, 4, 5, 6], dtype=np.float32)
    d_x = core.tensor_descriptor([2, 3, 1, 1], "float", "nchw")
    d_y = core.tensor_descriptor([1, 1, 1, 1], "float", "nchw")
    tx, ty = dev.put(v), dev.put(np.zeros(1, np.float32))
    core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor("max", "float", True), 1.0, d_x, tx, 0.0, d_y, ty)
    assert np.isnan(dev.get(ty, np.float32)[0])
    core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor("max", "float", False), 1.0, d_x, tx, 0.0, d_y, ty)
    assert dev.get(ty, np.float32)[0] == 6.0


@pytest.mark.parametrize("tag,np_t", [("float", np.float32), ("half", np.float16), ("bf16", None), ("double", np.float64)])
@pytest.mark.parametrize("op", ["max", "min", "amax"])
def test_nan_modes_on_every_min_max_path(fact, dev, oracle, tag, np_t, op):
    """A NaN among the reduced elements comes out as NaN with propagation on and is ignored with it
    off, through the row, column and generic kernels and, for the 16-bit types, through the packed
    forms (max.NaN.bf16x2 / f16x2); outputs whose elements hold no NaN are exact either way."""
    rng = np.random.default_rng(41)
    for shape, yshape in (([6, 32, 12, 16], [1, 32, 1, 1]), ([6, 32, 12, 16], [6, 1, 12, 16]), ([96, 96, 28, 28], [96, 1, 28, 28]),
                          ([16, 128, 28, 28], [1, 128, 1, 1]), ([2, 3, 4, 5], [2, 3, 4, 1])):
        n = int(np.prod(shape))
        xf = (rng.standard_normal(n) * 3).astype(np.float32)
        if tag == "bf16":
            bits = (xf.view(np.uint32) >> 16).astype(np.uint16)
            vals = (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
            store, nan_bits = bits, np.uint16(0x7FC0)
        else:
            store = xf.astype(np_t)
            vals = store.astype(np.float64)
            nan_bits = np_t(np.nan)
        hit = rng.choice(n, size=max(1, n // 997), replace=False)
        store = store.copy()
        store[hit] = nan_bits
        has_nan = np.zeros(n, bool)
        has_nan[hit] = True
        axes = tuple(i for i in range(4) if yshape[i] == 1 and shape[i] != 1)
        v = np.abs(vals) if op == "amax" else vals
        fill = -np.inf if op in ("max", "amax") else np.inf
        clean = np.where(has_nan, fill, v).reshape(shape)
        ref = clean.max(axis=axes) if op != "min" else clean.min(axis=axes)
        any_nan = has_nan.reshape(shape).any(axis=axes)
        xd, yd = core.tensor_descriptor(shape, tag, "nchw"), core.tensor_descriptor(yshape, tag, "nchw")
        tx = dev.put(store)
        for prop in (True, False):
            ty = dev.empty(ref.size * store.itemsize)
            core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor(op, "double" if tag == "double" else "float", prop),
                               1.0, xd, tx, 0.0, yd, ty)
            raw = dev.get(ty, store.dtype)
            got = (raw.astype(np.uint32) << 16).view(np.float32).astype(np.float64) if tag == "bf16" else raw.astype(np.float64)
            got = got.reshape(ref.shape)
            if prop:
                assert np.isnan(got[any_nan]).all(), (shape, yshape, fact.handle.last_kernel())
                assert np.array_equal(got[~any_nan], ref[~any_nan]), (shape, yshape, fact.handle.last_kernel())
            else:
                all_nan = ~np.isfinite(ref)   # an output all of whose elements are NaN: not produced by these inputs
                assert not all_nan.any()
                assert np.array_equal(got, ref), (shape, yshape, fact.handle.last_kernel())


def test_convolution_bwd_bias(fact, dev, oracle):
    """The bias gradient (cudnn/core.clj:344-350) is the (N,H,W) sum: db = alpha * sum(dy) + beta * db."""
    shape, bshape = [16, 48, 9, 7], [1, 48, 1, 1]
    dy = oracle.gen_normal(shape, 1.0, 11)
    db0 = np.linspace(-2, 2, 48, dtype=np.float32)
    for alpha, beta in ((1.0, 0.0), (0.5, 2.0)):
        want = db0.copy().reshape(bshape)
        oracle.reduce("add", dy, want, alpha=alpha, beta=beta)
        tdy, tdb = dev.put(dy), dev.put(db0)
        core.convolution_bwd_bias(fact.handle, alpha, core.tensor_descriptor(shape, "float", "nchw"), tdy, beta,
                                  core.tensor_descriptor(bshape, "float", "nchw"), tdb)
        got = dev.get(tdb, np.float32).reshape(bshape)
        scale = np.abs(dy.astype(np.float64)).sum(axis=(0, 2, 3), keepdims=True)
        assert (np.abs(got - want) <= np.maximum(1e-5 * np.abs(want), 12 * 6e-8 * abs(alpha) * scale)).all()
    # nhwc gradient, same result layout
    dyn = np.ascontiguousarray(dy.transpose(0, 2, 3, 1))
    want = np.zeros(bshape, np.float32)
    oracle.reduce("add", dy, want)
    tdy, tdb = dev.put(dyn), dev.put(np.zeros(48, np.float32))
    core.convolution_bwd_bias(fact.handle, 1.0, core.tensor_descriptor(shape, "float", "nhwc"), tdy, 0.0,
                              core.tensor_descriptor(bshape, "float", "nchw"), tdb)
    got = dev.get(tdb, np.float32).reshape(bshape)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-4)


LP_KINDS = ["norm-lp-max", "norm-lp-sum", "norm-lp-power-p-max", "norm-lp-power-p-sum"]


@pytest.mark.parametrize("kind", LP_KINDS)
@pytest.mark.parametrize("p,eps", [(1.0, 0.0), (2.0, 0.0), (2.0, 0.25), (3.0, 1e-3), (2.5, 0.0), (1.5, 1e12)])
def test_norm_lp_kinds(fact, dev, oracle, kind, p, eps):
    """oneDNN's norm reductions with p and epsilon (dnnl/constants.clj:393-402, `reduction` of
    dnnl/core.clj:796-803) against the oracle: row, column, split and generic plans; fp32 and fp64.
    Bar: 1e-5 relative (all terms are non-negative, nothing cancels); CUDA's powf is within a few ulp
    of the oracle's."""
    rng = np.random.default_rng(17)
    cases = [([6, 20, 12, 16], [1, 20, 1, 1]), ([6, 20, 12, 16], [6, 1, 12, 16]), ([2, 3, 4, 5], [2, 3, 4, 1]),
             ([4, 8, 64, 64], [4, 1, 1, 1]), ([3, 5, 7, 11], [1, 5, 1, 11])]
    for dtype, np_t, rel in (("float", np.float32, 1e-5), ("double", np.float64, 1e-12)):
        for shape, yshape in cases:
            n = int(np.prod(shape))
            data = (np.exp(0.5 * rng.standard_normal(n)) * np.where(rng.random(n) < 0.5, -1, 1)).astype(np_t)
            y0 = rng.standard_normal(int(np.prod(yshape))).astype(np_t)
            want = y0.copy().reshape(yshape)
            _, truth = oracle.reduce_lp(kind, p, eps, data.reshape(shape), want, alpha=1.5, beta=0.5, want_truth=True)
            tx, ty = dev.put(data), dev.put(y0)
            xd, yd = core.tensor_descriptor(shape, dtype, "nchw"), core.tensor_descriptor(yshape, dtype, "nchw")
            rtd = core.reduce_tensor_descriptor(kind, dtype, True, p=p, eps=eps)
            assert rtd.lp() == (p, eps)
            core.reduce_tensor(fact.handle, rtd, 1.5, xd, tx, 0.5, yd, ty)
            got = dev.get(ty, np_t).reshape(yshape).astype(np.float64)
            tv = 1.5 * truth + 0.5 * y0.reshape(yshape).astype(np.float64)
            assert (np.abs(got - tv) <= rel * np.abs(tv) + rel * np.abs(0.5 * y0.reshape(yshape))).all(), (dtype, shape, yshape)
            assert (np.abs(got - want.astype(np.float64)) <= 2 * rel * np.abs(tv) + rel).all(), (dtype, shape, yshape)
            rtd.release()


def test_norm_lp_matches_the_named_norms_bit_for_bit(fact, dev, oracle):
    """norm-lp-sum with p = 2, eps = 0 IS norm2 (same accumulation, same root), p = 1 IS norm1."""
    shape, yshape = [8, 32, 16, 16], [1, 32, 1, 1]
    data = oracle.gen_normal(shape, 1.0, 9).reshape(-1)
    xd, yd = core.tensor_descriptor(shape, "float", "nchw"), core.tensor_descriptor(yshape, "float", "nchw")
    tx = dev.put(data)
    outs = {}
    for name, args in (("norm2", ("norm2",)), ("lp2", ("norm-lp-sum", "float", True, None, 2.0, 0.0)),
                       ("norm1", ("norm1",)), ("lp1", ("norm-lp-sum", "float", True, None, 1.0, 0.0))):
        ty = dev.put(np.zeros(32, np.float32))
        core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor(*args), 1.0, xd, tx, 0.0, yd, ty)
        outs[name] = dev.get(ty, np.float32)
    assert np.array_equal(outs["norm2"], outs["lp2"])
    assert np.array_equal(outs["norm1"], outs["lp1"])


def test_norm_lp_bad_p(fact):
    from deep_diamond_b200.constants import DiamondError
    with pytest.raises(DiamondError):
        core.reduce_tensor_descriptor("norm-lp-sum", "float", True, p=0.5, eps=0.0)


@pytest.mark.parametrize("tag,np_t", [("float", np.float32), ("double", np.float64), ("half", np.float16)])
@pytest.mark.parametrize("op", ["max", "min", "amax"])
def test_flattened_indices(fact, dev, tag, np_t, op):
    """The reference's 4-argument reduce-tensor-descriptor (cudnn/core.clj:188-196) with :flattened:
    min / max / amax also report the position of the winning element as an offset into the
    row-major block of the reduced dims (original dim order), the first one among equals; other ops
    and :no-indices need no buffer.  Checked against numpy's argmax / argmin on duplicated and
    NaN-carrying data, on permuted strides too."""
    import torch
    rng = np.random.default_rng(77)
    cases = [([6, 20, 12, 16], [1, 20, 1, 1], "nchw"), ([6, 20, 12, 16], [6, 1, 12, 16], "nchw"), ([6, 20, 12, 16], [6, 20, 1, 1], "nhwc"),
             ([3, 5, 7, 11], [1, 5, 1, 11], "nchw"), ([4, 8, 64, 64], [4, 1, 1, 1], "nchw"), ([2, 3, 4, 5], [1, 1, 1, 1], "nhwc"),
             ([8, 24, 32, 32], [8, 1, 32, 32], "nchw")]   # 8192 outputs, unit-stride dim kept: a thread per output
    for shape, yshape, layout in cases:
        n = int(np.prod(shape))
        logical = rng.integers(-40, 40, size=shape).astype(np_t)        # many ties
        logical.reshape(-1)[rng.choice(n, 3, replace=False)] = np.nan
        axes = tuple(i for i in range(4) if yshape[i] == 1 and shape[i] != 1)
        kept = tuple(i for i in range(4) if i not in axes)
        # storage in the chosen layout
        if layout == "nhwc":
            store = np.ascontiguousarray(logical.transpose(0, 2, 3, 1)).reshape(-1)
        else:
            store = logical.reshape(-1).copy()
        xd = core.tensor_descriptor(shape, tag, layout)
        yd = core.tensor_descriptor(yshape, tag, "nchw")
        # reduced block flattened in original dim order, one row per output (outputs in row-major order of y)
        block = logical.transpose(kept + axes).reshape(int(np.prod([shape[i] for i in kept])) if kept else 1, -1).astype(np.float64)
        v = np.abs(block) if op == "amax" else block
        for prop in (True, False):
            rtd = core.reduce_tensor_descriptor(op, "double" if tag == "double" else "float", prop, "flattened")
            need = core.reduction_indices_size(fact.handle, rtd, xd, yd)
            assert need == block.shape[0] * 4
            ind = torch.full((block.shape[0],), 0x7fffffff, dtype=torch.int32, device=fact.device)
            ws = torch.empty(max(core.reduction_workspace_size(fact.handle, rtd, xd, yd), 16), dtype=torch.uint8, device=fact.device)
            ty = dev.empty(block.shape[0] * store.itemsize)
            core.reduce_tensor(fact.handle, rtd, ind, ws, 1.0, xd, dev.put(store), 0.0, yd, ty)
            assert fact.handle.last_kernel() == "reduce/positions"
            fact.synchronize()
            got = ind.cpu().numpy().astype(np.int64)
            if prop:
                filled = np.where(np.isnan(v), np.inf if op != "min" else -np.inf, v)   # a NaN wins
            else:
                filled = np.where(np.isnan(v), -np.inf if op != "min" else np.inf, v)   # a NaN never wins
            want = filled.argmin(axis=1) if op == "min" else filled.argmax(axis=1)
            assert np.array_equal(got, want), (shape, yshape, layout, op, prop)
            # and the value at that position is the reduction's result
            res = dev.get(ty, np_t).astype(np.float64)
            picked = v[np.arange(block.shape[0]), got]
            assert np.array_equal(np.isnan(res), np.isnan(picked)) and np.array_equal(res[~np.isnan(res)], picked[~np.isnan(res)])
    # no buffer needed without the setting, or for an op that has no position
    xd, yd = core.tensor_descriptor([2, 3, 4, 5], tag, "nchw"), core.tensor_descriptor([1, 3, 1, 1], tag, "nchw")
    assert core.reduction_indices_size(fact.handle, core.reduce_tensor_descriptor(op, "float", True), xd, yd) == 0
    assert core.reduction_indices_size(fact.handle, core.reduce_tensor_descriptor("add", "float", True, "flattened"), xd, yd) == 0
    from deep_diamond_b200._lib import DiamondError
    with pytest.raises(DiamondError):   # asked for, not given a buffer
        core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor(op, "float", True, "flattened"), 1.0, xd,
                           dev.put(np.zeros(120, np_t)), 0.0, yd, dev.empty(3 * 8))
