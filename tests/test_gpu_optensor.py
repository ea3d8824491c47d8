"""GPU parity: ddAddTensor / ddOpTensor / ddSumTensors / ddSetTensor / ddScaleTensor / ddTensorEquals
against the CPU oracle, bit for bit (one rounding per product and per sum on both sides).
Reference vectors: deep-diamond-dnnl/test/.../dnnl/core_test.clj:202-258 (scaled sums), :869-886
(binary add); bias add call sites deep-diamond-cuda/src/.../cudnn/directed.clj:508,579.
"""
import numpy as np
import pytest

from deep_diamond_b200 import core

pytestmark = pytest.mark.gpu


def rnd(shape, seed, lo=-1.0, hi=1.0):
    rng = np.random.default_rng(seed)
    return (rng.random(int(np.prod(shape)), dtype=np.float32) * (hi - lo) + lo).astype(np.float32)


@pytest.mark.parametrize("shape,bshape", [
    ([4, 32, 7, 7], [1, 32, 1, 1]),      # bias / per-channel scale, inner run not a multiple of 4
    ([4, 32, 14, 14], [1, 32, 1, 1]),    # inner run a multiple of 4: vector path
    ([3, 5, 2, 6], [3, 5, 2, 6]),        # same shape
    ([3, 5, 2, 6], [1, 1, 1, 1]),        # scalar
    ([3, 5, 2, 6], [1, 5, 1, 6]),        # two broadcast dims apart: strided kernel
    ([3, 5, 2, 6], [3, 1, 1, 1]),        # per-sample
])
@pytest.mark.parametrize("op", ["add", "mul", "min", "max", "sub", "div", "ge", "gt", "le", "lt", "eq", "ne"])
def test_op_tensor_broadcast(fact, dev, oracle, shape, bshape, op):
    a = rnd(shape, 1)
    b = rnd(bshape, 2, 0.5, 1.5)
    c0 = rnd(shape, 3)
    st, bst = oracle.default_strides(shape), oracle.default_strides(bshape)
    for (a1, a2, beta) in ((1.0, 1.0, 0.0), (1.0, 0.5, 0.0), (0.75, -2.0, 0.5)):
        want = c0.copy()
        oracle.binary(op, oracle.as_layout(a, shape, st), oracle.as_layout(b, bshape, bst),
                      oracle.as_layout(want, shape, st), alpha1=a1, alpha2=a2, beta=beta)
        ta, tb, tc = dev.put(a), dev.put(b), dev.put(c0)
        core.op_tensor(fact.handle, op, a1, core.tensor_descriptor(shape, "float", st), ta, a2,
                       core.tensor_descriptor(bshape, "float", bst), tb, beta,
                       core.tensor_descriptor(shape, "float", st), tc)
        got = dev.get(tc, np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (op, a1, a2, beta)


@pytest.mark.parametrize("op", ["add", "mul", "max"])
@pytest.mark.parametrize("shape,layout", [([6, 40, 7, 7], "nchw"), ([3, 24, 13, 13], "nchw"), ([5, 3, 1, 5], "nchw"),
                                          ([4, 36, 6, 6], "nhwc"), ([2, 1000, 3, 3], "nchw"), ([4, 6, 5, 6], "nhwc"),
                                          ([8, 10, 1, 3], "nchw")])
def test_channel_runs_that_are_not_whole_vectors(fact, dev, oracle, op, shape, layout):
    """Bias / per-channel scale where a channel's run (49, 169, 5, 9, 3 elements; 1 for nhwc) is not a
    multiple of four floats: A and C still move as 16-byte vectors and each element takes its own
    channel's value.  Three forms: a run at least a vector long (at most one run ends inside a
    vector), nhwc with a whole number of vectors per pixel (B read as vectors), and the element walk."""
    bshape = [1, shape[1], 1, 1]
    st = oracle.default_strides(shape) if layout == "nchw" else oracle.nhwc_strides(shape)
    bst = oracle.default_strides(bshape)
    a, b, c0 = rnd(shape, 21), rnd(bshape, 22, 0.5, 1.5), rnd(shape, 23)
    for (a1, a2, beta) in ((1.0, 1.0, 0.0), (0.75, -2.0, 0.5)):
        want = c0.copy()
        oracle.binary(op, oracle.as_layout(a, shape, st), oracle.as_layout(b, bshape, bst),
                      oracle.as_layout(want, shape, st), alpha1=a1, alpha2=a2, beta=beta)
        ta, tb, tc = dev.put(a), dev.put(b), dev.put(c0)
        core.op_tensor(fact.handle, op, a1, core.tensor_descriptor(shape, "float", st), ta, a2,
                       core.tensor_descriptor(bshape, "float", bst), tb, beta,
                       core.tensor_descriptor(shape, "float", st), tc)
        vector_b = layout == "nhwc" and shape[1] % 4 == 0
        assert fact.handle.last_kernel() == ("optensor/flat-bcast-vector" if vector_b else "optensor/flat-bcast-mixed")
        got = dev.get(tc, np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (op, a1, a2, beta)


@pytest.mark.parametrize("shape,layout,kernel", [([6, 40, 7, 7], "nchw", "optensor/flat-bcast-mixed"),
                                                 ([3, 24, 13, 13], "nchw", "optensor/flat-bcast-mixed"),
                                                 ([4, 40, 6, 6], "nhwc", "optensor/flat-bcast-vector"),
                                                 ([4, 12, 5, 6], "nhwc", "optensor/flat-bcast-mixed"),
                                                 ([8, 10, 1, 3], "nchw", "optensor/flat-bcast-mixed")])
def test_bias_on_bf16_maps_that_are_not_whole_vectors(fact, dev, oracle, shape, layout, kernel):
    """The same three forms with eight elements per vector (bf16): bias add y = 0.5*b[c] + y, bit-exact
    against the oracle (float arithmetic, one rounding to bf16)."""
    bshape = [1, shape[1], 1, 1]
    st = oracle.default_strides(shape) if layout == "nchw" else oracle.nhwc_strides(shape)
    to_bf16 = lambda v: (v.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    y0, b = to_bf16(rnd(shape, 31)), to_bf16(rnd(bshape, 32, 0.5, 1.5))
    want = y0.copy()
    oracle.add_tensor(0.5, oracle.as_layout(b, bshape, oracle.default_strides(bshape)), 1.0,
                      oracle.as_layout(want, shape, st), tag="bf16")
    ty, tb = dev.put(y0), dev.put(b)
    core.add_tensor(fact.handle, 0.5, core.tensor_descriptor(bshape, "bf16", "nchw"), tb, 1.0,
                    core.tensor_descriptor(shape, "bf16", st), ty)
    assert fact.handle.last_kernel() == kernel
    assert np.array_equal(dev.get(ty, np.uint16), want)


@pytest.mark.parametrize("op", ["add", "mul", "max"])
@pytest.mark.parametrize("bshape", [[1, 6, 1, 1], [4, 6, 8, 16], [1, 1, 1, 16], [4, 1, 8, 1]])
def test_op_tensor_rows_views(fact, dev, oracle, op, bshape):
    """A and C are channel windows of wider tensors (rows contiguous and 16-byte aligned), B a bias,
    a same-shape tensor, a row vector or a per-(n,h) scalar: the vectorised walk over views."""
    shape = [4, 6, 8, 16]
    win = [10 * 128, 128, 16, 1]                          # channels of a [4,10,8,16] parent
    span = oracle.span(shape, win)
    a, c0 = rnd([span], 11), rnd([span], 12)
    bst = oracle.default_strides(bshape)
    b = rnd(bshape, 13, 0.5, 1.5)
    for (a1, a2, beta) in ((1.0, 1.0, 0.0), (0.75, -2.0, 0.5)):
        want = c0.copy()
        oracle.binary(op, oracle.as_layout(a, shape, win), oracle.as_layout(b, bshape, bst),
                      oracle.as_layout(want, shape, win), alpha1=a1, alpha2=a2, beta=beta)
        ta, tb, tc = dev.put(a), dev.put(b), dev.put(c0)
        core.op_tensor(fact.handle, op, a1, core.tensor_descriptor(shape, "float", win), ta, a2,
                       core.tensor_descriptor(bshape, "float", bst), tb, beta,
                       core.tensor_descriptor(shape, "float", win), tc)
        assert fact.handle.last_kernel() == "optensor/rows", bshape
        got = dev.get(tc, np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (op, bshape, a1, a2, beta)


def test_add_tensor_bias_form_and_kernel_choice(fact, dev, oracle):
    shape, bshape = [8, 64, 14, 14], [1, 64, 1, 1]
    x, bias = rnd(shape, 4), rnd(bshape, 5, -0.1, 0.1)
    st, bst = oracle.default_strides(shape), oracle.default_strides(bshape)
    want = x.copy()
    oracle.add_tensor(0.5, oracle.as_layout(bias, bshape, bst), 1.0, oracle.as_layout(want, shape, st))
    tx, tb = dev.put(x), dev.put(bias)
    core.add_tensor(fact.handle, 0.5, core.tensor_descriptor(bshape, "float", bst), tb, 1.0,
                    core.tensor_descriptor(shape, "float", st), tx)
    assert fact.handle.last_kernel() == "optensor/flat-bcast"
    assert np.array_equal(dev.get(tx, np.float32).view(np.uint32), want.view(np.uint32))
    # beta == 0: y is not read, NaN in it does not propagate
    y = np.full(x.size, np.nan, dtype=np.float32)
    ty = dev.put(y)
    core.add_tensor(fact.handle, 2.0, core.tensor_descriptor(shape, "float", st), tx, 0.0,
                    core.tensor_descriptor(shape, "float", st), ty)
    assert np.array_equal(dev.get(ty, np.float32), 2.0 * want)
    # nhwc tensor with a channel bias: channel is the innermost dim
    sy = oracle.nhwc_strides(shape)
    want = x.copy()
    oracle.add_tensor(1.0, oracle.as_layout(bias, bshape, bst), 1.0, oracle.as_layout(want, shape, sy))
    tx = dev.put(x)
    core.add_tensor(fact.handle, 1.0, core.tensor_descriptor(bshape, "float", bst), tb, 1.0,
                    core.tensor_descriptor(shape, "float", sy), tx)
    assert np.array_equal(dev.get(tx, np.float32).view(np.uint32), want.view(np.uint32))


def test_reference_sum_and_binary_vectors(fact, dev):
    # core_test.clj:202-215 in-place scale; :217-236 two sources in place; :238-258 out of place
    d = core.tensor_descriptor([2, 3, 4, 5], "float", "nchw")
    buf = np.zeros(120, np.float32)
    buf[:2] = [-100, 20]
    t = dev.put(buf)
    core.sum_tensors(fact.handle, [2.0], [d], [t], d, t)
    assert dev.get(t, np.float32)[:2].tolist() == [-200.0, 40.0]
    src = np.zeros(120, np.float32); src[:2] = [-100, 10]
    dst = np.zeros(120, np.float32); dst[:2] = [-200, 20]
    ts, td = dev.put(src), dev.put(dst)
    core.sum_tensors(fact.handle, [2.0, 3.0], [d, d], [ts, td], d, td)   # dst = 2*src + 3*dst
    assert dev.get(td, np.float32)[:2].tolist() == [-800.0, 80.0]
    assert dev.get(ts, np.float32)[:2].tolist() == [-100.0, 10.0]
    s0 = np.zeros(120, np.float32); s0[:2] = [-100, 20]
    s1 = np.zeros(120, np.float32); s1[:2] = [-1000, 200]
    out = np.full(120, 1e5, np.float32)
    t0, t1, to = dev.put(s0), dev.put(s1), dev.put(out)
    core.sum_tensors(fact.handle, [2.0, 3.0], [d, d], [t0, t1], d, to)
    assert dev.get(to, np.float32)[:2].tolist() == [-3200.0, 640.0]
    # core_test.clj:869-886 binary add in place
    b0 = np.zeros(120, np.float32); b0[:2] = [-100, 20]
    b1 = np.zeros(120, np.float32); b1[:2] = [-200, 30]
    u0, u1 = dev.put(b0), dev.put(b1)
    core.op_tensor(fact.handle, "add", 1.0, d, u0, 1.0, d, u1, 0.0, d, u0)
    assert dev.get(u0, np.float32)[:2].tolist() == [-300.0, 50.0]


def test_sum_n_ary_matches_oracle(fact, dev, oracle):
    n_el = 4099
    srcs = [rnd([n_el], 10 + i) for i in range(5)]
    scales = [1.0, 0.5, -2.0, 1.0, 3.25]
    want = np.zeros(n_el, np.float32)
    oracle.scaled_sum(scales, srcs, want)
    d = core.tensor_descriptor([n_el], "float", [1])
    ts = [dev.put(s) for s in srcs]
    to = dev.put(np.zeros(n_el, np.float32))
    core.sum_tensors(fact.handle, scales, [d] * 5, ts, d, to)
    assert fact.handle.last_kernel() == "sum/flat"
    assert np.array_equal(dev.get(to, np.float32).view(np.uint32), want.view(np.uint32))


def test_set_and_scale_all_layouts(fact, dev, oracle):
    for dt, np_t in (("float", np.float32), ("double", np.float64), ("half", np.float16),
                     ("byte", np.int8), ("uint8", np.uint8), ("int", np.int32)):
        for shape, st in (([2, 3, 4, 5], [60, 20, 5, 1]), ([2, 2, 3, 2], [48, 100, 8, 3])):
            n = oracle.span(shape, st)
            base = np.full(n, 7, dtype=np_t)
            t = dev.put(base)
            d = core.tensor_descriptor(shape, dt, st)
            core.set_tensor(fact.handle, d, t, 3.0)
            got = dev.get(t, np_t)
            want = base.copy()
            oracle.as_layout(want, shape, st)[...] = 3
            assert np.array_equal(got, want)
            core.scale_tensor(fact.handle, 2.0, d, t)
            oracle.as_layout(want, shape, st)[...] = 6
            assert np.array_equal(dev.get(t, np_t), want)


def test_tensor_equals(fact, dev, oracle):
    import torch
    shape = [2, 3, 4, 5]
    x = rnd(shape, 20)
    flag = torch.zeros(1, dtype=torch.int32, device=fact.device)
    sx, sy = oracle.default_strides(shape), oracle.nhwc_strides(shape)
    y = np.zeros_like(x)
    oracle.reorder(oracle.as_layout(x, shape, sx), oracle.as_layout(y, shape, sy))
    tx, ty = dev.put(x), dev.put(y)
    dx, dy = core.tensor_descriptor(shape, "float", sx), core.tensor_descriptor(shape, "float", sy)
    core.tensor_equals(fact.handle, dx, tx, dy, ty, flag)
    fact.synchronize()
    assert int(flag.item()) == 0
    y[17] += 1.0
    ty = dev.put(y)
    core.tensor_equals(fact.handle, dx, tx, dy, ty, flag)
    fact.synchronize()
    assert int(flag.item()) != 0
    flag.zero_()
    core.tensor_equals(fact.handle, dx, tx, dx, tx, flag)
    fact.synchronize()
    assert int(flag.item()) == 0 and fact.handle.last_kernel() == "equals/flat"


def test_comparison_kinds_on_known_values(fact, dev):
    """oneDNN's comparison kinds (dnnl/constants.clj:359-371): 1 where the relation holds, else 0; a
    NaN compares false except under :ne; -0 equals +0."""
    a = np.array([1.0, 2.0, 3.0, np.nan, -0.0, 5.0, 7.0, 7.0], np.float32)
    b = np.array([2.0, 2.0, 1.0, 1.0, 0.0, np.nan, 7.0, 8.0], np.float32)
    d = core.tensor_descriptor([8], "float", [1])
    want = {"ge": a >= b, "gt": a > b, "le": a <= b, "lt": a < b, "eq": a == b, "ne": a != b}
    for op, w in want.items():
        tc = dev.put(np.full(8, -9.0, np.float32))
        core.op_tensor(fact.handle, op, 1.0, d, dev.put(a), 1.0, d, dev.put(b), 0.0, d, tc)
        assert dev.get(tc, np.float32).tolist() == w.astype(np.float32).tolist(), op


def test_equality_stops_early_and_stays_exact(fact, dev):
    """A mismatch anywhere (first element, last element, the scalar tail) raises the flag; equal
    tensors leave it alone; a flag already raised stays raised."""
    import torch
    n = (1 << 22) + 3
    x = np.random.default_rng(5).standard_normal(n).astype(np.float32)
    d = core.tensor_descriptor([n], "float", [1])
    tx = dev.put(x)
    for where in (None, 0, n // 2, n - 4, n - 1):
        y = x.copy()
        if where is not None:
            y[where] += 1.0
        flag = torch.zeros(1, dtype=torch.int32, device=fact.device)
        core.tensor_equals(fact.handle, d, tx, d, dev.put(y), flag)
        fact.synchronize()
        assert (int(flag.item()) != 0) == (where is not None), where
    flag = torch.ones(1, dtype=torch.int32, device=fact.device)
    core.tensor_equals(fact.handle, d, tx, d, tx, flag)
    fact.synchronize()
    assert int(flag.item()) != 0
