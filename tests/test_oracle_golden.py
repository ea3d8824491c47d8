"""Pins the CPU oracle: every known-answer vector the reference's own tests hold for the tensor hot
path, replayed through oracle/ (no GPU needed), plus the committed outputs of real oneDNN.

Abbreviations for the reference's test files:
  dnnl-core   deep-diamond-dnnl/test/uncomplicate/diamond/internal/dnnl/core_test.clj
  cudnn-core  deep-diamond-cuda/test/uncomplicate/diamond/internal/cudnn/core_test.clj
  tensor-t    deep-diamond-test/src/uncomplicate/diamond/tensor_test.clj
  dnn-t       deep-diamond-test/src/uncomplicate/diamond/dnn_test.clj
  dnnl-tz     deep-diamond-dnnl/test/uncomplicate/diamond/internal/dnnl/dnnl_tensor_test.clj
"""
import os

import numpy as np
import pytest

from conftest import ulp_diff_f32

NCHW = lambda o, s: o.default_strides(s)  # noqa: E731
NHWC = lambda o, s: o.nhwc_strides(s)     # noqa: E731


def lay(oracle, buf, shape, strides, offset=0):
    return oracle.as_layout(buf, shape, strides, offset)


# ----------------------------------------------------------------------------- reorder ---------

def test_reorder_nchw_nhwc_identity_and_s8(oracle):
    """dnnl-core :260-299 -- [2 2 3 2], data (range 24)."""
    dims = [2, 2, 3, 2]
    a = np.arange(24, dtype=np.float32)
    c = np.zeros(24, np.float32)
    oracle.reorder(lay(oracle, a, dims, NCHW(oracle, dims)), lay(oracle, c, dims, NHWC(oracle, dims)))
    assert not np.array_equal(a, c)
    assert np.linalg.norm(a) == np.linalg.norm(c)
    assert c.tolist() == [0, 6, 1, 7, 2, 8, 3, 9, 4, 10, 5, 11, 12, 18, 13, 19, 14, 20, 15, 21, 16, 22, 17, 23]
    b = np.zeros(24, np.float32)
    oracle.reorder(lay(oracle, a, dims, NCHW(oracle, dims)), lay(oracle, b, dims, NCHW(oracle, dims)))
    assert np.array_equal(a, b)
    d = np.full(24, -1, np.int8)
    oracle.reorder(lay(oracle, a, dims, NCHW(oracle, dims)), lay(oracle, d, dims, NHWC(oracle, dims)))
    assert int(d.astype(np.int64).sum()) == 276


def test_reorder_with_strides_round_trip(oracle):
    """dnnl-core :301-340 -- a -> b[48 100 8 3] -> c(nhwc) -> d(nchw); b -> b1 -> d1."""
    dims = [2, 2, 3, 2]
    bs = [48, 100, 8, 3]
    a = np.arange(24, dtype=np.float32)
    b = np.zeros(oracle.span(dims, bs), np.float32)
    b1 = np.zeros_like(b)
    c, d, d1 = np.zeros(24, np.float32), np.zeros(24, np.float32), np.zeros(24, np.float32)
    oracle.reorder(lay(oracle, a, dims, NCHW(oracle, dims)), lay(oracle, b, dims, bs))
    oracle.reorder(lay(oracle, b, dims, bs), lay(oracle, c, dims, NHWC(oracle, dims)))
    oracle.reorder(lay(oracle, b, dims, bs), lay(oracle, b1, dims, bs))
    oracle.reorder(lay(oracle, b1, dims, bs), lay(oracle, d1, dims, NCHW(oracle, dims)))
    oracle.reorder(lay(oracle, c, dims, NHWC(oracle, dims)), lay(oracle, d, dims, NCHW(oracle, dims)))
    assert np.array_equal(d, a) and np.array_equal(d1, a)
    assert np.linalg.norm(c) == np.linalg.norm(a)


def test_reorder_with_offsets(oracle):
    """dnnl-core :342-361 -- source read from element 2, destination written from element 5; the
    test then looks at the destination from element 2."""
    dims = [2, 2, 3, 2]
    a = np.arange(72, dtype=np.float32)
    b = np.zeros(72, np.float32)
    st = NCHW(oracle, dims)
    oracle.reorder(lay(oracle, a, dims, st, offset=2), lay(oracle, b, dims, st, offset=5))
    assert b[2:8].tolist() == [0, 0, 0, 2, 3, 4]
    assert b[2:27].tolist() == [0, 0, 0] + list(range(2, 24))


def test_transformer_and_subtensor(oracle):
    """tensor-t :152-169 -- [2 3 4 5] nchw -> nhwc; then only the first image after new data."""
    dims = [2, 3, 4, 5]
    x = np.arange(120, dtype=np.float32)
    y = np.zeros(120, np.float32)
    oracle.reorder(lay(oracle, x, dims, NCHW(oracle, dims)), lay(oracle, y, dims, NHWC(oracle, dims)))
    assert np.abs(y).sum() == np.abs(x).sum() and y[119] == 119.0
    x = np.arange(0, 1200, 10, dtype=np.float32)
    sub = [1, 3, 4, 5]
    oracle.reorder(lay(oracle, x, sub, NCHW(oracle, dims)), lay(oracle, y, sub, NHWC(oracle, dims)))
    assert y[34] == 310.0


def test_arbitrary_strides_transfer(oracle):
    """tensor-t :171-194 -- [2 3 2 1] through [48 16 5 2] -> [48 13 4 2] and [48 12 4 2] -> [48 14 4 2]."""
    dims = [2, 3, 2, 1]
    src = np.arange(12, dtype=np.float32)
    for s0, s1 in (([48, 16, 5, 2], [48, 13, 4, 2]), ([48, 12, 4, 2], [48, 14, 4, 2])):
        x = np.zeros(oracle.span(dims, s0), np.float32)
        y = np.zeros(oracle.span(dims, s1), np.float32)
        out = np.zeros(12, np.float32)
        oracle.reorder(lay(oracle, src, dims, NCHW(oracle, dims)), lay(oracle, x, dims, s0))
        oracle.reorder(lay(oracle, x, dims, s0), lay(oracle, y, dims, s1))
        oracle.reorder(lay(oracle, y, dims, s1), lay(oracle, out, dims, NCHW(oracle, dims)))
        assert np.array_equal(out, src)


def test_heterogenous_transfer_saturates(oracle):
    """tensor-t :205-221 -- s8 (range -6 6) -> f32 -> u8: negatives saturate to 0; sub-tensors at
    batch offsets 4, 2, 1."""
    dims = [6, 2, 1, 1]
    st = NCHW(oracle, dims)
    x = np.arange(-6, 6, dtype=np.int8)
    y = np.zeros(12, np.float32)
    z = np.zeros(12, np.uint8)
    oracle.reorder(lay(oracle, x, dims, st), lay(oracle, y, dims, st))
    assert np.abs(y).sum() == 36.0
    oracle.reorder(lay(oracle, y, dims, st), lay(oracle, z, dims, st))
    assert z.tolist() == [0, 0, 0, 0, 0, 0, 0, 1, 2, 3, 4, 5]
    sub = [2, 2, 1, 1]
    oracle.reorder(lay(oracle, x, sub, st, offset=8), lay(oracle, y, sub, st, offset=4))
    assert np.abs(y[4:8]).sum() == 14.0
    oracle.reorder(lay(oracle, y, sub, st, offset=4), lay(oracle, z, sub, st, offset=2))
    assert z[2:6].tolist() == [2, 3, 4, 5]
    assert z.tolist() == [0, 0, 2, 3, 4, 5, 0, 1, 2, 3, 4, 5]


def test_half_and_double_conversions(oracle):
    """dnnl-tz :35-51 (f32 <-> f16: 100 200 300 400 survive); cudnn-core :38-49 (s8 1..6 -> f64)."""
    x = np.array([100, 200, 300, 400], np.float32)
    h = np.zeros(4, np.float16)
    back = np.zeros(4, np.float32)
    oracle.reorder(x, h)
    oracle.reorder(h, back)
    assert back.tolist() == [100.0, 200.0, 300.0, 400.0]
    b = np.arange(1, 7, dtype=np.int8).reshape(2, 3, 1, 1)
    d = np.zeros((2, 3, 1, 1), np.float64)
    oracle.reorder(b, d)
    assert d.reshape(-1).tolist() == [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]


def test_f16_bf16_rounding_against_numpy(oracle):
    """RNE conversions agree with numpy's float16 cast and with a bit-level bf16 rule on edge values."""
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 1000,
                        np.array([65504, 65519.9, 65520, 1e-8, 6e-8, 6.1e-5, -0.0, np.inf, -np.inf], np.float32)])
    h = np.zeros(x.size, np.float16)
    oracle.reorder(x, h)
    with np.errstate(over="ignore"):
        assert np.array_equal(h.view(np.uint16), x.astype(np.float16).view(np.uint16))
    b = np.zeros(x.size, np.uint16)
    oracle.reorder(x, b, ytag="bf16")
    u = x.view(np.uint32).astype(np.uint64)
    want = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    assert np.array_equal(b, want)
    f = np.zeros(x.size, np.float32)
    oracle.reorder(b, f, xtag="bf16")
    assert np.array_equal(f.view(np.uint32), b.astype(np.uint32) << 16)


def test_batcher_and_shuffler_vectors(oracle):
    """tensor-t :263-297 -- x [7 2 1 1] strides [2 1 1 1] (values 1..14), y [3 2 1 1] strides [1 3 1 1]."""
    x = np.arange(1, 15, dtype=np.float32)
    sx, sy = [2, 1, 1, 1], [1, 3, 1, 1]

    def batch(src_n, dst_n, mb, y):
        sub = [mb, 2, 1, 1]
        oracle.reorder(lay(oracle, x, sub, sx, offset=src_n * sx[0]), lay(oracle, y, sub, sy, offset=dst_n * sy[0]))
        return y

    assert batch(0, 0, 3, np.zeros(6, np.float32)).tolist() == [1, 3, 5, 2, 4, 6]
    assert batch(1, 0, 3, np.zeros(6, np.float32)).tolist() == [3, 5, 7, 4, 6, 8]
    assert batch(1, 1, 2, np.zeros(6, np.float32)).tolist() == [0, 3, 5, 0, 4, 6]
    y = np.zeros(6, np.float32)          # shuffler [0 2 1] on (range 1 13)
    for dst_n, src_n in enumerate([0, 2, 1]):
        batch(src_n, dst_n, 1, y)
    assert y.tolist() == [1, 5, 3, 2, 6, 4]


# ----------------------------------------------------------------------------- eltwise ---------

def test_relu_forward_with_offsets_and_submemory(oracle):
    """dnnl-core :76-99, :146-181, :363-376."""
    buf = np.zeros(122, np.float32)
    buf[[0, 1, 2, 120, 121]] = [-100, -20, -200, -400, -500]
    v = lay(oracle, buf, [2, 3, 4, 5], [60, 20, 5, 1], offset=1)
    oracle.eltwise_fwd("relu", v, v)
    assert buf[[0, 1, 2, 120, 121]].tolist() == [-100.0, 0.0, 0.0, 0.0, -500.0]
    buf = np.zeros(120, np.float32)
    buf[[0, 1, 2, 59, 60, 119]] = [-100, -20, -200, -1, -2, -400]
    v = lay(oracle, buf, [1, 3, 4, 5], [60, 20, 5, 1], offset=60)
    oracle.eltwise_fwd("relu", v, v)
    assert buf[[0, 1, 2, 59, 60, 119]].tolist() == [-100.0, -20.0, -200.0, -1.0, 0.0, 0.0]
    buf = np.zeros(120, np.float32)
    buf[:2] = [-100, 20]
    oracle.eltwise_fwd("relu", buf, buf)
    assert buf[:2].tolist() == [0.0, 20.0]


def test_abs_on_offset_submemory(oracle):
    """dnnl-core :183-200 -- channel 1 of a [2 2 3 2] tensor holding -i."""
    buf = -np.arange(24, dtype=np.float32)
    v = lay(oracle, buf, [2, 1, 3, 2], [12, 6, 2, 1], offset=6)
    oracle.eltwise_fwd("abs", v, v)
    assert [buf[i] for i in (5, 6, 11, 12, 23)] == [-5.0, 6.0, 11.0, -12.0, 23.0]


def test_relu_backward(oracle):
    """dnnl-core :378-401 ([0 3 0 0 0 0], diff-dst aliases diff-src); dnn-t :28-54 ([0 0 1 2 7 0])."""
    x = np.zeros(6, np.float32)
    x[:2] = [-100, 20]
    g = np.arange(2, 8, dtype=np.float32)
    oracle.eltwise_bwd("relu", x, g, g)
    assert g.tolist() == [0, 3, 0, 0, 0, 0]
    x = np.array([-0.5, 0, 0.2, 1, 0.3, -0.7], np.float32)
    y = np.zeros(6, np.float32)
    oracle.eltwise_fwd("relu", x, y)
    assert np.allclose(y, [0, 0, 0.2, 1.0, 0.3, 0])
    g = np.array([-0.1, 0.1, 1, 2, 7, -0.6], np.float32)
    oracle.eltwise_bwd("relu", x, g, x)  # diff-src aliases src, like (activ-bluep src-tz src-tz)
    assert x.tolist() == [0, 0, 1, 2, 7, 0]


def test_logistic_forward_backward(oracle):
    """dnnl-core :403-427; dnn-t :56-82; cudnn-core :97-131."""
    x = np.array([-1, -0.5, 0, 0.1, 0.5, 0.7], np.float32)
    y = oracle.eltwise_fwd("logistic", x, np.zeros(6, np.float32))
    ref = np.array([0.2689414322376251, 0.377540647983551, 0.5, 0.5249792337417603, 0.622459352016449,
                    0.6681877970695496], np.float32)
    assert ulp_diff_f32(y, ref).max() <= 1
    g = np.array([-0.5, -0.2, -0.4, 0, 0.2, 0.3], np.float32)
    dx = oracle.eltwise_bwd("logistic", x, g, np.zeros(6, np.float32))
    refb = np.array([-0.09830597043037415, -0.04700074344873428, -0.10000000149011612, 0.0,
                     0.04700074344873428, 0.06651385873556137], np.float32)
    assert ulp_diff_f32(dx, refb).max() <= 2
    one = oracle.eltwise_bwd("sigmoid", np.array([-0.5], np.float32), np.array([-0.1], np.float32), np.zeros(1, np.float32))
    assert abs(float(one[0]) + 0.02350037172436714) < 1e-8
    assert abs(float(oracle.eltwise_fwd("sigmoid", np.array([0.7], np.float32), np.zeros(1, np.float32))[0]) - 0.6681877374649048) < 1e-7


def test_activation_alpha_beta_blend(oracle):
    """cudnn-core :51-95 -- y = 3*relu(x) + 2*y; dx = 300*relu'(x)*dy + 200*dx."""
    x = np.arange(-2, 118, dtype=np.float32)
    y = np.arange(120, dtype=np.float32)
    oracle.eltwise_fwd("relu", x, y, coef=0.0, alpha=3.0, beta=2.0)
    assert y[:5].tolist() == [0.0, 2.0, 4.0, 9.0, 14.0]
    dx = (np.arange(120) * 0.1 - 6).astype(np.float32)
    dy = (np.arange(120) * 0.01 - 0.6).astype(np.float32)
    oracle.eltwise_bwd("relu", x, dy, dx, alpha=300.0, beta=200.0)
    assert np.allclose(dx[:5], [-1200.0, -1180.0, -1160.0, -1311.0, -1288.0], rtol=1e-6)


# ----------------------------------------------------------------------------- sum / binary ----

def test_scaled_sums(oracle):
    """dnnl-core :202-258."""
    buf = np.zeros(120, np.float32)
    buf[:2] = [-100, 20]
    oracle.scaled_sum([2.0], [buf], buf)
    assert buf[:2].tolist() == [-200.0, 40.0]
    src = np.zeros(120, np.float32); src[:2] = [-100, 10]
    dst = np.zeros(120, np.float32); dst[:2] = [-200, 20]
    oracle.scaled_sum([2.0, 3.0], [src, dst], dst)
    assert dst[:2].tolist() == [-800.0, 80.0] and src[:2].tolist() == [-100.0, 10.0]
    s0 = np.zeros(120, np.float32); s0[:2] = [-100, 20]
    s1 = np.zeros(120, np.float32); s1[:2] = [-1000, 200]
    out = np.full(120, 1e5, np.float32)
    oracle.scaled_sum([2.0, 3.0], [s0, s1], out)
    assert out[:2].tolist() == [-3200.0, 640.0]


def test_binary_add_in_place_and_sum_layer(oracle):
    """dnnl-core :869-886; dnn-t :855-874 (sum layer: forward [4 6]; backward [2 3] [2 3])."""
    b0 = np.zeros(120, np.float32); b0[:2] = [-100, 20]
    b1 = np.zeros(120, np.float32); b1[:2] = [-200, 30]
    oracle.binary("add", b0, b1, b0)
    assert b0[:2].tolist() == [-300.0, 50.0]
    i0, i1 = np.array([1, 2], np.float32), np.array([3, 4], np.float32)
    oracle.scaled_sum([1.0, 1.0], [i0, i1], i0)
    assert i0.tolist() == [4.0, 6.0]
    oracle.scaled_sum([0.5], [i0], i0)
    i1[...] = i0
    assert i0.tolist() == [2.0, 3.0] and i1.tolist() == [2.0, 3.0]


# ----------------------------------------------------------------------------- reduction -------

def test_reductions(oracle):
    """dnnl-core :888-943; cudnn-core :149-178."""
    x = np.arange(120, dtype=np.float32).reshape(2, 3, 4, 5)
    y = np.zeros((2, 3, 4, 1), np.float32)
    oracle.reduce("sum", x, y)
    assert y.reshape(-1)[:3].tolist() == [10.0, 35.0, 60.0]
    m = np.zeros((1, 3, 1, 1), np.float32)
    oracle.reduce("max", x, m)
    assert m.reshape(-1).tolist() == [79.0, 99.0, 119.0]
    oracle.reduce("norm2", x, y)
    want = [np.float32(np.sqrt(sum(i * i for i in range(a, a + 5)))) for a in (0, 5, 10)]
    assert y.reshape(-1)[:3].tolist() == [float(v) for v in want]
    v = np.array([1, 2, 3, 4, 5, 6], np.float32).reshape(2, 3, 1, 1)
    s = np.zeros((1, 1, 1, 1), np.float32)
    oracle.reduce("add", v, s, alpha=3.0, beta=2.0)
    assert float(s.reshape(-1)[0]) == 63.0
    oracle.reduce("max", v, s, alpha=2.5)
    assert float(s.reshape(-1)[0]) == 15.0
    oracle.reduce("mul", v, s, alpha=1.5)
    assert float(s.reshape(-1)[0]) == 1080.0
    oracle.reduce("mean", v, s)
    assert float(s.reshape(-1)[0]) == 3.5


def test_reduction_norm_lp_kinds(oracle):
    """The four norm kinds of dnnl/constants.clj:393-402 with the p and epsilon that `reduction`
    passes (dnnl/core.clj:796-803).  norm-lp-sum, p = 2, eps = 0 over W of `range 120` is the known
    answer of dnnl-t/core_test.clj:926-943; the other kinds follow from the same sums by oneDNN's
    definitions and are checked against double-precision numpy."""
    x = np.arange(120, dtype=np.float32).reshape(2, 3, 4, 5)
    y = np.zeros((2, 3, 4, 1), np.float32)
    oracle.reduce_lp("norm-lp-sum", 2.0, 0.0, x, y)
    want = [np.float32(np.sqrt(sum(i * i for i in range(a, a + 5)))) for a in range(0, 120, 5)]
    assert y.reshape(-1).tolist() == [float(v) for v in want]
    xs = (x - 60.0).astype(np.float32)
    for p in (1.0, 2.0, 3.0, 2.5):
        s = (np.abs(xs.astype(np.float64)) ** p).sum(axis=3, keepdims=True)
        for eps in (0.0, 1e-3, 1e9):
            table = {"norm-lp-max": np.maximum(s, eps) ** (1 / p), "norm-lp-sum": (s + eps) ** (1 / p),
                     "norm-lp-power-p-max": np.maximum(s, eps), "norm-lp-power-p-sum": s + eps}
            for kind, ref in table.items():
                _, truth = oracle.reduce_lp(kind, p, eps, xs, y, want_truth=True)
                assert np.allclose(truth, ref, rtol=1e-12, atol=0), (kind, p, eps)
                assert np.allclose(y, ref, rtol=2e-6, atol=0), (kind, p, eps)
    # alpha / beta blend like every other reduction
    y[:] = 1.0
    oracle.reduce_lp("norm-lp-power-p-sum", 1.0, 0.5, xs, y, alpha=2.0, beta=3.0)
    assert np.array_equal(y, (2.0 * (np.abs(xs).sum(axis=3, keepdims=True) + 0.5) + 3.0).astype(np.float32))


def test_eltwise_kinds_of_the_dnnl_table(oracle):
    """The kinds of dnnl/constants.clj:277-308 beyond the cuDNN set.  The reference holds no known
    answer for them, so the restatement is pinned two ways: forward values against numpy / math on the
    definitions oneDNN documents, and every derivative against a central difference of its own forward
    (both in double)."""
    import math
    x = np.array([-3.0, -1.5, -0.25, 0.0, 0.25, 1.5, 3.0], np.float32)
    xd = x.astype(np.float64)
    sig = lambda t: 1.0 / (1.0 + np.exp(-t))
    erf = np.vectorize(math.erf)
    expect = {
        ("square", 0, 0): xd * xd, ("exp", 0, 0): np.exp(xd), ("swish", 1.25, 0): xd * sig(1.25 * xd),
        ("soft-relu", 1.5, 0): np.log1p(np.exp(1.5 * xd)) / 1.5,
        ("gelu-tanh", 0, 0): 0.5 * xd * (1 + np.tanh(math.sqrt(2 / math.pi) * (xd + 0.044715 * xd ** 3))),
        ("gelu-erf", 0, 0): 0.5 * xd * (1 + erf(xd / math.sqrt(2))),
        ("hardswish", 1 / 6, 0.5): xd * np.clip(xd / 6 + 0.5, 0, 1), ("clip", -0.75, 1.5): np.clip(xd, -0.75, 1.5),
        ("clip-v2", -0.75, 1.5): np.clip(xd, -0.75, 1.5), ("mish", 0, 0): xd * np.tanh(np.log1p(np.exp(xd))),
        ("round", 0, 0): np.round(xd),
    }
    for (kind, a, b), ref in expect.items():
        got = oracle.eltwise_fwd_truth(kind, x, coef=a, shift=b)
        assert np.allclose(got, ref, rtol=1e-12, atol=1e-15), kind
        got32 = oracle.eltwise_fwd(kind, x, np.zeros_like(x), coef=a, shift=b)
        assert np.allclose(got32, ref, rtol=3e-7, atol=1e-9), kind
    pos = np.abs(x) + np.float32(0.5)
    for (kind, a, b), ref in {("sqrt", 0, 0): np.sqrt(pos.astype(np.float64)), ("log", 0, 0): np.log(pos.astype(np.float64)),
                              ("pow", 0.5, 2.5): 0.5 * pos.astype(np.float64) ** 2.5}.items():
        assert np.allclose(oracle.eltwise_fwd_truth(kind, pos, coef=a, shift=b), ref, rtol=1e-12), kind
    assert oracle.eltwise_fwd("round", np.array([0.5, 1.5, 2.5, -0.5], np.float32), np.zeros(4, np.float32)).tolist() == [0, 2, 2, -0]
    # derivatives against central differences (points kept away from the kinks of clip and hardswish)
    pts = np.linspace(-4, 4, 161).astype(np.float32) + np.float32(0.0131)
    h = 2.0 ** -10
    for kind, a, b, dom in (("square", 0, 0, "any"), ("exp", 0, 0, "any"), ("swish", 1.25, 0, "any"), ("soft-relu", 1.5, 0, "any"),
                            ("gelu-tanh", 0, 0, "any"), ("gelu-erf", 0, 0, "any"), ("hardswish", 1 / 6, 0.5, "any"),
                            ("clip", -0.75, 1.5, "any"), ("clip-v2", -0.75, 1.5, "any"), ("mish", 0, 0, "any"),
                            ("sqrt", 0, 0, "pos"), ("log", 0, 0, "pos"), ("pow", 0.5, 2.5, "pos")):
        p = (np.abs(pts) + np.float32(0.25)) if dom == "pos" else pts
        lo, hi = (p - np.float32(h)).astype(np.float32), (p + np.float32(h)).astype(np.float32)
        num = (oracle.eltwise_fwd_truth(kind, hi, a, b) - oracle.eltwise_fwd_truth(kind, lo, a, b)) / (hi.astype(np.float64) - lo)
        der = oracle.eltwise_bwd_truth(kind, p, np.ones_like(p), a, b)
        assert np.allclose(num, der, rtol=2e-5, atol=2e-5), (kind, np.abs(num - der).max())
    # the *-dst-bwd kinds: the derivative written in terms of the forward result equals the one from the source
    g = np.ones_like(pts)
    for kind, base, a in (("tanh-dst-bwd", "tanh", 0), ("logistic-dst-bwd", "logistic", 0), ("elu-dst-bwd", "elu", 1.5),
                          ("exp-dst-bwd", "exp", 0), ("relu-dst-bwd", "relu", 0.25)):
        y = oracle.eltwise_fwd_truth(base, pts, coef=a)
        from_dst = oracle.eltwise_bwd_truth(kind, y.astype(np.float32), g, a)
        from_src = oracle.eltwise_bwd_truth(base, pts, g, a)
        assert np.allclose(from_dst, from_src, rtol=1e-5, atol=1e-6), kind
    ps = np.abs(pts) + np.float32(0.25)
    y = np.sqrt(ps.astype(np.float64))
    assert np.allclose(oracle.eltwise_bwd_truth("sqrt-dst-bwd", y.astype(np.float32), g), 0.5 / y, rtol=1e-6)


# ----------------------------------------------------------------------------- real oneDNN -----

def fixtures():
    return np.load(os.path.join(os.path.dirname(__file__), "golden", "onednn_fixtures.npz"))


def test_against_real_onednn_outputs(oracle):
    """Outputs of real oneDNN (see tests/golden/make_onednn_fixtures.py): relu, same-shape add/mul and
    f32->bf16 bit-exact; logistic within 2 ulp and tanh within 1 ulp of the oracle; gelu-erf within
    1.5e-6 absolute."""
    f = fixtures()
    assert "MKL-DNN" in str(f["onednn_version"]) or "oneDNN" in str(f["onednn_version"])
    x = f["x"]
    assert np.array_equal(oracle.eltwise_fwd("relu", x, np.zeros_like(x)), f["relu"])
    assert ulp_diff_f32(oracle.eltwise_fwd("logistic", x, np.zeros_like(x)), f["logistic"]).max() <= 2
    assert ulp_diff_f32(oracle.eltwise_fwd("tanh", x, np.zeros_like(x)), f["tanh"]).max() <= 1
    # gelu-erf: oneDNN's erf is a polynomial with an absolute error near 1e-6 (measured 7.4e-7 here)
    gelu = oracle.eltwise_fwd("gelu-erf", x, np.zeros_like(x))
    assert np.abs(gelu.astype(np.float64) - f["gelu_erf"]).max() <= 1.5e-6
    b = np.zeros(f["cvt_in"].size, np.uint16)
    oracle.reorder(f["cvt_in"], b, ytag="bf16")
    assert np.array_equal(b, f["cvt_bf16_bits"])
    s = np.zeros_like(f["a"])
    oracle.scaled_sum([1.0, 1.0], [f["a"], f["b"]], s)
    assert np.array_equal(s, f["add"])
    m = np.zeros_like(f["a"])
    oracle.binary("mul", f["a"], f["b"], m)
    assert np.array_equal(m, f["mul"])


def test_equals(oracle):
    """The typed compare of blas-plus.cu:9-101 (deep-diamond-cuda/src/device/...)."""
    x = np.arange(24, dtype=np.float32)
    y = np.zeros(24, np.float32)
    d = [2, 2, 3, 2]
    oracle.reorder(lay(oracle, x, d, NCHW(oracle, d)), lay(oracle, y, d, NHWC(oracle, d)))
    assert oracle.equals(lay(oracle, x, d, NCHW(oracle, d)), lay(oracle, y, d, NHWC(oracle, d)))
    y[3] += 1
    assert not oracle.equals(lay(oracle, x, d, NCHW(oracle, d)), lay(oracle, y, d, NHWC(oracle, d)))


def test_cost_known_answers(oracle):
    """deep-diamond-test/src/uncomplicate/diamond/dnn_test.clj:321-346: quadratic cost of
    a = [0.4 -1.3], y = [0.25 0.35] is 0.6862499438341274 with a - y = [0.15 -1.65]; sigmoid
    cross-entropy of a = [0.4 0.1], y = [0.25 0.65] is 1.0728740692138672 (float results)."""
    c, t, d = oracle.cost("quadratic", np.array([[0.4], [-1.3]]), np.array([[0.25], [0.35]]), want_diff=True)
    assert abs(c - 0.6862499438341274) < 1e-7 and abs(t - c) < 1e-7
    assert np.array_equal(d.reshape(-1), np.array([0.4, -1.3], np.float32) - np.array([0.25, 0.35], np.float32))
    c, t = oracle.cost("crossentropy", np.array([[0.4], [0.1]]), np.array([[0.25], [0.65]]))
    assert np.float32(c) == np.float32(1.0728740692138672)
    assert abs(t - c) < 1e-7
    c, _ = oracle.cost("mean-absolute", np.array([[0.4], [-1.3]]), np.array([[0.25], [0.35]]))
    assert abs(c - 0.9) < 1e-7
