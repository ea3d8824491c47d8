"""Seeded random differential tests: random ranks, extents, permuted and padded strides, data type
pairs, broadcast masks and reduce masks through the C ABI against the CPU oracle.  They walk the
generic paths (canonicalisation, dim merging, kernel-family choice, ragged tiles, index arithmetic)
that the hand-picked cases of the other files only sample.  Each case fills the destination with a
canary first, so a write outside the described view also fails the comparison.
"""
import os

import numpy as np
import pytest

from deep_diamond_b200 import core

pytestmark = pytest.mark.gpu

# DD_TEST_SEED_OFFSET=k shifts every generator's seed: the same tests over other random shapes
SEED_OFFSET = int(os.environ.get("DD_TEST_SEED_OFFSET", "0"))

NP = {"float": np.float32, "double": np.float64, "half": np.float16, "byte": np.int8,
      "int": np.int32, "uint8": np.uint8, "bf16": np.uint16, "long": np.int64}
TAG = {"float": "f32", "double": "f64", "half": "f16", "byte": "s8", "int": "s32", "uint8": "u8",
       "bf16": "bf16", "long": "s64"}


def random_layout(rng, shape, pad_prob=0.3):
    """Strides of a random dim permutation, with random padding between dims now and then."""
    order = list(rng.permutation(len(shape)))
    st, run = [0] * len(shape), 1
    for d in reversed(order):
        st[d] = run
        run *= shape[d]
        if rng.random() < pad_prob:
            run += int(rng.integers(1, 5))
    return st


def random_shape(rng, max_rank=5, big=False):
    rank = int(rng.integers(1, max_rank + 1))
    choices = [1, 1, 2, 3, 4, 5, 7, 8, 9, 12, 16, 17, 32, 33] + ([48, 64, 65, 96] if big else [])
    shape = [int(rng.choice(choices)) for _ in range(rank)]
    while np.prod(shape) > 300000:
        shape[int(rng.integers(0, rank))] = 1
    return shape


def values(rng, n, dt):
    if dt in ("float", "double"):
        return (rng.standard_normal(n) * 40).astype(NP[dt])
    if dt == "half":
        return (rng.standard_normal(n) * 40).astype(np.float16)
    if dt == "bf16":
        return ((rng.standard_normal(n) * 40).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    lo, hi = {"byte": (-128, 128), "uint8": (0, 256), "int": (-9000, 9000), "long": (-9000, 9000)}[dt]
    return rng.integers(lo, hi, n).astype(NP[dt])


def canary(n, np_t):
    b = np.empty(n, dtype=np_t)
    b.view(np.uint8)[:] = 0xA5
    return b


@pytest.mark.parametrize("seed", range(12))
def test_random_transforms(fact, dev, oracle, seed):
    rng = np.random.default_rng(1000 + 100 * SEED_OFFSET + seed)
    types = list(NP)
    for _ in range(25):
        shape = random_shape(rng, big=rng.random() < 0.5)
        sx, sy = random_layout(rng, shape), random_layout(rng, shape)
        if rng.random() < 0.3:
            sy = list(sx)                      # same layout: flat or row copies
        sdt = types[int(rng.integers(0, len(types)))]
        ddt = sdt if rng.random() < 0.4 else types[int(rng.integers(0, len(types)))]
        blend = rng.random() < 0.25
        alpha, beta = (float(rng.choice([0.5, 2.0, -1.0])), float(rng.choice([1.0, 0.5]))) if blend else (1.0, 0.0)
        xs = values(rng, oracle.span(shape, sx), sdt)
        y0 = values(rng, oracle.span(shape, sy), ddt) if blend else canary(oracle.span(shape, sy), NP[ddt])
        if blend and ddt in ("half", "bf16"):
            y0 = values(rng, oracle.span(shape, sy), ddt)
        want = y0.copy()
        oracle.reorder(oracle.as_layout(xs, shape, sx), oracle.as_layout(want, shape, sy), TAG[sdt], TAG[ddt], alpha, beta)
        tx, ty = dev.put(xs), dev.put(y0)
        core.transform_tensor(fact.handle, alpha, core.tensor_descriptor(shape, sdt, sx), tx, beta,
                              core.tensor_descriptor(shape, ddt, sy), ty)
        got = dev.get(ty, NP[ddt])
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (shape, sx, sy, sdt, ddt, alpha, beta,
                                                                            fact.handle.last_kernel())


@pytest.mark.parametrize("seed", range(6))
def test_random_op_tensors(fact, dev, oracle, seed):
    rng = np.random.default_rng(2000 + 100 * SEED_OFFSET + seed)
    ops = ["add", "mul", "min", "max", "sub"]
    for _ in range(25):
        shape = random_shape(rng, big=rng.random() < 0.5)
        bshape = [d if rng.random() < 0.5 else 1 for d in shape]
        same = rng.random() < 0.6
        sa = oracle.default_strides(shape) if same else random_layout(rng, shape)
        sc = list(sa) if same else random_layout(rng, shape)
        sb = random_layout(rng, bshape, 0.0)
        op = ops[int(rng.integers(0, len(ops)))]
        a1, a2, beta = float(rng.choice([1.0, 0.5, -2.0])), float(rng.choice([1.0, 0.25, 3.0])), float(rng.choice([0.0, 0.0, 1.0, 0.5]))
        a = values(rng, oracle.span(shape, sa), "float")
        b = values(rng, oracle.span(bshape, sb), "float")
        c0 = values(rng, oracle.span(shape, sc), "float")
        want = c0.copy()
        oracle.binary(op, oracle.as_layout(a, shape, sa), oracle.as_layout(b, bshape, sb),
                      oracle.as_layout(want, shape, sc), alpha1=a1, alpha2=a2, beta=beta)
        ta, tb, tc = dev.put(a), dev.put(b), dev.put(c0)
        core.op_tensor(fact.handle, op, a1, core.tensor_descriptor(shape, "float", sa), ta, a2,
                       core.tensor_descriptor(bshape, "float", sb), tb, beta,
                       core.tensor_descriptor(shape, "float", sc), tc)
        got = dev.get(tc, np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (shape, bshape, sa, sb, sc, op, a1, a2, beta,
                                                                            fact.handle.last_kernel())


@pytest.mark.parametrize("seed", range(8))
def test_random_reductions(fact, dev, oracle, seed):
    rng = np.random.default_rng(3000 + 100 * SEED_OFFSET + seed)
    ops = ["add", "avg", "max", "min", "amax", "norm1", "norm2"]
    for _ in range(20):
        shape = random_shape(rng, big=rng.random() < 0.6)
        yshape = [1 if rng.random() < 0.5 else d for d in shape]
        sx = oracle.default_strides(shape) if rng.random() < 0.6 else random_layout(rng, shape)
        sy = random_layout(rng, yshape, 0.2)
        op = ops[int(rng.integers(0, len(ops)))]
        alpha, beta = float(rng.choice([1.0, 1.0, 2.0])), float(rng.choice([0.0, 0.0, 0.5]))
        x = values(rng, oracle.span(shape, sx), "float")
        y0 = values(rng, oracle.span(yshape, sy), "float")
        want = y0.copy()
        _, truth = oracle.reduce(op, oracle.as_layout(x, shape, sx), oracle.as_layout(want, yshape, sy),
                                 alpha=alpha, beta=beta, want_truth=True)
        tx, ty = dev.put(x), dev.put(y0)
        core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor(op, "float"), alpha,
                           core.tensor_descriptor(shape, "float", sx), tx, beta,
                           core.tensor_descriptor(yshape, "float", sy), ty)
        got = dev.get(ty, np.float32)
        info = (shape, yshape, sx, sy, op, alpha, beta, fact.handle.last_kernel())
        if op in ("max", "min", "amax") and beta == 0.0:
            assert np.array_equal(got, want), info
        else:
            # untouched padding must be bit-identical; touched entries within the summation bound
            axes = tuple(i for i in range(len(shape)) if yshape[i] == 1 and shape[i] != 1)
            nred = int(np.prod([shape[i] for i in axes])) if axes else 1
            scale = np.abs(oracle.as_layout(x, shape, sx).astype(np.float64))
            scale = scale.sum(axis=axes, keepdims=True) if axes else scale
            if op == "avg":
                scale = scale / nred
            tol = np.maximum(1e-5 * np.abs(oracle.as_layout(want, yshape, sy).astype(np.float64)),
                             2 * (np.log2(max(nred, 2)) + 2) * 6e-8 * abs(alpha) * scale.reshape(yshape))
            d = np.abs(oracle.as_layout(got, yshape, sy).astype(np.float64) - oracle.as_layout(want, yshape, sy))
            assert (d <= tol).all(), info
            mask = np.ones(got.size, bool)
            idx = oracle.as_layout(np.arange(got.size), yshape, sy).reshape(-1)
            mask[idx] = False
            assert np.array_equal(got[mask].view(np.uint32), y0[mask].view(np.uint32)), info


@pytest.mark.parametrize("seed", range(4))
def test_random_activations_on_views(fact, dev, oracle, seed):
    rng = np.random.default_rng(4000 + 100 * SEED_OFFSET + seed)
    for _ in range(20):
        shape = random_shape(rng, big=True)
        sx, sy, sg = random_layout(rng, shape), random_layout(rng, shape), random_layout(rng, shape)
        mode = ["relu", "abs", "linear", "clipped-relu"][int(rng.integers(0, 4))]   # exact modes: bit compare
        coef = float(rng.choice([0.0, 0.1, 1.5]))
        x = values(rng, oracle.span(shape, sx), "float")
        g = values(rng, oracle.span(shape, sg), "float")
        y0 = canary(oracle.span(shape, sy), np.float32)
        want = y0.copy()
        oracle.eltwise_fwd(mode, oracle.as_layout(x, shape, sx), oracle.as_layout(want, shape, sy), coef=coef, shift=0.5)
        tx, ty = dev.put(x), dev.put(y0)
        ad = core.activation_descriptor(mode, True, coef, 0.5)
        xd, yd = core.tensor_descriptor(shape, "float", sx), core.tensor_descriptor(shape, "float", sy)
        core.activation_forward(fact.handle, ad, 1.0, xd, tx, 0.0, yd, ty)
        got = dev.get(ty, np.float32)
        assert np.array_equal(got.view(np.uint32) | (got == 0) * np.uint32(0x80000000),
                              want.view(np.uint32) | (want == 0) * np.uint32(0x80000000)), (shape, sx, sy, mode, coef)
        wantb = y0.copy()
        oracle.eltwise_bwd(mode, oracle.as_layout(x, shape, sx), oracle.as_layout(g, shape, sg),
                           oracle.as_layout(wantb, shape, sy), coef=coef)
        tg, tdx = dev.put(g), dev.put(y0)
        core.activation_backward(fact.handle, ad, 1.0, yd, None, core.tensor_descriptor(shape, "float", sg), tg,
                                 xd, tx, 0.0, yd, tdx)
        gotb = dev.get(tdx, np.float32)
        assert np.array_equal(gotb.view(np.uint32) | (gotb == 0) * np.uint32(0x80000000),
                              wantb.view(np.uint32) | (wantb == 0) * np.uint32(0x80000000)), (shape, sx, sg, sy, mode, coef)
