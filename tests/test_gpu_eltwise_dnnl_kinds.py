"""GPU parity: the activation kinds that only the reference's DNNL table names
(deep-diamond-dnnl/src/uncomplicate/diamond/internal/dnnl/constants.clj:277-308: square sqrt exp log
soft-relu swish gelu-tanh gelu-erf hardswish clip clip-v2 pow mish round and the *-dst-bwd kinds),
through ddActivationForward / ddActivationBackward against the CPU oracle.

Bars.  The few-instruction kinds (square, sqrt, clip, clip-v2, hardswish, round and the derivatives
that are a product or a quotient) are bit-exact against the oracle's float arithmetic.  The
transcendental kinds are compared with the definition evaluated in double and rounded once: forward
within ULP_FWD units of float32, or within 2^-24 * max(|x|, 1) absolutely -- the far negative tails of
swish, gelu and soft-relu are x * sigma(t) or exp(t) with |t| of 10 to 20, where the ONE rounding of t
in float is already |t| / 2 units of the (tiny) result: measured on B200, gelu-tanh is up to 98 units
off there and 1 unit everywhere else, gelu-erf 56 and 2, soft-relu 10 and 3, swish 8 and 1.  Backward:
within ULP_BWD units, or, around the zero crossings of a derivative (swish, gelu, mish), within
8 * 2^-24 * |dy| absolutely.  fp64 tensors: 1e-12 relative.
"""
import numpy as np
import pytest

from conftest import ulp_diff_f32
from deep_diamond_b200 import core

pytestmark = pytest.mark.gpu

# kind -> (coef a, shift b, input domain)
KINDS = {
    "square": (0.0, 0.0, "any"), "sqrt": (0.0, 0.0, "pos"), "exp": (0.0, 0.0, "any"), "log": (0.0, 0.0, "pos"),
    "soft-relu": (1.5, 0.0, "any"), "swish": (1.25, 0.0, "any"), "gelu-tanh": (0.0, 0.0, "any"),
    "gelu-erf": (0.0, 0.0, "any"), "hardswish": (1.0 / 6.0, 0.5, "any"), "clip": (-0.75, 1.5, "any"),
    "clip-v2": (-0.75, 1.5, "any"), "pow": (0.5, 2.5, "pos"), "mish": (0.0, 0.0, "any"), "round": (0.0, 0.0, "any"),
}
EXACT_FWD = {"square", "sqrt", "clip", "clip-v2", "hardswish", "round"}
EXACT_BWD = {"square", "sqrt", "clip", "clip-v2", "hardswish", "log"}
# measured on B200 (1 M normal(0, 2) inputs): forward exp 2, log 1, soft-relu 3, swish 1, gelu-tanh 1, gelu-erf 2,
# pow 1, mish 3 outside the absolute allowance; backward exp 3, pow 2, the others inside the allowance
ULP_FWD = {"exp": 2, "log": 2, "soft-relu": 4, "swish": 2, "gelu-tanh": 2, "gelu-erf": 4, "pow": 4, "mish": 4}
ULP_BWD = {"exp": 3, "soft-relu": 2, "swish": 2, "gelu-tanh": 2, "gelu-erf": 2, "pow": 4, "mish": 2}


def inputs(n, seed, domain):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n) * 2.0).astype(np.float32)
    x[:12] = [0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 2.5, -2.5, 1e-3, -1e-3, 19.0, -19.0]
    if domain == "pos":
        x = (np.abs(x) + np.float32(1e-3)).astype(np.float32)
    dy = rng.standard_normal(n).astype(np.float32)
    return x, dy


def run_fwd(fact, dev, kind, x, a, b, dtype="float", alpha=1.0, beta=0.0, y0=None):
    d = core.tensor_descriptor([x.size], dtype, [1])
    ad = core.activation_descriptor(kind, True, a, b)
    tx, ty = dev.put(x), dev.put(np.zeros_like(x) if y0 is None else y0)
    core.activation_forward(fact.handle, ad, alpha, d, tx, beta, d, ty)
    return dev.get(ty, x.dtype)


def run_bwd(fact, dev, kind, x, g, a, b, dtype="float", y=None):
    d = core.tensor_descriptor([x.size], dtype, [1])
    ad = core.activation_descriptor(kind, True, a, b)
    tx, tg, tdx = dev.put(x), dev.put(g), dev.put(np.zeros_like(x))
    ty = dev.put(y) if y is not None else None
    core.activation_backward(fact.handle, ad, 1.0, d, ty, d, tg, d, tx, 0.0, d, tdx)
    return dev.get(tdx, x.dtype)


@pytest.mark.parametrize("kind", sorted(KINDS))
def test_forward_fp32(fact, dev, oracle, kind):
    a, b, dom = KINDS[kind]
    x, _ = inputs(1 << 20, 11, dom)
    got = run_fwd(fact, dev, kind, x, a, b)
    assert fact.handle.last_kernel() == "activation-fwd/flat"
    want = oracle.eltwise_fwd(kind, x, np.zeros_like(x), coef=a, shift=b)
    if kind in EXACT_FWD:
        assert np.array_equal(got, want)
        return
    truth = oracle.eltwise_fwd_truth(kind, x, coef=a, shift=b).astype(np.float32)
    u = ulp_diff_f32(got, truth)
    small = np.abs(got.astype(np.float64) - truth) <= 2.0 ** -24 * np.maximum(np.abs(x), 1.0)
    print("%s forward: max %d ulp, %.2e of the elements above 1 ulp; max %d ulp where the error exceeds 2^-24 max(|x|,1)"
          % (kind, u.max(), (u > 1).mean(), u[~small].max(initial=0)))
    assert ((u <= ULP_FWD[kind]) | small).all()
    assert np.array_equal(want, truth)  # the oracle's float result IS the rounded double definition


@pytest.mark.parametrize("kind", sorted(k for k in KINDS if k != "round"))
def test_backward_fp32(fact, dev, oracle, kind):
    a, b, dom = KINDS[kind]
    x, g = inputs(1 << 20, 12, dom)
    got = run_bwd(fact, dev, kind, x, g, a, b)
    # swish and gelu-tanh have packed fp32 kernels of their own (two vectors per thread backward)
    assert fact.handle.last_kernel() == ("activation-bwd/flat-multi" if kind in ("swish", "gelu-tanh") else "activation-bwd/flat")
    want = oracle.eltwise_bwd(kind, x, g, np.zeros_like(x), coef=a, shift=b)
    if kind in EXACT_BWD:
        assert np.array_equal(got, want)
        return
    truth = oracle.eltwise_bwd_truth(kind, x, g, coef=a, shift=b)
    u = ulp_diff_f32(got, truth.astype(np.float32))
    near_zero = np.abs(got.astype(np.float64) - truth) <= 8 * 2.0 ** -24 * np.abs(g)
    print("%s backward: max %d ulp away from the derivative's zero crossings" % (kind, u[~near_zero].max(initial=0)))
    assert ((u <= ULP_BWD[kind]) | near_zero).all()


def test_round_has_no_backward(fact, dev):
    from deep_diamond_b200.constants import DiamondError
    x = np.ones(64, np.float32)
    with pytest.raises(DiamondError):
        run_bwd(fact, dev, "round", x, x, 0.0, 0.0)


DST = {"relu-dst-bwd": ("relu", 0.25, "any"), "tanh-dst-bwd": ("tanh", 0.0, "any"), "elu-dst-bwd": ("elu", 1.5, "any"),
       "sqrt-dst-bwd": ("sqrt", 0.0, "pos"), "logistic-dst-bwd": ("logistic", 0.0, "any"),
       "exp-dst-bwd": ("exp", 0.0, "any"), "clip-v2-dst-bwd": ("clip-v2", -0.75, "any")}


@pytest.mark.parametrize("kind", sorted(DST))
def test_dst_bwd_kinds(fact, dev, oracle, kind):
    """Forward = the kind it is named after (same bits); backward reads the forward RESULT (the y
    argument; x is not passed at all) and matches the oracle's arithmetic on that result bit for bit.
    Against the derivative taken from the source it agrees to the accuracy y carries."""
    base, a, dom = DST[kind]
    b = 1.5 if base == "clip-v2" else 0.0
    x, g = inputs(1 << 18, 13, dom)
    y = run_fwd(fact, dev, kind, x, a, b)
    assert np.array_equal(y, run_fwd(fact, dev, base, x, a, b))
    d = core.tensor_descriptor([x.size], "float", [1])
    ad = core.activation_descriptor(kind, True, a, b)
    ty, tg, tdx = dev.put(y), dev.put(g), dev.put(np.zeros_like(x))
    core.activation_backward(fact.handle, ad, 1.0, d, ty, d, tg, None, None, 0.0, d, tdx)
    got = dev.get(tdx, np.float32)
    want = oracle.eltwise_bwd(kind, y, g, np.zeros_like(x), coef=a, shift=b)
    assert np.array_equal(got, want)
    from_src = oracle.eltwise_bwd_truth(base, x, g, coef=a, shift=b)
    err = np.abs(got.astype(np.float64) - from_src)
    # 1 - y^2 and y (1 - y) lose what y has rounded away near saturation: bound by a few units of y's last place
    assert (err <= 1e-5 * np.abs(from_src) + 4 * 2.0 ** -24 * np.abs(g) * np.maximum(1.0, np.abs(y))).all()


@pytest.mark.parametrize("kind", ["swish", "gelu-erf", "hardswish", "mish", "pow"])
def test_fp64_and_views(fact, dev, oracle, kind):
    a, b, dom = KINDS[kind]
    rng = np.random.default_rng(5)
    x = rng.standard_normal(4096) * 2.0
    if dom == "pos":
        x = np.abs(x) + 1e-3
    g = rng.standard_normal(4096)
    got = run_fwd(fact, dev, kind, x, a, b, dtype="double")
    want = oracle.eltwise_fwd(kind, x, np.zeros_like(x), coef=a, shift=b)
    np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-300)
    gb = run_bwd(fact, dev, kind, x, g, a, b, dtype="double")
    wb = oracle.eltwise_bwd(kind, x, g, np.zeros_like(x), coef=a, shift=b)
    np.testing.assert_allclose(gb, wb, rtol=1e-11, atol=1e-14)
    # fp32 on views: a channel window (rows kernel) and an nhwc source into an nchw result (strided kernel),
    # with alpha / beta
    shape = [3, 8, 6, 8]
    xs = (np.abs(rng.standard_normal(3 * 12 * 6 * 8)) + 1e-3).astype(np.float32) if dom == "pos" \
        else rng.standard_normal(3 * 12 * 6 * 8).astype(np.float32)
    win = [12 * 48, 48, 8, 1]
    y0 = rng.standard_normal(3 * 8 * 48).astype(np.float32)
    dn = oracle.default_strides(shape)
    want = y0.copy()
    oracle.eltwise_fwd(kind, oracle.as_layout(xs, shape, win), oracle.as_layout(want, shape, dn), coef=a, shift=b,
                       alpha=0.5, beta=2.0)
    tx, ty = dev.put(xs), dev.put(y0)
    ad = core.activation_descriptor(kind, True, a, b)
    core.activation_forward(fact.handle, ad, 0.5, core.tensor_descriptor(shape, "float", win), tx, 2.0,
                            core.tensor_descriptor(shape, "float", dn), ty)
    assert fact.handle.last_kernel() == "activation-fwd/rows"
    got = dev.get(ty, np.float32)
    assert (ulp_diff_f32(got, want) <= 16).all() or np.allclose(got, want, rtol=2e-6, atol=1e-6)
    nhwc = oracle.nhwc_strides(shape)
    xs2 = xs[:3 * 8 * 48]
    want = np.zeros(3 * 8 * 48, np.float32)
    oracle.eltwise_fwd(kind, oracle.as_layout(xs2, shape, nhwc), oracle.as_layout(want, shape, dn), coef=a, shift=b)
    tx, ty = dev.put(xs2), dev.put(np.zeros_like(want))
    core.activation_forward(fact.handle, ad, 1.0, core.tensor_descriptor(shape, "float", nhwc), tx, 0.0,
                            core.tensor_descriptor(shape, "float", dn), ty)
    assert fact.handle.last_kernel() == "activation-fwd/strided"
    got = dev.get(ty, np.float32)
    xl = oracle.as_layout(xs2, shape, nhwc).reshape(-1)  # logical order = the dense result's order
    small = np.abs(got.astype(np.float64) - want) <= 2.0 ** -24 * np.maximum(np.abs(xl), 1.0)
    assert ((ulp_diff_f32(got, want) <= max(ULP_FWD.get(kind, 0), 1)) | small).all()


@pytest.mark.parametrize("dtype,np_t", [("half", np.float16)])
@pytest.mark.parametrize("kind", ["swish", "gelu-tanh", "square", "hardswish"])
def test_f16(fact, dev, oracle, kind, dtype, np_t):
    """16-bit tensors compute in float and round once more: at most one unit of the 16-bit type from
    the oracle (which rounds the double definition to float first, then to the 16-bit type)."""
    a, b, _ = KINDS[kind]
    x = (np.random.default_rng(3).standard_normal(1 << 16) * 2).astype(np_t)
    got = run_fwd(fact, dev, kind, x, a, b, dtype=dtype)
    want = oracle.eltwise_fwd(kind, x, np.zeros_like(x), coef=a, shift=b)
    gi, wi = got.view(np.int16).astype(np.int32), want.view(np.int16).astype(np.int32)
    same_sign = (gi < 0) == (wi < 0)
    assert ((np.abs(gi - wi) <= 1) & same_sign | (got == want)).all()


def test_activation_layers_of_the_dnnl_kinds(fact, oracle):
    """The kinds through the public layer API (`activation` blueprint -> training layer): forward into
    dst, backward from the upstream gradient; a *-dst-bwd kind keeps dst apart from the gradient."""
    from deep_diamond_b200 import dnn
    from deep_diamond_b200.tensor import native, output, tensor, transfer
    shape = [4, 8, 6, 6]
    x = oracle.gen_normal(shape, 1.0, 21).reshape(-1)
    g = oracle.gen_normal(shape, 1.0, 22).reshape(-1)
    for kind, opts in (("gelu-tanh", {}), ("swish", {"alpha": 1.0}), ("tanh-dst-bwd", {}), ("logistic-dst-bwd", {})):
        src = tensor(fact, shape, "float", "nchw")
        diff_src = tensor(fact, shape, "float", "nchw")
        layer = dnn.activation(fact, src, kind, opts)(src, diff_src)
        transfer(x.tolist(), src)
        dnn.forward(layer)
        y = np.array(list(native(output(layer))), np.float32)
        transfer(g.tolist(), dnn.diff_input(layer))
        dnn.backward(layer)
        dx = np.array(list(native(dnn.diff_output(layer))), np.float32)
        a = opts.get("alpha", 0.0)
        base = {"tanh-dst-bwd": "tanh", "logistic-dst-bwd": "logistic"}.get(kind, kind)
        ty = oracle.eltwise_fwd_truth(base, x, coef=a).astype(np.float32)
        td = oracle.eltwise_bwd_truth(base, x, g, coef=a)
        assert ((ulp_diff_f32(y, ty) <= 4) | (np.abs(y.astype(np.float64) - ty) <= 2.0 ** -24 * np.maximum(np.abs(x), 1))).all(), kind
        assert (np.abs(dx - td) <= 2e-6 * np.abs(td) + 1e-6 * np.abs(g)).all(), kind
