"""GPU parity: ddActivationForward / ddActivationBackward against the CPU oracle.

Bars: relu, linear, clipped-relu, abs bit-exact (signed zero compared by value); logistic, tanh, elu
within 2 ulp of the definition evaluated in double and rounded once (the "truth"), and within 2 ulp of
the fp32 oracle forward.  Backward is compared with the truth at 2 ulp, and with the fp32 oracle
(whose 1-f(x) cancels near saturation) at 2 ulp or 4*2^-24*|dy|, whichever is larger.
Reference vectors: deep-diamond-dnnl/test/.../dnnl/core_test.clj:363-427,
deep-diamond-cuda/test/.../cudnn/core_test.clj:51-147, deep-diamond-test/.../dnn_test.clj:28-82.
"""
import numpy as np
import pytest

from conftest import ulp_diff_f32
from deep_diamond_b200 import core

pytestmark = pytest.mark.gpu

MODES = ["relu", "logistic", "tanh", "elu", "linear", "clipped-relu", "abs"]
COEF = {"relu": 0.0, "logistic": 0.0, "tanh": 0.0, "elu": 1.0, "linear": 2.5, "clipped-relu": 1.5, "abs": 0.0}
EXACT = {"relu", "linear", "clipped-relu", "abs"}


def inputs(n, seed):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n) * 2.0).astype(np.float32)
    x[:16] = [0.0, -0.0, 1.0, -1.0, 1e-8, -1e-8, 1e-3, -1e-3, 20.0, -20.0, 88.0, -88.0, 100.0, -104.0, 0.5, -0.5]
    dy = rng.standard_normal(n).astype(np.float32)
    return x, dy


def gpu_fwd(fact, dev, mode, x, coef, shift=0.0, alpha=1.0, beta=0.0, y0=None, dtype="float"):
    d = core.tensor_descriptor([x.size], dtype, [1])
    ad = core.activation_descriptor(mode, True, coef, shift)
    dx = dev.put(x)
    dy = dev.put(y0 if y0 is not None else np.zeros_like(x))
    core.activation_forward(fact.handle, ad, alpha, d, dx, beta, d, dy)
    return dev.get(dy, x.dtype)


def gpu_bwd(fact, dev, mode, x, g, coef, alpha=1.0, beta=0.0, dx0=None, dtype="float"):
    d = core.tensor_descriptor([x.size], dtype, [1])
    ad = core.activation_descriptor(mode, True, coef)
    tx, tg = dev.put(x), dev.put(g)
    tdx = dev.put(dx0 if dx0 is not None else np.zeros_like(x))
    core.activation_backward(fact.handle, ad, alpha, d, None, d, tg, d, tx, beta, d, tdx)
    return dev.get(tdx, x.dtype)


@pytest.mark.parametrize("mode", MODES)
def test_forward_fp32(fact, dev, oracle, mode):
    x, _ = inputs(1 << 20, 1)
    coef = COEF[mode]
    shift = 0.25 if mode == "linear" else 0.0
    got = gpu_fwd(fact, dev, mode, x, coef, shift)
    want = oracle.eltwise_fwd(mode, x, np.zeros_like(x), coef=coef, shift=shift)
    assert fact.handle.last_kernel() == "activation-fwd/flat"
    if mode in EXACT:
        assert np.array_equal(got, want)  # value equality: -0.0 == +0.0
    else:
        truth = oracle.eltwise_fwd_truth(mode, x, coef=coef).astype(np.float32)
        assert ulp_diff_f32(got, truth).max() <= 2
        assert ulp_diff_f32(got, want).max() <= 2


@pytest.mark.parametrize("mode", MODES)
def test_backward_fp32(fact, dev, oracle, mode):
    x, g = inputs(1 << 20, 2)
    coef = COEF[mode]
    got = gpu_bwd(fact, dev, mode, x, g, coef)
    want = oracle.eltwise_bwd(mode, x, g, np.zeros_like(x), coef=coef)
    # the fp32 transcendental modes run the two-vectors-per-thread form of the flat kernel backward
    multi = mode in ("logistic", "sigmoid", "tanh", "elu")
    assert fact.handle.last_kernel() == ("activation-bwd/flat-multi" if multi else "activation-bwd/flat")
    if mode in EXACT:
        assert np.array_equal(got, want)
    else:
        truth = oracle.eltwise_bwd_truth(mode, x, g, coef=coef).astype(np.float32)
        tiny = np.abs(truth) < 1e-37  # denormal results: compare absolutely
        assert (ulp_diff_f32(got, truth)[~tiny]).max() <= 2
        assert np.abs(got[tiny].astype(np.float64) - truth[tiny]).max(initial=0) <= 1e-37
        ok = (ulp_diff_f32(got, want) <= 2) | (np.abs(got.astype(np.float64) - want) <= 4 * 2.0 ** -24 * np.abs(g))
        assert ok.all()


def test_alpha_beta_and_in_place(fact, dev, oracle):
    # cudnn core_test.clj:51-95: y = 3*relu(x) + 2*y ; dx = 300*relu'(x)*dy + 200*dx
    x = np.arange(-2, 118, dtype=np.float32)
    y0 = np.arange(120, dtype=np.float32)
    got = gpu_fwd(fact, dev, "relu", x, 42.0 * 0, alpha=3.0, beta=2.0, y0=y0)
    assert got[:5].tolist() == [0.0, 2.0, 4.0, 9.0, 14.0]
    want = oracle.eltwise_fwd("relu", x, y0.copy(), alpha=3.0, beta=2.0)
    assert np.array_equal(got, want)
    dx0 = (np.arange(120) * 0.1 - 6).astype(np.float32)
    dy = (np.arange(120) * 0.01 - 0.6).astype(np.float32)
    gb = gpu_bwd(fact, dev, "relu", x, dy, 0.0, alpha=300.0, beta=200.0, dx0=dx0)
    wb = oracle.eltwise_bwd("relu", x, dy, dx0.copy(), alpha=300.0, beta=200.0)
    assert np.array_equal(gb, wb)
    np.testing.assert_allclose(gb[:5], [-1200.0, -1180.0, -1160.0, -1311.0, -1288.0], rtol=1e-6)
    # in place: y is x (inference form)
    d = core.tensor_descriptor([2, 3, 4, 5], "float", "nchw")
    t = dev.put(x)
    core.activation_forward(fact.handle, core.activation_descriptor("relu", True, 0.0), 1.0, d, t, 0.0, d, t)
    assert np.array_equal(dev.get(t, np.float32), np.maximum(x, 0))


def test_reference_logistic_vectors(fact, dev):
    # dnnl core_test.clj:403-427
    x = np.array([-1, -0.5, 0, 0.1, 0.5, 0.7], dtype=np.float32)
    dy = np.array([-0.5, -0.2, -0.4, 0, 0.2, 0.3], dtype=np.float32)
    fwd = gpu_fwd(fact, dev, "logistic", x, 0.0)
    ref_fwd = np.array([0.2689414322376251, 0.377540647983551, 0.5, 0.5249792337417603,
                        0.622459352016449, 0.6681877970695496], dtype=np.float32)
    assert ulp_diff_f32(fwd, ref_fwd).max() <= 2
    bwd = gpu_bwd(fact, dev, "logistic", x, dy, 0.0)
    ref_bwd = np.array([-0.09830597043037415, -0.04700074344873428, -0.10000000149011612, 0.0,
                        0.04700074344873428, 0.06651385873556137], dtype=np.float32)
    assert ulp_diff_f32(bwd, ref_bwd).max() <= 2
    # cudnn core_test.clj:97-131
    one = gpu_bwd(fact, dev, "sigmoid", np.array([-0.5], np.float32), np.array([-0.1], np.float32), 0.0)
    assert abs(float(one[0]) - (-0.02350037172436714)) < 1e-8


def test_nan_and_inf(fact, dev, oracle):
    x = np.array([np.nan, np.inf, -np.inf, 0.0] * 4, dtype=np.float32)
    for mode in MODES:
        got = gpu_fwd(fact, dev, mode, x, COEF[mode])
        want = oracle.eltwise_fwd(mode, x, np.zeros_like(x), coef=COEF[mode])
        assert np.array_equal(np.isnan(got), np.isnan(want)), mode
        fin = ~np.isnan(want)
        assert np.array_equal(got[fin], want[fin]), mode


@pytest.mark.parametrize("dtype,np_t", [("double", np.float64), ("half", np.float16)])
def test_other_float_types(fact, dev, oracle, dtype, np_t):
    x32, g32 = inputs(4096 + 3, 3)
    x, g = x32.astype(np_t), g32.astype(np_t)
    for mode in ("relu", "tanh", "logistic", "elu"):
        got = gpu_fwd(fact, dev, mode, x, COEF[mode], dtype=dtype)
        want = oracle.eltwise_fwd(mode, x, np.zeros_like(x), coef=COEF[mode])
        tol = 1e-14 if dtype == "double" else 1e-3
        np.testing.assert_allclose(got.astype(np.float64), want.astype(np.float64), rtol=tol, atol=tol * 1e-3)
        gb = gpu_bwd(fact, dev, mode, x, g, COEF[mode], dtype=dtype)
        wb = oracle.eltwise_bwd(mode, x, g, np.zeros_like(x), coef=COEF[mode])
        tol = 1e-12 if dtype == "double" else 2e-3
        np.testing.assert_allclose(gb.astype(np.float64), wb.astype(np.float64), rtol=tol, atol=tol)


def test_bf16(fact, dev, oracle):
    x32, _ = inputs(4096, 4)
    xb = (x32.view(np.uint32) >> 16).astype(np.uint16)
    d = core.tensor_descriptor([xb.size], "bf16", [1])
    tx, ty = dev.put(xb), dev.put(np.zeros_like(xb))
    core.activation_forward(fact.handle, core.activation_descriptor("relu", True, 0.0), 1.0, d, tx, 0.0, d, ty)
    got = dev.get(ty, np.uint16)
    want = oracle.eltwise_fwd("relu", xb, np.zeros_like(xb), tag="bf16")
    gf = (got.astype(np.uint32) << 16).view(np.float32)
    wf = (want.astype(np.uint32) << 16).view(np.float32)
    assert np.array_equal(gf, wf)


def test_strided_views(fact, dev, oracle):
    # sub-memory with offsets: dnnl core_test.clj:146-200 (abs on channel 1 of a [2 2 3 2] tensor)
    buf = -np.arange(24, dtype=np.float32)
    want = buf.copy()
    sub_shape, st = [2, 1, 3, 2], [12, 6, 2, 1]
    oracle.eltwise_fwd("abs", oracle.as_layout(want, sub_shape, st, offset=6),
                       oracle.as_layout(want, sub_shape, st, offset=6))
    assert want[5] == -5 and want[6] == 6 and want[11] == 11 and want[12] == -12 and want[23] == 23
    t = dev.put(buf)
    d = core.tensor_descriptor(sub_shape, "float", st)
    core.activation_forward(fact.handle, core.activation_descriptor("abs", True, 0.0), 1.0, d,
                            t.data_ptr() + 6 * 4, 0.0, d, t.data_ptr() + 6 * 4)
    assert np.array_equal(dev.get(t, np.float32), want)
    assert fact.handle.last_kernel() == "activation-fwd/strided"
    # nchw source, nhwc destination
    shape = [2, 6, 3, 4]
    x = np.random.default_rng(5).standard_normal(int(np.prod(shape))).astype(np.float32)
    sx, sy = oracle.default_strides(shape), oracle.nhwc_strides(shape)
    w = np.zeros_like(x)
    oracle.eltwise_fwd("relu", oracle.as_layout(x, shape, sx), oracle.as_layout(w, shape, sy))
    tx, ty = dev.put(x), dev.put(np.zeros_like(x))
    core.activation_forward(fact.handle, core.activation_descriptor("relu", True, 0.0), 1.0,
                            core.tensor_descriptor(shape, "float", sx), tx, 0.0,
                            core.tensor_descriptor(shape, "float", sy), ty)
    assert np.array_equal(dev.get(ty, np.float32), w)


@pytest.mark.parametrize("mode", ["relu", "tanh", "logistic", "elu", "abs"])
def test_rows_views(fact, dev, oracle, mode):
    """Activation forward and backward on a channel window of a wider tensor (rows contiguous,
    16-byte aligned): the vectorised walk over views; untouched channels keep their bits."""
    shape, parent = [4, 6, 8, 16], [4, 10, 8, 16]
    st = [10 * 128, 128, 16, 1]
    rng = np.random.default_rng(12)
    xs = (rng.standard_normal(int(np.prod(parent))) * 2).astype(np.float32)
    gs = rng.standard_normal(int(np.prod(parent))).astype(np.float32)
    coef = COEF[mode]
    off = 2 * 128                                           # channels 2..7
    want = np.full(xs.size, 7.0, np.float32)
    oracle.eltwise_fwd(mode, oracle.as_layout(xs, shape, st, offset=off), oracle.as_layout(want, shape, st, offset=off), coef=coef)
    tx, ty = dev.put(xs), dev.put(np.full(xs.size, 7.0, np.float32))
    d = core.tensor_descriptor(shape, "float", st)
    ad = core.activation_descriptor(mode, True, coef)
    core.activation_forward(fact.handle, ad, 1.0, d, tx.data_ptr() + off * 4, 0.0, d, ty.data_ptr() + off * 4)
    assert fact.handle.last_kernel() == "activation-fwd/rows"
    got = dev.get(ty, np.float32)
    if mode in EXACT:
        assert np.array_equal(got, want)
    else:
        assert ulp_diff_f32(got, want).max() <= 2
    wantb = np.full(xs.size, -3.0, np.float32)
    oracle.eltwise_bwd(mode, oracle.as_layout(xs, shape, st, offset=off), oracle.as_layout(gs, shape, st, offset=off),
                       oracle.as_layout(wantb, shape, st, offset=off), coef=coef)
    tg, tdx = dev.put(gs), dev.put(np.full(xs.size, -3.0, np.float32))
    core.activation_backward(fact.handle, ad, 1.0, d, None, d, tg.data_ptr() + off * 4, d, tx.data_ptr() + off * 4,
                             0.0, d, tdx.data_ptr() + off * 4)
    assert fact.handle.last_kernel() == "activation-bwd/rows"
    gotb = dev.get(tdx, np.float32)
    if mode in EXACT:
        assert np.array_equal(gotb, wantb)
    else:
        ok = (ulp_diff_f32(gotb, wantb) <= 2) | (np.abs(gotb.astype(np.float64) - wantb) <= 4 * 2.0 ** -24 * np.abs(gs))
        assert ok.all()


def _round_to_bf16(x64):
    """float64 -> bfloat16 bit patterns, rounded to nearest even ONCE (not through float32)."""
    f32 = x64.astype(np.float32)
    u = f32.view(np.uint32)
    lo = u & np.uint32(0xFFFF0000)
    hi = lo + np.uint32(0x10000)
    with np.errstate(invalid="ignore", over="ignore"):
        dlo = np.abs(x64 - lo.view(np.float32).astype(np.float64))
        dhi = np.abs(hi.view(np.float32).astype(np.float64) - x64)
    odd = ((lo >> np.uint32(16)) & np.uint32(1)).astype(bool)
    up = (dhi < dlo) | ((dhi == dlo) & odd)
    out = np.where(up, hi, lo)
    out = np.where(np.isnan(x64), np.uint32(0x7FC00000), out)
    out = np.where(np.isinf(x64), u, out)
    return (out >> np.uint32(16)).astype(np.uint16)


def _ordered16(bits):
    i = bits.astype(np.int64)
    return np.where(i >= 0x8000, 0x8000 - i, i)


@pytest.mark.parametrize("dtype", ["half", "bf16"])
@pytest.mark.parametrize("mode", ["tanh", "logistic", "elu"])
def test_every_16_bit_input(fact, dev, mode, dtype):
    """All 65536 bit patterns of f16 / bf16 through forward and backward (dy = 1): at most one unit
    of the 16-bit type from the definition evaluated in double and rounded once."""
    bits = np.arange(65536, dtype=np.uint16)
    if dtype == "half":
        x64 = bits.view(np.float16).astype(np.float64)
        one = np.ones(65536, np.float16).view(np.uint16)
    else:
        with np.errstate(invalid="ignore"):           # signalling NaN patterns among the inputs
            x64 = (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        one = np.full(65536, 0x3F80, np.uint16)
    with np.errstate(over="ignore", invalid="ignore"):
        e = np.exp(-np.abs(x64))
        if mode == "logistic":
            f = np.where(x64 >= 0, 1 / (1 + e), e / (1 + e))
            df = e / (1 + e) ** 2
        elif mode == "tanh":
            f, e2 = np.tanh(x64), np.exp(-2 * np.abs(x64))
            df = 4 * e2 / (1 + e2) ** 2
        else:
            f = np.where(x64 > 0, x64, np.expm1(np.minimum(x64, 0)))
            df = np.where(x64 > 0, 1.0, np.exp(np.minimum(x64, 0)))
    d = core.tensor_descriptor([65536], dtype, [1])
    ad = core.activation_descriptor(mode, True, 1.0 if mode == "elu" else 0.0)
    tx, ty, tg, tdx = dev.put(bits), dev.put(np.zeros_like(bits)), dev.put(one), dev.put(np.zeros_like(bits))
    core.activation_forward(fact.handle, ad, 1.0, d, tx, 0.0, d, ty)
    core.activation_backward(fact.handle, ad, 1.0, d, None, d, tg, d, tx, 0.0, d, tdx)
    for got, ref in ((dev.get(ty, np.uint16), f), (dev.get(tdx, np.uint16), df)):
        if dtype == "half":
            with np.errstate(over="ignore"):
                want = ref.astype(np.float16).view(np.uint16)
            nan_got = np.isnan(got.view(np.float16))
        else:
            want = _round_to_bf16(ref)
            nan_got = np.isnan((got.astype(np.uint32) << 16).view(np.float32))
        nan_want = np.isnan(ref)
        assert np.array_equal(nan_got, nan_want)
        diff = np.abs(_ordered16(got) - _ordered16(want))[~nan_want]
        assert diff.max() <= 1, (mode, dtype, int(diff.max()), int((diff > 0).sum()))


def _ordered(t):
    """float32 tensor -> int64 keys that are monotone in the float order (ulp distance = key diff)."""
    import torch
    i = t.view(torch.int32).to(torch.int64)
    return torch.where(i < 0, -(2 ** 31) - i, i)


@pytest.mark.parametrize("mode,bwd", [("logistic", False), ("tanh", False), ("logistic", True),
                                      ("tanh", True), ("elu", True), ("elu", False)])
def test_every_float32_input(fact, dev, mode, bwd):
    """All 2^32 float32 bit patterns through the kernel, against the definition evaluated in double on
    the device and rounded once.  Bar: 2 ulp (1 ulp is what is actually reached; printed)."""
    import torch
    chunk = 1 << 27
    ad = core.activation_descriptor(mode, True, COEF[mode])
    d = core.tensor_descriptor([chunk], "float", [1])
    out = torch.empty(chunk, dtype=torch.float32, device=fact.device)
    ones = torch.ones(chunk, dtype=torch.float32, device=fact.device)
    worst, worst_at = 0, (0.0, 0.0, 0.0)
    for start in range(0, 1 << 32, chunk):
        bits = torch.arange(start, start + chunk, dtype=torch.int64, device=fact.device)
        x = bits.to(torch.int32).view(torch.float32) if start + chunk <= (1 << 31) else \
            (bits - (1 << 32)).to(torch.int32).view(torch.float32)
        if bwd:
            core.activation_backward(fact.handle, ad, 1.0, d, None, d, ones, d, x, 0.0, d, out)
        else:
            core.activation_forward(fact.handle, ad, 1.0, d, x, 0.0, d, out)
        fact.synchronize()
        xd = x.double()
        if mode == "logistic":
            e = torch.exp(-xd.abs())
            truth = e / (1 + e) ** 2 if bwd else torch.where(xd >= 0, 1 / (1 + e), e / (1 + e))
        elif mode == "tanh":
            e = torch.exp(-2 * xd.abs())
            truth = 4 * e / (1 + e) ** 2 if bwd else torch.tanh(xd)
        else:
            truth = torch.where(xd > 0, torch.ones_like(xd), torch.exp(xd)) if bwd else \
                torch.where(xd > 0, xd, torch.expm1(xd))
        t32 = truth.float()
        fin = torch.isfinite(t32) & torch.isfinite(x)
        diff = (_ordered(out) - _ordered(t32)).abs()
        diff = torch.where(fin, diff, torch.zeros_like(diff))
        # signed zero: -0.0 and +0.0 are one key apart in this ordering but equal in value
        diff = torch.where((out == 0) & (t32 == 0), torch.zeros_like(diff), diff)
        w = int(diff.max().item())
        if w > worst:
            worst = w
            at = int(diff.argmax().item())
            worst_at = (float(x[at]), float(out[at]), float(t32[at]))
        nan_in = torch.isnan(x)
        assert bool((torch.isnan(out) == nan_in).all()), "NaN must propagate and only NaN"
    print("%s %s: worst ulp distance over all float32 inputs = %d" % (mode, "bwd" if bwd else "fwd", worst))
    assert worst <= 2, "x=%r got=%r truth=%r" % worst_at
