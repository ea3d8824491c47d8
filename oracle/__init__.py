"""CPU oracle for the tensor hot path -- TEST INFRASTRUCTURE, not product code.

A ctypes front end to ``dd_oracle.c`` (a plain-C restatement of what the reference's DNNL backend
computes for reorder, eltwise, binary, sum and reduction; see that file's header for the
reference file:line each function follows and for how parity is pinned).  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / reference arm of ``bench.py`` may import this
package.  The GPU library never calls into it.

Arrays are numpy arrays; a tensor with a layout is a numpy *view* whose logical shape is the
tensor's dims and whose strides are the layout (see ``as_layout``).  bfloat16 data is carried in
``uint16`` arrays with an explicit ``"bf16"`` tag.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libdd_oracle.so")
_lib = None

# data type codes shared with include/dd_b200.h
F32, F64, F16, S8, S32, U8, BF16, S64 = 0, 1, 2, 3, 4, 6, 9, 15
CODES = {"f32": F32, "float": F32, "f64": F64, "double": F64, "f16": F16, "half": F16,
         "s8": S8, "byte": S8, "int8": S8, "s32": S32, "int": S32, "u8": U8, "uint8": U8,
         "bf16": BF16, "s64": S64, "long": S64}
NP_OF = {F32: np.float32, F64: np.float64, F16: np.float16, S8: np.int8, S32: np.int32,
         U8: np.uint8, BF16: np.uint16, S64: np.int64}
ACT = {"sigmoid": 0, "logistic": 0, "relu": 1, "tanh": 2, "clipped-relu": 3, "elu": 4,
       "linear": 5, "identity": 5, "abs": 6,
       # elu as oneDNN's fp32 kernels form it, alpha * (float(exp(x)) - 1): forward only, oracle only
       "elu-fp32-exp-minus-1": 7,
       # the rest of the reference's oneDNN table (dnnl/constants.clj:277-308)
       "square": 20, "sqrt": 21, "exp": 22, "log": 23, "soft-relu": 24, "swish": 25, "gelu": 26, "gelu-tanh": 26,
       "gelu-erf": 27, "hardswish": 28, "clip": 29, "clip-v2": 30, "pow": 31, "mish": 32, "round": 33,
       "relu-dst-bwd": 34, "tanh-dst-bwd": 35, "elu-dst-bwd": 36, "sqrt-dst-bwd": 37, "logistic-dst-bwd": 38,
       "sigmoid-dst-bwd": 38, "exp-dst-bwd": 39, "clip-v2-dst-bwd": 40}
BINOP = {"add": 0, "mul": 1, "min": 2, "max": 3, "sub": 4, "div": 5,
         "ge": 6, "gt": 7, "le": 8, "lt": 9, "eq": 10, "ne": 11}
REDOP = {"add": 0, "sum": 0, "mul": 1, "min": 2, "max": 3, "amax": 4, "avg": 5, "mean": 5,
         "norm1": 6, "norm2": 7, "mul-no-zeros": 8}


def build(force=False):
    """Compiles dd_oracle.c with gcc (idempotent)."""
    src = os.path.join(_HERE, "dd_oracle.c")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
        return _LIB_PATH
    subprocess.run(["make", "-C", _HERE, "-B", "libdd_oracle.so"], check=True,
                   capture_output=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def code_of(arr, tag=None):
    if tag is not None:
        return CODES[tag] if isinstance(tag, str) else int(tag)
    for c, t in NP_OF.items():
        if arr.dtype == t and c != BF16:
            return c
    raise TypeError("no data type code for %s" % arr.dtype)


def _i64(seq):
    return (ctypes.c_int64 * len(seq))(*[int(v) for v in seq])


def _desc(arr):
    """(dims, element strides, base pointer) of a numpy view."""
    item = arr.dtype.itemsize
    for s in arr.strides:
        if s % item:
            raise ValueError("strides must be whole elements")
    return _i64(arr.shape), _i64([s // item for s in arr.strides]), ctypes.c_void_p(arr.ctypes.data)


def default_strides(shape):
    st, run = [], 1
    for d in reversed(shape):
        st.append(run)
        run *= max(int(d), 1)
    return list(reversed(st))


def nhwc_strides(shape):
    """Channels (dim 1) innermost, then spatial dims, then batch: [4 1 2 2] for [3 2 2 1]."""
    nd = len(shape)
    st = [0] * nd
    st[1] = 1
    run = shape[1]
    for i in range(nd - 1, 1, -1):
        st[i] = run
        run *= shape[i]
    st[0] = run
    return st


def span(shape, strides):
    return 1 + sum((d - 1) * s for d, s in zip(shape, strides))


def as_layout(buf, shape, strides, offset=0):
    """A logical-shape view over the 1-D storage array ``buf`` with element strides ``strides``."""
    item = buf.dtype.itemsize
    need = offset + span(shape, strides)
    if need > buf.size:
        raise ValueError("buffer too small: need %d elements, have %d" % (need, buf.size))
    return np.lib.stride_tricks.as_strided(buf[offset:], shape=tuple(shape),
                                           strides=tuple(s * item for s in strides))


def alloc_layout(shape, strides, dtype, fill=0):
    buf = np.full(span(shape, strides), fill, dtype=dtype)
    return buf, as_layout(buf, shape, strides)


def reorder(x, y, xtag=None, ytag=None, alpha=1.0, beta=0.0):
    """y = alpha*convert(x) + beta*y over equal logical shapes (views with any strides)."""
    assert x.shape == y.shape
    dims, xs, xp = _desc(x)
    _, ys, yp = _desc(y)
    rc = lib().oracle_reorder(len(x.shape), dims, code_of(x, xtag), xs, xp, code_of(y, ytag), ys, yp,
                              ctypes.c_double(alpha), ctypes.c_double(beta))
    assert rc == 0
    return y


def eltwise_fwd(alg, x, y, coef=0.0, shift=0.0, alpha=1.0, beta=0.0, nanprop=True, tag=None):
    assert x.shape == y.shape and x.dtype == y.dtype
    dims, xs, xp = _desc(x)
    _, ys, yp = _desc(y)
    rc = lib().oracle_eltwise_fwd(ACT[alg], ctypes.c_double(coef), ctypes.c_double(shift),
                                  int(bool(nanprop)), code_of(x, tag), len(x.shape), dims, xs, xp,
                                  ys, yp, ctypes.c_double(alpha), ctypes.c_double(beta))
    assert rc == 0
    return y


def eltwise_bwd(alg, x, dy, dx, coef=0.0, alpha=1.0, beta=0.0, tag=None, shift=0.0):
    """``x`` is the forward source; for the ``*-dst-bwd`` kinds pass the forward result there."""
    assert x.shape == dy.shape == dx.shape
    dims, xs, xp = _desc(x)
    _, gs, gp = _desc(dy)
    _, os_, op = _desc(dx)
    rc = lib().oracle_eltwise_bwd_ex(ACT[alg], ctypes.c_double(coef), ctypes.c_double(shift), code_of(x, tag),
                                     len(x.shape), dims, xs, xp, gs, gp, os_, op, ctypes.c_double(alpha),
                                     ctypes.c_double(beta))
    assert rc == 0
    return dx


def eltwise_fwd_truth(alg, x, coef=0.0, shift=0.0):
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    out = np.empty(x.size, dtype=np.float64)
    lib().oracle_eltwise_fwd_truth(ACT[alg], ctypes.c_double(coef), ctypes.c_double(shift),
                                   ctypes.c_int64(x.size), ctypes.c_void_p(x.ctypes.data),
                                   ctypes.c_void_p(out.ctypes.data))
    return out


def eltwise_bwd_truth(alg, x, dy, coef=0.0, shift=0.0):
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    dy = np.ascontiguousarray(dy, dtype=np.float32).ravel()
    out = np.empty(x.size, dtype=np.float64)
    lib().oracle_eltwise_bwd_truth_ex(ACT[alg], ctypes.c_double(coef), ctypes.c_double(shift),
                                      ctypes.c_int64(x.size), ctypes.c_void_p(x.ctypes.data),
                                      ctypes.c_void_p(dy.ctypes.data), ctypes.c_void_p(out.ctypes.data))
    return out


def binary(op, a, b, c, alpha1=1.0, alpha2=1.0, beta=0.0, tag=None):
    """c = op(alpha1*a, alpha2*bcast(b)) + beta*c; b's dims equal c's or are 1."""
    assert a.shape == c.shape and len(b.shape) == len(c.shape)
    dims, as_, ap = _desc(a)
    bdims, bs, bp = _desc(b)
    _, cs, cp = _desc(c)
    rc = lib().oracle_binary(BINOP[op], code_of(c, tag), len(c.shape), dims, ctypes.c_double(alpha1),
                             as_, ap, ctypes.c_double(alpha2), bdims, bs, bp, ctypes.c_double(beta),
                             cs, cp)
    assert rc == 0
    return c


def add_tensor(alpha, x, beta, y, tag=None):
    """y = alpha*bcast(x) + beta*y (the cudnnAddTensor form)."""
    return binary("add", y, x, y, alpha1=beta, alpha2=alpha, beta=0.0, tag=tag)


def scaled_sum(scales, srcs, dst, tag=None):
    """dst = sum_i scales[i]*srcs[i] over dense same-layout arrays (dst may be srcs[0])."""
    n = len(srcs)
    sc = (ctypes.c_float * n)(*[float(s) for s in scales])
    ptrs = (ctypes.c_void_p * n)(*[s.ctypes.data for s in srcs])
    rc = lib().oracle_sum(n, sc, code_of(dst, tag), ctypes.c_int64(dst.size), ptrs,
                          ctypes.c_void_p(dst.ctypes.data))
    assert rc == 0
    return dst


def reduce(op, x, y, alpha=1.0, beta=0.0, nanprop=True, tag=None, want_truth=False):
    """y = alpha*reduce(x) + beta*y over the dims where y's extent is 1."""
    assert len(x.shape) == len(y.shape)
    xd, xs, xp = _desc(x)
    yd, ys, yp = _desc(y)
    truth = np.empty(y.size, dtype=np.float64) if want_truth else None
    tp = ctypes.c_void_p(truth.ctypes.data) if want_truth else ctypes.c_void_p(0)
    rc = lib().oracle_reduce(REDOP[op], code_of(x, tag), int(bool(nanprop)), len(x.shape), xd, xs, xp,
                             yd, ys, yp, ctypes.c_double(alpha), ctypes.c_double(beta), tp)
    assert rc == 0
    return (y, truth.reshape(y.shape)) if want_truth else y


LP_REDOP = {"norm-lp-max": 9, "norm-lp-sum": 10, "norm-lp-power-p-max": 11, "norm-lp-power-p-sum": 12}


def reduce_lp(op, p, eps, x, y, alpha=1.0, beta=0.0, tag=None, want_truth=False):
    """oneDNN's norm reductions with exponent ``p`` and ``eps`` (dnnl/constants.clj:393-402):
    S = sum |x|^p over the dims where y's extent is 1, then max(S,eps)^(1/p), (S+eps)^(1/p),
    max(S,eps) or S+eps."""
    assert len(x.shape) == len(y.shape)
    xd, xs, xp = _desc(x)
    yd, ys, yp = _desc(y)
    truth = np.empty(y.size, dtype=np.float64) if want_truth else None
    tp = ctypes.c_void_p(truth.ctypes.data) if want_truth else ctypes.c_void_p(0)
    rc = lib().oracle_reduce_lp(LP_REDOP[op], ctypes.c_double(p), ctypes.c_double(eps), code_of(x, tag),
                                len(x.shape), xd, xs, xp, yd, ys, yp, ctypes.c_double(alpha),
                                ctypes.c_double(beta), tp)
    assert rc == 0
    return (y, truth.reshape(y.shape)) if want_truth else y


def equals(x, y, tag=None):
    dims, xs, xp = _desc(x)
    _, ys, yp = _desc(y)
    return bool(lib().oracle_equals(code_of(x, tag), len(x.shape), dims, xs, xp, ys, yp))


COST = {"quadratic": 0, "mean-absolute": 1, "crossentropy": 2}


def cost(kind, a, y, batch=None, want_diff=False):
    """(cost, truth[, a - y]) of dense float32 arrays per base/internal/cost.clj:20-40; ``batch`` is
    the divisor of the cross-entropy (the extent of the batch dim), default ``a.shape[0]``."""
    a32 = np.ascontiguousarray(a, dtype=np.float32)
    y32 = np.ascontiguousarray(y, dtype=np.float32)
    assert a32.shape == y32.shape
    d = np.empty(a32.size, dtype=np.float32) if want_diff else None
    c, t = ctypes.c_double(), ctypes.c_double()
    rc = lib().oracle_cost(COST[kind], ctypes.c_int64(a32.size),
                           ctypes.c_int64(a32.shape[0] if batch is None else batch),
                           ctypes.c_void_p(a32.ctypes.data), ctypes.c_void_p(y32.ctypes.data),
                           ctypes.c_void_p(d.ctypes.data if want_diff else 0), ctypes.byref(c), ctypes.byref(t))
    assert rc == 0
    return (c.value, t.value, d.reshape(a32.shape)) if want_diff else (c.value, t.value)


def num_threads():
    return int(lib().oracle_num_threads())


def set_num_threads(n):
    """Overrides OMP_NUM_THREADS (launchers such as torch.distributed.run set it to 1)."""
    lib().oracle_set_num_threads(int(n))
    return num_threads()


# ---------------------------------------------------------------- synthetic inputs ------------
# Seeded generators for the benchmark configurations (their shapes, value distributions and seeds).
# Shared by the GPU and CPU legs so both see identical inputs.

def gen_uniform(shape, lo, hi, seed):
    rng = np.random.default_rng(seed)
    return (rng.random(size=shape, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def gen_normal(shape, sigma, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(size=shape, dtype=np.float32) * np.float32(sigma)).astype(np.float32)


def gen_signed_lognormal(shape, seed):
    rng = np.random.default_rng(seed)
    mag = np.exp(rng.standard_normal(size=shape, dtype=np.float32))
    sign = np.where(rng.random(size=shape, dtype=np.float32) < 0.5, np.float32(-1), np.float32(1))
    return (mag * sign).astype(np.float32)


def quantize_s8(x):
    """The int8 copy of the reorder configuration: scale 1/127, round-to-nearest-even, saturate."""
    return np.clip(np.rint(x * np.float32(127.0)), -128, 127).astype(np.int8)


def ulp_diff_f32(a, b):
    """Distance in units of float32 last place between two float32 arrays (NaN == NaN -> 0)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, np.int64(-(2 ** 31)) - ia, ia)  # monotone mapping of the float order
    ib = np.where(ib < 0, np.int64(-(2 ** 31)) - ib, ib)
    d = np.abs(ia - ib)
    both_nan = np.isnan(a) & np.isnan(b)
    return np.where(both_nan, 0, d)
