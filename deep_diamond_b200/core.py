"""Functional core over the C ABI -- the counterpart of the reference's
deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/core.clj (descriptor builders and
op wrappers taking keywords and vectors), with the same function names in snake_case and the same
argument order.  Citations below are to that file unless another path is given.
"""
import ctypes

from . import _lib
from ._lib import DiamondError, check, lib
from .constants import (ACTIVATION_MODE, ACTIVATION_NAME, DATA_TYPE, DATA_TYPE_NAME,
                        DATA_TYPE_WIDTH, OP_TENSOR, REDUCE_INDICES, REDUCE_NAME, REDUCE_OP, enc_keyword,
                        layout_strides)


def _ptr(x):
    """Device address of `x`: an int, a torch tensor, or anything with ``device_ptr()``."""
    if x is None:
        return None
    if isinstance(x, int):
        return ctypes.c_void_p(x)
    if hasattr(x, "device_ptr"):
        return ctypes.c_void_p(x.device_ptr())
    if hasattr(x, "data_ptr"):
        return ctypes.c_void_p(x.data_ptr())
    raise TypeError("cannot take a device address of %r" % type(x))


def _scalar(value, dtype_code):
    """Host scalar in the C type the data type asks for (``cast-prim``, cudnn/tensor.clj:193-194):
    double for :double tensors, float otherwise."""
    return ctypes.c_double(float(value)) if dtype_code == 1 else ctypes.c_float(float(value))


class Handle:
    """The library handle bound to one CUDA stream (``cudnn-context``, :33-43)."""

    def __init__(self, stream=None):
        h = ctypes.c_void_p()
        check(lib.ddCreate(ctypes.byref(h)), None, "ddCreate")
        self.ptr = h
        self.stream = None
        if stream is not None:
            self.set_stream(stream)

    def set_stream(self, stream):
        raw = getattr(stream, "cuda_stream", stream)  # torch.cuda.Stream or a raw address
        check(lib.ddSetStream(self.ptr, ctypes.c_void_p(raw or 0)), self.ptr, "ddSetStream")
        self.stream = stream
        return self

    def launch_count(self):
        n = ctypes.c_uint64()
        check(lib.ddGetLaunchCount(self.ptr, ctypes.byref(n)), self.ptr)
        return int(n.value)

    def last_kernel(self):
        return lib.ddGetLastKernelName(self.ptr).decode()

    def device_fault(self):
        """0 unless a kernel of this handle gave up a bounded wait (read after a synchronize)."""
        w = ctypes.c_int(0)
        check(lib.ddGetDeviceFault(self.ptr, ctypes.byref(w)), self.ptr)
        return int(w.value)

    def release(self):
        if self.ptr is not None and self.ptr.value:
            lib.ddDestroy(self.ptr)
            self.ptr = None
        return True


def b200_context(stream=None):
    return Handle(stream)


def get_stream(handle):
    """``get-cudnn-stream`` (:45-46)."""
    s = ctypes.c_void_p()
    check(lib.ddGetStream(handle.ptr, ctypes.byref(s)), handle.ptr)
    return s.value or 0


class TensorDescriptor:
    """Backend tensor descriptor: shape + data type + strides (``CUTensorDescriptor``,
    cudnn/impl.clj:98-148).  Equality is structural, like the reference's."""

    def __init__(self, shape, data_type, strides):
        self.dims = [int(d) for d in shape]
        self.dtype_code = enc_keyword(DATA_TYPE, data_type, "data type") if not isinstance(data_type, int) else data_type
        self.data_type = DATA_TYPE_NAME[self.dtype_code]
        self.strides = [int(s) for s in strides]
        d = ctypes.c_void_p()
        check(lib.ddCreateTensorDescriptor(ctypes.byref(d)), None, "ddCreateTensorDescriptor")
        n = len(self.dims)
        st = lib.ddSetTensorNdDescriptor(d, self.dtype_code, n, (ctypes.c_int64 * n)(*self.dims),
                                         (ctypes.c_int64 * n)(*self.strides))
        if st != 0:
            lib.ddDestroyTensorDescriptor(d)
            check(st, None, "ddSetTensorNdDescriptor")
        self.ptr = d

    # TensorDescriptor protocol (base/tensor.clj:87-94)
    @property
    def shape(self):
        return list(self.dims)

    @property
    def layout(self):
        return list(self.strides)

    def __eq__(self, other):
        return (isinstance(other, TensorDescriptor) and self.dims == other.dims
                and self.dtype_code == other.dtype_code and self.strides == other.strides)

    def __hash__(self):
        return hash((tuple(self.dims), self.dtype_code, tuple(self.strides)))

    def __repr__(self):
        return "{:shape %s :data-type :%s :layout %s}" % (self.dims, self.data_type, self.strides)

    def view(self):
        return TensorDescriptor(self.dims, self.dtype_code, self.strides)

    def release(self):
        if self.ptr is not None:
            lib.ddDestroyTensorDescriptor(self.ptr)
            self.ptr = None
        return True

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def tensor_descriptor(shape, data_type, layout):
    """``tensor-descriptor`` (:48-70): layout is a keyword or a stride vector."""
    shape = [int(d) for d in shape]
    if any(d < 1 for d in shape):
        raise DiamondError("Tensor dimensions must be positive.", {"shape": shape})
    return TensorDescriptor(shape, data_type, layout_strides(shape, layout))


def desc(x):
    """``desc`` of the DescProvider protocol: the backend descriptor of a tensor-like thing."""
    if isinstance(x, TensorDescriptor):
        return x
    if hasattr(x, "desc"):
        return x.desc
    raise TypeError("no tensor descriptor in %r" % type(x))


def equal_desc(a, b):
    """``equal-desc?`` (:72-78)."""
    return desc(a) == desc(b)


def data_type(td):
    return desc(td).data_type


def dims(td):
    return list(desc(td).dims)


def ndims(td):
    return len(desc(td).dims)


def strides(td):
    return list(desc(td).strides)


def bytesize(td):
    n = ctypes.c_size_t()
    check(lib.ddGetTensorSizeInBytes(desc(td).ptr, ctypes.byref(n)), None)
    return int(n.value)


def set_tensor(handle, desc_x, x, value):
    """``set-tensor`` (:100-106)."""
    d = desc(desc_x)
    v = _scalar(value, d.dtype_code)
    check(lib.ddSetTensor(handle.ptr, d.ptr, _ptr(x), ctypes.byref(v)), handle.ptr, "ddSetTensor")
    return handle


def scale_tensor(handle, alpha, desc_x, x):
    """``scale-tensor`` (:108-115)."""
    d = desc(desc_x)
    a = _scalar(alpha, d.dtype_code)
    check(lib.ddScaleTensor(handle.ptr, d.ptr, _ptr(x), ctypes.byref(a)), handle.ptr, "ddScaleTensor")
    return handle


def add_tensor(handle, alpha, desc_x, x, beta, desc_y, y):
    """``add-tensor`` (:117-129): y = alpha*bcast(x) + beta*y."""
    dx, dy = desc(desc_x), desc(desc_y)
    a, b = _scalar(alpha, dx.dtype_code), _scalar(beta, dy.dtype_code)
    check(lib.ddAddTensor(handle.ptr, ctypes.byref(a), dx.ptr, _ptr(x), ctypes.byref(b), dy.ptr,
                          _ptr(y)), handle.ptr, "ddAddTensor")
    return handle


def op_tensor(handle, op, alpha1, desc_a, a, alpha2, desc_b, b, beta, desc_c, c):
    """C = op(alpha1*A, alpha2*bcast(B)) + beta*C -- the binary primitive of the DNNL side
    (``binary``, deep-diamond-dnnl/src/uncomplicate/diamond/internal/dnnl/core.clj:430-447)."""
    da, db, dc = desc(desc_a), desc(desc_b), desc(desc_c)
    a1, a2, bt = _scalar(alpha1, da.dtype_code), _scalar(alpha2, db.dtype_code), _scalar(beta, dc.dtype_code)
    check(lib.ddOpTensor(handle.ptr, enc_keyword(OP_TENSOR, op, "op"), ctypes.byref(a1), da.ptr,
                         _ptr(a), ctypes.byref(a2), db.ptr, _ptr(b), ctypes.byref(bt), dc.ptr,
                         _ptr(c)), handle.ptr, "ddOpTensor")
    return handle


def sum_tensors(handle, scales, descs, srcs, desc_dst, dst):
    """dst = sum_i scales[i]*srcs[i] in one pass (``sum!``,
    deep-diamond-dnnl/src/uncomplicate/diamond/internal/dnnl/core.clj:392-426)."""
    n = len(srcs)
    sc = (ctypes.c_float * n)(*[float(s) for s in scales])
    dp = (ctypes.c_void_p * n)(*[desc(d).ptr.value for d in descs])
    sp = (ctypes.c_void_p * n)(*[_ptr(s).value for s in srcs])
    check(lib.ddSumTensors(handle.ptr, n, sc, dp, sp, desc(desc_dst).ptr, _ptr(dst)), handle.ptr,
          "ddSumTensors")
    return handle


def transform_tensor(handle, alpha, desc_x, buf_x, beta, desc_y, buf_y):
    """``transform-tensor`` (:131-144): y = alpha*convert(x) + beta*y across layouts and types."""
    dx, dy = desc(desc_x), desc(desc_y)
    a, b = _scalar(alpha, dx.dtype_code), _scalar(beta, dy.dtype_code)
    check(lib.ddTransformTensor(handle.ptr, ctypes.byref(a), dx.ptr, _ptr(buf_x), ctypes.byref(b),
                                dy.ptr, _ptr(buf_y)), handle.ptr, "ddTransformTensor")
    return handle


def gather_transform(handle, src_offsets, dst_offsets, desc_x, buf_x, desc_y, buf_y):
    """All the sub-tensor copies of one shuffler invocation in a single launch (the reference issues
    one transform-tensor per column, cudnn/tensor.clj:306-317)."""
    n = len(src_offsets)
    so = (ctypes.c_int64 * n)(*[int(v) for v in src_offsets])
    do = (ctypes.c_int64 * n)(*[int(v) for v in dst_offsets])
    check(lib.ddGatherTransform(handle.ptr, n, so, do, desc(desc_x).ptr, _ptr(buf_x),
                                desc(desc_y).ptr, _ptr(buf_y)), handle.ptr, "ddGatherTransform")
    return handle


def multi_transform(handle, pairs):
    """All the sub-tensor copies of a branch / concatenate pass in one launch.  `pairs` is a list of
    (x, y) tensors (anything with ``desc`` and a device address); the reference runs one
    transform-tensor per pair (cudnn/directed.clj:1331-1333, 1402-1409)."""
    n = len(pairs)
    xd = (ctypes.c_void_p * n)(*[desc(x).ptr.value for x, _ in pairs])
    yd = (ctypes.c_void_p * n)(*[desc(y).ptr.value for _, y in pairs])
    xp = (ctypes.c_void_p * n)(*[_ptr(x).value for x, _ in pairs])
    yp = (ctypes.c_void_p * n)(*[_ptr(y).value for _, y in pairs])
    check(lib.ddMultiTransform(handle.ptr, n, xd, xp, yd, yp), handle.ptr, "ddMultiTransform")
    return handle


COST_KIND = {"quadratic": 0, "mean-absolute": 1, "crossentropy": 2}


def cost_diff(handle, kind, desc_a, a, y, d, cost):
    """d = a - y and its cost in one pass (`cost`: one device element)."""
    check(lib.ddCostDiff(handle.ptr, enc_keyword(COST_KIND, kind, "cost"), desc(desc_a).ptr, _ptr(a), _ptr(y),
                         _ptr(d), _ptr(cost)), handle.ptr, "ddCostDiff")
    return handle


def tensor_equals(handle, desc_x, x, desc_y, y, device_flag):
    check(lib.ddTensorEquals(handle.ptr, desc(desc_x).ptr, _ptr(x), desc(desc_y).ptr, _ptr(y),
                             _ptr(device_flag)), handle.ptr, "ddTensorEquals")
    return handle


# =========================== Activation ============================================

class ActivationDescriptor:
    def __init__(self, mode, relu_nan_opt=True, coef=0.0, shift=0.0):
        d = ctypes.c_void_p()
        check(lib.ddCreateActivationDescriptor(ctypes.byref(d)), None)
        self.ptr = d
        self.mode = enc_keyword(ACTIVATION_MODE, mode, "activation mode")
        check(lib.ddSetActivationDescriptorEx(d, self.mode, 1 if relu_nan_opt else 0, float(coef),
                                              float(shift)), None, "ddSetActivationDescriptor")

    def release(self):
        if self.ptr is not None:
            lib.ddDestroyActivationDescriptor(self.ptr)
            self.ptr = None
        return True


def activation_descriptor(mode, relu_nan_opt=True, coef=0.0, shift=0.0):
    """``activation-descriptor`` (:148-164).  Given a descriptor, returns its contents as a map."""
    if isinstance(mode, ActivationDescriptor):
        m, n, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_double()
        check(lib.ddGetActivationDescriptor(mode.ptr, ctypes.byref(m), ctypes.byref(n), ctypes.byref(c)), None)
        return {"mode": ACTIVATION_NAME[m.value], "relu-nan-opt": bool(n.value), "coef": c.value}
    return ActivationDescriptor(mode, relu_nan_opt, coef, shift)


def activation_forward(handle, ad, alpha, desc_x, buf_x, beta, desc_y, buf_y):
    """``activation-forward`` (:166-172): y = alpha*act(x) + beta*y."""
    dx, dy = desc(desc_x), desc(desc_y)
    a, b = _scalar(alpha, dx.dtype_code), _scalar(beta, dy.dtype_code)
    check(lib.ddActivationForward(handle.ptr, ad.ptr, ctypes.byref(a), dx.ptr, _ptr(buf_x),
                                  ctypes.byref(b), dy.ptr, _ptr(buf_y)), handle.ptr,
          "ddActivationForward")
    return handle


def activation_backward(handle, ad, alpha, desc_y, buf_y, desc_dy, buf_dy, desc_x, buf_x, beta,
                        desc_dx, buf_dx):
    """``activation-backward`` (:174-184): dx = alpha*act'(x)*dy + beta*dx.  y is read by the
    ``*-dst-bwd`` kinds only (they take the derivative from the forward result)."""
    dyy, ddy, ddx = desc(desc_y), desc(desc_dy), desc(desc_dx)
    dx = desc(desc_x) if desc_x is not None else None  # may be absent for a *-dst-bwd kind
    a, b = _scalar(alpha, ddy.dtype_code), _scalar(beta, ddx.dtype_code)
    check(lib.ddActivationBackward(handle.ptr, ad.ptr, ctypes.byref(a), dyy.ptr, _ptr(buf_y),
                                   ddy.ptr, _ptr(buf_dy), dx.ptr if dx is not None else None,
                                   _ptr(buf_x) if buf_x is not None else None, ctypes.byref(b),
                                   ddx.ptr, _ptr(buf_dx)), handle.ptr, "ddActivationBackward")
    return handle


# ============================ Reduce ==============================================

class ReduceTensorDescriptor:
    def __init__(self, op, comp_type="float", nan_opt=True, indices=None, p=None, eps=None):
        d = ctypes.c_void_p()
        check(lib.ddCreateReduceTensorDescriptor(ctypes.byref(d)), None)
        self.ptr = d
        self.op = enc_keyword(REDUCE_OP, op, "reduce op")
        comp = enc_keyword(DATA_TYPE, comp_type, "data type")
        if p is None and eps is None:
            st = lib.ddSetReduceTensorDescriptor(d, self.op, comp, 1 if nan_opt else 0)
        else:
            st = lib.ddSetReduceTensorDescriptorLp(d, self.op, comp, 1 if nan_opt else 0,
                                                   2.0 if p is None else float(p), 0.0 if eps is None else float(eps))
        if st == 0 and indices is not None:
            st = lib.ddSetReduceTensorDescriptorIndices(d, enc_keyword(REDUCE_INDICES, indices, "reduce indices"))
        if st != 0:
            lib.ddDestroyReduceTensorDescriptor(d)
            check(st, None, "ddSetReduceTensorDescriptor")

    def lp(self):
        """(p, eps) of the norm kinds."""
        p, eps = ctypes.c_double(), ctypes.c_double()
        check(lib.ddGetReduceTensorDescriptorLp(self.ptr, ctypes.byref(p), ctypes.byref(eps)), None)
        return p.value, eps.value

    def release(self):
        if self.ptr is not None:
            lib.ddDestroyReduceTensorDescriptor(self.ptr)
            self.ptr = None
        return True


def reduce_tensor_descriptor(op, comp_type="float", nan_opt=True, indices=None, p=None, eps=None):
    """``reduce-tensor-descriptor`` (:188-203), whose fourth argument is ``indices`` (``"flattened"``:
    min / max / amax also report where the result was found; ``"no-indices"``).  ``p`` and ``eps``
    are the two extra arguments of the DNNL backend's ``reduction`` (dnnl/core.clj:796-803), read by
    the ``norm-lp-*`` kinds."""
    return ReduceTensorDescriptor(op, comp_type, nan_opt, indices, p, eps)


def reduction_indices_size(handle, rtd, desc_x, desc_y):
    n = ctypes.c_size_t()
    check(lib.ddGetReductionIndicesSize(handle.ptr, rtd.ptr, desc(desc_x).ptr, desc(desc_y).ptr,
                                        ctypes.byref(n)), handle.ptr)
    return int(n.value)


def reduction_workspace_size(handle, rtd, desc_x, desc_y):
    """``reduction-workspace-size`` (:209-211)."""
    n = ctypes.c_size_t()
    check(lib.ddGetReductionWorkspaceSize(handle.ptr, rtd.ptr, desc(desc_x).ptr, desc(desc_y).ptr,
                                          ctypes.byref(n)), handle.ptr)
    return int(n.value)


def reduce_tensor(handle, rtd, *args):
    """``reduce-tensor`` (:213-231).  The 10-argument arity takes caller-owned indices and
    workspace; the 6-argument arity uses the handle's own scratch -- where the reference allocates
    and frees two device buffers on every call (:223-231), this one allocates nothing."""
    ind, ind_bytes = None, 0
    if len(args) == 8:
        indices, workspace, alpha, desc_x, buf_x, beta, desc_y, buf_y = args
        ws = _ptr(workspace)
        ws_bytes = workspace.numel() * workspace.element_size() if hasattr(workspace, "numel") else 0
        if indices is not None:
            ind = _ptr(indices)
            ind_bytes = indices.numel() * indices.element_size() if hasattr(indices, "numel") else 0
    elif len(args) == 6:
        alpha, desc_x, buf_x, beta, desc_y, buf_y = args
        ws, ws_bytes = None, 0
    else:
        raise TypeError("reduce_tensor takes 6 or 8 arguments after the descriptor")
    dx, dy = desc(desc_x), desc(desc_y)
    a, b = _scalar(alpha, dx.dtype_code), _scalar(beta, dy.dtype_code)
    check(lib.ddReduceTensor(handle.ptr, rtd.ptr, ind, ind_bytes, ws, ws_bytes, ctypes.byref(a), dx.ptr,
                             _ptr(buf_x), ctypes.byref(b), dy.ptr, _ptr(buf_y)), handle.ptr,
          "ddReduceTensor")
    return handle


def convolution_bwd_bias(handle, alpha, desc_dy, buf_dy, beta, desc_db, buf_db):
    """``convolution-bwd-bias`` (cudnn/core.clj:344-350): db = alpha * sum(dy over N,H,W) + beta * db."""
    ddy, ddb = desc(desc_dy), desc(desc_db)
    a, b = _scalar(alpha, ddy.dtype_code), _scalar(beta, ddb.dtype_code)
    check(lib.ddConvolutionBackwardBias(handle.ptr, ctypes.byref(a), ddy.ptr, _ptr(buf_dy), ctypes.byref(b),
                                        ddb.ptr, _ptr(buf_db)), handle.ptr, "ddConvolutionBackwardBias")
    return handle


def data_type_width(dt):
    """``data-type-width`` (cudnn/constants.clj:126-148)."""
    return DATA_TYPE_WIDTH[enc_keyword(DATA_TYPE, dt, "data type") if not isinstance(dt, int) else dt]


__all__ = [n for n in dir() if not n.startswith("_")] + ["_lib"]
