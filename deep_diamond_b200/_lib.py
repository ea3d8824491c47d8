"""ctypes binding of libdd_b200.so -- the counterpart of the reference's raw FFI layer
(deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/impl.clj: one function per C
call plus ``with-check``, impl.clj:30-41).

The library must have been built (``python deep_diamond_b200/build.py``); importing this module
without it raises: there is no fallback path.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# DD_B200_LIBRARY names another build of the same library (e.g. the `--tune` build of build.py)
LIB_PATH = os.environ.get("DD_B200_LIBRARY") or os.path.join(_HERE, "libdd_b200.so")


class DiamondError(RuntimeError):
    """The analogue of the reference's ``ex-info`` with ``{:type :code}`` (cudnn/impl.clj:30-33,
    ``dragan-says-ex``)."""

    def __init__(self, message, data=None):
        super().__init__(message if not data else "%s %s" % (message, data))
        self.data = dict(data or {})


STATUS = {
    0: "success", 1: "not-initialized", 2: "alloc-failed", 3: "bad-param", 4: "internal-error",
    5: "invalid-value", 6: "arch-mismatch", 7: "mapping-error", 8: "execution-failed",
    9: "not-supported", 10: "timeout", 11: "comm-failed",
}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "libdd_b200.so is missing at %s: build it with `python deep_diamond_b200/build.py` "
        "(there is no CPU or library fallback for these ops)" % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

_vp = ctypes.c_void_p
_i64p = ctypes.POINTER(ctypes.c_int64)
_int = ctypes.c_int
_i64 = ctypes.c_int64
_dbl = ctypes.c_double
_sz = ctypes.c_size_t

_SIGS = {
    "ddCreate": [ctypes.POINTER(_vp)],
    "ddDestroy": [_vp],
    "ddSetStream": [_vp, _vp],
    "ddGetStream": [_vp, ctypes.POINTER(_vp)],
    "ddGetLaunchCount": [_vp, ctypes.POINTER(ctypes.c_uint64)],
    "ddCreateTensorDescriptor": [ctypes.POINTER(_vp)],
    "ddDestroyTensorDescriptor": [_vp],
    "ddSetTensor4dDescriptor": [_vp, _int, _int, _i64, _i64, _i64, _i64],
    "ddSetTensor4dDescriptorEx": [_vp, _int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64],
    "ddSetTensorNdDescriptor": [_vp, _int, _int, _i64p, _i64p],
    "ddSetTensorNdDescriptorEx": [_vp, _int, _int, _int, _i64p],
    "ddGetTensorNdDescriptor": [_vp, _int, ctypes.POINTER(_int), ctypes.POINTER(_int), _i64p, _i64p],
    "ddGetTensorSizeInBytes": [_vp, ctypes.POINTER(_sz)],
    "ddSetTensor": [_vp, _vp, _vp, _vp],
    "ddScaleTensor": [_vp, _vp, _vp, _vp],
    "ddAddTensor": [_vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "ddOpTensor": [_vp, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "ddSumTensors": [_vp, _int, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(_vp),
                     ctypes.POINTER(_vp), _vp, _vp],
    "ddTransformTensor": [_vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "ddGatherTransform": [_vp, _int, _i64p, _i64p, _vp, _vp, _vp, _vp],
    "ddTensorEquals": [_vp, _vp, _vp, _vp, _vp, _vp],
    "ddMultiTransform": [_vp, _int, ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(_vp),
                         ctypes.POINTER(_vp)],
    "ddCostDiff": [_vp, _int, _vp, _vp, _vp, _vp, _vp],
    "ddCreateActivationDescriptor": [ctypes.POINTER(_vp)],
    "ddDestroyActivationDescriptor": [_vp],
    "ddSetActivationDescriptor": [_vp, _int, _int, _dbl],
    "ddSetActivationDescriptorEx": [_vp, _int, _int, _dbl, _dbl],
    "ddGetActivationDescriptor": [_vp, ctypes.POINTER(_int), ctypes.POINTER(_int),
                                  ctypes.POINTER(_dbl)],
    "ddActivationForward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "ddActivationBackward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "ddCreateReduceTensorDescriptor": [ctypes.POINTER(_vp)],
    "ddDestroyReduceTensorDescriptor": [_vp],
    "ddSetReduceTensorDescriptor": [_vp, _int, _int, _int],
    "ddSetReduceTensorDescriptorLp": [_vp, _int, _int, _int, ctypes.c_double, ctypes.c_double],
    "ddGetReduceTensorDescriptorLp": [_vp, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)],
    "ddSetReduceTensorDescriptorIndices": [_vp, _int],
    "ddGetReduceTensorDescriptor": [_vp, ctypes.POINTER(_int), ctypes.POINTER(_int),
                                    ctypes.POINTER(_int)],
    "ddGetReductionIndicesSize": [_vp, _vp, _vp, _vp, ctypes.POINTER(_sz)],
    "ddGetReductionWorkspaceSize": [_vp, _vp, _vp, _vp, ctypes.POINTER(_sz)],
    "ddReduceTensor": [_vp, _vp, _vp, _sz, _vp, _sz, _vp, _vp, _vp, _vp, _vp, _vp],
    "ddConvolutionBackwardBias": [_vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "ddReduceTensorNoAlloc": [_vp, _int, _int, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_char_p, _sz],
    "ddShardedGetUniqueId": [_vp],
    "ddShardedCreate": [ctypes.POINTER(_vp), _vp, _int, _int, _vp],
    "ddShardedDestroy": [_vp],
    "ddShardedReduceTensor": [_vp, _vp, _int, _i64, _vp, _vp, _vp, _vp, _vp, _vp],
    "ddShardedPeerDetach": [_vp],
    "ddShardedSetJoinLimit": [_dbl],
    "ddResetCounters": [_vp],
    "ddGetDeviceFault": [_vp, ctypes.POINTER(ctypes.c_int)],
    "ddShardedCheck": [_vp],
    "ddShardedPeerExport": [_vp, _vp],
    "ddShardedPeerAttach": [_vp, _vp],
    "ddShardedPeerConfigure": [_vp, _int, _dbl],
    "ddShardedPeerStatus": [_vp, ctypes.POINTER(_int)],
}
for _name, _args in _SIGS.items():
    _f = getattr(lib, _name)
    _f.argtypes = _args
    _f.restype = _int
lib.ddGetErrorString.argtypes = [_int]
lib.ddGetErrorString.restype = ctypes.c_char_p
lib.ddGetLastErrorMessage.argtypes = [_vp]
lib.ddGetLastErrorMessage.restype = ctypes.c_char_p
lib.ddGetLastKernelName.argtypes = [_vp]
lib.ddGetLastKernelName.restype = ctypes.c_char_p
lib.ddGetVersion.argtypes = []
lib.ddGetVersion.restype = _sz

EXPORTS = sorted(list(_SIGS) + ["ddGetErrorString", "ddGetLastErrorMessage", "ddGetLastKernelName",
                                "ddGetVersion"])


def check(status, handle=None, what=""):
    """``with-check``: turns a non-zero status into DiamondError carrying {type, code}."""
    if status != 0:
        name = lib.ddGetErrorString(status).decode()
        detail = lib.ddGetLastErrorMessage(handle).decode() if handle else ""
        raise DiamondError("%s failed: %s%s" % (what or "libdd_b200 call", name,
                                                 (" (" + detail + ")") if detail else ""),
                           {"type": STATUS.get(status, "unknown"), "code": status})
    return status
