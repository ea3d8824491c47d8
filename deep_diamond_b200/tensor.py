"""Public tensor API -- the counterpart of the reference's
deep-diamond-base/src/uncomplicate/diamond/tensor.clj (``desc tensor transformer connector batcher
shuffler view-tz offset! with-diamond *diamond-factory*``, :61-83, :211-400) plus the handful of
Neanderthal generics the reference's tensor tests call on tensors (``transfer! asum nrm2 entry!
view-vctr native dim zero``).  Function names are the reference's in snake_case (``offset!`` ->
``offset_``, ``transfer!`` -> ``transfer``, ``entry!`` -> ``entry_``); keywords are strings.
"""
import contextlib

import numpy as np

from . import factory as _f
from ._lib import DiamondError
from .constants import default_strides

_diamond_factory = None  # *diamond-factory* (:61-72)


def diamond_factory():
    return _diamond_factory


def set_diamond_factory(fact):
    global _diamond_factory
    _diamond_factory = fact
    return fact


@contextlib.contextmanager
def with_diamond(factory_fn, *params):
    """``with-diamond`` (:74-83): binds a fresh factory for the body and releases it after."""
    global _diamond_factory
    prev = _diamond_factory
    _diamond_factory = factory_fn(*params)
    try:
        yield _diamond_factory
    finally:
        _diamond_factory.release()
        _diamond_factory = prev


class TensorDescriptorImpl:
    """General, technology-agnostic descriptor (``TensorDescriptorImpl``, :164-209)."""

    def __init__(self, shape, data_type=None, layout=None):
        self.shape = list(shape)
        self.data_type = data_type
        self.layout = layout if layout is None or isinstance(layout, str) else list(layout)

    def __eq__(self, other):
        return (isinstance(other, TensorDescriptorImpl) and self.shape == other.shape
                and self.data_type == other.data_type and self.layout == other.layout)

    __hash__ = None

    def __repr__(self):
        return "{:shape %s, :data-type %s, :layout %s}" % (self.shape, self.data_type, self.layout)

    def connector(self, out):
        return connector(output(out).diamond_factory().create_tensor_desc(self), out)


def desc(shape, type=None, layout=None):  # noqa: A002 - the reference's parameter name
    """``desc`` (:211-248).  ``desc(shape, layout)`` and ``desc(tdesc)`` arities included."""
    if not isinstance(shape, (list, tuple)):
        return desc(_f._shape_of(shape), _dtype_name(shape), _f._layout_of(shape))
    if layout is None and type is not None and (isinstance(type, (list, tuple)) or
                                                (isinstance(type, str) and _looks_like_layout(type, shape))):
        type, layout = None, type
    ok_layout = (layout is None or (isinstance(layout, str) and len(layout) == len(shape))
                 or (isinstance(layout, (list, tuple)) and len(layout) == len(shape)))
    if not ok_layout:
        raise DiamondError("The requested descriptor would most likely be inconsistent.",
                           {"shape": list(shape), "type": type, "layout": layout})
    return TensorDescriptorImpl(shape, type, layout)


def _looks_like_layout(word, shape):
    from .constants import DATA_TYPE
    return word not in DATA_TYPE


def _dtype_name(x):
    dt = _f._dtype_of(x)
    if isinstance(dt, int):
        from .constants import DATA_TYPE_NAME
        return DATA_TYPE_NAME[dt]
    return dt


def default_desc(shape, type=None):  # noqa: A002
    """``default-desc`` (:250-257)."""
    if not isinstance(shape, (list, tuple)):
        return default_desc(_f._shape_of(shape), _dtype_name(shape))
    return desc(list(shape), type, default_strides(shape))


def shape(x):
    return _f._shape_of(x)


def layout(x):
    return _f._layout_of(x)


def data_type(x):
    return _dtype_name(x)


def _is_factory(x):
    return hasattr(x, "create_tensor")


def tensor(*args):
    """``tensor`` (:259-307): (fact shape type layout [batch-index]) | (shape type layout) |
    (fact desc) | (desc)."""
    if args and _is_factory(args[0]):
        fact, rest = args[0].diamond_factory(), args[1:]
    else:
        fact, rest = _diamond_factory, args
    if fact is None:
        raise DiamondError("No diamond factory is bound.", {})
    if len(rest) == 1:
        d = rest[0]
        lay = _f._layout_of(d)
        bi = 1 if isinstance(lay, str) and "t" in lay else 0
        return fact.create_tensor(fact.create_tensor_desc(d), bi, True)
    shp, typ, lay = rest[0], rest[1], rest[2]
    if len(rest) > 3:
        bi = int(rest[3])
    else:
        bi = 1 if isinstance(lay, str) and "t" in lay else 0
    if not (isinstance(shp, (list, tuple)) and 0 <= bi <= len(shp) - 1):
        raise DiamondError("Incompatible tensor constructor arguments.",
                           {"shape": type(shp).__name__, "batch-index": bi})
    if any(int(d) < 0 for d in shp):
        raise DiamondError("Tensor dimensions must not be negative.", {"shape": list(shp)})
    return fact.create_tensor(fact.create_tensor_desc(list(shp), typ, lay), bi, True)


def offset_(tz, n):
    """``offset!`` (:309-312)."""
    return tz.offset(int(n))


def transformer(x, y):
    """``transformer`` (:314-336)."""
    return x.diamond_factory().create_transformer(x, y)


def batch_size(x):
    """``batch-size`` (:338-344)."""
    return _f._shape_of(x)[x.batch_index()]


def batcher(x, y, mb_size=None):
    """``batcher`` (:346-373)."""
    if mb_size is None:
        mb_size = min(batch_size(x), batch_size(y))
    return x.diamond_factory().create_batcher(x, y, int(mb_size))


def shuffler(x, y):
    """``shuffler`` (:375-400)."""
    return x.diamond_factory().create_shuffler(x, y)


def input(x):  # noqa: A001 - the reference's name
    return x.input()


def output(x):
    return x.output()


def revert(x):
    return x.revert()


def view_tz(x, sub=None):
    return x.view_tz(sub)


def connector(in_, out):
    """``connector`` of ConnectorCreator (:145-160, :207-209; cudnn/tensor.clj:104-113,498-503).
    Either side may be a tensor (or a transfer) or a descriptor / layout keyword."""
    if isinstance(in_, str):  # a layout keyword on the input side (:150-160)
        in_out = input(out)
        fact = in_out.diamond_factory()
        in_desc = fact.create_tensor_desc(in_out.shape, in_out.desc.dtype_code, in_)
        if in_desc.strides == in_out.layout:
            return output(out).view()
        in_tz = fact.create_tensor(in_desc, output(out).batch_index(), False)
        return fact.create_transformer(in_tz, output(out).view())
    if hasattr(in_, "connector") and not isinstance(in_, TensorDescriptorImpl):
        return in_.connector(out)  # tensor / transformer / batcher on the input side
    # descriptor on the input side, tensor-like on the output side
    out_tz = output(out)
    fact = out_tz.diamond_factory()
    in_desc = fact.create_tensor_desc(in_)
    if in_desc == input(out).desc:
        return out.view()
    if in_desc == out_tz.desc:
        return out_tz.view()
    in_tz = fact.create_tensor(in_desc, out_tz.batch_index(), False)
    return fact.create_transformer(in_tz, out_tz.view())


# ---------------------------------------------------------------- Neanderthal generics --------

def transfer(source, destination):
    """``transfer!``: see factory.transfer; vector views of device tensors stand for their tensor."""
    src = source.tz if isinstance(source, VectorView) else source
    if isinstance(destination, VectorView):
        _f.transfer(src, destination.tz)
        return destination
    return _f.transfer(src, destination)



def transfer_async(source, destination):
    """``transfer`` on the factory's copy streams: returns a ``Pending`` (see factory.transfer_async)."""
    src = source.tz if isinstance(source, VectorView) else source
    dst = destination.tz if isinstance(destination, VectorView) else destination
    return _f.transfer_async(src, dst)


def native(x):
    if isinstance(x, (_f.HostTensor, np.ndarray, list)):
        return x
    if isinstance(x, VectorView):
        return native(x.tz).storage
    return x.host()


host = native


def dim(x):
    return x.dim() if hasattr(x, "dim") else len(x)


def zero(x):
    return x.zero()


def raw(x):
    return x.raw()


def contiguous(x):
    """``contiguous?``"""
    return x.is_contiguous()


def buffer(x):
    return x.buffer()


def release(x):
    return x.release()


class VectorView:
    """``view-vctr`` of a device tensor: the storage seen as a flat vector (contiguous tensors only,
    cudnn/tensor.clj:472-474 with ``check-contiguous``)."""

    def __init__(self, tz):
        if not tz.is_contiguous():
            raise DiamondError("This operation is supported only on contiguous tensors. "
                               "Please use a copy or create a transformer.", {"x": repr(tz)})
        self.tz = tz

    def dim(self):
        return self.tz.nc

    def __eq__(self, other):
        if isinstance(other, VectorView):
            a, b = native(self), native(other)
            return a.dtype == b.dtype and np.array_equal(a, b)
        return NotImplemented

    __hash__ = None


def view_vctr(x):
    if isinstance(x, _f.HostTensor):
        return x.storage
    if isinstance(x, np.ndarray):
        return x.reshape(-1)
    return VectorView(x)


def vctr(like, values):
    """A host vector of `like`'s data type holding `values` (Neanderthal's ``vctr``)."""
    code = like.desc.dtype_code if hasattr(like, "desc") else like.dtype_code
    return _f._encode(np.asarray(values, dtype=np.float64), code)


def entry(v, i):
    if isinstance(v, VectorView):
        return float(native(v)[i])
    if isinstance(v, _f.HostTensor):
        return v.values()[i]
    return float(v[i])


def entry_(x, value):
    """``entry!``: set all entries."""
    tz = x.tz if isinstance(x, VectorView) else x
    tz.fact.set_all(value, tz)
    return x


def _tz(x):
    return x.tz if isinstance(x, VectorView) else x


def asum(x):
    if isinstance(x, _f.HostTensor):
        return float(np.abs(np.asarray(x.values(), dtype=np.float64)).sum())
    if isinstance(x, np.ndarray):
        return float(np.abs(x.astype(np.float64)).sum())
    return _tz(x).fact.asum(_tz(x))


def nrm2(x):
    if isinstance(x, (_f.HostTensor, np.ndarray)):
        v = np.asarray(x.values() if isinstance(x, _f.HostTensor) else x, dtype=np.float64)
        return float(np.sqrt((v * v).sum()))
    return _tz(x).fact.nrm2(_tz(x))


def amax(x):
    return _tz(x).fact.amax(_tz(x))


def sum(x):  # noqa: A001
    return _tz(x).fact.sum(_tz(x))


def axpy(alpha, x, y):
    """``axpy!``: y = alpha*x + y (x may broadcast along dims of extent 1)."""
    return _tz(y).fact.axpy(alpha, _tz(x), _tz(y))


def axpby(alpha, x, beta, y):
    return _tz(y).fact.axpby(alpha, _tz(x), beta, _tz(y))


def scal(alpha, x):
    """``scal!``"""
    return _tz(x).fact.scal(alpha, _tz(x))


def copy(x, y):
    """``copy!``"""
    return _tz(y).fact.copy(_tz(x), _tz(y))
