"""The B200 backend objects: factory, tensor, transformer, batcher, shuffler and the tensor engine.

Mirrors, type for type, the reference's cuDNN backend
  deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/tensor.clj   (CUDnnTensor :332-533,
      CUDnnTransformer :158-207, CUDnnBatcher :211-279, CUDnnShuffler :281-328, transfer! :542-625)
  deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/factory.clj  (TensorEngine :161-322,
      CUDnnFactory :324-431)
with every cuDNN / Neanderthal-CUDA call replaced by a libdd_b200 call.  PyTorch supplies device
memory, streams and host<->device copies only.
"""
import itertools

import numpy as np
import torch

from . import core
from ._lib import DiamondError
from .constants import DATA_TYPE, DATA_TYPE_NAME, DATA_TYPE_WIDTH, NUMPY_TYPE, default_strides, enc_keyword

DOES_NOT_FIT_MSG = "Source and destination shapes have to fit."


def _span(shape, strides):
    return 1 + sum((d - 1) * s for d, s in zip(shape, strides))


# ====================== Host mirror ==============================================

class HostTensor:
    """A host-side mirror: raw storage (numpy) plus the descriptor it was read under.  Stands where
    the reference hands out a DNNL tensor from ``native`` (cudnn/tensor.clj:396-401).  Iterating it
    yields the storage in memory order, which is what ``(seq (native tz))`` does there."""

    def __init__(self, shape, data_type, strides, storage=None):
        self.shape = [int(d) for d in shape]
        self.dtype_code = enc_keyword(DATA_TYPE, data_type, "data type") if not isinstance(data_type, int) else data_type
        self.data_type = DATA_TYPE_NAME[self.dtype_code]
        self.layout = [int(s) for s in strides]
        n = _span(self.shape, self.layout) if all(d > 0 for d in self.shape) else 0
        self.storage = np.zeros(n, dtype=NUMPY_TYPE[self.dtype_code]) if storage is None else storage

    def __iter__(self):
        return iter(self.values())

    def __len__(self):
        return len(self.storage)

    def __getitem__(self, i):
        return self.values()[i]

    def values(self):
        """Storage as Python numbers (bf16 decoded to float)."""
        if self.dtype_code == 9:
            return (self.storage.astype(np.uint32) << 16).view(np.float32).tolist()
        return self.storage.tolist()

    def logical(self):
        """The tensor as a numpy view of logical shape (strided, no copy)."""
        item = self.storage.dtype.itemsize
        return np.lib.stride_tricks.as_strided(self.storage, shape=tuple(self.shape),
                                               strides=tuple(s * item for s in self.layout))

    def __eq__(self, other):
        return (isinstance(other, HostTensor) and self.shape == other.shape
                and self.dtype_code == other.dtype_code and self.layout == other.layout
                and np.array_equal(self.storage, other.storage))

    __hash__ = None

    def __repr__(self):
        return "{:shape %s :data-type :%s :layout %s} %s" % (self.shape, self.data_type, self.layout,
                                                             self.values()[:16])


class ZeroDescriptor:
    """Descriptor of a tensor with a zero extent.  The C library (like cuDNN) only takes positive
    extents, so such tensors never reach it: the reference keeps a general descriptor for them too
    (cudnn/tensor.clj:119-122) and turns their transformers into no-ops (:204-207)."""

    ptr = None

    def __init__(self, shape, dtype_code, strides):
        self.dims, self.dtype_code, self.strides = [int(d) for d in shape], dtype_code, [int(s) for s in strides]
        self.data_type = DATA_TYPE_NAME[dtype_code]

    shape = property(lambda self: list(self.dims))
    layout = property(lambda self: list(self.strides))

    def __eq__(self, other):
        return (isinstance(other, ZeroDescriptor) and self.dims == other.dims
                and self.dtype_code == other.dtype_code and self.strides == other.strides)

    __hash__ = None

    def view(self):
        return self

    def release(self):
        return True


# ====================== Tensor ==================================================

class B200Tensor:
    """Device tensor: one CUDA buffer + a descriptor (``CUDnnTensor``, cudnn/tensor.clj:332-503).

    `alloc` is the torch uint8 tensor that owns (or shares) the memory; `base` is the byte offset of
    this tensor's origin inside it and `position` the element offset set by ``offset!``."""

    def __init__(self, fact, alloc, base, capacity, tdesc, n_index, master):
        self.fact = fact
        self.alloc = alloc
        self.base = int(base)
        self.capacity = int(capacity)  # elements available from `base`
        self.position = 0
        self.desc = tdesc
        self.nc = int(np.prod(tdesc.dims)) if tdesc.dims else 0
        self.n_index = int(n_index)
        self.master = master
        self.width = DATA_TYPE_WIDTH[tdesc.dtype_code]
        self.storage_elems = _span(tdesc.dims, tdesc.strides) if self.nc > 0 else 0

    # --- protocols ---------------------------------------------------------------
    @property
    def shape(self):
        return list(self.desc.dims)

    @property
    def data_type(self):
        return self.desc.data_type

    @property
    def layout(self):
        return list(self.desc.strides)

    def batch_index(self):
        return self.n_index

    def diamond_factory(self):
        return self.fact

    def device(self):
        return "cuda"

    def dim(self):
        return self.nc

    def device_ptr(self):
        return self.alloc.data_ptr() + self.base + self.position * self.width

    def buffer(self):
        """Identity of the underlying memory at the current offset (tests compare buffers)."""
        return self.device_ptr()

    def is_contiguous(self):
        """``isContiguous`` (:419-420): as many logical entries as storage entries."""
        return self.nc == self.storage_elems

    def info(self):
        return {"data-type": self.data_type, "class": type(self).__name__, "device": "cuda",
                "shape": self.shape, "strides": self.layout, "master": self.master}

    def release(self):
        self.alloc = None
        return True

    # Transfer / Revert / IFn: a tensor is its own input and output
    def input(self):
        return self

    def output(self):
        return self

    def diff_input(self):
        return self

    def diff_output(self):
        return self

    def revert(self):
        return self

    def __call__(self):
        return self

    def view(self):
        """``view`` (:470-471): same memory at the current offset, not a master."""
        return B200Tensor(self.fact, self.alloc, self.base + self.position * self.width,
                          self.capacity - self.position, self.desc.view(), self.n_index, False)

    def view_tz(self, sub=None):
        """``view-tz`` (:476-490): a sub-tensor over the same memory.  `sub` is a batch count, a
        shape, or a descriptor (shape + optional data type and strides)."""
        if sub is None:
            return self
        if isinstance(sub, (int, np.integer)):
            dims = list(self.desc.dims)
            dims[self.n_index] = int(sub)
            sub_desc = core.tensor_descriptor(dims, self.desc.dtype_code, self.desc.strides)
        else:
            shp = _shape_of(sub)
            dt = _dtype_of(sub)
            dt = self.desc.dtype_code if dt is None else dt
            lay = _layout_of(sub)
            sub_desc = core.tensor_descriptor(shp, dt, lay if lay is not None else self.desc.strides)
        need = _span(sub_desc.dims, sub_desc.strides) * DATA_TYPE_WIDTH[sub_desc.dtype_code]
        avail = (self.capacity - self.position) * self.width
        if need > avail:
            raise DiamondError("Insufficient buffer size.", {"desc-size": need, "buffer-size": avail})
        w = DATA_TYPE_WIDTH[sub_desc.dtype_code]
        return B200Tensor(self.fact, self.alloc, self.base + self.position * self.width,
                          avail // w, sub_desc, self.n_index, False)

    def offset(self, ofst):
        """``offset`` of the Offset protocol (:491-497): moves the tensor's origin."""
        ofst = int(ofst)
        if not 0 <= ofst <= self.capacity:
            raise DiamondError("There isn't enough capacity in the underlying buffer for this offset.",
                               {"requested": ofst, "available": self.capacity})
        self.position = ofst
        return self

    def connector(self, out_desc):
        """``connector`` (:498-503): a view if the descriptors agree, else allocate + transformer."""
        od = self.fact.create_tensor_desc(out_desc)
        if core.equal_desc(self.desc, od):
            return self.view()
        out_tz = self.fact.create_tensor(od, self.n_index, False)
        return B200Transformer(self.fact.handle, self.view(), out_tz)

    # Container
    def raw(self, fact=None):
        f = (fact or self.fact)
        return f.create_tensor(f.create_tensor_desc(self.shape, self.desc.dtype_code, default_strides(self.shape)),
                               self.n_index, False)

    def zero(self, fact=None):
        f = (fact or self.fact)
        return f.create_tensor(f.create_tensor_desc(self.shape, self.desc.dtype_code, default_strides(self.shape)),
                               self.n_index, True)

    def host(self):
        """``host``/``native`` (:396-401): storage copied to the host under the same descriptor."""
        return self.fact.download(self)

    native = host

    def __eq__(self, other):
        """``equals`` (:336-340): equal descriptors, both contiguous, equal contents."""
        if other is self:
            return True
        if not isinstance(other, B200Tensor):
            return False
        if not core.equal_desc(self.desc, other.desc):
            return False
        if not (self.is_contiguous() and other.is_contiguous()):
            return False
        return self.fact.equals_block(self, other)

    __hash__ = None

    def __repr__(self):
        return "{:shape %s :data-type :%s :layout %s}" % (self.shape, self.data_type, self.layout)


def _shape_of(x):
    if isinstance(x, (list, tuple)):
        return [int(d) for d in x]
    if isinstance(x, dict):
        return list(x.get("shape", []))
    s = x.shape
    return list(s() if callable(s) else s)


def _dtype_of(x):
    if isinstance(x, (list, tuple)):
        return None
    if isinstance(x, dict):
        return x.get("data-type")
    if hasattr(x, "desc") and hasattr(x.desc, "dtype_code"):
        return x.desc.dtype_code
    if hasattr(x, "dtype_code"):
        return x.dtype_code
    return getattr(x, "data_type", None)


def _layout_of(x):
    if isinstance(x, (list, tuple)):
        return None
    if isinstance(x, dict):
        return x.get("layout") or x.get("format") or x.get("strides")
    return getattr(x, "layout", None)


# ====================== Transformer =============================================

class NoOpTransformer:
    """For zero-sized tensors (base/internal/common.clj:49-89)."""

    def __init__(self, in_tz, out_tz):
        self.in_tz, self.out_tz = in_tz, out_tz

    def input(self):
        return self.in_tz

    def output(self):
        return self.out_tz

    def __call__(self, *_):
        return self.out_tz

    def release(self):
        return True


class B200Transformer:
    """``CUDnnTransformer`` (:158-207): invoking it reorders/convert-copies input into output."""

    def __init__(self, hdl, in_tz, out_tz):
        self.hdl, self.in_tz, self.out_tz = hdl, in_tz, out_tz

    def release(self):
        self.in_tz.release()
        self.out_tz.release()
        return True

    def __eq__(self, other):
        return other is self or (isinstance(other, B200Transformer)
                                 and self.in_tz.shape == other.in_tz.shape and self.out_tz == other.out_tz)

    __hash__ = None

    def revert(self):
        return B200Transformer(self.hdl, self.out_tz.view(), self.in_tz.view())

    def view(self):
        return B200Transformer(self.hdl, self.in_tz.view(), self.out_tz.view())

    def input(self):
        return self.in_tz

    def output(self):
        return self.out_tz

    def __call__(self, hdl2=None):
        core.transform_tensor(hdl2 or self.hdl, 1.0, self.in_tz.desc, self.in_tz, 0.0,
                              self.out_tz.desc, self.out_tz)
        return self.out_tz

    def connector(self, out_desc):
        od = self.out_tz.fact.create_tensor_desc(out_desc)
        if core.equal_desc(self.out_tz.desc, od):
            return self
        return self.in_tz.connector(od)


def b200_transformer(hdl, in_tz, out_tz):
    if any(d == 0 for d in in_tz.shape) and any(d == 0 for d in out_tz.shape):
        return NoOpTransformer(in_tz, out_tz)
    return B200Transformer(hdl, in_tz, out_tz)


# ====================== Batcher / Shuffler ======================================

class B200Batcher:
    """``CUDnnBatcher`` (:211-279): copies mini-batch `src_n` of the source into slot `dst_n` of the
    destination (sub-tensors along the batch dim, any layouts and data types)."""

    def __init__(self, hdl, src_tz, dst_tz, mb_size):
        self.hdl = hdl
        self.mb_size = max(1, int(mb_size))
        self.src_tz, self.dst_tz = src_tz, dst_tz
        self.src_sub = src_tz.view_tz(self.mb_size)
        self.dst_sub = dst_tz.view_tz(self.mb_size)
        self.src_cnt = src_tz.shape[src_tz.n_index]
        self.src_stride_n = self.src_sub.layout[src_tz.n_index]
        self.dst_cnt = dst_tz.shape[dst_tz.n_index]
        self.dst_stride_n = self.dst_sub.layout[dst_tz.n_index]

    def release(self):
        return True

    def view(self):
        return B200Batcher(self.hdl, self.src_tz.view(), self.dst_tz.view(), self.mb_size)

    def input(self):
        return self.src_tz

    def output(self):
        return self.dst_tz

    def check(self, src_n, dst_n):
        if not (0 <= src_n <= self.src_cnt - self.mb_size and 0 <= dst_n <= self.dst_cnt - self.mb_size):
            raise DiamondError("Requested subtensor is outside of bounds.",
                               {"src-index": src_n, "src-cnt": self.src_cnt, "dst-index": dst_n,
                                "dst-cnt": self.dst_cnt, "mb-size": self.mb_size})

    def __call__(self, src_n=0, dst_n=0, hdl2=None):
        src_n, dst_n = int(src_n), int(dst_n)
        self.check(src_n, dst_n)
        self.src_sub.offset(self.src_stride_n * src_n)
        self.dst_sub.offset(self.dst_stride_n * dst_n)
        core.transform_tensor(hdl2 or self.hdl, 1.0, self.src_sub.desc, self.src_sub, 0.0,
                              self.dst_sub.desc, self.dst_sub)
        return self.dst_tz

    def connector(self, dst_desc):
        od = self.dst_tz.fact.create_tensor_desc(dst_desc)
        if core.equal_desc(self.dst_tz.desc, od):
            return self
        return self.dst_tz.connector(od)


class B200Shuffler:
    """``CUDnnShuffler`` (:281-328).  The reference runs one single-sample batcher call per column;
    here all columns of an invocation go out as ONE gather launch."""

    def __init__(self, hdl, src_tz, dst_tz):
        self.hdl = hdl
        self.batcher = B200Batcher(hdl, src_tz, dst_tz, 1)
        self.batch_size = src_tz.shape[src_tz.n_index]
        self.mb_size = dst_tz.shape[dst_tz.n_index]

    def release(self):
        return True

    def view(self):
        return B200Shuffler(self.hdl, self.batcher.src_tz.view(), self.batcher.dst_tz.view())

    def input(self):
        return self.batcher.input()

    def output(self):
        return self.batcher.output()

    def __call__(self, cols=None, hdl2=None):
        b = self.batcher
        if cols is None:
            cols = [int(v) for v in np.random.randint(0, self.batch_size, size=self.mb_size)]
        cols = [int(c) for c in cols]
        for dst_n, src_n in enumerate(cols):
            b.check(src_n, dst_n)
        if cols:
            b.src_sub.offset(0)
            b.dst_sub.offset(0)
            core.gather_transform(hdl2 or self.hdl, [b.src_stride_n * c for c in cols],
                                  [b.dst_stride_n * i for i in range(len(cols))],
                                  b.src_sub.desc, b.src_sub, b.dst_sub.desc, b.dst_sub)
        return self.output()

    def connector(self, dst_desc):
        return self.batcher.connector(dst_desc)


# ====================== Factory =================================================

class Pending:
    """A host<->device copy in flight on one of the factory's copy streams (``transfer_async``)."""

    def __init__(self, fact, event, result):
        self.fact, self.event, self.result = fact, event, result

    def wait(self):
        """Blocks the host until the copy has finished; returns what was copied into."""
        if self.event is not None:
            self.event.synchronize()
        return self.result

    def done(self):
        return self.event is None or self.event.query()

    def before_overwrite(self):
        """Makes the factory's stream wait for this copy without blocking the host: call it right
        before the call that overwrites the SOURCE of a device -> host copy (uploads issued after
        it wait too, since an upload starts behind what the factory's stream holds)."""
        if self.event is not None:
            self.fact.stream.wait_event(self.event)
        return self


class CapturedCalls:
    """A CUDA graph of library calls on a factory's tensors (see ``B200Factory.capture``).  The capture
    runs on a side stream the factory's handle is switched to for its duration; replays are enqueued
    on the factory's own stream, in order with everything else on it."""

    def __init__(self, fact, fn, warmup=1):
        self.fact = fact
        side = torch.cuda.Stream(device=fact.device)
        side.wait_stream(fact.stream)
        fact.handle.set_stream(side)
        try:
            with torch.cuda.stream(side):
                for _ in range(max(0, int(warmup))):
                    fn()
                side.synchronize()
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, stream=side):
                    fn()
        finally:
            fact.handle.set_stream(fact.stream)
        fact.stream.wait_stream(side)

    def __call__(self):
        with torch.cuda.stream(self.fact.stream):
            self.graph.replay()
        return self

    def release(self):
        self.graph = None
        return True


class B200Factory:
    """``CUDnnFactory`` (cudnn/factory.clj:324-431): creates descriptors, tensors, transformers,
    batchers, shufflers and layer blueprints, and carries the tensor engine (:161-322)."""

    def __init__(self, device=None, stream=None):
        if not torch.cuda.is_available():
            raise DiamondError("The B200 factory needs a CUDA device; there is no CPU fallback.",
                               {"type": "not-initialized"})
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        torch.cuda.set_device(self.device)
        self.stream = stream if stream is not None else torch.cuda.current_stream(self.device)
        self.handle = core.Handle(self.stream)
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._scalar = torch.zeros(2, dtype=torch.float64, device=self.device)
        self._reduce_desc = {}
        self._h2d = self._d2h = None   # copy streams of transfer_async, made on first use
        self.master = True

    # DiamondFactoryProvider / FlowProvider
    def diamond_factory(self):
        return self

    def native_diamond_factory(self):
        return HOST_FACTORY

    def flow(self):
        return self.stream

    def release(self):
        for r in self._reduce_desc.values():
            r.release()
        self._reduce_desc = {}
        if self.handle is not None:
            self.handle.release()
            self.handle = None
        return True

    def synchronize(self):
        self.stream.synchronize()

    def capture(self, fn, warmup=1):
        """Records the library calls `fn` makes (layer forwards / backwards, transformers, reductions
        on fixed tensors) into a CUDA graph and returns a ``CapturedCalls`` whose call replays them
        with one launch.  A Python + ctypes call costs 10-20 us of host time, more than the smaller
        kernels run; a replayed graph keeps a chain of them launch-bound no longer.  `fn` must only
        enqueue work on this factory (no host reads, no allocation of new tensors)."""
        return CapturedCalls(self, fn, warmup)

    # TensorFactory (base/internal/protocols.clj:36-52)
    def create_tensor_desc(self, shape, dtype=None, fmt=None):
        if dtype is None and fmt is None and not isinstance(shape, (list, tuple)):
            tdesc = shape
            if isinstance(tdesc, (core.TensorDescriptor, ZeroDescriptor)):
                return tdesc
            if hasattr(tdesc, "desc") and isinstance(tdesc.desc, (core.TensorDescriptor, ZeroDescriptor)):
                return tdesc.desc
            shape, dtype, fmt = _shape_of(tdesc), _dtype_of(tdesc), _layout_of(tdesc)
        shape = [int(d) for d in shape]
        if any(d < 0 for d in shape):
            raise DiamondError("Tensor dimensions must not be negative.", {"shape": shape})
        if any(d == 0 for d in shape):
            from .constants import layout_strides
            code = dtype if isinstance(dtype, int) else enc_keyword(DATA_TYPE, dtype if dtype is not None else "float", "data type")
            return ZeroDescriptor(shape, code, layout_strides([max(d, 1) for d in shape], fmt))
        return core.tensor_descriptor(shape, dtype if dtype is not None else "float", fmt)

    def create_tensor(self, tensor_desc, batch_index=0, init=True):
        td = self.create_tensor_desc(tensor_desc)
        nbytes = 1 if isinstance(td, ZeroDescriptor) else max(1, core.bytesize(td))
        with torch.cuda.stream(self.stream):
            alloc = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        tz = B200Tensor(self, alloc, 0, nbytes // DATA_TYPE_WIDTH[td.dtype_code], td, batch_index, True)
        if init:
            self.set_all(0.0, tz)
        return tz

    def create_transformer(self, in_tz, out_tz):
        return b200_transformer(self.handle, in_tz.view(), out_tz.view())

    def create_shuffler(self, src_tz, dst_tz):
        return B200Shuffler(self.handle, src_tz.view(), dst_tz.view())

    def create_batcher(self, src_tz, dst_tz, mb_size):
        return B200Batcher(self.handle, src_tz.view(), dst_tz.view(), mb_size)

    def tensor_engine(self, dtype=None):
        return self

    # DnnFactory: only the hot-path blueprints exist here (base/internal/protocols.clj:68-110)
    def activ_blueprint(self, src_desc, activ, alpha, beta):
        from . import dnn
        return dnn.b200_activ_blueprint(self, src_desc, activ, alpha, beta)

    def sum_blueprint(self, src_descs):
        from . import dnn
        return dnn.B200SumBlueprint(self, [self.create_tensor_desc(d).view() for d in src_descs])

    def activ_op_blueprint(self, src_desc, activ, alpha, beta):
        """The operation-level blueprint is the layer-level one here: an activation is one kernel."""
        return self.activ_blueprint(src_desc, activ, alpha, beta)

    def concat_blueprint(self, src_descs, conc_dim, dst_type=None):
        from . import dnn
        return dnn.B200ConcatBlueprint(self, src_descs, conc_dim, dst_type)

    def branch_blueprint(self, src_desc, split_dim, dst_descs):
        from . import dnn
        return dnn.B200BranchBlueprint(self, src_desc, split_dim, dst_descs)

    def split_blueprint(self, src_desc, n):
        from . import dnn
        return dnn.B200SplitBlueprint(self, src_desc, n)

    def create_workspace(self, byte_size):
        return torch.empty(max(1, int(byte_size)), dtype=torch.uint8, device=self.device)

    # CostFactory (base/internal/protocols.clj:125-129)
    def quadratic_cost(self, last_layer, train_tz):
        from . import dnn
        return dnn.B200Cost(last_layer, train_tz, "quadratic")

    def mean_absolute_cost(self, last_layer, train_tz):
        from . import dnn
        return dnn.B200Cost(last_layer, train_tz, "mean-absolute")

    def crossentropy_cost(self, last_layer, train_tz):
        from . import dnn
        return dnn.B200CustomCost(last_layer, train_tz, "crossentropy")

    def inner_product_blueprint(self, *_):
        raise DiamondError("The B200 engine covers the tensor hot path only; use another factory "
                           "for contractions.", {"type": "not-supported"})

    fc_blueprint = convolution_blueprint = pooling_blueprint = batch_norm_blueprint = inner_product_blueprint
    gaussian_dropout_blueprint = rnn_op_blueprint = rnn_blueprint = abbreviate_blueprint = inner_product_blueprint

    # ------------------------------------------------------------------ host <-> device -------
    def upload(self, host_array, tz):
        """Raw storage copy host -> device (``set-vector!``)."""
        n = tz.storage_elems
        arr = np.ascontiguousarray(host_array).reshape(-1)
        if arr.size < n:
            raise DiamondError(DOES_NOT_FIT_MSG, {"source": arr.size, "destination": n})
        src = torch.from_numpy(arr[:n].view(np.uint8))
        with torch.cuda.stream(self.stream):
            dst = self._bytes(tz)
            dst.copy_(src, non_blocking=False)
        return tz

    def download(self, tz):
        """Raw storage copy device -> host under the tensor's own descriptor."""
        with torch.cuda.stream(self.stream):
            raw = self._bytes(tz).cpu().numpy()
        storage = raw.view(NUMPY_TYPE[tz.desc.dtype_code]).copy()
        return HostTensor(tz.shape, tz.desc.dtype_code, tz.layout, storage)

    def download_into(self, tz, host_array):
        """Raw storage copy device -> a caller-owned (ideally pinned) numpy array of the same dtype."""
        dst = torch.from_numpy(host_array.reshape(-1)[:tz.storage_elems].view(np.uint8))
        with torch.cuda.stream(self.stream):
            dst.copy_(self._bytes(tz), non_blocking=False)
        return host_array

    def _copy_streams(self):
        if self._h2d is None:
            self._h2d = torch.cuda.Stream(device=self.device)
            self._d2h = torch.cuda.Stream(device=self.device)

    def upload_async(self, host_array, tz):
        """Raw storage copy pinned host -> device on the factory's upload stream.  The copy starts once
        the work already given to the factory's stream is done (the destination may still be in
        use) and everything given to it afterwards waits for the copy; a download in flight on the
        other copy stream is NOT waited for, so both directions of the link run at once."""
        self._copy_streams()
        n = tz.storage_elems
        arr = np.ascontiguousarray(host_array).reshape(-1)
        if arr.size < n:
            raise DiamondError(DOES_NOT_FIT_MSG, {"source": arr.size, "destination": n})
        src = torch.from_numpy(arr[:n].view(np.uint8))
        self._h2d.wait_stream(self.stream)
        tz.alloc.record_stream(self._h2d)   # the allocator must not hand this memory out again before the copy ran
        with torch.cuda.stream(self._h2d):
            self._bytes(tz).copy_(src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._h2d)
        self.stream.wait_stream(self._h2d)
        return Pending(self, ev, tz)

    def download_async(self, tz, host_array):
        """Raw storage copy device -> a caller-owned pinned numpy array on the factory's download
        stream, after the work already given to the factory's stream.  Later work does not wait
        for it: use ``Pending.wait`` before reading the array and ``Pending.before_overwrite``
        before anything writes `tz` again."""
        self._copy_streams()
        dst = torch.from_numpy(host_array.reshape(-1)[:tz.storage_elems].view(np.uint8))
        self._d2h.wait_stream(self.stream)
        tz.alloc.record_stream(self._d2h)
        with torch.cuda.stream(self._d2h):
            dst.copy_(self._bytes(tz), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._d2h)
        return Pending(self, ev, host_array)

    def _bytes(self, tz):
        start = tz.base + tz.position * tz.width
        return tz.alloc[start:start + tz.storage_elems * tz.width]

    # ------------------------------------------------------------------ tensor engine ---------
    # (``TensorEngine``, cudnn/factory.clj:161-322: Neanderthal's BLAS protocol on tensors)
    def equals_block(self, x, y):
        """``equals-block`` (cudnn/factory.clj:123-133,163-164)."""
        with torch.cuda.stream(self.stream):
            self._flag.zero_()
        core.tensor_equals(self.handle, x.desc, x, y.desc, y, self._flag)
        with torch.cuda.stream(self.stream):
            return int(self._flag.item()) == 0

    def copy(self, x, y):
        """``copy`` (:166-168): transform-tensor with alpha 1, beta 0."""
        if x.nc == 0 and y.nc == 0:
            return y
        core.transform_tensor(self.handle, 1.0, x.desc, x, 0.0, y.desc, y)
        return y

    def axpy(self, alpha, x, y):
        """``axpy`` (:169-171): y = alpha*x + y with broadcasting of x."""
        core.add_tensor(self.handle, alpha, x.desc, x, 1.0, y.desc, y)
        return y

    def axpby(self, alpha, x, beta, y):
        """``axpby`` (:194-196)."""
        core.add_tensor(self.handle, alpha, x.desc, x, beta, y.desc, y)
        return y

    def scal(self, alpha, x):
        """``scal`` (:183-185)."""
        core.scale_tensor(self.handle, alpha, x.desc, x)
        return x

    def set_all(self, value, x):
        """``set-all`` (:191-193)."""
        if x.nc > 0:
            core.set_tensor(self.handle, x.desc, x, value)
        return x

    def _whole_reduce(self, op, x):
        """Whole-tensor scalar reductions (``asum nrm2 amax sum``, :175-190): one reduce-tensor call
        into a single element, read back (this synchronises, as the reference's does)."""
        if x.nc == 0:
            return 0.0
        if x.desc.dtype_code not in (0, 1, 2, 9):
            raise DiamondError("Reductions need a floating point tensor.", {"data-type": x.data_type})
        rtd = self._reduce_desc.get(op)
        if rtd is None:
            rtd = self._reduce_desc[op] = core.reduce_tensor_descriptor(op, "float", True)
        ydesc = core.tensor_descriptor([1] * len(x.shape), x.desc.dtype_code, [1] * len(x.shape))
        core.reduce_tensor(self.handle, rtd, 1.0, x.desc, x, 0.0, ydesc, self._scalar)
        with torch.cuda.stream(self.stream):
            raw = self._scalar.view(torch.uint8)[:x.width].cpu().numpy()
        if x.desc.dtype_code == 9:
            return float((raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)[0])
        return float(raw.view(NUMPY_TYPE[x.desc.dtype_code])[0])

    def asum(self, x):
        return self._whole_reduce("norm1", x)

    def nrm1(self, x):
        return self._whole_reduce("norm1", x)

    def nrm2(self, x):
        return self._whole_reduce("norm2", x)

    def nrmi(self, x):
        return self._whole_reduce("amax", x)

    def amax(self, x):
        return self._whole_reduce("amax", x)

    def sum(self, x):
        return self._whole_reduce("add", x)


class HostFactory:
    """Creates host mirrors.  It computes nothing: host tensors only carry data to and from the
    device (the reference uses its DNNL factory here, cudnn/factory.clj:342-343,447)."""

    def diamond_factory(self):
        return self

    def native_diamond_factory(self):
        return self

    def create_tensor_desc(self, shape, dtype=None, fmt=None):
        from .constants import layout_strides
        if dtype is None and fmt is None and not isinstance(shape, (list, tuple)):
            shape, dtype, fmt = _shape_of(shape), _dtype_of(shape), _layout_of(shape)
        return HostTensor(shape, dtype if dtype is not None else "float",
                          layout_strides(shape, fmt), storage=np.zeros(0))

    def create_tensor(self, tdesc, batch_index=0, init=True):
        return HostTensor(tdesc.shape, tdesc.dtype_code, tdesc.layout)

    def release(self):
        return True


HOST_FACTORY = HostFactory()


def b200_factory(device=None, stream=None):
    """``cudnn-factory`` (cudnn/factory.clj:481-494)."""
    return B200Factory(device, stream)


# ====================== transfer! ===============================================

def transfer_async(source, destination):
    """``transfer!`` without blocking the host, for the two raw-copy cases (a C-contiguous numpy array
    of the tensor's own data type, ideally pinned, to or from a contiguous device tensor): the copy
    runs on a copy stream of its own, uploads and downloads on different ones, and a ``Pending`` is
    returned.  Every other combination is done at once by ``transfer`` and comes back finished.
    The reference has no counterpart (its ``transfer!`` is synchronous, cudnn/tensor.clj:546-608)."""
    if (isinstance(destination, B200Tensor) and isinstance(source, np.ndarray) and destination.is_contiguous()
            and source.dtype == NUMPY_TYPE[destination.desc.dtype_code] and destination.desc.dtype_code != 9
            and source.flags["C_CONTIGUOUS"] and source.size >= destination.nc and destination.nc > 0):
        return destination.fact.upload_async(source, destination)
    if (isinstance(source, B200Tensor) and isinstance(destination, np.ndarray) and source.is_contiguous()
            and destination.dtype == NUMPY_TYPE[source.desc.dtype_code] and source.desc.dtype_code != 9
            and destination.flags["C_CONTIGUOUS"] and destination.size >= source.nc and source.nc > 0):
        return source.fact.download_async(source, destination)
    result = transfer(source, destination)
    fact = destination.fact if isinstance(destination, B200Tensor) else getattr(source, "fact", None)
    return Pending(fact, None, result)


def _host_values(source, n, dtype_code):
    """`n` values from a host sequence in the storage dtype of `dtype_code`; a numpy array that already
    has that dtype is used as is (no copy, so pinned buffers stay pinned)."""
    want = NUMPY_TYPE[dtype_code]
    if isinstance(source, np.ndarray) and source.dtype == want and dtype_code != 9:
        flat = source.reshape(-1)
        if flat.size < n:
            raise DiamondError(DOES_NOT_FIT_MSG, {"source": flat.size, "destination": n})
        return flat[:n]
    return _encode(_take(source, n, np.float64 if dtype_code in (0, 1, 2, 9) else np.int64), dtype_code)


def _take(source, n, np_dtype):
    if isinstance(source, np.ndarray):
        flat = source.reshape(-1)
        if flat.size < n:
            raise DiamondError(DOES_NOT_FIT_MSG, {"source": flat.size, "destination": n})
        return flat[:n].astype(np_dtype)
    vals = list(itertools.islice(iter(source), n))
    if len(vals) < n:  # a shorter sequence fills a prefix, like Neanderthal's transfer!
        vals = vals + [0] * (n - len(vals))
    return np.asarray(vals).astype(np_dtype)


def _encode(values, dtype_code):
    """Python/numpy numbers -> storage dtype (bf16 through round-to-nearest-even)."""
    if dtype_code == 9:
        f = np.asarray(values, dtype=np.float32).view(np.uint32)
        return ((f + 0x7FFF + ((f >> 16) & 1)) >> 16).astype(np.uint16)
    return np.asarray(values).astype(NUMPY_TYPE[dtype_code])


def transfer(source, destination):
    """``transfer!`` (cudnn/tensor.clj:542-625): moves data between tensors, host mirrors and plain
    sequences / arrays, converting layout and data type where they differ."""
    if hasattr(destination, "input") and not isinstance(destination, (B200Tensor, HostTensor)):
        transfer(source, destination.input())  # [Object Transformer] (:610-613)
        return destination
    if hasattr(source, "output") and not isinstance(source, (B200Tensor, HostTensor)):
        return transfer(source.output(), destination)  # [Transformer Object] (:615-617)

    if isinstance(source, B200Tensor) and isinstance(destination, B200Tensor):
        source.fact.copy(source, destination)  # :542-544
        return destination

    if isinstance(source, B200Tensor) and source.nc == 0:
        return destination

    if isinstance(destination, B200Tensor):
        fact = destination.fact
        if any(d == 0 for d in destination.shape):
            return destination
        if isinstance(source, HostTensor):  # [DnnlTensor CUDnnTensor] (:546-562)
            if source.shape != destination.shape:
                raise DiamondError(DOES_NOT_FIT_MSG, {"source": source.shape, "destination": destination.shape})
            if (source.dtype_code == destination.desc.dtype_code and source.layout == destination.layout):
                return fact.upload(source.storage, destination)
            # stage: raw upload under the source's own descriptor, then a device-side transform
            stage = fact.create_tensor(core.tensor_descriptor(source.shape, source.dtype_code, source.layout), 0, False)
            fact.upload(source.storage, stage)
            fact.copy(stage, destination)
            return destination
        # [Object CUDnnTensor] (:582-594)
        if destination.is_contiguous():
            return fact.upload(_host_values(source, destination.nc, destination.desc.dtype_code), destination)
        conn = fact.create_tensor(core.tensor_descriptor(destination.shape, destination.desc.dtype_code,
                                                         default_strides(destination.shape)), 0, False)
        fact.upload(_host_values(source, destination.nc, destination.desc.dtype_code), conn)
        fact.copy(conn, destination)
        return destination

    if isinstance(source, B200Tensor):
        fact = source.fact
        if isinstance(destination, HostTensor):  # [CUDnnTensor DnnlTensor] (:564-580)
            if source.shape != destination.shape:
                raise DiamondError(DOES_NOT_FIT_MSG, {"source": source.shape, "destination": destination.shape})
            if not (source.desc.dtype_code == destination.dtype_code and source.layout == destination.layout):
                stage = fact.create_tensor(core.tensor_descriptor(destination.shape, destination.dtype_code,
                                                                  destination.layout), 0, False)
                fact.copy(source, stage)
                source = stage
            destination.storage[...] = fact.download(source).storage
            return destination
        # [CUDnnTensor Object] (:596-608): a numpy array or list to fill
        if (isinstance(destination, np.ndarray) and source.is_contiguous()
                and destination.dtype == NUMPY_TYPE[source.desc.dtype_code] and source.desc.dtype_code != 9
                and destination.flags["C_CONTIGUOUS"] and destination.size >= source.nc):
            return fact.download_into(source, destination)  # straight into the caller's buffer
        if source.is_contiguous():
            host = fact.download(source)
        else:
            conn = fact.create_tensor(core.tensor_descriptor(source.shape, source.desc.dtype_code,
                                                             default_strides(source.shape)), 0, False)
            fact.copy(source, conn)
            host = fact.download(conn)
        vals = host.values()
        if isinstance(destination, np.ndarray):
            flat = destination.reshape(-1)
            flat[:len(vals)] = np.asarray(vals[:flat.size], dtype=destination.dtype)
        else:
            for i, v in enumerate(vals[:len(destination)]):
                destination[i] = v
        return destination

    if isinstance(destination, HostTensor):  # plain data into a host mirror
        n = len(destination.storage)
        destination.storage[...] = _encode(_take(source, n, np.float64), destination.dtype_code)
        return destination
    raise DiamondError("No transfer! defined for these arguments.",
                       {"source": type(source).__name__, "destination": type(destination).__name__})
