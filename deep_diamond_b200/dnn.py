"""The two layer entry points on the hot path: ``activation`` / ``activ`` and ``sum``.

Counterpart of deep-diamond-base/src/uncomplicate/diamond/dnn.clj (:56-108, :537-557) on top of the
backend layer objects the cuDNN backend defines in
deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/directed.clj (activation :49-233,
:352-363; sum :1722-1833).  A blueprint is called with source tensors to make a layer; a layer has
``forward`` / ``backward`` and the Transfer / DiffTransfer accessors.
"""
import builtins as _builtins

from . import core
from . import tensor as _t
from ._lib import DiamondError


class B200ActivationInference:
    """``CUDnnActivationInference`` (:49-77): in place on the data tensor."""

    def __init__(self, hdl, bluep, ad, data_tz, linear):
        self.hdl, self.bluep, self.ad, self.data_tz, self.linear = hdl, bluep, ad, data_tz, linear

    def input(self):
        return self.data_tz

    def output(self):
        return self.data_tz

    def __call__(self):
        if not self.linear:
            core.activation_forward(self.hdl, self.ad, 1.0, self.data_tz.desc, self.data_tz, 0.0,
                                    self.data_tz.desc, self.data_tz)
        return self.data_tz

    def release(self):
        return True


class B200ActivationTraining:
    """``CUDnnActivationTraining`` (:125-177).  dst doubles as the incoming-gradient buffer except
    for sigmoid, which gets its own (:223-231)."""

    def __init__(self, hdl, bluep, ad, src_tz, dst_tz, diff_dst_tz, diff_src_tz):
        self.hdl, self.bluep, self.ad = hdl, bluep, ad
        self.src_tz, self.dst_tz, self.diff_dst_tz, self.diff_src_tz = src_tz, dst_tz, diff_dst_tz, diff_src_tz

    def input(self):
        return self.src_tz

    def output(self):
        return self.dst_tz

    def diff_input(self):
        return self.diff_dst_tz

    def diff_output(self):
        return self.diff_src_tz

    def __call__(self):
        self.forward()
        return self.dst_tz

    def forward(self):
        core.activation_forward(self.hdl, self.ad, 1.0, self.src_tz.desc, self.src_tz, 0.0,
                                self.dst_tz.desc, self.dst_tz)
        return self

    def backward(self):
        core.activation_backward(self.hdl, self.ad, 1.0, self.dst_tz.desc, self.dst_tz,
                                 self.diff_dst_tz.desc, self.diff_dst_tz, self.src_tz.desc, self.src_tz,
                                 0.0, self.diff_src_tz.desc, self.diff_src_tz)
        return self

    def release(self):
        return True


class B200LinearActivationTraining:
    """``CUDnnLinearActivationTraining`` (:79-123): two copies."""

    def __init__(self, hdl, bluep, src_tz, dst_tz, diff_src_tz):
        self.hdl, self.bluep, self.src_tz, self.dst_tz, self.diff_src_tz = hdl, bluep, src_tz, dst_tz, diff_src_tz

    def input(self):
        return self.src_tz

    def output(self):
        return self.dst_tz

    def diff_input(self):
        return self.dst_tz

    def diff_output(self):
        return self.diff_src_tz

    def __call__(self):
        self.forward()
        return self.dst_tz

    def forward(self):
        _t.copy(self.src_tz, self.dst_tz)
        return self

    def backward(self):
        _t.copy(self.dst_tz, self.diff_src_tz)
        return self

    def release(self):
        return True


class B200ActivationBlueprint:
    """``CUDnnActivationBlueprint`` (:179-233)."""

    def __init__(self, fact, activ, ad, inf_desc, train_desc, diff_desc):
        self.fact, self.activ, self.ad = fact, activ, ad
        self.inf_desc, self.train_desc, self.diff_desc = inf_desc, train_desc, diff_desc

    @property
    def shape(self):
        return self.train_desc.shape

    @property
    def data_type(self):
        return self.train_desc.data_type

    @property
    def layout(self):
        return self.train_desc.layout

    def diamond_factory(self):
        return self.fact

    def info(self):
        return {"activation": self.activ}

    def __call__(self, src_tz, diff_src_tz=None):
        linear = self.activ in ("linear", "identity")
        if diff_src_tz is None:
            return B200ActivationInference(self.fact.handle, self, self.ad, src_tz, linear)
        dst_tz = self.fact.create_tensor(self.diff_desc.view(), diff_src_tz.batch_index(), False)
        if linear:
            return B200LinearActivationTraining(self.fact.handle, self, src_tz, dst_tz, diff_src_tz)
        # a kind whose derivative reads the forward result needs that result kept apart from the
        # incoming gradient (the *-dst-bwd kinds of the DNNL table), like sigmoid in the reference
        if self.activ in ("sigmoid", "logistic") or self.activ.endswith("-dst-bwd"):
            diff_dst_tz = self.fact.create_tensor(self.diff_desc.view(), dst_tz.batch_index(), False)
            return B200ActivationTraining(self.fact.handle, self, self.ad, src_tz, dst_tz, diff_dst_tz, diff_src_tz)
        return B200ActivationTraining(self.fact.handle, self, self.ad, src_tz, dst_tz, dst_tz, diff_src_tz)

    def release(self):
        self.ad.release()
        return True


def b200_activ_blueprint(fact, data_desc, activ, alpha, beta=0.0):
    """``cudnn-activ-blueprint`` (:352-363); `alpha` is the activation coefficient, `beta` the shift
    of :linear (oneDNN's second eltwise argument)."""
    d = fact.create_tensor_desc(data_desc)
    if activ == "softmax":
        raise DiamondError("softmax is outside the B200 engine's scope.", {"type": "not-supported"})
    ad = core.activation_descriptor(activ, True, alpha, beta)
    return B200ActivationBlueprint(fact, activ, ad, d.view(), d.view(), d.view())


def activation(*args):
    """``activation`` (dnn.clj:56-94): (fact src-provider activ [args]) or (activ [args]) which
    returns a function of (fact src-provider) / (src-provider)."""
    if args and hasattr(args[0], "create_tensor"):
        fact, src_provider, activ = args[0], args[1], args[2]
        opts = args[3] if len(args) > 3 and args[3] else {}
        alpha = opts.get("alpha", 1.0 if activ == "linear" else 0.0)
        beta = opts.get("beta", 0.0)
        return fact.diamond_factory().activ_blueprint(src_provider, activ, alpha, beta)
    activ = args[0]
    opts = args[1] if len(args) > 1 else None

    def make(*a):
        if len(a) == 2:
            return activation(a[0], a[1], activ, opts)
        return activation(_t.diamond_factory(), a[0], activ, opts)
    return make


def activ(activ_kw, args=None):
    """``activ`` (dnn.clj:96-108)."""
    return activation(activ_kw, args)


class B200Sum:
    """``CUDnnSum`` (:1722-1779).  forward: src0 += the other sources, as ONE n-ary pass (the
    reference loops n-1 ``axpy!`` calls, :1762-1766); backward: src0 /= n, copied to the rest."""

    def __init__(self, fact, bluep, src_tzs, prop_diff):
        self.fact, self.bluep, self.src_tzs, self.prop_diff = fact, bluep, list(src_tzs), prop_diff

    def input(self):
        return self.src_tzs

    def output(self):
        return self.src_tzs[0]

    def diff_input(self):
        return self.src_tzs[0]

    def diff_output(self):
        return self.src_tzs

    def parameters(self):
        return []

    def _sum(self):
        s0 = self.src_tzs[0]
        if len(self.src_tzs) > 1:
            core.sum_tensors(self.fact.handle, [1.0] * len(self.src_tzs), [t.desc for t in self.src_tzs],
                             self.src_tzs, s0.desc, s0)
        return s0

    def forward(self, _=None):
        self._sum()
        return self

    def backward(self, _=None):
        if self.prop_diff:
            s0 = _t.scal(1.0 / len(self.src_tzs), self.src_tzs[0])
            for tz in self.src_tzs[1:]:
                _t.copy(s0, tz)
        return self

    def __call__(self):
        return self._sum()

    def release(self):
        return True


class B200SumBlueprint:
    """``CUDnnSumBlueprint`` (:1785-1829)."""

    def __init__(self, fact, src_descs):
        self.fact, self.src_descs = fact, src_descs

    @property
    def shape(self):
        return self.src_descs[0].shape

    @property
    def data_type(self):
        return self.src_descs[0].data_type

    @property
    def layout(self):
        return self.src_descs[0].layout

    def diamond_factory(self):
        return self.fact

    def __call__(self, prev_layer, prop_diff=False, _=None):
        return B200Sum(self.fact, self, [_t.output(p) for p in prev_layer], prop_diff)

    def release(self):
        return True


def sum(*args):  # noqa: A001 - the reference's name
    """``sum`` (dnn.clj:537-557): (fact src-descs) or () returning a function."""
    if not args:
        def make(*a):
            if len(a) == 2:
                return sum(a[0], a[1])
            return sum(_t.diamond_factory(), a[0])
        return make
    fact, src_descs = args
    return fact.diamond_factory().sum_blueprint(src_descs)


def forward(layer, *a):
    return layer.forward(*a)


def backward(layer, *a):
    return layer.backward(*a)


def diff_input(layer):
    return layer.diff_input()


def diff_output(layer):
    return layer.diff_output()


# ====================== branch / concatenate / split ============================================
# Counterparts of cudnn/directed.clj:1289-1549 (branch, concat) and :1553-1710 (split).  Where the
# reference invokes one transformer per sub-tensor, a pass here is ONE ddMultiTransform launch.

def concat_offsets(split_dim, sub_shapes):
    """``concat-offsets`` (deep-diamond-base/src/uncomplicate/diamond/internal/utils.clj:88-92)."""
    acc = [0]
    for s in sub_shapes:
        acc.append(acc[-1] + int(s[split_dim]))
    return acc[:-1]


def concat_dst_shape(conc_dim, src_shapes):
    """``concat-dst-shape`` (utils.clj:98-100)."""
    out = list(src_shapes[0])
    out[conc_dim] = _builtins.sum(int(s[conc_dim]) for s in src_shapes)  # this module defines its own `sum`
    return out


class _Pairs:
    """A list of (source, destination) tensor pairs copied by one launch."""

    def __init__(self, fact, pairs):
        self.fact, self.pairs = fact, pairs

    def __call__(self):
        core.multi_transform(self.fact.handle, self.pairs)


class B200Branch:
    """``CUDnnBranchInference`` / ``CUDnnBranchTraining`` (:1289-1404) for both branch (one source
    cut along `dim` into several destinations) and concatenate (the mirror image)."""

    def __init__(self, fact, bluep, is_branch, data_tz, diff_data, fwd_pairs, bwd_pairs, prop_diff):
        self.fact, self.bluep, self.is_branch, self.data_tz, self.diff_data = fact, bluep, is_branch, data_tz, diff_data
        self.fwd, self.bwd, self.prop_diff = _Pairs(fact, fwd_pairs), (_Pairs(fact, bwd_pairs) if bwd_pairs else None), prop_diff
        self._fwd_pairs, self._bwd_pairs = fwd_pairs, bwd_pairs

    def input(self):
        return self.data_tz if self.is_branch else [x for x, _ in self._fwd_pairs]

    def output(self):
        return [y for _, y in self._fwd_pairs] if self.is_branch else self.data_tz

    def diff_input(self):
        return [x for x, _ in self._bwd_pairs] if self.is_branch else self.data_tz

    def diff_output(self):
        return self.diff_data if self.is_branch else [y for _, y in self._bwd_pairs]

    def parameters(self):
        return []

    def forward(self, _=None):
        self.fwd()
        return self

    def backward(self, _=None):
        if self.prop_diff and self.bwd is not None:
            self.bwd()
        return self

    def __call__(self):
        self.fwd()
        return self.output()

    def release(self):
        return True


def _sub_views(tz, dim, sub_shapes):
    """Sub-tensors of `tz` laid end to end along `dim` (same strides, element offsets of
    ``concat-offsets`` times the stride of `dim`)."""
    views = []
    for shp, off in zip(sub_shapes, concat_offsets(dim, sub_shapes)):
        v = tz.view()
        v.offset(off * tz.layout[dim])
        views.append(v.view_tz(_t.desc(list(shp), tz.data_type, tz.layout)))
    return views


class B200BranchBlueprint:
    """``CUDnnBranchBlueprint`` (:1406-1466)."""

    def __init__(self, fact, src_desc, branch_dim, dst_descs):
        self.fact, self.branch_dim = fact, int(branch_dim)
        self.src_desc = fact.create_tensor_desc(src_desc)
        self.dst_descs = [fact.create_tensor_desc(d) if not isinstance(d, _t.TensorDescriptorImpl) or d.data_type
                          else fact.create_tensor_desc(d.shape, self.src_desc.dtype_code, d.layout) for d in dst_descs]
        self.dst_dims = [list(d.shape) for d in self.dst_descs]

    @property
    def shape(self):
        return [d.shape for d in self.dst_descs]

    def diamond_factory(self):
        return self.fact

    def __call__(self, prev_layer, prop_diff=None, _=None):
        src_tz = _t.output(prev_layer)
        dst_tzs = [self.fact.create_tensor(d.view(), 0, True) for d in self.dst_descs]
        fwd = list(zip(_sub_views(src_tz, self.branch_dim, self.dst_dims), dst_tzs))
        if prop_diff is None:
            return B200Branch(self.fact, self, True, src_tz, None, fwd, None, False)
        diff_src_tz = prev_layer.diff_input() if hasattr(prev_layer, "diff_input") else src_tz
        bwd = list(zip(dst_tzs, _sub_views(diff_src_tz, self.branch_dim, self.dst_dims)))
        return B200Branch(self.fact, self, True, src_tz, diff_src_tz, fwd, bwd, prop_diff)

    def release(self):
        return True


class B200ConcatBlueprint:
    """``CUDnnConcatBlueprint`` (:1468-1549): destination has default strides."""

    def __init__(self, fact, src_descs, conc_dim, dst_type=None):
        self.fact, self.conc_dim = fact, int(conc_dim)
        self.src_descs = [fact.create_tensor_desc(d) for d in src_descs]
        self.src_dims = [list(d.shape) for d in self.src_descs]
        dst_shape = concat_dst_shape(self.conc_dim, self.src_dims)
        from .constants import default_strides
        self.dst_desc = fact.create_tensor_desc(dst_shape, dst_type or self.src_descs[0].dtype_code,
                                                default_strides(dst_shape))

    @property
    def shape(self):
        return self.dst_desc.shape

    def diamond_factory(self):
        return self.fact

    def __call__(self, prev_layer, prop_diff=None, _=None):
        src_tzs = [_t.output(p).view() for p in prev_layer]
        dst_tz = self.fact.create_tensor(self.dst_desc.view(), 0, True)
        subs = _sub_views(dst_tz, self.conc_dim, self.src_dims)
        fwd = list(zip(src_tzs, subs))
        if prop_diff is None:
            return B200Branch(self.fact, self, False, dst_tz, None, fwd, None, False)
        diff_src_tzs = [(p.diff_input() if hasattr(p, "diff_input") else _t.output(p)).view() for p in prev_layer]
        bwd = list(zip(subs, diff_src_tzs))
        return B200Branch(self.fact, self, False, dst_tz, diff_src_tzs, fwd, bwd, prop_diff)

    def release(self):
        return True


class B200Split:
    """``CUDnnSplitInference`` / ``CUDnnSplitTraining`` (:1553-1660): forward hands out the source n
    times; backward = mean of the n incoming gradients, here one n-ary sum launch (the reference
    zero-fills and runs n ``axpy!`` passes, :1649-1653)."""

    def __init__(self, fact, bluep, n, src_tz, diff_tzs, prop_diff):
        self.fact, self.bluep, self.n, self.src_tz, self.diff_tzs, self.prop_diff = fact, bluep, n, src_tz, diff_tzs, prop_diff

    def input(self):
        return self.src_tz

    def output(self):
        return [self.src_tz] * self.n

    def diff_input(self):
        return self.diff_tzs

    def diff_output(self):
        return self.src_tz

    def parameters(self):
        return []

    def forward(self, _=None):
        return self

    def backward(self, _=None):
        if self.prop_diff and self.diff_tzs:
            core.sum_tensors(self.fact.handle, [1.0 / self.n] * self.n, [t.desc for t in self.diff_tzs],
                             self.diff_tzs, self.src_tz.desc, self.src_tz)
        return self

    def __call__(self):
        return self.output()

    def release(self):
        return True


class B200SplitBlueprint:
    """``CUDnnSplitBlueprint`` (:1662-1710)."""

    def __init__(self, fact, src_desc, n):
        self.fact, self.n = fact, int(n)
        self.src_desc = fact.create_tensor_desc(src_desc)

    def diamond_factory(self):
        return self.fact

    def __call__(self, prev_layer, prop_diff=None, _=None):
        src_tz = _t.output(prev_layer)
        if prop_diff is None:
            return B200Split(self.fact, self, self.n, src_tz, None, False)
        diffs = [self.fact.create_tensor(self.src_desc.view(), 0, True) for _ in range(self.n)]
        return B200Split(self.fact, self, self.n, src_tz, diffs, prop_diff)

    def release(self):
        return True


def branch(fact, src_desc, branch_dim, dst_descs):
    """``branch`` (dnn.clj:477-508)."""
    return B200BranchBlueprint(fact.diamond_factory(), src_desc, branch_dim, dst_descs)


def concatenate(fact, conc_dim, src_descs, dst_type=None):
    """``concatenate`` (dnn.clj:411-443)."""
    return B200ConcatBlueprint(fact.diamond_factory(), src_descs, conc_dim, dst_type)


def split(fact, src_desc, n):
    """``split`` (dnn.clj:510-535)."""
    return B200SplitBlueprint(fact.diamond_factory(), src_desc, n)


# ====================== cost ====================================================================

class B200Cost:
    """``CUDnnUniversalCost`` (cudnn/directed.clj:367-412) for :quadratic and :mean-absolute
    (base/internal/cost.clj:20-34).  Invoking it writes a - y into the previous layer's diff-input and
    returns the cost, both from ONE kernel; the reference runs connector + ``axpy! -1`` + ``nrm2``."""

    def __init__(self, prev_layer, train_tz, kind):
        import torch
        self.prev_layer, self.train_tz, self.kind = prev_layer, train_tz, kind
        self.fact = train_tz.fact
        self.a = _t.output(prev_layer)
        self.a_y = prev_layer.diff_input() if hasattr(prev_layer, "diff_input") else self.a
        if not (core.equal_desc(self.a.desc, train_tz.desc) and core.equal_desc(self.a_y.desc, train_tz.desc)):
            raise DiamondError("The B200 cost needs the output, its gradient and the target in one layout.",
                               {"output": repr(self.a), "target": repr(train_tz)})
        self._cost = torch.zeros(1, dtype=torch.float64, device=self.fact.device)

    def input(self):
        return self.a

    def output(self):
        return self.a

    def diff_input(self):
        return self.train_tz

    def diff_output(self):
        return self.a_y

    def forward(self):
        return self

    def backward(self):
        core.cost_diff(self.fact.handle, self.kind, self.train_tz.desc, self.a, self.train_tz, self.a_y, self._cost)
        if hasattr(self.prev_layer, "backward"):
            self.prev_layer.backward()
        return self

    def __call__(self):
        import torch
        core.cost_diff(self.fact.handle, self.kind, self.train_tz.desc, self.a, self.train_tz, self.a_y, self._cost)
        with torch.cuda.stream(self.fact.stream):
            view = self._cost.view(torch.float32) if self.train_tz.desc.dtype_code == 0 else self._cost
            return float(view[0].item())


class B200CustomCost(B200Cost):
    """``CUDnnCustomCost`` (cudnn/directed.clj:413-458) with ``crossentropy-cost!``
    (base/internal/cost.clj:34-40).  Invoking it only reads: the cost of (y, a) comes from one pass
    where the reference runs two logs, two linear-fracs, two products, an axpy and an asum.
    ``backward`` writes a - y into the previous layer's gradient after its linear part (``diff-z``:
    the activation layer's diff-output here) and, like the reference, does not call the previous
    layer's backward."""

    def __init__(self, prev_layer, train_tz, kind):
        import torch
        self.prev_layer, self.train_tz, self.kind = prev_layer, train_tz, kind
        self.fact = train_tz.fact
        self.a = _t.output(prev_layer)
        if hasattr(prev_layer, "diff_z"):
            self.a_y = prev_layer.diff_z()
        elif hasattr(prev_layer, "diff_output"):
            self.a_y = prev_layer.diff_output()
        else:
            self.a_y = _t.tensor(self.fact, train_tz.desc)
        if not (core.equal_desc(self.a.desc, train_tz.desc) and core.equal_desc(self.a_y.desc, train_tz.desc)):
            raise DiamondError("The B200 cost needs the output, its gradient and the target in one layout.",
                               {"output": repr(self.a), "target": repr(train_tz)})
        self._cost = torch.zeros(1, dtype=torch.float64, device=self.fact.device)

    def backward(self):
        core.cost_diff(self.fact.handle, "mean-absolute", self.train_tz.desc, self.a, self.train_tz, self.a_y,
                       self._cost)
        return self

    def __call__(self):
        import torch
        core.cost_diff(self.fact.handle, self.kind, self.train_tz.desc, self.a, self.train_tz, None, self._cost)
        with torch.cuda.stream(self.fact.stream):
            view = self._cost.view(torch.float32) if self.train_tz.desc.dtype_code == 0 else self._cost
            return float(view[0].item())


def cost(layer, train_tz, cost_kw="quadratic"):
    """``cost`` (dnn.clj:559-581)."""
    if cost_kw not in core.COST_KIND:
        raise DiamondError("This cost function is not supported.", {"cost": cost_kw})
    if cost_kw == "crossentropy":
        return B200CustomCost(layer, train_tz, cost_kw)
    return B200Cost(layer, train_tz, cost_kw)
