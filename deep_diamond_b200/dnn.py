"""The two layer entry points on the hot path: ``activation`` / ``activ`` and ``sum``.

Counterpart of deep-diamond-base/src/uncomplicate/diamond/dnn.clj (:56-108, :537-557) on top of the
backend layer objects the cuDNN backend defines in
deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/directed.clj (activation :49-233,
:352-363; sum :1722-1833).  A blueprint is called with source tensors to make a layer; a layer has
``forward`` / ``backward`` and the Transfer / DiffTransfer accessors.
"""
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
        if self.activ in ("sigmoid", "logistic"):
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
