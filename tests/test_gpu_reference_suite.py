"""The reference's factory-parametric suites, transcribed function for function and run against the
B200 factory through the public API.  This is how the reference accepts a backend: its cuDNN suite
just calls these with its own factory (deep-diamond-cuda/test/.../cudnn_tensor_test.clj:70-94,
directed_test.clj:16-53).

Sources: deep-diamond-test/src/uncomplicate/diamond/tensor_test.clj (tt) and dnn_test.clj (dt).
"""
import itertools

import numpy as np
import pytest

from deep_diamond_b200 import core, dnn
from deep_diamond_b200 import tensor as T
from deep_diamond_b200._lib import DiamondError
from deep_diamond_b200.tensor import (asum, batcher, connector, desc, entry, entry_, input, native, offset_,
                                      output, shuffler, tensor, transfer, transformer, view_tz, view_vctr)

pytestmark = pytest.mark.gpu


def seq(x):
    return list(native(x))


def test_tensor(fact):
    """tt :22-27"""
    tz = tensor(fact, [2, 3, 4, 5], "float", "nchw")
    assert asum(tz) == 0.0
    assert asum(entry_(tz, 1)) == 120.0
    assert T.shape(tz) == [2, 3, 4, 5]


def test_zero(fact):
    """tt :29-35"""
    tz = tensor(fact, [2, 3, 4, 5], "float", "nchw")
    tz_zero = T.zero(tz)
    assert asum(tz) == 0.0
    assert asum(entry_(tz, 1)) == 120.0
    assert asum(tz_zero) == 0.0


def test_create(fact):
    """tt :37-48"""
    t1 = tensor(fact, [1, 1, 1, 1], "float", "nchw")
    td3221 = desc([3, 2, 2, 1], "float", "nhwc")
    t3221 = tensor(fact, td3221)
    with pytest.raises(DiamondError):
        tensor(fact, [1, -1, 1, 1], "float", "nchw")
    assert T.dim(t1) == 1 and T.shape(t1) == [1, 1, 1, 1] and T.layout(t1) == [1, 1, 1, 1]
    assert T.data_type(t1) == "float"
    assert T.dim(t3221) == 12 and T.layout(t3221) == [4, 1, 2, 2]


def test_equality(fact):
    """tt :50-63"""
    x1 = tensor(fact, [2, 1, 2, 3], "float", "nchw")
    y1 = tensor(fact, [2, 1, 2, 3], "float", "nchw")
    y3 = tensor(fact, [2, 1, 2, 3], "float", "nhwc")
    y4 = tensor(fact, [2, 1, 2, 2], "float", "nchw")
    x5 = tensor(fact, [2, 2, 2, 2], "float", "nchw")
    y5 = tensor(fact, [2, 2, 2, 2], "float", "nhwc")
    assert (x1 == None) is False  # noqa: E711
    assert x1 == y1
    assert not (x1 == y3) and not (x1 == y4) and not (x5 == y5)
    assert transfer(itertools.count(), x1) == transfer(itertools.count(), y1)


def test_release(fact):
    """tt :65-69"""
    t1 = tensor(fact, [2, 3, 1, 1], "float", "nchw")
    assert T.release(view_tz(t1)) is True and T.release(t1) is True


def test_transfer(fact):
    """tt :71-87 with both factories the B200 one (the reference also runs it as fact0 = fact1)."""
    x1 = tensor(fact, [2, 1, 2, 1], "float", "nchw")
    x2 = tensor(fact, [2, 1, 2, 1], "float", "nchw")
    y1 = tensor(fact, [2, 1, 2, 1], "float", "nchw")
    y2 = tensor(fact, [2, 1, 1, 1], "float", [1, 1, 1, 1])
    assert transfer(np.array([1, 2, 3, 4], np.float32), x1) is x1
    assert list(transfer(x1, np.zeros(4, np.float32))) == [1.0, 2.0, 3.0, 4.0]
    assert seq(transfer(np.array([4, 3, 2, 1], np.float32), x1)) == [4.0, 3.0, 2.0, 1.0]
    assert seq(transfer([10, 20, 30, 40], x1)) == [10.0, 20.0, 30.0, 40.0]
    assert transfer(x1, x2) is x2 and seq(x2) == [10.0, 20.0, 30.0, 40.0]
    assert transfer(x1, y1) is y1 and seq(y1) == [10.0, 20.0, 30.0, 40.0]
    assert entry_(y1, 100) is y1
    assert seq(transfer(y1, x1)) == [100.0] * 4
    with pytest.raises(DiamondError):
        transfer(x2, y2)


def test_transfer_to_and_from_host_mirror(fact):
    """tt :71-87 with fact1 = the native (host) factory, as cudnn_tensor_test.clj:79 runs it."""
    host = fact.native_diamond_factory()
    x1 = tensor(fact, [2, 1, 2, 1], "float", "nchw")
    y1 = tensor(host, [2, 1, 2, 1], "float", "nchw")
    transfer([10, 20, 30, 40], x1)
    assert transfer(x1, y1) is y1 and list(y1) == [10.0, 20.0, 30.0, 40.0]
    transfer([100, 100, 100, 100], y1)
    assert seq(transfer(y1, x1)) == [100.0] * 4
    y2 = tensor(host, [2, 1, 1, 1], "float", [1, 1, 1, 1])
    with pytest.raises(DiamondError):
        transfer(x1, y2)


def test_contiguous(fact):
    """tt :89-96"""
    x1 = tensor(fact, [2, 3, 2, 2], "float", "nchw")
    assert T.contiguous(x1)
    transfer(itertools.count(), x1)
    assert view_tz(x1, [2, 3, 2, 2]) == x1
    assert seq(view_tz(x1, [1, 3, 2, 2])) == [float(i) for i in range(12)]
    assert T.contiguous(x1)


def test_subtensor(fact):
    """tt :98-117"""
    tz_x = tensor(fact, [6, 1, 1, 1], "float", [1, 1, 1, 1])
    sub_x = view_tz(tz_x, [2, 1, 1, 1])
    sub_y = view_tz(tz_x, desc([1, 3, 1, 1], [3, 1, 1, 1]))
    sub_z = view_tz(tz_x, 4)
    transfer(itertools.count(), tz_x)
    assert seq(tz_x) == [0.0, 1.0, 2.0, 3.0, 4.0, 5.0]
    assert seq(sub_x) == [0.0, 1.0] and seq(sub_y) == [0.0, 1.0, 2.0] and seq(sub_z) == [0.0, 1.0, 2.0, 3.0]
    sub_y.offset(3)
    assert seq(sub_y) == [3.0, 4.0, 5.0] and seq(sub_x) == [0.0, 1.0]
    sub_z.offset(1)
    assert seq(sub_z) == [1.0, 2.0, 3.0, 4.0] and seq(sub_x) == [0.0, 1.0]
    assert seq(tz_x) == [0.0, 1.0, 2.0, 3.0, 4.0, 5.0]
    entry_(view_vctr(sub_y), 0)
    assert seq(tz_x) == [0.0, 1.0, 2.0, 0.0, 0.0, 0.0]


def test_transformer(fact):
    """tt :152-169"""
    tz_x = tensor(fact, [2, 3, 4, 5], "float", "nchw")
    tz_y = tensor(fact, [2, 3, 4, 5], "float", "nhwc")
    tz_sub_x = view_tz(tz_x, [1, 3, 4, 5])
    tz_sub_y = view_tz(tz_y, [1, 3, 4, 5])
    transform = transformer(tz_x, tz_y)
    sub_transform = transformer(tz_sub_x, tz_sub_y)
    assert entry(view_vctr(native(transfer(itertools.count(), tz_x))), 119) == 119.0
    assert entry(view_vctr(native(tz_y)), 119) == 0.0
    assert T.buffer(input(transform)) == T.buffer(tz_x)
    assert T.buffer(output(transform)) == T.buffer(tz_y)
    assert transform() == tz_y
    assert asum(tz_y) == asum(tz_x)
    assert entry(view_vctr(native(tz_y)), 119) == 119.0
    transfer(range(0, 1000, 10), tz_x)
    assert sub_transform() == tz_sub_y
    assert entry(view_vctr(native(tz_y)), 34) == 310.0


def test_transformer_any(fact):
    """tt :171-182"""
    tz_x = tensor(fact, [2, 3, 2, 1], "float", [48, 16, 5, 2])
    in_x = connector(desc([2, 3, 2, 1], "float", "nchw"), tz_x)
    tz_y = tensor(fact, [2, 3, 2, 1], "float", [48, 13, 4, 2])
    out_y = connector(tz_y, desc([2, 3, 2, 1], "float", "nchw"))
    transform = transformer(tz_x, tz_y)
    transfer(itertools.count(), input(in_x))
    in_x()
    transform()
    out_y()
    assert output(out_y) == input(in_x)


def test_transfer_any(fact):
    """tt :184-194"""
    tz_x = tensor(fact, [2, 3, 2, 1], "float", [48, 12, 4, 2])
    in_x = connector(desc([2, 3, 2, 1], "float", "nchw"), tz_x)
    tz_y = tensor(fact, [2, 3, 2, 1], "float", [48, 14, 4, 2])
    out_y = connector(tz_y, desc([2, 3, 2, 1], "float", "nchw"))
    transfer(itertools.count(), input(in_x))
    in_x()
    transfer(tz_x, tz_y)
    out_y()
    assert asum(output(out_y)) == float(sum(range(12)))


def test_transfer_view_tz(fact):
    """tt :196-203"""
    tz = tensor(fact, [1, 3, 3, 1], "float", "nchw")
    entry_(tz, 100.0)
    ibtz = view_tz(tz, [1, 2, 1, 1])
    offset_(ibtz, 1)
    offset_(ibtz, 1)
    transfer(range(1, 3), ibtz)
    assert seq(tz) == [100.0, 1.0, 100.0, 100.0, 2.0, 100.0, 100.0, 100.0, 100.0]


def test_heterogenous_transfer(fact):
    """tt :205-221"""
    tz_x = tensor(fact, [6, 2, 1, 1], "byte", "nchw")
    sub_x = offset_(view_tz(tz_x, 2), 2 * 4)
    tz_y = tensor(fact, [6, 2, 1, 1], "float", "nchw")
    sub_y = offset_(view_tz(tz_y, 2), 2 * 2)
    tz_z = tensor(fact, [6, 2, 1, 1], "uint8", "nchw")
    sub_z = offset_(view_tz(tz_z, 2), 2 * 1)
    transfer(range(-6, 6), tz_x)
    assert seq(tz_x) == list(range(-6, 6))
    transfer(tz_x, tz_y)
    assert asum(transfer(tz_x, tz_y)) == 36.0
    assert seq(transfer(tz_y, tz_z)) == [0, 0, 0, 0, 0, 0, 0, 1, 2, 3, 4, 5]
    assert asum(native(transfer(sub_x, sub_y))) == 14.0
    assert seq(transfer(sub_y, sub_z)) == [2, 3, 4, 5]
    assert seq(tz_z) == [0, 0, 2, 3, 4, 5, 0, 1, 2, 3, 4, 5]


def test_pull_push_connectors(fact):
    """tt :223-261"""
    tz_x = tensor(fact, [2, 3, 4, 5], "float", "nchw")
    connection = connector(tz_x, desc([2, 3, 4, 5], "float", "nhwc"))       # pull, different
    assert entry(view_vctr(native(transfer(itertools.count(), tz_x))), 119) == 119.0
    assert T.buffer(input(connection)) == T.buffer(tz_x)
    assert T.buffer(input(connection)) != T.buffer(output(connection))
    assert entry(native(view_vctr(connection())), 119) == 119.0
    same = connector(tz_x, desc([2, 3, 4, 5], "float", "nchw"))              # pull, same
    assert T.buffer(input(same)) == T.buffer(tz_x) == T.buffer(output(same))
    assert entry(native(view_vctr(same())), 119) == 119.0
    tz_y = tensor(fact, [2, 3, 4, 5], "float", "nchw")
    push = connector(desc([2, 3, 4, 5], "float", "nhwc"), tz_y)              # push, different
    assert entry(native(transfer(itertools.count(), view_vctr(input(push)))), 119) == 119.0
    assert T.buffer(output(push)) == T.buffer(tz_y)
    assert T.buffer(input(push)) != T.buffer(output(push))
    assert entry(native(view_vctr(push())), 119) == 119.0
    push_same = connector(desc([2, 3, 4, 5], "float", "nchw"), tz_y)         # push, same
    assert T.buffer(output(push_same)) == T.buffer(tz_y) == T.buffer(input(push_same))


def test_shuffler(fact):
    """tt :263-275"""
    tz_x = tensor(fact, [6, 2, 1, 1], "float", [2, 1, 1, 1])
    tz_y = tensor(fact, [3, 2, 1, 1], "float", [1, 3, 1, 1])
    shuff = shuffler(tz_x, tz_y)
    transfer(range(1, 13), tz_x)
    assert seq(tz_x) == [float(i) for i in range(1, 13)]
    assert seq(tz_y) == [0.0] * 6
    shuff([0, 2, 1])
    assert seq(tz_y) == [1.0, 5.0, 3.0, 2.0, 6.0, 4.0]
    assert fact.handle.last_kernel().startswith("transform/gather")
    with pytest.raises(DiamondError):
        shuff([0, 2, 1, 1])
    with pytest.raises(DiamondError):
        shuff([0, 2, 8])
    assert shuff([0, 1]) == tz_y


def _batcher_checks(tz_x, tz_y, batch, batch_2):
    assert seq(tz_y) == [0.0] * 6
    assert batch(0, 0) == tz_y
    assert seq(tz_y) == [1.0, 3.0, 5.0, 2.0, 4.0, 6.0]
    transfer(itertools.repeat(0), tz_y)
    assert batch(1, 0) == tz_y
    assert seq(tz_y) == [3.0, 5.0, 7.0, 4.0, 6.0, 8.0]
    transfer(itertools.repeat(0), tz_y)
    assert batch_2(1, 1) == tz_y
    assert seq(tz_y) == [0.0, 3.0, 5.0, 0.0, 4.0, 6.0]
    for bad in ((8,), (0, -1), (7, -1), (-1,)):
        with pytest.raises(DiamondError):
            batch(*bad)


def test_batcher(fact):
    """tt :277-297"""
    tz_x = tensor(fact, [7, 2, 1, 1], "float", [2, 1, 1, 1])
    tz_y = tensor(fact, [3, 2, 1, 1], "float", [1, 3, 1, 1])
    batch, batch_2 = batcher(tz_x, tz_y, 3), batcher(tz_x, tz_y, 2)
    transfer(range(1, 15), tz_x)
    assert seq(tz_x) == [float(i) for i in range(1, 15)]
    _batcher_checks(tz_x, tz_y, batch, batch_2)


def test_batcher_tnc(fact):
    """tt :299-326"""
    tz_x_ntc = tensor(fact, [2, 7, 1], "float", "ntc")
    tz_x = tensor(fact, [2, 7, 1], "float", "tnc")
    tz_y = tensor(fact, [2, 3, 1], "float", "tnc")
    assert tz_x.batch_index() == 1
    sub_x = view_tz(tz_x, 3)
    batch, batch_2 = batcher(tz_x, tz_y, 3), batcher(tz_x, tz_y, 2)
    transfer(range(1, 15), tz_x)
    assert seq(transfer(sub_x, tensor(fact, [2, 3, 1], "float", "tnc"))) == [1.0, 2.0, 3.0, 8.0, 9.0, 10.0]
    sub_x.offset(3)
    assert seq(transfer(sub_x, tensor(fact, [2, 3, 1], "float", "tnc"))) == [4.0, 5.0, 6.0, 11.0, 12.0, 13.0]
    transfer(range(1, 15), tz_x_ntc)
    transfer(tz_x_ntc, tz_x)
    assert seq(tz_x) == [1.0, 3.0, 5.0, 7.0, 9.0, 11.0, 13.0, 2.0, 4.0, 6.0, 8.0, 10.0, 12.0, 14.0]
    _batcher_checks(tz_x, tz_y, batch, batch_2)


def test_half_and_bf16_storage(fact):
    """cudnn_tensor_test.clj:49-68 (f32 <-> f16, 100..400 survive) and the same for the new :bf16."""
    src = tensor(fact, [1, 4, 1, 1], "float", "nchw")
    transfer([100, 200, 300, 400], src)
    for dt in ("half", "bf16"):
        mid = tensor(fact, [1, 4, 1, 1], dt, "nchw")
        back = tensor(fact, [1, 4, 1, 1], "float", "nchw")
        transfer(src, mid)
        transfer(mid, back)
        assert seq(back) == [100.0, 200.0, 300.0, 400.0]
        assert list(native(mid)) == [100.0, 200.0, 300.0, 400.0]


# ---------------------------------------------------------------------------------- dnn -------

def vctr_of(tz, values):
    return T.vctr(tz, values).tolist()


def test_activation_relu(fact):
    """dt :28-54"""
    src_tz = tensor(fact, [1, 3, 2, 1], "float", "nchw")
    activ_bluep = dnn.activation(fact, src_tz, "relu")
    activ_infer = activ_bluep(src_tz)
    activ_train = activ_bluep(src_tz, src_tz)
    transfer([-0.5, 0, 0.2, 1, 0.3, -0.7], src_tz)
    assert seq(activ_infer()) == vctr_of(src_tz, [0, 0, 0.2, 1.0, 0.3, 0])
    assert seq(input(activ_infer)) == vctr_of(src_tz, [0, 0, 0.2, 1.0, 0.3, 0])
    assert seq(output(activ_infer)) == vctr_of(src_tz, [0, 0, 0.2, 1.0, 0.3, 0])
    transfer([-0.5, 0, 0.2, 1, 0.3, -0.7], src_tz)
    dnn.forward(activ_train)
    assert seq(input(activ_train)) == vctr_of(src_tz, [-0.5, 0, 0.2, 1, 0.3, -0.7])
    assert seq(output(activ_train)) == vctr_of(src_tz, [0, 0, 0.2, 1.0, 0.3, 0])
    transfer([-0.1, 0.1, 1, 2, 7, -0.6], dnn.diff_input(activ_train))
    dnn.backward(activ_train)
    assert seq(dnn.diff_output(activ_train)) == vctr_of(src_tz, [0, 0, 1, 2, 7.0, 0])


def test_activation_sigmoid(fact):
    """dt :56-82"""
    src_tz = tensor(fact, [1, 1, 1, 1], "float", "nchw")
    activ_bluep = dnn.activation(fact, src_tz, "sigmoid")
    activ_infer = activ_bluep(src_tz)
    activ_train = activ_bluep(src_tz, src_tz)
    transfer([0.7], src_tz)
    assert abs(seq(activ_infer())[0] - 0.6681877374649048) < 1e-6
    assert abs(seq(input(activ_infer))[0] - 0.6681877374649048) < 1e-6
    transfer([-0.5], src_tz)
    dnn.forward(activ_train)
    assert seq(input(activ_train)) == vctr_of(src_tz, [-0.5])
    assert abs(seq(output(activ_train))[0] - 0.3775407) < 1e-6
    transfer([-0.1], dnn.diff_input(activ_train))
    dnn.backward(activ_train)
    assert abs(seq(input(activ_train))[0] - (-0.02350037172436714)) < 1e-8


def test_activation_linear_tanh_elu(fact):
    """Activation kinds the shared suite does not exercise: layers against the C-level oracle."""
    import oracle
    x = [-1.5, -0.2, 0.0, 0.4, 2.0, 5.0]
    g = [1.0, -2.0, 0.5, 3.0, -1.0, 0.25]
    for kind, args in (("tanh", None), ("elu", {"alpha": 1.0}), ("linear", {"alpha": 2.0, "beta": 0.5})):
        src = tensor(fact, [1, 6, 1, 1], "float", "nchw")
        dsrc = tensor(fact, [1, 6, 1, 1], "float", "nchw")
        layer = dnn.activation(fact, src, kind, args)(src, dsrc)
        transfer(x, src)
        dnn.forward(layer)
        xa, ga = np.array(x, np.float32), np.array(g, np.float32)
        if kind == "linear":   # the cuDNN-style linear training layer is a pair of copies
            assert seq(output(layer)) == vctr_of(src, x)
        else:
            want = oracle.eltwise_fwd(kind, xa, np.zeros(6, np.float32), coef=(args or {}).get("alpha", 0.0))
            assert np.allclose(seq(output(layer)), want, rtol=3e-7, atol=0)
        transfer(g, dnn.diff_input(layer))
        dnn.backward(layer)
        if kind == "linear":
            assert seq(dnn.diff_output(layer)) == vctr_of(src, g)
        else:
            wantb = oracle.eltwise_bwd(kind, xa, ga, np.zeros(6, np.float32), coef=(args or {}).get("alpha", 0.0))
            assert np.allclose(seq(dnn.diff_output(layer)), wantb, rtol=3e-7, atol=0)


def test_sum(fact):
    """dt :855-874"""
    input0_tz = tensor(fact, [1, 2, 1, 1], "float", "nchw")
    input1_tz = tensor(fact, [1, 2, 1, 1], "float", "nchw")
    sum_bluep = dnn.sum(fact, [input0_tz, input1_tz])
    sum_train = sum_bluep([input0_tz, input1_tz], True, None)
    transfer([1, 2], input0_tz)
    transfer([3, 4], input1_tz)
    assert dnn.forward(sum_train, None) is sum_train
    assert seq(output(sum_train)) == [4.0, 6.0]
    transfer([0, 0], input1_tz)
    assert seq(input1_tz) == [0.0, 0.0]
    assert dnn.backward(sum_train, None) is sum_train
    assert seq(input0_tz) == [2.0, 3.0] and seq(input1_tz) == [2.0, 3.0]


def test_blas_generics_on_tensors(fact):
    """axpy! / scal! / copy! / nrm2 / amax on tensors: the TensorEngine of cudnn/factory.clj:161-196."""
    x = tensor(fact, [2, 3, 1, 1], "float", "nchw")
    y = tensor(fact, [2, 3, 1, 1], "float", "nchw")
    bias = tensor(fact, [1, 3, 1, 1], "float", "nchw")
    transfer([1, 2, 3, 4, 5, 6], x)
    transfer([10, 20, 30], bias)
    T.copy(x, y)
    T.axpy(2.0, x, y)
    assert seq(y) == [3.0, 6.0, 9.0, 12.0, 15.0, 18.0]
    T.axpy(1.0, bias, y)                     # bias broadcast over the batch
    assert seq(y) == [13.0, 26.0, 39.0, 22.0, 35.0, 48.0]
    T.scal(0.5, y)
    assert seq(y) == [6.5, 13.0, 19.5, 11.0, 17.5, 24.0]
    T.axpby(1.0, x, -1.0, y)
    assert seq(y) == [-5.5, -11.0, -16.5, -7.0, -12.5, -18.0]
    assert abs(T.nrm2(x) - np.sqrt(91.0)) < 1e-5 and T.amax(y) == 18.0 and T.sum(x) == 21.0


def test_concatenate(fact):
    """dt :657-684"""
    input0_tz = tensor(fact, [1, 1, 2, 2], "float", "nchw")
    input1_tz = tensor(fact, [1, 2, 2, 2], "float", "nchw")
    concat_bluep = dnn.concatenate(fact, 1, [input0_tz, input1_tz, input0_tz], None)
    concat_inf = concat_bluep([input0_tz, input1_tz, input0_tz])
    concat_train = concat_bluep([input0_tz, input1_tz, input0_tz], True, None)
    transfer(range(4), input0_tz)
    transfer(range(10, 90, 10), input1_tz)
    want = [0.0, 1.0, 2.0, 3.0, 10.0, 20.0, 30.0, 40.0, 50.0, 60.0, 70.0, 80.0, 0.0, 1.0, 2.0, 3.0]
    n0 = fact.handle.launch_count()
    assert seq(concat_inf()) == want
    assert fact.handle.launch_count() - n0 == 1 and fact.handle.last_kernel().startswith("multi-transform")
    assert dnn.forward(concat_train, None) is concat_train
    assert seq(output(concat_train)) == want
    transfer(itertools.repeat(0.0), input0_tz)
    transfer(itertools.repeat(0.0), input1_tz)
    assert seq(input0_tz) == [0.0] * 4
    assert dnn.backward(concat_train, None) is concat_train
    assert seq(input0_tz) == [0.0, 1.0, 2.0, 3.0]
    assert seq(input1_tz) == [10.0, 20.0, 30.0, 40.0, 50.0, 60.0, 70.0, 80.0]


def test_branch(fact):
    """dt :686-710"""
    dst0_desc = desc([1, 1, 2, 2], "float", "nchw")
    dst1_desc = desc([1, 2, 2, 2], "float", "nchw")
    input_tz = tensor(fact, [1, 3, 2, 2], "float", "nchw")
    branch_bluep = dnn.branch(fact, input_tz, 1, [dst0_desc, dst1_desc])
    branch_inf = branch_bluep(input_tz)
    branch_train = branch_bluep(input_tz, True, None)
    data = [0.0, 1.0, 2.0, 3.0, 10.0, 20.0, 30.0, 40.0, 50.0, 60.0, 70.0, 80.0]
    transfer(data, input_tz)
    assert [seq(t) for t in branch_inf()] == [data[:4], data[4:]]
    assert dnn.forward(branch_train, None) is branch_train
    assert [seq(t) for t in output(branch_train)] == [data[:4], data[4:]]
    transfer(itertools.repeat(0.0), input_tz)
    assert seq(input_tz) == [0.0] * 12
    assert dnn.backward(branch_train, None) is branch_train
    assert seq(input_tz) == data


def test_split(fact):
    """dt :876-898"""
    input_tz = tensor(fact, [1, 2, 1, 1], "float", "nchw")
    split_bluep = dnn.split(fact, input_tz, 2)
    split_inf = split_bluep(input_tz)
    split_train = split_bluep(input_tz, True, None)
    transfer([1.0, 2.0], input_tz)
    assert [seq(t) for t in split_inf()] == [[1.0, 2.0], [1.0, 2.0]]
    assert dnn.forward(split_train, None) is split_train
    assert [seq(t) for t in output(split_train)] == [[1.0, 2.0], [1.0, 2.0]]
    transfer(itertools.repeat(0.0), input_tz)
    transfer([1.0, 2.0], dnn.diff_input(split_train)[0])
    transfer([3.0, 4.0], dnn.diff_input(split_train)[1])
    assert dnn.backward(split_train, None) is split_train
    assert seq(input_tz) == [2.0, 3.0]


def test_quadratic_and_mean_absolute_cost(fact):
    """dt :321-334 (the cost numbers; the network in front of it is outside this engine, so the cost
    sits directly on an output tensor): quadratic 0.68625, gradient [0.15 -1.65]."""
    out_tz = tensor(fact, [2, 1], "float", "nc")
    train_tz = tensor(fact, [2, 1], "float", "nc")
    quad = dnn.cost(out_tz, train_tz, "quadratic")
    transfer([0.25, 0.35], train_tz)
    transfer([0.4, -1.3], out_tz)
    assert abs(quad() - 0.6862499438341274) < 1e-6
    assert np.allclose(seq(out_tz), [0.15, -1.65], rtol=1e-6)      # a - y lands in the diff-input
    transfer([0.4, -1.3], out_tz)
    mae = dnn.cost(out_tz, train_tz, "mean-absolute")
    assert abs(mae() - (0.15 + 1.65) / 2) < 1e-6
    with pytest.raises(DiamondError):
        dnn.cost(out_tz, train_tz, "hinge")


def test_crossentropy_cost(fact):
    """dt :335-346: y = [0.25 0.65], a = [0.4 0.1] -> 1.0728740692138672; invoking the cost leaves
    the output alone, backward leaves a - y in the gradient after the linear part."""
    out_tz = tensor(fact, [2, 1], "float", "nc")
    train_tz = tensor(fact, [2, 1], "float", "nc")
    ce = dnn.cost(out_tz, train_tz, "crossentropy")
    transfer([0.25, 0.65], train_tz)
    transfer([0.4, 0.1], out_tz)
    assert abs(ce() - 1.0728740692138672) < 2e-7
    assert seq(out_tz) == vctr_of(out_tz, [0.4, 0.1])
    assert ce.backward() is ce
    assert np.allclose(seq(dnn.diff_output(ce)), [0.15, -0.55], rtol=1e-6)
    # behind a sigmoid layer the gradient lands in the layer's diff-output (its diff-z)
    src_tz = tensor(fact, [2, 1], "float", "nc")
    dsrc_tz = tensor(fact, [2, 1], "float", "nc")
    layer = dnn.activation(fact, src_tz, "sigmoid")(src_tz, dsrc_tz)
    transfer([-0.4054651, -2.1972246], src_tz)                 # logit(0.4), logit(0.1)
    layer.forward()
    ce2 = dnn.cost(layer, train_tz, "crossentropy")
    assert abs(ce2() - 1.0728740692138672) < 1e-6
    ce2.backward()
    assert np.allclose(seq(dnn.diff_output(layer)), [0.15, -0.55], atol=1e-6)


def test_costs_against_oracle(fact):
    """All three costs on [64, 1000] outputs against the oracle's float restatement and its double
    truth (1e-5 relative), a - y bit-exact; float and double tensors."""
    import oracle
    rng = np.random.default_rng(77)
    a = rng.uniform(0.001, 0.999, (64, 1000)).astype(np.float32)
    y = (rng.random((64, 1000)) < 0.1).astype(np.float32) * 0.9 + 0.05
    for dt, npt in (("float", np.float32), ("double", np.float64)):
        for kind in ("quadratic", "mean-absolute", "crossentropy"):
            out_tz = tensor(fact, [64, 1000], dt, "nc")
            train_tz = tensor(fact, [64, 1000], dt, "nc")
            transfer(a.astype(npt).reshape(-1), out_tz)
            transfer(y.astype(npt).reshape(-1), train_tz)
            c = dnn.cost(out_tz, train_tz, kind)
            got = c()
            want, truth, diff = oracle.cost(kind, a, y, want_diff=True)
            assert abs(got - truth) <= 1e-5 * abs(truth), (dt, kind, got, truth)
            assert abs(got - want) <= 1e-5 * abs(want), (dt, kind, got, want)
            if kind == "crossentropy":      # invoking it only reads; backward writes a - y
                assert np.array_equal(np.array(seq(out_tz), dtype=npt), a.astype(npt).reshape(-1))
                c.backward()
            d = np.array(seq(dnn.diff_output(c)), dtype=npt)
            if dt == "float":
                assert np.array_equal(d.astype(np.float32), diff.reshape(-1)), (dt, kind)
            else:
                assert np.array_equal(d, (a.astype(np.float64) - y.astype(np.float64)).reshape(-1)), (dt, kind)


def test_branch_concat_large_against_oracle(fact, dev):
    """Branch then concatenate of a [8, 96, 14, 14] tensor cut 32/48/16 along channels, against the
    oracle's per-sub-tensor reorders: the 16-byte path of the multi-copy kernel."""
    import oracle
    shape = [8, 96, 14, 14]
    parts = [[8, 32, 14, 14], [8, 48, 14, 14], [8, 16, 14, 14]]
    x = oracle.gen_uniform(shape, -1, 1, 3).reshape(-1)
    src = tensor(fact, shape, "float", "nchw")
    transfer(x, src)
    br = dnn.branch(fact, src, 1, [desc(p, "float", "nchw") for p in parts])(src)
    outs = br()
    assert fact.handle.last_kernel() == "multi-transform/vec"
    xv = x.reshape(shape)
    c0 = 0
    for p, t in zip(parts, outs):
        want = np.ascontiguousarray(xv[:, c0:c0 + p[1]]).reshape(-1)
        c0 += p[1]
        assert np.array_equal(np.asarray(seq(t), np.float32), want)
    cat = dnn.concatenate(fact, 1, outs)(outs)
    assert np.array_equal(np.asarray(seq(cat()), np.float32), x)


def test_zero_sized_tensors(fact):
    """Zero extents never reach the C library: descriptors stay general, transformers are no-ops
    (cudnn/tensor.clj:119-122, 204-207) and transfers do nothing (:584, :598)."""
    z = tensor(fact, [0, 3, 2, 2], "float", "nchw")
    w = tensor(fact, [0, 3, 2, 2], "float", "nhwc")
    assert T.dim(z) == 0 and T.shape(z) == [0, 3, 2, 2] and asum(z) == 0.0
    assert transformer(z, w)() is not None
    assert transfer([1, 2, 3], z) is z
    assert transfer(z, w) is w
    assert entry_(z, 1.0) is z


def test_factory_protocol_surface(fact):
    """The factory answers every DnnFactory / CostFactory method of base/internal/protocols.clj:68-129:
    the hot-path ones build blueprints, the contraction ones refuse like the cuDNN factory's
    missing pieces."""
    src = tensor(fact, [2, 4, 1, 1], "float", "nchw")
    f = fact.diamond_factory()
    assert f.activ_op_blueprint(src, "relu", 0.0, 0.0) is not None
    assert f.split_blueprint(src, 2)(src)() is not None
    parts = [desc([2, 1, 1, 1], "float", "nchw"), desc([2, 3, 1, 1], "float", "nchw")]
    transfer(range(8), src)
    outs = f.branch_blueprint(src, 1, parts)(src)()
    assert [seq(t) for t in outs] == [[0.0, 4.0], [1.0, 2.0, 3.0, 5.0, 6.0, 7.0]]
    cat = f.concat_blueprint(parts, 1)(outs)
    assert seq(cat()) == [float(i) for i in range(8)]
    train = tensor(fact, [2, 4, 1, 1], "float", "nchw")
    for make in (f.quadratic_cost, f.mean_absolute_cost, f.crossentropy_cost):
        assert callable(make(src, train))
    for name in ("inner_product_blueprint", "fc_blueprint", "convolution_blueprint", "pooling_blueprint",
                 "batch_norm_blueprint", "gaussian_dropout_blueprint", "rnn_op_blueprint", "rnn_blueprint",
                 "abbreviate_blueprint"):
        with pytest.raises(DiamondError):
            getattr(f, name)(src)


def test_captured_layer_chain_replays(fact):
    """A chain of layers recorded once with ``capture`` and replayed as one graph launch gives the
    same bits as the calls made one by one, also after the inputs change."""
    rng = np.random.default_rng(5)
    shape = [4, 8, 6, 6]
    src = tensor(fact, shape, "float", "nchw")
    dsrc = tensor(fact, shape, "float", "nchw")
    nhwc = tensor(fact, shape, "float", "nhwc")
    layer = dnn.activation(fact, src, "tanh")(src, dsrc)
    tr = transformer(dsrc, nhwc)

    def step():                     # the gradient fed back is the output itself (same buffer for tanh)
        layer.forward()
        layer.backward()
        tr()

    calls = fact.capture(step)
    for seed in (1, 2):
        x = rng.standard_normal(int(np.prod(shape))).astype(np.float32)
        transfer(x, src)
        step()
        want = seq(nhwc)
        transfer(x, src)
        transfer(itertools.repeat(0.0), nhwc)
        n0 = fact.handle.launch_count()
        calls()
        assert fact.handle.launch_count() == n0          # no library call on the host: one graph launch
        assert seq(nhwc) == want
    calls.release()


def test_crossentropy_log_accuracy(fact, dev):
    """The cross-entropy kernel's own log (two at a time, packed arithmetic), element by element:
    with y = 1 the cost of a one-element tensor is |log(a)|, with y = 0 it is |log(1.0000001 - a)|.
    4000 values from the smallest normal float up to 1, dense near 1 where log cancels: within
    2 ulp of the double-precision log; zero and denormal inputs take the library path."""
    import torch
    from conftest import ulp_diff_f32
    rng = np.random.default_rng(3)
    a = np.concatenate([
        np.exp(rng.uniform(np.log(1.2e-38), 0.0, 2000)),
        1.0 - np.exp(rng.uniform(np.log(1e-7), np.log(0.5), 1500)),
        np.array([0.5, 0.25, 0.70710677, 0.70710683, 0.9999999, 1.0, 1e-40, 3e-39]),
    ]).astype(np.float32)
    n = a.size
    ta = dev.put(a)
    ones, zeros = dev.put(np.ones(n, np.float32)), dev.put(np.zeros(n, np.float32))
    out = torch.zeros(2 * n, dtype=torch.float32, device=fact.device)
    d = core_desc([1, 1])
    for i in range(n):
        core.cost_diff(fact.handle, "crossentropy", d, ta.data_ptr() + 4 * i, ones.data_ptr() + 4 * i, None,
                       out.data_ptr() + 4 * i)
        core.cost_diff(fact.handle, "crossentropy", d, ta.data_ptr() + 4 * i, zeros.data_ptr() + 4 * i, None,
                       out.data_ptr() + 4 * (n + i))
    fact.synchronize()
    got = out.cpu().numpy()
    want_log = np.abs(np.log(a.astype(np.float64))).astype(np.float32)
    assert ulp_diff_f32(got[:n], want_log).max() <= 2
    one_minus = (np.float32(1.0000001) - a).astype(np.float32)          # formed in float like the kernel
    want_l1 = np.abs(np.log(one_minus.astype(np.float64))).astype(np.float32)
    assert ulp_diff_f32(got[n:], want_l1).max() <= 2


def core_desc(shape):
    from deep_diamond_b200 import core as _core
    return _core.tensor_descriptor(shape, "float", "nc")


def test_transfer_async_pipeline(fact):
    """Uploads and downloads on the factory's copy streams: results equal the synchronous path, a
    download started before its source is overwritten still delivers the old contents once
    ``before_overwrite`` guards the overwrite, and mixed cases fall back to ``transfer``."""
    import torch
    shape = [8, 16, 32, 32]
    n = int(np.prod(shape))
    rng = np.random.default_rng(9)
    src = tensor(fact, shape, "float", "nchw")
    dst = tensor(fact, shape, "float", "nchw")
    layer = dnn.activation(fact, src, "relu")(src, dst)
    hx = [torch.from_numpy(rng.standard_normal(n).astype(np.float32)).pin_memory() for _ in range(3)]
    hy = [torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(3)]
    pend = []
    for i in range(3):
        T.transfer_async(hx[i].numpy(), src)
        if pend:
            pend[-1].before_overwrite()               # the previous result is still being read
        layer.forward()
        pend.append(T.transfer_async(layer.output(), hy[i].numpy()))
    for i, p in enumerate(pend):
        assert p.wait() is not None and p.done()
        assert np.array_equal(hy[i].numpy(), np.maximum(hx[i].numpy(), 0.0)), i
    # a list source is not a raw copy: done at once, returned finished
    p = T.transfer_async([1.0] * n, src)
    assert p.done() and p.wait() is src
    assert seq(src)[:3] == [1.0, 1.0, 1.0]
