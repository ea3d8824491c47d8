"""GPU parity of ddReduceTensor, one case per launch plan: shapes picked so that each kernel of
csrc/dd_reduce_kernels.cuh and each way of combining split partials is the one that runs (asserted
through ddGetLastKernelName), each against the CPU oracle on the same seeded input.  The shapes are
the per-GPU shards of the benchmark configurations and their neighbours.  The call replaced:
cudnn/core.clj:213-231 (`reduce-tensor`); the oracle follows dnnl/core.clj:796-803.
"""
import numpy as np
import pytest

from deep_diamond_b200 import core
from test_gpu_reduce import run_reduce

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("op", ["add", "avg", "norm2", "max", "amax"])
@pytest.mark.parametrize("shape,yshape,kernel", [
    ([8, 1024, 32, 32], [1, 1024, 1, 1], "reduce/row-lean"),    # 2 chunks per run, 128-thread CTAs, no split
    ([8, 1024, 32, 32], [8, 1, 1, 1], "reduce/row-lean"),       # one long run per output, folded into rows; ~70 splits
    ([32, 64, 28, 28], [1, 64, 1, 1], "reduce/row-lean"),       # 784-long runs: 4 chunks of 64 lanes, split over r1 (arrival counters)
    ([32, 256, 28, 28], [1, 256, 1, 1], "reduce/row-lean"),     # the same with 256 outputs: 8 splits of 4 runs
    ([37, 200, 28, 28], [1, 200, 1, 1], "reduce/row-lean"),     # uneven: 9 splits of 4 runs and one of 1
    ([2, 3, 28, 28], [1, 3, 1, 1], "reduce/row"),               # short reductions: warp groups, general walk
    ([3, 5, 7, 1030], [3, 5, 7, 1], "reduce/row"),              # runs that are not 16-byte aligned
    ([8, 1024, 32, 32], [8, 1, 32, 32], "reduce/col-cluster"),  # 8 splits of a tile as one cluster
    ([16, 1024, 32, 32], [16, 1, 32, 32], "reduce/col-cluster"),  # 4 splits
    ([64, 64, 16, 16], [1, 64, 16, 16], "reduce/col"),          # no split: the general column kernel
    ([256, 20, 28, 28], [256, 1, 28, 28], "reduce/col"),        # 784 columns: tile width narrowed by padding
])
def test_each_plan_against_the_oracle(fact, dev, oracle, op, shape, yshape, kernel):
    run_reduce(fact, dev, oracle, op, shape, yshape, seed=hash((op, tuple(shape))) % 1000, expect=kernel)
    assert fact.handle.last_kernel() == kernel


@pytest.mark.parametrize("op", ["add", "avg", "norm1", "norm2", "max", "min", "amax", "mul"])
@pytest.mark.parametrize("shape", [[64, 256, 7, 7], [16, 96, 13, 13], [9, 8, 3, 5], [40, 4, 1, 50]])
def test_dense_odd_runs_reduce_in_two_stages(fact, dev, oracle, op, shape):
    """Per-channel reductions of nchw tensors whose maps are not whole 16-byte vectors (49, 169, 15
    elements; and rows of 50 that are not 16-byte aligned from one channel to the next): a column reduce over
    n with (c, h, w) as one kept dim, then a fold of each channel's run."""
    n, c, h, w = shape
    run_reduce(fact, dev, oracle, op, shape, [1, c, 1, 1], seed=71, expect="reduce/col+fold-runs")


@pytest.mark.parametrize("op", ["add", "avg", "norm2", "max", "min", "amax"])
@pytest.mark.parametrize("shape", [[16, 64, 7, 7], [3, 256, 13, 13], [1, 96, 3, 5], [5, 40, 1, 6]])
def test_odd_kept_rows_reduce_in_periodic_sets(fact, dev, oracle, op, shape):
    """Reductions over C of nchw tensors whose maps are not whole vectors (49, 169, 15, 6 elements):
    four (or two) consecutive channel rows are, so the column reduce runs over groups of them and a
    second launch folds the interleaved sets."""
    n, c, h, w = shape
    run_reduce(fact, dev, oracle, op, shape, [n, 1, h, w], seed=73, expect="reduce/col+fold-sets")


def test_two_launch_forms_blend_with_alpha_and_beta(fact, dev, oracle):
    """y = alpha * reduce(x) + beta * y through both two-launch forms (the blend happens in the
    second launch), and double precision through the first."""
    run_reduce(fact, dev, oracle, "add", [32, 48, 7, 7], [1, 48, 1, 1], alpha=0.5, beta=2.0, seed=74,
               expect="reduce/col+fold-runs")
    run_reduce(fact, dev, oracle, "norm2", [32, 48, 7, 7], [1, 48, 1, 1], alpha=-1.5, beta=0.25, seed=75,
               expect="reduce/col+fold-runs")
    run_reduce(fact, dev, oracle, "max", [8, 64, 7, 7], [8, 1, 7, 7], alpha=0.5, beta=2.0, seed=76,
               expect="reduce/col+fold-sets")
    run_reduce(fact, dev, oracle, "avg", [8, 64, 5, 5], [8, 1, 5, 5], alpha=3.0, beta=-1.0, seed=77,
               expect="reduce/col+fold-sets")
    run_reduce(fact, dev, oracle, "add", [16, 24, 3, 3], [1, 24, 1, 1], seed=78, dtype="double",
               expect="reduce/col+fold-runs")
    run_reduce(fact, dev, oracle, "amax", [4, 64, 3, 3], [4, 1, 3, 3], seed=79, dtype="double",
               expect="reduce/col+fold-sets")


def test_bias_gradient_on_seven_by_seven_maps(fact, dev, oracle):
    """ddConvolutionBackwardBias (sum of dy over n, h, w) on [32, 512, 7, 7]: the same two-stage plan."""
    shape = [32, 512, 7, 7]
    dyv = oracle.gen_signed_lognormal(shape, 72)
    want = dyv.astype(np.float64).sum(axis=(0, 2, 3))
    mag = np.abs(dyv.astype(np.float64)).sum(axis=(0, 2, 3))
    tdy, tdb = dev.put(dyv), dev.put(np.zeros(512, np.float32))
    core.convolution_bwd_bias(fact.handle, 1.0, core.tensor_descriptor(shape, "float", "nchw"), tdy, 0.0,
                              core.tensor_descriptor([1, 512, 1, 1], "float", "nchw"), tdb)
    assert fact.handle.last_kernel() == "reduce/col+fold-runs"
    got = dev.get(tdb, np.float32).astype(np.float64)
    assert (np.abs(got - want) <= 1e-5 * np.abs(want) + 64 * 6e-8 * mag).all()


def test_hundreds_of_splits_folded_by_a_warp(fact, dev, oracle):
    """One output over 6.4 M elements: more than 32 splits, so the last arrival folds the partials
    with a whole warp; and the same through the entry point that has no arrival counters (its
    partials are folded by the separate finishing kernel), which must give the same bits."""
    from test_zz_no_alloc import no_alloc_reduce
    shape, yshape = [32, 256, 28, 28], [1, 1, 1, 1]
    for op in ("add", "norm2", "max"):
        run_reduce(fact, dev, oracle, op, shape, yshape, seed=5, expect="reduce/row-lean")
    x = oracle.gen_signed_lognormal(shape, 6)
    xd, yd = core.tensor_descriptor(shape, "float", "nchw"), core.tensor_descriptor(yshape, "float", "nchw")
    rtd = core.reduce_tensor_descriptor("add", "float")
    need = core.reduction_workspace_size(fact.handle, rtd, xd, yd)
    assert need > 32 * 4                                   # more than 32 partials
    tx = dev.put(x)
    a, b = dev.put(np.zeros(1, np.float32)), dev.put(np.zeros(1, np.float32))
    core.reduce_tensor(fact.handle, rtd, 1.0, xd, tx, 0.0, yd, a)
    st, msg = no_alloc_reduce(fact, "add", xd, tx, yd, b)
    assert st == 0, msg
    assert dev.get(a, np.uint32)[0] == dev.get(b, np.uint32)[0]
    truth = float(x.astype(np.float64).sum())
    assert abs(float(dev.get(a, np.float32)[0]) - truth) <= 32 * 6e-8 * float(np.abs(x.astype(np.float64)).sum())


@pytest.mark.parametrize("tag,np_t,to16", [("half", np.float16, None), ("bf16", np.uint16, "bf16")])
@pytest.mark.parametrize("op,shape,yshape,kernel", [
    ("max", [96, 96, 28, 28], [96, 1, 28, 28], "reduce/col-lean"),    # 98 vectors: 14 lanes along the kept dim
    ("add", [96, 96, 28, 28], [96, 1, 28, 28], "reduce/col-lean"),
    ("add", [16, 128, 28, 28], [1, 128, 1, 1], "reduce/row-lean"),
    ("add", [70, 256, 28, 28], [1, 256, 1, 1], "reduce/row-cluster"),   # 16 splits of 5 runs: 14 used, 2 empty
    ("max", [70, 256, 28, 28], [1, 256, 1, 1], "reduce/row-cluster"),
    ("add", [64, 200, 28, 28], [1, 200, 1, 1], "reduce/row-cluster"),   # 16 splits of 4 runs, all used
    ("max", [8, 256, 32, 32], [8, 1, 32, 32], "reduce/col-cluster"),
    # 14 x 14 maps: runs of 196 elements start on 8-byte boundaries only, so 8-byte loads
    ("max", [32, 512, 14, 14], [32, 1, 14, 14], "reduce/col+fold-sets"),  # pairs of rows are whole vectors
    ("add", [32, 512, 14, 14], [32, 1, 14, 14], "reduce/col+fold-sets"),
    ("max", [32, 14, 14, 14], [32, 1, 14, 14], "reduce/col-v8"),          # too few rows for that: 8-byte loads
    ("add", [32, 15, 14, 14], [32, 1, 14, 14], "reduce/col-v8"),          # an odd number of rows
    ("add", [32, 512, 14, 14], [1, 512, 1, 1], "reduce/col+fold-runs"),  # dense odd runs: column reduce over n, then a fold of each run
    ("add", [6, 512, 14, 14], [1, 512, 1, 1], "reduce/row-v8"),           # too few rows for that: 8-byte loads along the runs
    ("max", [2, 6, 14, 14], [1, 6, 1, 1], "reduce/row-v8"),
    ("add", [3, 5, 7, 10], [3, 1, 7, 10], "reduce/col"),          # 70 elements per row: not a multiple of 4
])
def test_sixteen_bit_types(fact, dev, oracle, tag, np_t, to16, op, shape, yshape, kernel):
    """16-bit storage, fp32 accumulation; the result is rounded once to the 16-bit type, so it must be
    within one unit of that type of the oracle's (which rounds the same way)."""
    rng = np.random.default_rng(11)
    xf = rng.standard_normal(int(np.prod(shape))).astype(np.float32)
    if to16 == "bf16":
        x = (xf.view(np.uint32) >> 16).astype(np.uint16)          # truncated to bf16 bit patterns
        xv = (x.astype(np.uint32) << 16).view(np.float32)
    else:
        x = xf.astype(np.float16)
        xv = x.astype(np.float32)
    axes = tuple(i for i in range(4) if yshape[i] == 1 and shape[i] != 1)
    ref = xv.reshape(shape).astype(np.float64)
    ref = ref.max(axis=axes) if op == "max" else ref.sum(axis=axes)
    xd, yd = core.tensor_descriptor(shape, tag, "nchw"), core.tensor_descriptor(yshape, tag, "nchw")
    ty = dev.empty(int(np.prod(yshape)) * 2)
    core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor(op, "float"), 1.0, xd, dev.put(x), 0.0, yd, ty)
    assert fact.handle.last_kernel() == kernel
    got16 = dev.get(ty, np_t)
    got = (got16.astype(np.uint32) << 16).view(np.float32) if to16 == "bf16" else got16.astype(np.float32)
    got = got.reshape(ref.shape).astype(np.float64)
    if op == "max":
        assert np.array_equal(got, ref)
    else:
        unit = 2.0 ** (-7 if to16 == "bf16" else -10)                 # one unit of the 16-bit type, relative
        mag = np.abs(xv.reshape(shape).astype(np.float64)).sum(axis=axes)
        assert (np.abs(got - ref) <= unit * np.abs(ref) + 64 * 6e-8 * mag).all()
