"""GPU parity of the 1-byte transposing reorder whose tiles the copy engine (TMA) loads: bit for bit
against the CPU oracle, on tensors large enough that the library picks that kernel, with edges that
are ragged in both tiled dims, with and without a batch dim, both directions, int8 and uint8.

That kernel is an alternative to the register-staged tile kernel (it measured within a few per cent
of it either way), chosen per handle by DD_B200_TILE_TMA=1 in the environment of ddCreate: the
tests here run on such a handle, and one checks that a default handle keeps the other kernel.

The reorder itself is the reference's transformer between an nchw and an nhwc int8 tensor
(deep-diamond-dnnl/test/uncomplicate/diamond/internal/dnnl/core_test.clj:260-361 at the C level).
"""
import os

import numpy as np
import pytest

from deep_diamond_b200 import core
from test_gpu_transform import nchw, nhwc, perm_strides, run_case

pytestmark = pytest.mark.gpu

TMA = "transform/tile-tma"


@pytest.fixture(scope="module")
def fact():
    """A factory whose handle was created with the TMA form switched on."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from deep_diamond_b200 import b200_factory
    old = os.environ.get("DD_B200_TILE_TMA")
    os.environ["DD_B200_TILE_TMA"] = "1"
    try:
        f = b200_factory()
    finally:
        if old is None:
            del os.environ["DD_B200_TILE_TMA"]
        else:
            os.environ["DD_B200_TILE_TMA"] = old
    yield f
    f.release()


@pytest.fixture(scope="module")
def dev(fact):
    from conftest import Dev
    return Dev(fact)


def test_a_default_handle_keeps_the_register_kernel(oracle):
    from conftest import Dev
    from deep_diamond_b200 import b200_factory
    f = b200_factory()
    try:
        shape = [64, 256, 28, 28]
        run_case(f, Dev(f), oracle, shape, nchw(shape), nhwc(shape), "byte", "byte", seed=50, expect="transform/tile")
    finally:
        f.release()


def clean(fact):
    fact.synchronize()
    assert fact.handle.device_fault() == 0


@pytest.mark.parametrize("dt", ["byte", "uint8"])
def test_benchmark_shard_both_ways(fact, dev, oracle, dt):
    shape = [256, 256, 28, 28]  # one GPU's eighth of the [2048,256,28,28] int8 reorder
    run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), dt, dt, seed=51, expect=TMA)
    run_case(fact, dev, oracle, shape, nhwc(shape), nchw(shape), dt, dt, seed=52, expect=TMA)
    clean(fact)


@pytest.mark.parametrize("shape", [
    [192, 144, 12, 40],   # A = 480 bytes (30 vectors), B = 144: partial tiles along both
    [80, 272, 16, 48],    # A = 768, B = 272 (two full tiles of 128 and one of 16)
    [40, 1024, 32, 32],   # A = 1024: full tiles only
    [700, 48, 16, 16],    # B below one tile, many batches
    [67, 400, 4, 148],    # A = 592 (37 vectors, prime), odd batch count
])
def test_ragged_edges_and_batches(fact, dev, oracle, shape):
    run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), "byte", "byte", seed=53, expect=TMA)
    run_case(fact, dev, oracle, shape, nhwc(shape), nchw(shape), "byte", "byte", seed=54, expect=TMA)
    clean(fact)


def test_plain_matrix_transposition(fact, dev, oracle):
    # no batch dim: [4096, 6000] bytes, row-major to column-major
    shape = [4096, 6000]
    run_case(fact, dev, oracle, shape, [6000, 1], [1, 4096], "uint8", "uint8", seed=55, expect=TMA)
    clean(fact)


def test_padded_source_rows(fact, dev, oracle):
    # the source is a window of a wider parent: rows of 784 bytes in a pitch of 800, channel pitch
    # 800 * 1, batch pitch 260 channels; the destination is dense nhwc
    shape = [128, 256, 28, 28]
    sx = [260 * 800, 800, 28, 1]
    run_case(fact, dev, oracle, shape, sx, nhwc(shape), "byte", "byte", seed=56, expect=TMA)
    clean(fact)


def test_two_batch_dims_stay_with_the_register_kernel(fact, dev, oracle):
    # n and h both outside the transposed pair (c <-> w) and not mergeable: the tensor map of the
    # TMA form has three dims (A, B, one batch dim)
    shape = [64, 128, 12, 256]
    sx = perm_strides(shape, [0, 1, 2, 3])   # n c h w
    sy = perm_strides(shape, [2, 0, 3, 1])   # h n w c
    run_case(fact, dev, oracle, shape, sx, sy, "byte", "byte", seed=57, expect="transform/tile")
    clean(fact)


def test_small_tensors_stay_with_the_register_kernel(fact, dev, oracle):
    shape = [2, 144, 4, 40]
    run_case(fact, dev, oracle, shape, nchw(shape), nhwc(shape), "byte", "byte", seed=58, expect="transform/tile")
    clean(fact)


def test_back_to_back_calls_share_nothing(fact, dev, oracle):
    """Two reorders in a row on one stream (the second launch may start while the first drains):
    each output is complete and the inverse brings the source back."""
    shape = [192, 256, 28, 28]
    n = int(np.prod(shape))
    rng = np.random.default_rng(59)
    xs = rng.integers(-128, 128, n).astype(np.int8)
    dx, dm, dz = dev.put(xs), dev.put(np.zeros(n, np.int8)), dev.put(np.zeros(n, np.int8))
    a = core.tensor_descriptor(shape, "byte", nchw(shape))
    b = core.tensor_descriptor(shape, "byte", nhwc(shape))
    for _ in range(3):
        core.transform_tensor(fact.handle, 1.0, a, dx, 0.0, b, dm)
        assert fact.handle.last_kernel() == TMA
        core.transform_tensor(fact.handle, 1.0, b, dm, 0.0, a, dz)
    clean(fact)
    assert np.array_equal(dev.get(dz, np.int8), xs)
    want = xs.reshape(shape).transpose(0, 2, 3, 1).reshape(-1)
    assert np.array_equal(dev.get(dm, np.int8), want)
