"""The reduce entry point that allocates nothing, ddReduceTensorNoAlloc, called through the C ABI.

It exists for callers that may not allocate device memory at the point of the call (a latency-critical
loop, a process whose memory pool owns the whole GPU, a host that forbids allocation after start-up)
and therefore cannot create a library handle either.  Its split-reduction partials live in a fixed
array inside the library, so this test checks (1) that its results equal ddReduceTensor's exactly --
same plan, same kernels -- on two calls in a row that both go through that array, (2) that a
reduction too large for the array is refused with a readable reason, and (3) that stale contents of
the array from an earlier call do not leak into a later one.  The file sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest

from deep_diamond_b200 import _lib, core

pytestmark = pytest.mark.gpu

OPS = {"add": 0, "max": 3, "avg": 5, "norm2": 7}


def no_alloc_reduce(fact, op, xd, x, yd, y, alpha=1.0, beta=0.0, nan_opt=1):
    err = ctypes.create_string_buffer(512)
    a, b = ctypes.c_float(alpha), ctypes.c_float(beta)
    st = _lib.lib.ddReduceTensorNoAlloc(ctypes.c_void_p(fact.stream.cuda_stream), OPS[op], nan_opt,
                                        ctypes.byref(a), xd.ptr, core._ptr(x), ctypes.byref(b), yd.ptr,
                                        core._ptr(y), err, len(err))
    return st, err.value.decode()


CASES = [
    ("norm2", [4, 64, 32, 32], [4, 1, 1, 1]),      # row kernel, reduce range split over CTAs
    ("add", [2048, 8, 1, 16], [1, 8, 1, 16]),      # column kernel, split
    ("avg", [1, 1, 1, 1 << 20], [1, 1, 1, 1]),     # one output, many splits
    ("max", [64, 16, 32, 32], [1, 16, 1, 1]),      # split, exact op
]


def test_matches_the_handle_entry_point_on_consecutive_calls(fact, dev):
    import torch
    rng = np.random.default_rng(40)
    for round_ in range(2):                         # two passes over all cases: calls in a row
        for op, shape, yshape in CASES:
            x = (np.exp(rng.standard_normal(int(np.prod(shape)))) *
                 np.where(rng.random(int(np.prod(shape))) < 0.5, -1, 1)).astype(np.float32)
            y0 = rng.standard_normal(int(np.prod(yshape))).astype(np.float32)
            xd = core.tensor_descriptor(shape, "float", "nchw")
            yd = core.tensor_descriptor(yshape, "float", "nchw")
            tx = dev.put(x)
            t_ref, t_new = dev.put(y0), dev.put(y0)
            rtd = core.reduce_tensor_descriptor(op, "float")
            assert core.reduction_workspace_size(fact.handle, rtd, xd, yd) > 0   # it does use scratch
            core.reduce_tensor(fact.handle, rtd, 1.5, xd, tx, 0.5, yd, t_ref)
            st, msg = no_alloc_reduce(fact, op, xd, tx, yd, t_new, alpha=1.5, beta=0.5)
            assert st == 0, msg
            got, want = dev.get(t_new, np.float32), dev.get(t_ref, np.float32)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (op, shape, round_)
    torch.cuda.synchronize()


def test_refuses_what_does_not_fit(fact, dev):
    # a reduction whose plan needs more scratch than the built-in array holds (few tiles of outputs,
    # a long reduced range: many splits per output)
    rtd = core.reduce_tensor_descriptor("add", "float")
    need = 0
    for rows, cols in ((8192, 2048), (256, 20000), (65536, 1024), (32768, 4096)):
        xd = core.tensor_descriptor([rows, cols], "float", [cols, 1])
        yd = core.tensor_descriptor([1, cols], "float", [cols, 1])
        need = core.reduction_workspace_size(fact.handle, rtd, xd, yd)
        if need > (64 << 10):
            break
    assert need > (64 << 10)
    tx = dev.empty(rows * cols * 4, fill=0)
    ty = dev.empty(cols * 4, fill=0)
    st, msg = no_alloc_reduce(fact, "add", xd, tx, yd, ty)
    assert st == 9 and "scratch" in msg and str(need) in msg     # DD_STATUS_NOT_SUPPORTED
    st, msg = no_alloc_reduce(fact, "add", xd, None, yd, ty)
    assert st == 3 and msg                                       # DD_STATUS_BAD_PARAM


def test_unsplit_reductions_and_other_types(fact, dev, oracle):
    # plans that need no scratch at all go through the same entry point
    x = np.arange(120, dtype=np.float32)
    xd = core.tensor_descriptor([2, 3, 4, 5], "float", "nchw")
    yd = core.tensor_descriptor([1, 3, 1, 1], "float", "nchw")
    ty = dev.put(np.zeros(3, np.float32))
    st, msg = no_alloc_reduce(fact, "max", xd, dev.put(x), yd, ty)
    assert st == 0, msg
    assert dev.get(ty, np.float32).tolist() == [79.0, 99.0, 119.0]


def test_device_memory_does_not_move(fact, dev):
    """Free device memory is the same before and after the calls: nothing is allocated or freed on
    the way.  (One warm-up call per plan first: the CUDA runtime loads a kernel's code, and with it
    the library's built-in array, the first time that kernel is used.)"""
    import torch
    rng = np.random.default_rng(41)
    prepared = []
    for op, shape, yshape in CASES:
        x = rng.standard_normal(int(np.prod(shape))).astype(np.float32)
        xd = core.tensor_descriptor(shape, "float", "nchw")
        yd = core.tensor_descriptor(yshape, "float", "nchw")
        tx, ty = dev.put(x), dev.put(np.zeros(int(np.prod(yshape)), np.float32))
        st, msg = no_alloc_reduce(fact, op, xd, tx, yd, ty)
        assert st == 0, msg
        prepared.append((op, xd, tx, yd, ty))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(2):
        for op, xd, tx, yd, ty in prepared:
            st, msg = no_alloc_reduce(fact, op, xd, tx, yd, ty)
            assert st == 0, msg
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
