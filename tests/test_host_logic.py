"""CPU-only checks: the C-ABI library loads and exports every symbol the header declares, the host
logic (layout keywords, descriptors, argument validation that needs no device) behaves like the
reference's, and the multi-rank logic of the sharded reduce agrees with a single-rank reduce
(world size 2 over gloo).  No kernel is launched here.
"""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from deep_diamond_b200 import _lib
    header = open(os.path.join(ROOT, "include", "dd_b200.h")).read()
    declared = set(re.findall(r"DD_API\s+[\w\s\*]+?\b(dd[A-Z]\w+)\s*\(", header))
    assert len(declared) >= 50
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, missing
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    assert lib.ddGetVersion() == 100


def test_error_strings_and_descriptor_calls_without_a_device():
    from deep_diamond_b200 import _lib, core
    from deep_diamond_b200._lib import DiamondError
    assert _lib.lib.ddGetErrorString(3) == b"DD_STATUS_BAD_PARAM"
    assert _lib.lib.ddGetErrorString(0) == b"DD_STATUS_SUCCESS"
    d = core.tensor_descriptor([3, 2, 2, 1], "float", "nhwc")
    assert core.strides(d) == [4, 1, 2, 2] and core.dims(d) == [3, 2, 2, 1] and core.data_type(d) == "float"
    assert core.bytesize(d) == 48
    assert core.bytesize(core.tensor_descriptor([2, 2, 3, 2], "float", [48, 100, 8, 3])) == (1 + 48 + 100 + 16 + 3) * 4
    assert core.equal_desc(d, core.tensor_descriptor([3, 2, 2, 1], "float", [4, 1, 2, 2]))
    assert not core.equal_desc(d, core.tensor_descriptor([3, 2, 2, 1], "int", "nhwc"))
    # cudnn core_test.clj:30-36: rank-3 descriptors are native here (no padding to 4)
    tnc = core.tensor_descriptor([2, 3, 4], "float", [12, 4, 1])
    assert core.dims(tnc) == [2, 3, 4] and core.strides(tnc) == [12, 4, 1]
    for bad in (([2, 3], "f128", [3, 1]), ([1, 1], "byte", "xxx"), ([2, -1, 1, 1], "float", "nchw"),
                ([2, 3], "float", [3])):
        with pytest.raises(DiamondError):
            core.tensor_descriptor(*bad)
    ad = core.activation_descriptor("relu", True, 42.0)
    assert core.activation_descriptor(ad) == {"mode": "relu", "relu-nan-opt": True, "coef": 42.0}
    assert core.activation_descriptor(core.activation_descriptor("sigmoid", True, 42.0))["mode"] == "logistic"
    with pytest.raises(DiamondError):
        core.activation_descriptor("softsign")
    with pytest.raises(DiamondError):
        core.reduce_tensor_descriptor("median")
    with pytest.raises(DiamondError):
        core.reduce_tensor_descriptor("add", "half")


def test_layout_keywords():
    from deep_diamond_b200.constants import default_strides, layout_strides
    assert layout_strides([2, 3, 4, 5], "nchw") == [60, 20, 5, 1]
    assert layout_strides([2, 3, 4, 5], "nhwc") == [60, 1, 15, 3]
    assert layout_strides([2, 7, 1], "tnc") == [7, 1, 1]
    assert layout_strides([2, 7, 1], "ntc") == [1, 2, 1]
    assert layout_strides([2, 3], "nc") == [3, 1] and layout_strides([2, 3], "cn") == [1, 2]
    assert layout_strides([2, 3, 4, 5, 6], "ncdhw") == default_strides([2, 3, 4, 5, 6])
    assert layout_strides([4], "x") == [1]
    assert default_strides([2, 3, 4, 5]) == [60, 20, 5, 1] and default_strides([]) == []


def test_general_descriptor_and_the_no_fallback_rule():
    from deep_diamond_b200 import tensor as T
    from deep_diamond_b200._lib import DiamondError
    d = T.desc([2, 3, 2, 4], "nhwc")
    assert (d.shape, d.data_type, d.layout) == ([2, 3, 2, 4], None, "nhwc")
    assert T.desc([2, 3], "float", "nc").data_type == "float"
    assert T.default_desc([2, 3, 4], "float").layout == [12, 4, 1]
    with pytest.raises(DiamondError):
        T.desc([2, 3], "float", "nchw")
    import torch
    if not torch.cuda.is_available():
        from deep_diamond_b200 import b200_factory
        with pytest.raises(DiamondError):   # no device: the factory refuses, nothing falls back to the CPU
            b200_factory()


def test_shard_arithmetic():
    from deep_diamond_b200 import sharded
    from deep_diamond_b200._lib import DiamondError
    assert sharded.shard_range(64, 8, 3) == (24, 32)
    assert sharded.shard_shape([2048, 256, 28, 28], 8) == [256, 256, 28, 28]
    assert sharded.spans_sharded_dim([8, 1024, 32, 32], [1, 1024, 1, 1])
    assert not sharded.spans_sharded_dim([8, 1024, 32, 32], [8, 1, 32, 32])
    with pytest.raises(DiamondError):
        sharded.shard_range(10, 4, 0)


_WORKER = r'''
import os, sys
import numpy as np
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
import oracle
from deep_diamond_b200 import sharded

dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%s" % sys.argv[2], rank=int(sys.argv[3]), world_size=2)
rank, world = dist.get_rank(), dist.get_world_size()
full = oracle.gen_signed_lognormal([8, 6, 5, 4], 5)
lo, hi = sharded.shard_range(full.shape[0], world, rank)
mine = np.ascontiguousarray(full[lo:hi])
ok = True
for op, pre in (("add", "add"), ("avg", "add"), ("norm2", None), ("max", "max"), ("norm1", "norm1")):
    yshape = (1, 6, 1, 1)
    # local pre-finish partial: sum, sum|x|, sum x^2 or max over this rank's slice
    if op == "norm2":
        part = (mine.astype(np.float64) ** 2).sum(axis=(0, 2, 3), keepdims=True)
    else:
        part = np.zeros(yshape, np.float32)
        oracle.reduce(pre, mine, part)
    gathered = [None, None]
    dist.all_gather_object(gathered, np.asarray(part, dtype=np.float64))
    got = sharded.combine_partials_host(op, gathered, mine.size // 6, world)
    want = np.zeros(yshape, np.float32)
    _, truth = oracle.reduce(op, full, want, want_truth=True)
    ok = ok and np.allclose(got, truth, rtol=1e-5, atol=1e-5)
# the handle swap of the peer exchange: every rank ends up with all handles in rank order
handles = sharded.gather_in_rank_order(bytes([rank + 1]) * sharded.PEER_HANDLE_BYTES, dist.all_gather_object, world)
ok = ok and handles == [bytes([1]) * 64, bytes([2]) * 64]
flags = [None, None]
dist.all_gather_object(flags, bool(ok))
dist.barrier()
dist.destroy_process_group()
sys.exit(0 if all(flags) else 1)
'''


def test_sharded_reduce_logic_world_size_2_gloo(tmp_path):
    """Two CPU ranks each hold half the batch; local partial + combine + finish equals the reduce of
    the whole tensor for sum, mean, norm2, max, norm1 (the arithmetic ddShardedReduceTensor runs with
    NCCL in place of the gather)."""
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(port), str(r)]) for r in range(2)]
    codes = [p.wait(timeout=180) for p in procs]
    assert codes == [0, 0]


def test_uneven_shards_and_global_count():
    from deep_diamond_b200 import sharded
    from deep_diamond_b200._lib import DiamondError
    # 10 images over 4 ranks: the first two ranks own one more
    assert [sharded.shard_range(10, 4, r, even=False) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    with pytest.raises(DiamondError):
        sharded.shard_range(3, 4, 0, even=False)          # a rank would be left without a batch entry
    # elements folded into one output over all ranks, whatever this rank's share of the batch is
    assert sharded.global_reduced_count([3, 64, 16, 16], [1, 64, 1, 1], 10) == 10 * 16 * 16
    assert sharded.global_reduced_count([2, 64, 16, 16], [1, 64, 1, 1], 10) == 10 * 16 * 16
    assert sharded.global_reduced_count([3, 64, 16, 16], [1, 1, 1, 1], 10) == 10 * 64 * 16 * 16
    # the mean over unevenly sharded data: combine the partial sums, divide by the GLOBAL count
    rng = np.random.default_rng(3)
    full = rng.standard_normal((10, 6, 5, 4))
    parts = []
    for r in range(4):
        lo, hi = sharded.shard_range(10, 4, r, even=False)
        parts.append(full[lo:hi].sum(axis=(0, 2, 3)))
    got = np.stack(parts).sum(axis=0) / sharded.global_reduced_count([3, 6, 5, 4], [1, 6, 1, 1], 10)
    assert np.allclose(got, full.mean(axis=(0, 2, 3)))


_TEARDOWN_WORKER = r'''
import datetime, os, sys, time
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from deep_diamond_b200 import sharded
from deep_diamond_b200._lib import DiamondError

rank, world, mode = int(sys.argv[3]), 2, sys.argv[4]
store = dist.TCPStore("127.0.0.1", int(sys.argv[2]), world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=60))
if mode == "teardown":
    # The order of the collective tear-down, with stand-ins for the library calls (no GPU here): a rank
    # may free the buffer it exported only after EVERY rank has closed its mappings.  Rank 1 is slow
    # to detach; rank 0 must still find both detached when it frees.
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    log = []

    def detach():
        if rank == 1:
            time.sleep(1.0)
        store.add("detached", 1)
        log.append("detach")

    def destroy():
        log.append("destroy with %d detached" % store.add("detached", 0))
    sharded.collective_release(detach, dist.barrier, destroy)
    ok = log == ["detach", "destroy with 2 detached"]
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)
else:
    # The bounded join: rank 1 never announces itself; rank 0 gives up after its limit and says who
    # is missing.  No communicator is created, nothing touches a GPU.
    if rank == 1:
        time.sleep(3.0)          # arrives after rank 0 has given up, and never joins
        sys.exit(0)
    t0 = time.time()
    try:
        sharded.join_with_limit(store, rank, world, 1.0)
        sys.exit(1)
    except DiamondError as e:
        took = time.time() - t0
        ok = e.data.get("type") == "timeout" and e.data.get("missing-ranks") == [1] and took < 2.5
        sys.exit(0 if ok else 1)
'''


@pytest.mark.parametrize("mode", ["teardown", "join"])
def test_collective_teardown_order_and_bounded_join_gloo(tmp_path, mode):
    """World size 2 on CPU.  `teardown`: detach -> host barrier -> destroy, so that no rank frees the
    buffer it exported while another still has it mapped.  `join`: a rank that never joins makes the
    others fail with a timeout after the limit instead of blocking in the communicator set-up."""
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = tmp_path / "worker.py"
    script.write_text(_TEARDOWN_WORKER)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(port), str(r), mode]) for r in range(2)]
    codes = [p.wait(timeout=180) for p in procs]
    assert codes == [0, 0]


def test_release_of_an_attached_handle_needs_the_barrier():
    """`ShardedHandle.release` refuses to free an attached exchange without the ranks' barrier."""
    from deep_diamond_b200 import sharded
    from deep_diamond_b200._lib import DiamondError

    class Fake(sharded.ShardedHandle):
        def __init__(self):                       # no library call: only the release logic is under test
            self.ptr, self.peer_attached, self.world_size, self.calls = object(), True, 2, []

        def detach(self):
            self.calls.append("detach")
            self.peer_attached = False

        def destroy(self):
            self.calls.append("destroy")
            self.ptr = None
    h = Fake()
    with pytest.raises(DiamondError):
        h.release()
    assert h.calls == []
    h.release(barrier=lambda: h.calls.append("barrier"))
    assert h.calls == ["detach", "barrier", "destroy"]
