"""Multi-GPU: the batch-sharded reduce (local partial -> combine across ranks -> finish) on 2 GPUs of
one box, one process per GPU, against the CPU oracle on the whole tensor, over both combine paths
(the library's peer-exchange kernel and NCCL).  Skipped on a single-GPU box; the multi-rank host
logic is also covered on CPU by tests/test_host_logic.py (gloo, world size 2).

The bounded wait of the exchange kernel is tested on ONE GPU with a failure made on the host: a
handle that claims two ranks whose second rank does not exist, so the flag it waits for is never
set; the kernel gives up after the configured limit, records which rank it waited for, writes no
result and returns normally."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_sharded_reduce_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sharded_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), worker]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


def test_peer_exchange_wait_runs_out(fact, dev):
    import numpy as np
    from deep_diamond_b200 import core, sharded
    from deep_diamond_b200._lib import DiamondError
    sh = sharded.ShardedHandle(fact, 2, 0, None)             # rank 0 of 2, no NCCL
    try:
        own = sh.peer_export()
        sh.peer_attach([own, own])                            # "rank 1" is this rank's own buffer: nobody signals for it
        shape = [4, 64, 16, 16]
        x = dev.put(np.ones(shape, np.float32))
        y0 = np.full(64, -7.0, np.float32)
        y = dev.put(y0)
        for fused, kernel in ((True, "reduce/row+peer-exchange"), (False, "reduce/peer-exchange")):
            sh.peer_configure(use_peer=True, wait_seconds=0.05, fused=fused)
            sh.reduce_tensor(core.reduce_tensor_descriptor("add", "float"), 1.0,
                             core.tensor_descriptor(shape, "float", "nchw"), x, 0.0,
                             core.tensor_descriptor([1, 64, 1, 1], "float", "nchw"), y, spans=True)
            assert fact.handle.last_kernel() == kernel
            with pytest.raises(DiamondError) as e:
                sh.peer_status()
            assert e.value.data["type"] == "timeout" and "rank 1" in str(e.value)
            assert np.array_equal(dev.get(y, np.float32), y0)     # the kernel that gave up wrote nothing
        # the context is still usable
        z = dev.put(np.zeros(64, np.float32))
        core.reduce_tensor(fact.handle, core.reduce_tensor_descriptor("add", "float"), 1.0,
                           core.tensor_descriptor(shape, "float", "nchw"), x, 0.0,
                           core.tensor_descriptor([1, 64, 1, 1], "float", "nchw"), z)
        assert np.array_equal(dev.get(z, np.float32), np.full(64, 4 * 256, np.float32))
    finally:
        sh.release(barrier=lambda: None)      # the only "peer" is this process itself


def test_sharded_without_any_transport_is_refused(fact, dev):
    import numpy as np
    from deep_diamond_b200 import core, sharded
    from deep_diamond_b200._lib import DiamondError
    sh = sharded.ShardedHandle(fact, 2, 0, None)
    try:
        x = dev.put(np.ones([2, 4, 2, 2], np.float32))
        y = dev.put(np.zeros(4, np.float32))
        with pytest.raises(DiamondError):
            sh.reduce_tensor(core.reduce_tensor_descriptor("add", "float"), 1.0,
                             core.tensor_descriptor([2, 4, 2, 2], "float", "nchw"), x, 0.0,
                             core.tensor_descriptor([1, 4, 1, 1], "float", "nchw"), y, spans=True)
    finally:
        sh.release()
