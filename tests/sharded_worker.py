"""One rank of the multi-GPU reduce test (launched by tests/test_gpu_sharded.py under
torch.distributed.run).  Every rank builds the same full tensor from a seed, keeps its own batch
slice on its GPU, runs ddShardedReduceTensor over both combine paths (the library's peer exchange
and NCCL), and checks the (replicated) result against the CPU oracle's reduction of the whole
tensor."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def within(got, want, full, alpha, axes):
    scale = np.abs(full.astype(np.float64)).sum(axis=axes, keepdims=True)
    return bool((np.abs(got - want) <= np.maximum(1e-5 * np.abs(want), 16 * 6e-8 * abs(alpha) * scale)).all())


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import oracle
    from deep_diamond_b200 import b200_factory, core, sharded
    fact = b200_factory(local)
    sh = sharded.create_from_torch_distributed(fact)
    assert sh.check() and sh.peer_attached
    full_shape = [4 * world, 64, 16, 16]
    full = oracle.gen_signed_lognormal(full_shape, 5)
    lo, hi = sharded.shard_range(full_shape[0], world, rank)
    mine = np.ascontiguousarray(full[lo:hi])
    x = torch.from_numpy(mine).to(fact.device)
    shard_shape = list(mine.shape)
    xd = core.tensor_descriptor(shard_shape, "float", "nchw")
    failures = []
    for path in ("fused", "peer", "nccl"):
        sh.peer_configure(use_peer=(path != "nccl"), fused=(path == "fused"))
        for op in ("add", "avg", "norm2", "norm1", "max", "min", "amax"):
            for alpha, beta in ((1.0, 0.0), (2.0, 0.5)):
                yshape = [1, 64, 1, 1]
                y0 = np.linspace(-1, 1, 64, dtype=np.float32)
                want = y0.copy().reshape(yshape)
                oracle.reduce(op, full, want, alpha=alpha, beta=beta)
                y = torch.from_numpy(y0.copy()).to(fact.device)
                yd = core.tensor_descriptor(yshape, "float", "nchw")
                sh.reduce_tensor(core.reduce_tensor_descriptor(op, "float"), alpha, xd, x, beta, yd, y)
                fact.synchronize()
                want_kernel = {"fused": "reduce/row+peer-exchange", "peer": "reduce/peer-exchange",
                               "nccl": "reduce/finish"}[path]
                if fact.handle.last_kernel() != want_kernel:
                    failures.append((path, "kernel", fact.handle.last_kernel()))
                got = y.cpu().numpy().reshape(yshape)
                if op in ("max", "min", "amax") and beta == 0.0:
                    ok = np.array_equal(got, want)
                else:
                    ok = within(got, want, full, alpha, (0, 2, 3))
                if not ok:
                    failures.append((path, op, alpha, beta, float(np.abs(got - want).max())))
        # oneDNN's norm kinds with p and epsilon: the ranks exchange sums of |x|^p, epsilon and the root follow
        for kind, pw, eps in (("norm-lp-sum", 3.0, 0.5), ("norm-lp-power-p-max", 2.0, 1e6), ("norm-lp-max", 1.0, 0.0)):
            want = np.zeros([1, 64, 1, 1], np.float32)
            oracle.reduce_lp(kind, pw, eps, full, want)
            y = torch.zeros(64, device=fact.device)
            sh.reduce_tensor(core.reduce_tensor_descriptor(kind, "float", True, p=pw, eps=eps), 1.0, xd, x, 0.0,
                             core.tensor_descriptor([1, 64, 1, 1], "float", "nchw"), y)
            fact.synchronize()
            got = y.cpu().numpy().reshape(want.shape)
            if not (np.abs(got - want) <= 1e-5 * np.abs(want)).all():
                failures.append((path, kind, pw, eps, float(np.abs(got - want).max())))
        # all ranks must hold identical bits for the replicated results
        y = torch.zeros(64, device=fact.device)
        sh.reduce_tensor(core.reduce_tensor_descriptor("add", "float"), 1.0, xd, x, 0.0,
                         core.tensor_descriptor([1, 64, 1, 1], "float", "nchw"), y)
        gathered = [torch.zeros_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        if any(not torch.equal(g, gathered[0]) for g in gathered):
            failures.append((path, "replicas differ"))
    sh.peer_configure(use_peer=True, fused=True)

    # the fused form through the col kernel (sum over N only, 4096 outputs) and with split rows
    # (few outputs, long ranges: the per-output arrival counters feed the push)
    for fshape, yshape, axes in (([4 * world, 16, 16, 16], [1, 16, 16, 16], (0,)),
                                 ([2 * world, 2, 64, 64], [1, 2, 1, 1], (0, 2, 3))):
        ffull = oracle.gen_signed_lognormal(fshape, 9)
        flo, fhi = sharded.shard_range(fshape[0], world, rank)
        fx = torch.from_numpy(np.ascontiguousarray(ffull[flo:fhi])).to(fact.device)
        want = np.zeros(yshape, np.float32)
        oracle.reduce("add", ffull, want)
        y = torch.zeros(int(np.prod(yshape)), device=fact.device)
        for _ in range(3):
            sh.reduce_tensor(core.reduce_tensor_descriptor("add", "float"), 1.0,
                             core.tensor_descriptor([fhi - flo] + fshape[1:], "float", "nchw"), fx, 0.0,
                             core.tensor_descriptor(yshape, "float", "nchw"), y)
        fact.synchronize()
        if not fact.handle.last_kernel().endswith("+peer-exchange"):
            failures.append(("fused kernel expected", fshape, fact.handle.last_kernel()))
        if not within(y.cpu().numpy().reshape(yshape), want, ffull, 1.0, axes):
            failures.append(("fused", fshape))

    sh.peer_configure(use_peer=True)

    # many outputs (several CTAs of the exchange kernel): sum over N only
    yshape = [1, 64, 16, 16]
    want = np.zeros(yshape, np.float32)
    oracle.reduce("add", full, want)
    y = torch.zeros(int(np.prod(yshape)), device=fact.device)
    yd = core.tensor_descriptor(yshape, "float", "nchw")
    rtd = core.reduce_tensor_descriptor("add", "float")
    for _ in range(5):          # calls in a row alternate the exchange's two parities
        y.zero_()
        sh.reduce_tensor(rtd, 1.0, xd, x, 0.0, yd, y)
    fact.synchronize()
    if not within(y.cpu().numpy().reshape(yshape), want, full, 1.0, (0,)):
        failures.append(("sum over N, 16384 outputs",))

    # a captured launch replayed: the call number lives on the device, so replays stay in step
    side = torch.cuda.Stream(device=fact.device)
    side.wait_stream(fact.stream)
    fact.handle.set_stream(side)
    with torch.cuda.stream(side):
        sh.reduce_tensor(rtd, 1.0, xd, x, 0.0, yd, y)
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(3):
                sh.reduce_tensor(rtd, 1.0, xd, x, 0.0, yd, y)
        for _ in range(4):
            y.zero_()
            g.replay()
        side.synchronize()
    fact.handle.set_stream(fact.stream)
    if not within(y.cpu().numpy().reshape(yshape), want, full, 1.0, (0,)):
        failures.append(("graph replay",))

    # double precision accumulators through the exchange
    fulld = full.astype(np.float64)
    xdbl = torch.from_numpy(np.ascontiguousarray(fulld[lo:hi])).to(fact.device)
    wantd = np.zeros([1, 64, 1, 1], np.float64)
    oracle.reduce("norm2", fulld, wantd)
    yd64 = torch.zeros(64, dtype=torch.float64, device=fact.device)
    sh.reduce_tensor(core.reduce_tensor_descriptor("norm2", "double"), 1.0,
                     core.tensor_descriptor(shard_shape, "double", "nchw"), xdbl, 0.0,
                     core.tensor_descriptor([1, 64, 1, 1], "double", "nchw"), yd64)
    fact.synchronize()
    if not np.allclose(yd64.cpu().numpy().reshape(wantd.shape), wantd, rtol=1e-12):
        failures.append(("norm2 double",))

    # a reduction that keeps the sharded dim needs no exchange: result stays sharded
    yshape = [shard_shape[0], 1, 16, 16]
    want = np.zeros(yshape, np.float32)
    oracle.reduce("max", mine, want)
    y = torch.zeros(int(np.prod(yshape)), device=fact.device)
    sh.reduce_tensor(core.reduce_tensor_descriptor("max", "float"), 1.0, xd, x, 0.0,
                     core.tensor_descriptor(yshape, "float", "nchw"), y)
    fact.synchronize()
    if not np.array_equal(y.cpu().numpy().reshape(yshape), want):
        failures.append(("max over C (local)",))

    # uneven shards: 4 * world + 1 images, rank 0 owns one more; the mean divides by the global count
    # that the caller passes.  Both combine paths.
    ushape = [4 * world + 1, 64, 16, 16]
    ufull = oracle.gen_signed_lognormal(ushape, 11)
    ulo, uhi = sharded.shard_range(ushape[0], world, rank, even=False)
    ux = torch.from_numpy(np.ascontiguousarray(ufull[ulo:uhi])).to(fact.device)
    uxd = core.tensor_descriptor([uhi - ulo] + ushape[1:], "float", "nchw")
    for path in ("peer", "nccl"):
        sh.peer_configure(use_peer=(path == "peer"))
        for op in ("avg", "add", "norm2"):
            want = np.zeros([1, 64, 1, 1], np.float32)
            oracle.reduce(op, ufull, want)
            y = torch.zeros(64, device=fact.device)
            sh.reduce_tensor(core.reduce_tensor_descriptor(op, "float"), 1.0, uxd, ux, 0.0,
                             core.tensor_descriptor([1, 64, 1, 1], "float", "nchw"), y, global_batch=ushape[0])
            fact.synchronize()
            if not within(y.cpu().numpy().reshape(want.shape), want, ufull, 1.0, (0, 2, 3)):
                failures.append(("uneven shards", path, op))
    sh.peer_configure(use_peer=True)
    # a global count below the local one is refused
    import ctypes
    from deep_diamond_b200._lib import DiamondError, check, lib
    one, zero = core._scalar(1.0, 0), core._scalar(0.0, 0)
    try:
        check(lib.ddShardedReduceTensor(sh.ptr, core.reduce_tensor_descriptor("avg", "float").ptr, 1, 3,
                                        ctypes.byref(one), uxd.ptr, core._ptr(ux), ctypes.byref(zero),
                                        core.tensor_descriptor([1, 64, 1, 1], "float", "nchw").ptr, core._ptr(y)),
              fact.handle.ptr, "ddShardedReduceTensor")
        failures.append(("global count below the local one was accepted",))
    except DiamondError as e:
        if e.data.get("type") != "bad-param":
            failures.append(("unexpected error for a bad global count", str(e)))

    # a small shard: 32 or fewer reduced elements per rank still takes the structured (row) form
    sshape = [2 * world, 64, 2, 2]
    sfull = oracle.gen_signed_lognormal(sshape, 13)
    slo, shi = sharded.shard_range(sshape[0], world, rank)
    sx = torch.from_numpy(np.ascontiguousarray(sfull[slo:shi])).to(fact.device)
    want = np.zeros([1, 64, 1, 1], np.float32)
    oracle.reduce("add", sfull, want)
    y = torch.zeros(64, device=fact.device)
    sh.reduce_tensor(core.reduce_tensor_descriptor("add", "float"), 1.0,
                     core.tensor_descriptor([shi - slo] + sshape[1:], "float", "nchw"), sx, 0.0,
                     core.tensor_descriptor([1, 64, 1, 1], "float", "nchw"), y)
    fact.synchronize()
    if not within(y.cpu().numpy().reshape(want.shape), want, sfull, 1.0, (0, 2, 3)):
        failures.append(("small shard",))

    if sh.peer_status() != 0:
        failures.append(("peer status",))
    flag = torch.tensor([len(failures)], device=fact.device)
    dist.all_reduce(flag)
    # collective tear-down: detach, host barrier, destroy
    sh.release(barrier=dist.barrier)
    fact.release()
    dist.destroy_process_group()
    if failures:
        print("rank", rank, "failures:", failures, flush=True)
    sys.exit(1 if int(flag.item()) else 0)


if __name__ == "__main__":
    main()
