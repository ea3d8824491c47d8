"""Batch-dim sharding over the GPUs of one box: one process per GPU, each holding its own slice of
every tensor.  The reference has nothing like it (one CUDA context, one stream,
deep-diamond-cuda/src/clojure/uncomplicate/diamond/internal/cudnn/factory.clj:481-494); its closest
primitives are the batch sub-tensors of ``view-tz`` / ``offset!`` (cudnn/tensor.clj:478-497), whose
arithmetic `shard_range` repeats.

Reorder, eltwise and broadcast op-tensor need no communication: every rank just runs the
single-GPU call on its slice.  Only a reduction that spans the sharded dim exchanges data: the
local partial results (a few KB) are combined across the ranks and finished, either by the
library's own peer exchange (one kernel per rank pushing into every rank's buffer over NVLink) or
by an NCCL all-reduce on the compute stream followed by a finishing kernel.
"""
import ctypes

import numpy as np

from . import core
from ._lib import DiamondError, check, lib

UNIQUE_ID_BYTES = 128
PEER_HANDLE_BYTES = 64
PEER_MAX_RANKS = 8


def shard_range(n, world_size, rank):
    """[lo, hi) of the batch entries rank `rank` owns: equal slices, n divisible by world_size."""
    if n % world_size:
        raise DiamondError("The batch dim must divide evenly over the ranks.",
                           {"batch": n, "world-size": world_size})
    per = n // world_size
    return rank * per, (rank + 1) * per


def shard_shape(shape, world_size, batch_index=0):
    s = list(shape)
    lo, hi = shard_range(s[batch_index], world_size, 0)
    s[batch_index] = hi - lo
    return s


def spans_sharded_dim(x_shape, y_shape, batch_index=0):
    """True when the reduction y <- x folds the sharded (batch) dim."""
    return y_shape[batch_index] == 1 and x_shape[batch_index] != 1


def get_unique_id():
    buf = (ctypes.c_ubyte * UNIQUE_ID_BYTES)()
    check(lib.ddShardedGetUniqueId(buf), None, "ddShardedGetUniqueId")
    return bytes(buf)


class ShardedHandle:
    """The library's communicator for one rank (wraps ddShardedCreate).  ``unique_id=None`` makes a
    handle without NCCL that can only combine over the peer exchange."""

    def __init__(self, fact, world_size, rank, unique_id):
        self.fact, self.world_size, self.rank = fact, world_size, rank
        h = ctypes.c_void_p()
        idbuf = (ctypes.c_ubyte * UNIQUE_ID_BYTES).from_buffer_copy(unique_id) if unique_id is not None else None
        check(lib.ddShardedCreate(ctypes.byref(h), fact.handle.ptr, world_size, rank, idbuf),
              fact.handle.ptr, "ddShardedCreate")
        self.ptr = h
        self.peer_attached = False

    def reduce_tensor(self, rtd, alpha, desc_x, x, beta, desc_y, y, spans=None):
        dx, dy = core.desc(desc_x), core.desc(desc_y)
        if spans is None:
            spans = spans_sharded_dim(dx.dims, dy.dims)
        a, b = core._scalar(alpha, dx.dtype_code), core._scalar(beta, dy.dtype_code)
        check(lib.ddShardedReduceTensor(self.ptr, rtd.ptr, 1 if spans else 0, ctypes.byref(a), dx.ptr,
                                        core._ptr(x), ctypes.byref(b), dy.ptr, core._ptr(y)),
              self.fact.handle.ptr, "ddShardedReduceTensor")
        return y

    def peer_export(self):
        """This rank's exchange-buffer handle (64 bytes) for the other processes of the box."""
        buf = (ctypes.c_ubyte * PEER_HANDLE_BYTES)()
        check(lib.ddShardedPeerExport(self.ptr, buf), self.fact.handle.ptr, "ddShardedPeerExport")
        return bytes(buf)

    def peer_attach(self, handles):
        """`handles`: every rank's exported handle, in rank order."""
        if len(handles) != self.world_size or any(len(hd) != PEER_HANDLE_BYTES for hd in handles):
            raise DiamondError("One 64-byte handle per rank is needed.",
                               {"world-size": self.world_size, "handles": len(handles)})
        blob = b"".join(handles)
        buf = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
        check(lib.ddShardedPeerAttach(self.ptr, buf), self.fact.handle.ptr, "ddShardedPeerAttach")
        self.peer_attached = True
        return self

    def peer_configure(self, use_peer=None, wait_seconds=None, fused=False):
        """use_peer False: NCCL; True: the peer exchange as a kernel of its own after the local
        pass (`fused=True`: pushed from inside the reduce kernel where the plan allows); None:
        leave as is."""
        mode = -1 if use_peer is None else (0 if not use_peer else (2 if fused else 1))
        check(lib.ddShardedPeerConfigure(self.ptr, mode, 0.0 if wait_seconds is None else float(wait_seconds)),
              self.fact.handle.ptr, "ddShardedPeerConfigure")
        return self

    def peer_status(self):
        """Synchronises the stream; raises DiamondError (type timeout) when a bounded wait of the
        exchange ran out, else returns 0."""
        st = ctypes.c_int(0)
        check(lib.ddShardedPeerStatus(self.ptr, ctypes.byref(st)), self.fact.handle.ptr, "ddShardedPeerStatus")
        return st.value

    def check(self):
        check(lib.ddShardedCheck(self.ptr), self.fact.handle.ptr, "ddShardedCheck")
        return True

    def release(self):
        if self.ptr is not None:
            lib.ddShardedDestroy(self.ptr)
            self.ptr = None
        return True


def gather_in_rank_order(payload, all_gather_object, world_size):
    """Every rank's `payload` as a list indexed by rank, through any all-gather of Python objects
    (``torch.distributed.all_gather_object`` over gloo or nccl)."""
    out = [None] * world_size
    all_gather_object(out, payload)
    return out


def create_from_torch_distributed(fact, peer=True, nccl=True):
    """Builds the library communicator for this rank from an initialised torch.distributed group:
    rank 0 makes the NCCL id, the group broadcasts it (any transport: gloo or nccl); with `peer`
    the ranks also swap exchange-buffer handles and attach the peer exchange (boxes of up to 8
    GPUs), which then carries the reductions."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(), dist.get_rank()
    payload = [None]
    if nccl:
        payload = [get_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(payload, src=0)
    with torch.cuda.device(fact.device):
        sh = ShardedHandle(fact, world, rank, payload[0])
        if peer and world <= PEER_MAX_RANKS:
            handles = gather_in_rank_order(sh.peer_export(), dist.all_gather_object, world)
            try:
                sh.peer_attach(handles)
                mine = None
            except DiamondError as e:       # e.g. no peer access between two of the GPUs
                mine = str(e)
            errors = gather_in_rank_order(mine, dist.all_gather_object, world)
            if any(errors):
                # the exchange needs every rank: all fall back to NCCL together, or fail together
                sh.peer_attached = False
                sh.peer_configure(use_peer=False)
                if not nccl:
                    raise DiamondError("The peer exchange could not be attached on every rank.",
                                       {"errors": [e for e in errors if e]})
        return sh


def combine_partials_host(op, partials, local_count, world_size):
    """What the all-reduce + finish step computes, on host arrays (used by the CPU tests of the
    multi-rank logic): `partials` is one array per rank of pre-finish accumulators."""
    stack = np.stack([np.asarray(p, dtype=np.float64) for p in partials])
    if op in ("add", "avg", "norm1", "norm2"):
        acc = stack.sum(axis=0)
    elif op in ("mul", "mul-no-zeros"):
        acc = stack.prod(axis=0)
    elif op == "min":
        acc = stack.min(axis=0)
    else:
        acc = stack.max(axis=0)
    if op == "avg":
        acc = acc / (local_count * world_size)
    if op == "norm2":
        acc = np.sqrt(acc)
    return acc
