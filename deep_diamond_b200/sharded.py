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


def shard_range(n, world_size, rank, even=True):
    """[lo, hi) of the batch entries rank `rank` owns.  `even`: equal slices, n must divide by
    world_size.  Otherwise the first ``n % world_size`` ranks own one entry more (every rank needs
    at least one, so n >= world_size)."""
    if even:
        if n % world_size:
            raise DiamondError("The batch dim must divide evenly over the ranks.",
                               {"batch": n, "world-size": world_size})
        per = n // world_size
        return rank * per, (rank + 1) * per
    if n < world_size:
        raise DiamondError("Every rank needs at least one batch entry.", {"batch": n, "world-size": world_size})
    per, extra = divmod(n, world_size)
    lo = rank * per + min(rank, extra)
    return lo, lo + per + (1 if rank < extra else 0)


def global_reduced_count(x_shape_local, y_shape, global_batch, batch_index=0):
    """Elements folded into one output over all ranks: what ddShardedReduceTensor divides a mean by."""
    n = 1
    for i, (xd, yd) in enumerate(zip(x_shape_local, y_shape)):
        if yd == 1:                          # a reduced dim (or an extent of 1 on both sides)
            n *= global_batch if i == batch_index else xd
    return n


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

    def reduce_tensor(self, rtd, alpha, desc_x, x, beta, desc_y, y, spans=None, global_batch=None):
        """`global_batch`: the un-sharded batch size when the ranks own unequal slices (a mean then
        divides by the global element count); None = equal slices."""
        dx, dy = core.desc(desc_x), core.desc(desc_y)
        if spans is None:
            spans = spans_sharded_dim(dx.dims, dy.dims)
        count = 0 if global_batch is None else global_reduced_count(dx.dims, dy.dims, global_batch)
        a, b = core._scalar(alpha, dx.dtype_code), core._scalar(beta, dy.dtype_code)
        check(lib.ddShardedReduceTensor(self.ptr, rtd.ptr, 1 if spans else 0, count, ctypes.byref(a), dx.ptr,
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

    def peer_configure(self, use_peer=None, wait_seconds=None, fused=None):
        """use_peer False: NCCL.  True: the peer exchange; `fused` then picks its form: None = the
        library's choice (reduce + exchange in ONE kernel where every output can be collected by the
        thread that finished it, else a small exchange kernel after the local pass), True = fused
        wherever the plan allows, False = always the separate exchange kernel.  use_peer None leaves
        the path as it is."""
        mode = -1 if use_peer is None else (0 if not use_peer else (1 if fused is None else (2 if fused else 3)))
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

    def detach(self):
        """Step 1 of the collective tear-down: waits for this rank's work and closes its mappings of
        the other ranks' exchange buffers."""
        if self.ptr is not None:
            check(lib.ddShardedPeerDetach(self.ptr), self.fact.handle.ptr, "ddShardedPeerDetach")
            self.peer_attached = False
        return True

    def destroy(self):
        if self.ptr is not None:
            lib.ddShardedDestroy(self.ptr)
            self.ptr = None
        return True

    def release(self, barrier=None):
        """Tear-down.  With an attached exchange it is collective: pass the ranks' host barrier
        (e.g. ``torch.distributed.barrier``); every rank detaches, all meet at the barrier, then
        every rank frees what it exported (see `collective_release`)."""
        if self.ptr is None:
            return True
        if self.peer_attached and self.world_size > 1 and barrier is None:
            raise DiamondError("Releasing a sharded handle with an attached peer exchange is collective: "
                               "pass the ranks' host barrier.", {"world-size": self.world_size})
        return collective_release(self.detach, barrier or (lambda: None), self.destroy)


def collective_release(detach, barrier, destroy):
    """The order every rank follows to take the peer exchange down: close the own mappings of the
    other ranks' buffers, meet all ranks on the host, only then free the buffer the others had
    mapped.  Freeing it earlier leaves a late peer storing into freed memory."""
    detach()
    barrier()
    destroy()
    return True


def join_with_limit(store, rank, world_size, seconds, key="dd-b200-join"):
    """Bounded rendezvous before the (unbounded) communicator set-up: every rank announces itself in
    `store` (anything with ``set(key, value)`` and ``wait(keys, timedelta)``, e.g. a
    ``torch.distributed.TCPStore`` or the default group's store) and waits for all the others, at most
    `seconds`.  Raises DiamondError of type timeout naming the ranks that never arrived."""
    import datetime
    store.set("%s/%d" % (key, rank), b"1")
    missing = []
    limit = datetime.timedelta(seconds=float(seconds))
    for r in range(world_size):
        try:
            store.wait(["%s/%d" % (key, r)], limit)
        except Exception:                   # the store raises on timeout (RuntimeError / DistStoreError)
            missing.append(r)
            limit = datetime.timedelta(milliseconds=1)     # the limit is for the whole join, not per rank
    if missing:
        raise DiamondError("Not every rank joined within the limit.",
                           {"type": "timeout", "missing-ranks": missing, "seconds": float(seconds)})
    return True


def gather_in_rank_order(payload, all_gather_object, world_size):
    """Every rank's `payload` as a list indexed by rank, through any all-gather of Python objects
    (``torch.distributed.all_gather_object`` over gloo or nccl)."""
    out = [None] * world_size
    all_gather_object(out, payload)
    return out


def create_from_torch_distributed(fact, peer=True, nccl=True, join_seconds=None, store=None):
    """Builds the library communicator for this rank from an initialised torch.distributed group:
    rank 0 makes the NCCL id, the group broadcasts it (any transport: gloo or nccl); with `peer`
    the ranks also swap exchange-buffer handles and attach the peer exchange (boxes of up to 8
    GPUs), which then carries the reductions.  With `join_seconds` and a `store` the ranks first
    check, within that limit, that all of them have arrived (`join_with_limit`); the library's own
    limit on the communicator set-up is set to the same value."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(), dist.get_rank()
    if join_seconds is not None:
        if store is not None:
            join_with_limit(store, rank, world, join_seconds)
        check(lib.ddShardedSetJoinLimit(float(join_seconds)), None, "ddShardedSetJoinLimit")
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
