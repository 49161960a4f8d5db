"""Process-per-GPU data parallelism over torch.distributed (NCCL on GPUs, gloo in CPU tests): the
`Var.mpi_all_reduce` surface of the reference (python/jittor/extern/mpi/ops/mpi_all_reduce_op.cc:27-61)
without MPI. Rank and world size come from the torchrun environment."""
import os

import torch
import torch.distributed as tdist

from . import var as V


def init(backend=None):
    """Joins the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (a no-op for one process)."""
    if tdist.is_initialized() or int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    tdist.init_process_group(backend=backend)
    if backend == "nccl" and os.environ.get("B200JT_PEER_ALLREDUCE", "1") != "0":
        connect_peers()


_PEER = None


def connect_peers(data_bytes=None, wait_ms=None):
    """Sets up the NVLink peer all-reduce kernel for messages up to `data_bytes` (collective; see peer.PeerComm).
    Larger messages, other dtypes and jobs where the set-up fails keep going through NCCL."""
    global _PEER
    from . import peer
    if _PEER is not None:
        _PEER.close()
    _PEER = peer.PeerComm.connect(data_bytes, wait_ms)
    return _PEER


def peer_comm():
    return _PEER


def all_reduce_sum(src, out=None):
    """Sum of a device tensor over the ranks, in stream order: the peer kernel when it applies, else NCCL."""
    if _PEER is not None and _PEER.usable(src):
        return _PEER.all_reduce(src, torch.empty_like(src) if out is None else out, "add")
    if out is None:
        out = src.clone()
    elif out.data_ptr() != src.data_ptr():
        out.copy_(src)
    tdist.all_reduce(out, op=tdist.ReduceOp.SUM)
    return out


_OVERLAP = {"active": False, "stream": None, "scope": None}


class overlap_collectives:
    """Inside this block an all-reduce of the path runs on a side stream beside the kernels that follow it, instead of
    between them: the collective's kernel is capped to a few CTAs and the persistent kernels leave `sms` SMs free for it
    (the reference runs every collective in order on stream 0, python/jittor/extern/cuda/nccl/ops/nccl_all_reduce_op.cc:57).
    A result is waited for by whatever reads it first; leaving the block joins the side stream, so everything issued inside
    is ordered before what follows. Every rank must enter and leave the block at the same points. Without the peer
    kernel (one process, or NCCL only) the block changes nothing.

    defer=True holds the all-reduces back until flush() (or until one of their results is read, or the block ends) and then
    issues them back to back on the side stream: the ranks are not tied together between the kernels that produce the
    messages, the SMs are only reserved from the flush on, and the whole exchange runs beside whatever is launched after
    the flush -- the bucketed form of a data-parallel step (python/jittor/optim.py:389-438 gathers gradients the same way)."""

    def __init__(self, sms=None, blocks=None, defer=False):
        # beside persistent kernels the collective gets 8 SMs; a held-back exchange runs beside whatever follows the flush
        # and is the only thing between the step and its end, so it gets 24 (measured on 2 GPUs: 16 blocks move 2 x 4 MiB
        # + 2 x 16 KiB in 0.21 ms, 48 blocks in well under the 0.14 ms of the kernel they run beside)
        self.sms = int(os.environ.get("B200JT_OVERLAP_SMS", 24 if defer else 8)) if sms is None else sms
        self.blocks = int(os.environ.get("B200JT_OVERLAP_BLOCKS", 2 * self.sms)) if blocks is None else blocks
        self.defer = defer
        self.queue = []

    def _reserve(self):
        from . import _capi as C
        C.check(C.lib.b200jt_set_sm_reserve(self.sms), "set_sm_reserve")
        C.check(C.lib.b200jt_peer_comm_set_max_blocks(_PEER._h, self.blocks), "peer max blocks")

    def __enter__(self):
        self.on = _PEER is not None and not _OVERLAP["active"]
        if self.on:
            if _OVERLAP["stream"] is None:
                _OVERLAP["stream"] = torch.cuda.Stream(priority=-1)
            _OVERLAP["active"] = True
            _OVERLAP["scope"] = self
            if not self.defer:
                self._reserve()
        return self

    def flush(self):
        """Issues the held-back all-reduces (every rank at the same point of its program)."""
        if not (self.on and self.queue):
            return
        self._reserve()
        side, cur = _OVERLAP["stream"], torch.cuda.current_stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for src, out, handle in self.queue:
                _PEER.all_reduce(src, out, "add")
                src.record_stream(side)
                out.record_stream(cur)
        join = _StreamJoin(side)
        for _, _, handle in self.queue:
            handle.join = join
        self.queue = []

    def __exit__(self, *exc):
        from . import _capi as C
        if self.on:
            self.flush()
            torch.cuda.current_stream().wait_stream(_OVERLAP["stream"])
            _OVERLAP["active"] = False
            _OVERLAP["scope"] = None
            C.lib.b200jt_set_sm_reserve(0)
            C.lib.b200jt_peer_comm_set_max_blocks(_PEER._h, 0)
        return False


class _StreamJoin:
    """Handle kept by a Var whose value is produced on the side stream: wait() orders the current stream after it."""

    def __init__(self, stream):
        self.event = torch.cuda.Event()
        self.event.record(stream)

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


class _Deferred:
    """Handle of an all-reduce that a defer block holds back: reading the result first makes the block flush."""

    def __init__(self, scope):
        self.scope, self.join = scope, None

    def wait(self):
        if self.join is None:
            self.scope.flush()
        if self.join is not None:
            self.join.wait()


def all_reduce_sum_overlapped(src):
    """(result, join handle or None): the sum over the ranks, issued on the side stream when an overlap block is open and
    the peer kernel takes the message; otherwise in stream order."""
    if not (_OVERLAP["active"] and _PEER is not None and _PEER.usable(src)):
        return all_reduce_sum(src), None
    scope = _OVERLAP["scope"]
    if scope is not None and scope.defer:
        out, handle = torch.empty_like(src), _Deferred(scope)
        scope.queue.append((src, out, handle))
        return out, handle
    side, cur = _OVERLAP["stream"], torch.cuda.current_stream()
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        out = _PEER.all_reduce(src, torch.empty_like(src), "add")
    src.record_stream(side)
    out.record_stream(cur)
    return out, _StreamJoin(side)


def in_mpi():
    return tdist.is_available() and tdist.is_initialized() and tdist.get_world_size() > 1


def world_size():
    return tdist.get_world_size() if in_mpi() else 1


def rank():
    return tdist.get_rank() if in_mpi() else 0


def mpi_all_reduce(x, op="add"):
    """op 'add' or 'mean'; 'mean' is all_reduce(add) / world_size as in the reference (:32-37).
    Without a process group the input is forwarded unchanged (:28-31)."""
    x = V.to_var(x)
    if not in_mpi():
        return x
    if op == "mean":
        return mpi_all_reduce(x, "add") / world_size()
    if op != "add":
        raise ValueError(f"Not supported MPI op {op}")
    return V.Var(x.shape, x.dtype, V.Op("mpi_all_reduce", [x], op="add"))


def mpi_broadcast(x, root=0):
    """Every rank receives root's value (python/jittor/extern/mpi/ops/mpi_broadcast_op.cc; the CUDA relay is
    ncclBroadcast, python/jittor/extern/cuda/nccl/ops/nccl_broadcast_op.cc). Eager: the value is needed now."""
    x = V.to_var(x)
    if not in_mpi():
        return x
    x.sync()
    out = x._data.clone()
    tdist.broadcast(out, src=root)
    return V.Var(x.shape, x.dtype, data=out)


def mpi_reduce(x, op="add", root=0):
    """The root rank receives the sum (or, for "mean", the sum divided by the number of ranks) over all ranks; the other
    ranks receive zeros (python/jittor/extern/mpi/ops/mpi_reduce_op.cc:28-60,92; CUDA relay
    ncclReduce, python/jittor/extern/cuda/nccl/ops/nccl_reduce_op.cc:56). Without a process group x is returned unchanged.
    Eager, like mpi_broadcast."""
    x = V.to_var(x)
    if not in_mpi():
        return x
    if op == "mean":
        return mpi_reduce(x, "add", root) / world_size()
    if op != "add":
        raise ValueError(f"Not supported MPI op {op}")
    x.sync()
    out = x._data.clone()
    tdist.reduce(out, dst=root, op=tdist.ReduceOp.SUM)
    if rank() != root:
        out.zero_()                    # the reference clears the result on the other ranks (mpi_reduce_op.cc:93-95)
    return V.Var(x.shape, x.dtype, data=out)


def all_reduce_buckets(tensors, bucket_bytes=None):
    """Sums a list of tensors over the ranks in as few collectives as possible: tensors of one dtype are packed back
    to back into flat buckets of at most `bucket_bytes` (default: what the peer kernel takes in one call, else 32 MiB),
    each bucket is reduced once, and the results are returned as views into the buckets, in the input order. This
    replaces the reference's one all-reduce per gradient (python/jittor/optim.py:196-198)."""
    if not tensors:
        return []
    if bucket_bytes is None:
        bucket_bytes = _PEER.max_bytes if _PEER is not None else 32 << 20
    out = [None] * len(tensors)
    by_dtype = {}
    for i, t in enumerate(tensors):
        by_dtype.setdefault(t.dtype, []).append(i)
    for dtype, ids in by_dtype.items():
        bucket, used = [], 0
        esize = tensors[ids[0]].element_size()

        def flush():
            nonlocal bucket, used
            if not bucket:
                return
            flat = torch.empty(used // esize, dtype=dtype, device=tensors[bucket[0]].device)
            off = 0
            for i in bucket:
                n = tensors[i].numel()
                flat[off:off + n].copy_(tensors[i].reshape(-1))
                off += _round_up(n * esize, 16) // esize
            flat = all_reduce_sum(flat, out=flat)
            off = 0
            for i in bucket:
                n = tensors[i].numel()
                out[i] = flat[off:off + n].view(tensors[i].shape)
                off += _round_up(n * esize, 16) // esize
            bucket, used = [], 0

        for i in ids:
            nbytes = _round_up(tensors[i].numel() * esize, 16)       # 16-byte slots keep every view vector-aligned
            if bucket and used + nbytes > bucket_bytes:
                flush()
            bucket.append(i)
            used += nbytes
        flush()
    return out


def _round_up(n, m):
    return (n + m - 1) // m * m


# ---- departure of a rank between steps -------------------------------------------------------------------------------
# A collective whose peer is gone can only end in a time-out (NCCL) or a bounded wait running out (the peer kernel).
# Ranks therefore announce that they leave through the job's key-value store, between steps and with nothing of theirs
# in flight, and the others ask the store before their next step instead of finding out on the device.
def _store():
    return tdist.distributed_c10d._get_default_store()


def leave():
    """Announces that this rank stops taking part (call between steps; then exit or idle)."""
    if in_mpi():
        _store().set(f"b200jt/left/{rank()}", "1")


def departed():
    """Ranks that have announced their departure (one non-blocking store query per rank)."""
    if not in_mpi():
        return []
    st = _store()
    return [r for r in range(world_size()) if r != rank() and st.check([f"b200jt/left/{r}"])]


def check_peers():
    """Raises before the next collective is launched if a peer has left."""
    gone = departed()
    if gone:
        from ._capi import B200Error
        raise B200Error(f"rank(s) {gone} left the job: the next collective would never complete")
