"""Host side of the NVLink peer all-reduce kernel (csrc/peer_allreduce.cu): segment set-up and handle exchange
over the existing process group, and the call the executor makes in place of the reference's NCCL relay
(python/jittor/extern/cuda/nccl/ops/nccl_all_reduce_op.cc:46-58).

`PeerComm.connect()` is collective: either every rank ends up with a communicator or none does (then the executor
keeps using NCCL), so ranks can never disagree on which path a given all-reduce takes."""
import ctypes
import os

import torch
import torch.distributed as tdist

from . import _capi as C

HANDLE_BYTES = 64
DTYPES = ("float32", "float64", "int32", "int64", "float16", "bfloat16")


def _dtype_code(t):
    name = str(t.dtype).replace("torch.", "")
    if name not in DTYPES:
        return None
    return C.DTYPE_CODES[name]


class PeerComm:
    def __init__(self, handle, rank, world, max_bytes):
        self._h, self.rank, self.world, self.max_bytes = handle, rank, world, max_bytes

    @classmethod
    def connect(cls, data_bytes=None, wait_ms=None):
        """Builds the communicator over the default process group (all ranks on this node, 2..8 of them).
        Returns None on every rank if any rank could not export or map a segment."""
        world, rank = tdist.get_world_size(), tdist.get_rank()
        if world < 2 or world > 8 or int(os.environ.get("LOCAL_WORLD_SIZE", world)) != world:
            return None
        data_bytes = data_bytes or int(os.environ.get("B200JT_PEER_BYTES", 8 << 20))
        wait_ms = wait_ms or float(os.environ.get("B200JT_PEER_WAIT_MS", 20000))
        C.require_cuda()
        seg, handle = ctypes.c_void_p(), ctypes.create_string_buffer(HANDLE_BYTES)
        ok = C.lib.b200jt_peer_segment_create(data_bytes, ctypes.byref(seg), handle) == 0
        mine = (ok, handle.raw if ok else b"", C.lib.b200jt_last_error().decode(errors="replace") if not ok else "")
        everyone = [None] * world
        tdist.all_gather_object(everyone, mine)
        comm = ctypes.c_void_p()
        if all(e[0] for e in everyone):
            blob = b"".join(e[1] for e in everyone)
            ok = C.lib.b200jt_peer_comm_create(rank, world, seg, blob, data_bytes, wait_ms, ctypes.byref(comm)) == 0
        else:
            ok = False
        err = "" if ok else C.lib.b200jt_last_error().decode(errors="replace")
        verdicts = [None] * world
        tdist.all_gather_object(verdicts, (ok, err))
        if not all(v[0] for v in verdicts):
            if ok:
                C.lib.b200jt_peer_comm_destroy(comm)       # frees the segment it took over
            elif seg:
                C.lib.b200jt_peer_segment_destroy(seg)     # exported here, but the job as a whole could not connect
            if rank == 0:
                why = next((v[1] for v in verdicts if not v[0] and v[1]), "") or next((e[2] for e in everyone if not e[0]), "")
                print(f"[jittor_b200] peer all-reduce unavailable, using NCCL: {why}", flush=True)
            return None
        tdist.barrier()                      # nobody flags a segment before everyone has mapped it
        return cls(comm, rank, world, data_bytes)

    def usable(self, t):
        return (t.is_cuda and t.is_contiguous() and _dtype_code(t) is not None
                and 0 < t.numel() * t.element_size() <= self.max_bytes)

    def all_reduce(self, src, dst, op="add"):
        """dst = op over the ranks of src (same shape and dtype; may be the same tensor); on the current stream."""
        C.check(C.lib.b200jt_peer_all_reduce(self._h, ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst.data_ptr()),
                                             src.numel(), _dtype_code(src), op.encode(), C.stream_ptr()),
                "peer_all_reduce")
        return dst

    def close(self):
        if self._h:
            C.lib.b200jt_peer_comm_destroy(self._h)
            self._h = None


class LocalJob:
    """All ranks of a job on one device, played by a single cooperative launch (tests; no process group)."""

    def __init__(self, world, data_bytes=1 << 20, wait_ms=2000.0):
        C.require_cuda()
        self.world, self.max_bytes = world, data_bytes
        self._comms = (ctypes.c_void_p * world)()
        C.check(C.lib.b200jt_peer_comm_create_local(world, data_bytes, wait_ms, self._comms), "peer_comm_create_local")

    def all_reduce(self, srcs, dsts, op="add"):
        n = self.world
        sp = (ctypes.c_void_p * n)(*[s.data_ptr() for s in srcs])
        dp = (ctypes.c_void_p * n)(*[d.data_ptr() for d in dsts])
        C.check(C.lib.b200jt_peer_all_reduce_local(self._comms, n, sp, dp, srcs[0].numel(), _dtype_code(srcs[0]),
                                                   op.encode(), C.stream_ptr()), "peer_all_reduce_local")
        return dsts

    def rank_alone(self, rank, src, dst, op="add"):
        """Launches ONE rank of the job only: its peers never arrive, so its waits run out (failure-path test)."""
        C.check(C.lib.b200jt_peer_all_reduce(self._comms[rank], ctypes.c_void_p(src.data_ptr()),
                                             ctypes.c_void_p(dst.data_ptr()), src.numel(), _dtype_code(src),
                                             op.encode(), C.stream_ptr()), "peer_all_reduce")

    def close(self):
        for c in self._comms:
            if c:
                C.lib.b200jt_peer_comm_destroy(c)
        self._comms = (ctypes.c_void_p * self.world)()
