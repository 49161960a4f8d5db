"""Worker of tests/test_dist_gloo.py: run under torchrun with 2 ranks on CPU (gloo)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import jittor_b200 as jt                      # noqa: E402
from jittor_b200 import dist, executor, nn    # noqa: E402


def main():
    dist.init("gloo")
    rank, world = dist.rank(), dist.world_size()
    assert dist.in_mpi() and world == 2
    # 1. the all-reduce node sums the ranks' tensors (host tensors stand in for device buffers)
    v = jt.Var([4], "float32")
    v._data = torch.full((4,), float(rank + 1))
    out = v.mpi_all_reduce("add")
    out.sync().wait()
    assert torch.equal(out._data, torch.full((4,), 3.0)), out._data
    # 2. 'mean' is add / world_size, as in the reference
    m = v.mpi_all_reduce("mean")
    assert m._op.kind == "binary" and m._op.attrs["op"] == "divide"
    assert m._op.inputs[0]._op.kind == "mpi_all_reduce" and m._op.inputs[1]._const == 2
    # 3. sync BatchNorm (+ReLU, fed by a conv) is still recognised as one plan with the all-reduce inside
    x, w = jt.Var([4, 8, 10, 10], "float32"), jt.Var([16, 8, 3, 3], "float32")
    bn = nn.BatchNorm(16, is_train=True, sync=True)
    y = nn.relu(bn(nn.conv2d(x, w, None, 1, 1, 1)))
    plan = executor._match_batchnorm(y)
    assert plan is not None and plan.leaves[:2] == [x, w]
    xb, wb = jt.Var([4, 64, 16, 16], "bfloat16"), jt.Var([64, 64, 3, 3], "bfloat16")
    bnb = nn.BatchNorm(64, is_train=True, sync=True)
    with jt.flag_scope(amp_reg=2):
        yb = nn.relu(bnb(nn.conv2d(xb, wb, None, 1, 1, 1)))
    planb = executor._match_batchnorm(yb)
    assert yb.dtype == "bfloat16" and planb is not None and planb.leaves[:2] == [xb, wb]
    # 4. rank-divergent data, identical reduction: packed statistics message
    stats = torch.tensor([float(rank), 10.0 * (rank + 1)])
    torch.distributed.all_reduce(stats)
    assert stats.tolist() == [1.0, 30.0]
    # 5. bucketed gradient exchange: mixed dtypes and sizes, a bucket limit that forces several collectives
    gen = torch.Generator().manual_seed(7 + rank)
    shapes = [(3, 5), (1,), (17,), (4, 4, 4), (2, 9)]
    ts = [torch.randn(s, generator=gen) for s in shapes] + [torch.randint(0, 9, (11,), generator=gen, dtype=torch.int32)]
    want = []
    for t in ts:
        w = t.clone()
        torch.distributed.all_reduce(w)
        want.append(w)
    for limit in (64, 1 << 20):
        got = dist.all_reduce_buckets([t.clone() for t in ts], bucket_bytes=limit)
        for g, w, t in zip(got, want, ts):
            assert g.shape == t.shape and g.dtype == t.dtype and torch.equal(g, w), (limit, g, w)
    # 6. parameter broadcast from rank 0
    p = jt.Var([3], "float32")
    p._data = torch.full((3,), float(10 + rank))
    b = dist.mpi_broadcast(p, 0)
    assert torch.equal(b._data, torch.full((3,), 10.0))
    # 6b. reduce to a root: the root holds the sum (or mean), the other rank zeros
    q = jt.Var([3], "float32")
    q._data = torch.full((3,), float(1 + rank))
    for root in (0, 1):
        r = dist.mpi_reduce(q, "add", root)
        assert torch.equal(r._data, torch.full((3,), 3.0 if rank == root else 0.0)), (root, r._data)
    m = q.mpi_reduce("mean", 1)
    assert m._op.kind == "binary" and m._op.attrs["op"] == "divide"
    # 7. a rank leaves between steps: the other one learns of it from the store, not from a collective that hangs
    import time
    assert dist.departed() == []
    dist.check_peers()
    torch.distributed.barrier()
    if rank == 1:
        dist.leave()
        print(f"rank {rank} ok")
        return
    deadline = time.time() + 30
    while dist.departed() != [1] and time.time() < deadline:
        time.sleep(0.05)
    assert dist.departed() == [1]
    try:
        dist.check_peers()
        raise AssertionError("check_peers did not raise")
    except jt.B200Error as e:
        assert "rank(s) [1] left" in str(e)
    print(f"rank {rank} ok")


if __name__ == "__main__":
    main()
