"""Worker of tests/test_peer_multi_gpu.py: run under torchrun with one rank per GPU (NCCL). Checks the peer
all-reduce kernel against NCCL on the same tensors, then the Var-level all-reduce and sync BatchNorm through it."""
import os
import sys

import torch
import torch.distributed as tdist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import jittor_b200 as jt                      # noqa: E402
from jittor_b200 import _capi as C, dist, nn  # noqa: E402


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init("nccl")
    rank, world = dist.rank(), dist.world_size()
    pc = dist.peer_comm()
    assert pc is not None, "peer communicator was not set up"
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    for rep in range(3):
        for dtype in (torch.float32, torch.int32, torch.bfloat16):
            for count in (1, 512, 4099, 100_000, 1 << 20, (2 << 20) - 3):
                if count * torch.empty(0, dtype=dtype).element_size() > pc.max_bytes:
                    continue
                if dtype.is_floating_point:
                    x = torch.randn(count, generator=g, device="cuda").to(dtype)
                else:
                    x = torch.randint(0, 100, (count,), generator=g, device="cuda", dtype=dtype)
                got = pc.all_reduce(x, torch.empty_like(x))
                # rank-ordered reference: gather every rank's tensor and add them in order
                parts = [torch.empty_like(x) for _ in range(world)]
                tdist.all_gather(parts, x)
                acc = parts[0].float() if dtype == torch.bfloat16 else parts[0].clone()
                for p in parts[1:]:
                    acc = acc + (p.float() if dtype == torch.bfloat16 else p)
                assert torch.equal(got, acc.to(dtype)), (rep, dtype, count)
    # Var-level: scatter-add onto a shared output, all-reduced
    idx = torch.randint(0, 1 << 16, (1 << 20,), generator=g, device="cuda", dtype=torch.int32)
    val = torch.randint(0, 100, (1 << 20,), generator=g, device="cuda", dtype=torch.int32)
    out = jt.array(val).reindex_reduce("add", [1 << 16], ["@e0(i0)"], extras=[jt.array(idx)]).mpi_all_reduce("add")
    got = out.sync()._data
    local = torch.zeros(1 << 16, dtype=torch.int32, device="cuda").index_add_(0, idx.long(), val)
    tdist.all_reduce(local)
    assert torch.equal(got, local)
    # the same all-reduce run BESIDE the next scatter (side stream, capped blocks, reserved SMs): same bits, also from a
    # captured graph replayed several times
    parts = []
    for k in range(3):
        ik = torch.randint(0, 1 << 20, (1 << 22,), generator=g, device="cuda", dtype=torch.int32)
        vk = torch.randint(0, 100, (1 << 22,), generator=g, device="cuda", dtype=torch.int32)
        parts.append((jt.array(vk), jt.array(ik)))

    def step():
        with dist.overlap_collectives():
            return [v.reindex_reduce("add", [1 << 20], ["@e0(i0)"], extras=[i]).mpi_all_reduce("add").sync() for v, i in parts]

    want = [v.reindex_reduce("add", [1 << 20], ["@e0(i0)"], extras=[i]).mpi_all_reduce("add").torch().clone() for v, i in parts]
    for o, w_ in zip(step(), want):
        assert torch.equal(o.torch(), w_)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    tdist.barrier()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step()
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    for o, w_ in zip(outs, want):
        assert torch.equal(o._data.view(-1), w_.view(-1))
    assert C.lib.b200jt_device_status() == 0

    # the same step with the all-reduces held back and issued together (defer), directly and from a captured graph;
    # a result read before the flush makes the block flush by itself
    def step_deferred():
        with dist.overlap_collectives(defer=True) as scope:
            outs = [v.reindex_reduce("add", [1 << 20], ["@e0(i0)"], extras=[i]).mpi_all_reduce("add").sync() for v, i in parts]
            scope.flush()
            tail = (parts[0][0] + 1).sync()                  # a kernel that runs beside the exchange
            return outs, tail
    outs, _ = step_deferred()
    for o, w_ in zip(outs, want):
        assert torch.equal(o.torch(), w_)
    with dist.overlap_collectives(defer=True):
        early = parts[0][0].reindex_reduce("add", [1 << 20], ["@e0(i0)"], extras=[parts[0][1]]).mpi_all_reduce("add")
        assert torch.equal((early + 0).torch(), want[0])   # read inside the block, before any flush
    torch.cuda.synchronize()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step_deferred()
    torch.cuda.current_stream().wait_stream(side)
    tdist.barrier()
    torch.cuda.synchronize()
    graph2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph2):
        outs2, _ = step_deferred()
    for _ in range(5):
        graph2.replay()
    torch.cuda.synchronize()
    for o, w_ in zip(outs2, want):
        assert torch.equal(o._data.view(-1), w_.view(-1))
    assert C.lib.b200jt_device_status() == 0
    # sync BatchNorm statistics over the ranks' batches
    x = torch.randn(8, 64, 16, 16, generator=g, device="cuda")
    bn = nn.BatchNorm(64, is_train=True, sync=True)
    y = nn.relu(bn(jt.array(x))).sync()._data
    allx = [torch.empty_like(x) for _ in range(world)]
    tdist.all_gather(allx, x)
    full = torch.cat(allx)
    mean = full.mean((0, 2, 3), keepdim=True)
    var = full.var((0, 2, 3), unbiased=False, keepdim=True)
    want = torch.relu((x - mean) / torch.sqrt(var + 1e-5))
    assert torch.allclose(y, want, rtol=1e-4, atol=1e-4), (y - want).abs().max()
    # data-parallel SGD: each rank holds a slice of the batch; the bucketed, averaged gradients must give every rank
    # the parameters of a single-process run over the whole batch
    from jittor_b200 import optim
    gw = torch.Generator(device="cuda").manual_seed(5)
    w0 = torch.randn(16, 4, generator=gw, device="cuda")
    b0 = torch.randn(4, generator=gw, device="cuda")
    xs = torch.randn(8, 16, generator=g, device="cuda")
    ys = torch.randn(8, 4, generator=g, device="cuda")
    w, b = jt.array(w0.clone()), jt.array(b0.clone())
    opt = optim.SGD([w, b], lr=0.1, momentum=0.9)
    for _ in range(3):
        d = nn.matmul(jt.array(xs), w) + b - jt.array(ys)
        opt.step((d * d).sum() * (1.0 / 8))
    ax = [torch.empty_like(xs) for _ in range(world)]
    ay = [torch.empty_like(ys) for _ in range(world)]
    tdist.all_gather(ax, xs)
    tdist.all_gather(ay, ys)
    fx, fy = torch.cat(ax), torch.cat(ay)
    tw, tb = w0.clone().requires_grad_(), b0.clone().requires_grad_()
    topt = torch.optim.SGD([tw, tb], lr=0.1, momentum=0.9)
    for _ in range(3):
        topt.zero_grad()
        (((fx @ tw + tb - fy) ** 2).sum() / fx.shape[0]).backward()
        topt.step()
    assert torch.allclose(w.torch(), tw.detach(), rtol=1e-4, atol=1e-5), (w.torch() - tw).abs().max()
    assert torch.allclose(b.torch(), tb.detach(), rtol=1e-4, atol=1e-5)
    assert C.lib.b200jt_device_status() == 0
    tdist.barrier()
    print(f"rank {rank} ok", flush=True)


if __name__ == "__main__":
    main()
