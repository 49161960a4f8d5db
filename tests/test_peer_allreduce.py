"""The NVLink peer all-reduce kernel with every rank of the job on ONE device (one cooperative launch plays all
ranks), against a rank-ordered sum computed by torch: bit-exact, since the kernel adds in rank order too."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rank_ordered(srcs, op):
    acc_t = torch.float32 if srcs[0].dtype in (torch.bfloat16, torch.float16) else srcs[0].dtype
    acc = srcs[0].to(acc_t)
    for s in srcs[1:]:
        s = s.to(acc_t)
        acc = acc + s if op == "add" else (torch.maximum(acc, s) if op == "maximum" else torch.minimum(acc, s))
    return acc.to(srcs[0].dtype)


def make(world, count, dtype, seed, offset=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = []
    for _ in range(world):
        if dtype.is_floating_point:
            t = torch.randn(count + offset, generator=g, device="cuda", dtype=torch.float32).to(dtype)
        else:
            t = torch.randint(-1000, 1000, (count + offset,), generator=g, device="cuda", dtype=dtype)
        out.append(t[offset:])
    return out


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.int32, torch.bfloat16, torch.float64, torch.int64, torch.float16])
def test_local_job_matches_rank_ordered_sum(world, dtype):
    from jittor_b200 import peer
    job = peer.LocalJob(world, data_bytes=2 << 20)
    try:
        # one-shot sizes (incl. ragged tails and one element), then two-shot sizes (> 256 KiB), repeated so that both
        # staging halves and growing epochs are exercised, with and without 16-byte aligned pointers
        for seed, (count, offset) in enumerate([(1, 0), (512, 0), (4099, 0), (4096, 1), (65536 + 3, 0),
                                                (300_000, 0), (262_147, 1), (2 << 20, 0), (512, 0), (300_000, 0)]):
            count = min(count, (2 << 20) // torch.empty(0, dtype=dtype).element_size())
            srcs = make(world, count, dtype, seed, offset)
            dsts = [torch.full_like(s, 7) for s in srcs]
            job.all_reduce(srcs, dsts, "add")
            want = rank_ordered(srcs, "add")
            for d in dsts:
                assert torch.equal(d, want), (world, dtype, count, offset)
    finally:
        job.close()


@pytest.mark.parametrize("op", ["maximum", "minimum"])
def test_local_job_max_min_and_in_place(op):
    from jittor_b200 import peer
    job = peer.LocalJob(4, data_bytes=1 << 20)
    try:
        for count in (1000, 200_000):
            srcs = make(4, count, torch.float32, 3)
            want = rank_ordered(srcs, op)
            job.all_reduce(srcs, srcs, op)              # dst aliases src
            for s in srcs:
                assert torch.equal(s, want)
    finally:
        job.close()


def test_message_larger_than_the_segment_is_rejected():
    from jittor_b200 import peer, _capi as C
    job = peer.LocalJob(2, data_bytes=1 << 16)
    try:
        srcs = make(2, (1 << 16) // 4 + 1, torch.float32, 0)
        with pytest.raises(C.B200Error, match="exceeds"):
            job.all_reduce(srcs, [torch.empty_like(s) for s in srcs])
    finally:
        job.close()


def test_absent_peer_runs_into_the_wait_bound_and_leaves_the_context_usable():
    """One rank of a two-rank job is launched alone: nothing ever sets the flag it waits for, the wait gives up
    after its bound, the status word says so, and the device keeps working."""
    from jittor_b200 import peer, _capi as C
    assert C.lib.b200jt_device_status() == 0
    job = peer.LocalJob(2, data_bytes=1 << 16, wait_ms=50.0)
    try:
        src = torch.ones(1024, device="cuda")
        dst = torch.zeros(1024, device="cuda")
        job.rank_alone(0, src, dst)
        assert C.lib.b200jt_device_status() == 5
        assert C.lib.b200jt_device_status() == 0        # cleared by the read
    finally:
        job.close()
    job = peer.LocalJob(2, data_bytes=1 << 16)
    try:
        srcs = make(2, 1024, torch.float32, 1)
        dsts = job.all_reduce(srcs, [torch.empty_like(s) for s in srcs])
        assert torch.equal(dsts[0], rank_ordered(srcs, "add"))
    finally:
        job.close()


def test_alternating_message_sizes_keep_all_blocks_on_one_call_count():
    """The block count follows the message size; blocks a small call leaves idle must still advance with the call
    count, or a later large call would mix staging halves between its blocks. Sizes in 16-byte packs: 512 / 600 / 512
    (one and two blocks), then one-block and 128-block messages in turn, one-shot and two-shot."""
    from jittor_b200 import peer
    job = peer.LocalJob(4, data_bytes=4 << 20)
    try:
        counts = [2048, 2400, 2048, 4, 1 << 18, 4, 1 << 20, 2400, 1 << 18, 1, 1 << 20]
        for seed, count in enumerate(counts * 2):
            srcs = make(4, count, torch.float32, 100 + seed)
            dsts = [torch.full_like(s, -3) for s in srcs]
            job.all_reduce(srcs, dsts, "add")
            want = rank_ordered(srcs, "add")
            for d in dsts:
                assert torch.equal(d, want), (seed, count)
    finally:
        job.close()
