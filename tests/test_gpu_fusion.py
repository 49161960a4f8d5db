"""GPU parity of the fused-chain kernels (csrc/chain_jit.cu, csrc/fused_chain.cu, fusion.py): every case is computed four
ways -- fused through the kernel compiled for the chain (one launch, asserted through the executor's plan counter; a
failed compilation is an error here), fused through the interpreting kernel (must be the same bits), op by op with fusion
switched off, and by the CPU oracle's element-wise / reduce restatements. Fused and unfused results must be the same bits for element-wise chains (both round
every intermediate to its dtype); reductions and the oracle are compared with the fp32 1e-5 (bf16 2e-2) mixed tolerance."""
import numpy as np
import pytest
import torch

from oracle import meta_ops_ref as ref
from tests.golden_cases import check

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def jt():
    import jittor_b200
    return jittor_b200


def bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16().float().numpy()


def run_both(jt, build, arrays, reduces=False):
    """build(*Vars) -> Var. Returns (fused numpy, unfused numpy, plans run by the fused sync). The compiled and the
    interpreting kernel must agree bit for bit on element-wise chains; with a reduce in the chain (reduces=True) the two
    fold in different orders (4 against 8 elements per thread) and are compared with the float tolerance."""
    from jittor_b200 import executor
    vs = [jt.array(a) for a in arrays]
    for v in vs:
        v.sync()
    import os
    saved = os.environ.get("B200JT_CHAIN_JIT")
    try:
        os.environ["B200JT_CHAIN_JIT"] = "2"            # the compiled kernel, or an error
        out = build(*vs)
        before = executor.counters["plans"]
        fused = out.numpy()
        plans = executor.counters["plans"] - before
        os.environ["B200JT_CHAIN_JIT"] = "0"            # the interpreting kernel
        interpreted = build(*vs).numpy()
    finally:
        if saved is None:
            os.environ.pop("B200JT_CHAIN_JIT", None)
        else:
            os.environ["B200JT_CHAIN_JIT"] = saved
    if reduces:
        check(fused, interpreted, False, rtol=2e-2 if fused.dtype != np.float32 else 1e-5)
    else:
        assert np.array_equal(fused, interpreted, equal_nan=True), "compiled and interpreted chains differ"
    with jt.flag_scope(b200_fuse_chains=0):
        unfused = build(*vs).numpy()
    return fused, unfused, plans


@pytest.mark.parametrize("shape", [(32768 // 64, 4096), (37, 53), (5, 6, 7), (1, 9), (300, 1000)])
def test_scale_shift_and_relu_bias(jt, shape):
    from jittor_b200 import nn
    rng = np.random.default_rng(sum(shape))
    x = rng.normal(size=shape).astype(np.float32)
    w, b = rng.normal(size=shape[-1:]).astype(np.float32), rng.normal(size=shape[-1:]).astype(np.float32)
    fused, unfused, plans = run_both(jt, lambda X, W, B: X * W + B, [x, w, b])
    assert plans == 1 and np.array_equal(fused, unfused)
    check(fused, ref.binary(ref.binary(x, w, "multiply"), b, "add"), False)
    fused, unfused, plans = run_both(jt, lambda X, B: nn.relu(X + B), [x, b])
    assert plans == 1 and np.array_equal(fused, unfused)
    check(fused, np.maximum(x + b, 0), False)


@pytest.mark.parametrize("shape", [(512, 4096), (37, 53), (64, 1000), (3, 5, 70), (130, 8)])
def test_multiply_then_row_reduce(jt, shape):
    rng = np.random.default_rng(sum(shape) + 1)
    a, b = rng.normal(size=shape).astype(np.float32), rng.normal(size=shape).astype(np.float32)
    for op, npf in (("add", np.sum), ("maximum", np.max), ("minimum", np.min), ("mean", np.mean)):
        fused, unfused, plans = run_both(jt, lambda A, B: (A * B).reduce(op, -1), [a, b], reduces=True)
        assert plans == 1
        want = ref.reduce(ref.binary(a, b, "multiply"), op, (-1,))
        check(fused, want, False)
        check(unfused, want, False)
    # keepdims, and two trailing axes at once
    if len(shape) == 3:
        fused, _, plans = run_both(jt, lambda A, B: (A + B).sum([1, 2], keepdims=True), [a, b], reduces=True)
        assert plans == 1
        check(fused, ref.reduce(a + b, "add", (1, 2), True), False)


def test_centre_and_scale_rows(jt):
    rng = np.random.default_rng(3)
    x = (rng.normal(size=(257, 771)) * 3 + 1).astype(np.float32)

    def build(X):
        m = X.mean(1, keepdims=True)
        v = ((X - m) * (X - m)).mean(1, keepdims=True)
        return (X - m) / (v + 1e-5).sqrt()

    fused, unfused, plans = run_both(jt, build, [x], reduces=True)
    assert plans == 1
    xd = x.astype(np.float64)
    want = ((xd - xd.mean(1, keepdims=True)) / np.sqrt(xd.var(1, keepdims=True) + 1e-5)).astype(np.float32)
    check(fused, want, False, rtol=1e-4)
    check(unfused, want, False, rtol=1e-4)


def _softmax_by_hand(x):
    e = (x - x.max(-1, keepdims=True)).exp()
    return e / e.sum(-1, keepdims=True)


@pytest.mark.parametrize("rows,cols", [(64, 4096), (33, 1000), (7, 10)])
def test_softmax_backward_chain_one_launch(jt, rows, cols):
    """Reverse mode through a softmax written with meta-ops (no backward rule of its own): five row statements, one launch."""
    rng = np.random.default_rng(rows)
    x, dy = rng.normal(size=(rows, cols)).astype(np.float32), rng.normal(size=(rows, cols)).astype(np.float32)
    fused, unfused, plans = run_both(jt, lambda X, DY: jt.grad((_softmax_by_hand(X) * DY).sum(), X), [x, dy], reduces=True)
    assert plans == 1
    y = ref.softmax(x, -1).astype(np.float64)
    want = (y * (dy - (y * dy).sum(-1, keepdims=True))).astype(np.float32)
    check(fused, want, False, rtol=1e-4)
    check(unfused, want, False, rtol=1e-4)


def test_channel_scale_shift_relu_bf16(jt):
    """x[N,C,H,W] * w[C] + b[C] then ReLU with bfloat16 results kept (amp_reg bit 2): inputs broadcast over non-trailing
    axes, every intermediate rounded to bfloat16 as op by op."""
    from jittor_b200 import nn
    rng = np.random.default_rng(9)
    x = bf16_round(rng.normal(size=(6, 24, 9, 11)))
    w, b = rng.normal(size=24).astype(np.float32), rng.normal(size=24).astype(np.float32)

    def build(X, W, B):
        with jt.flag_scope(amp_reg=2):
            return nn.relu(X * W.broadcast(X, [0, 2, 3]) + B.broadcast(X, [0, 2, 3]))

    from jittor_b200 import executor
    X, W, B = jt.array(torch.from_numpy(x).bfloat16()), jt.array(w), jt.array(b)
    out = build(X, W, B)
    assert out.dtype == "bfloat16"
    before = executor.counters["plans"]
    fused = out.numpy()
    assert executor.counters["plans"] - before == 1
    with jt.flag_scope(b200_fuse_chains=0):
        unfused = build(X, W, B).numpy()
    assert np.array_equal(fused, unfused)
    want = np.maximum(bf16_round(bf16_round(x * w[None, :, None, None]) + b[None, :, None, None]), 0)
    check(fused, bf16_round(want), False, rtol=2e-2)


def test_mixed_ops_and_comparisons(jt):
    rng = np.random.default_rng(12)
    a = rng.uniform(0.5, 2.0, size=(45, 130)).astype(np.float32)
    b = rng.uniform(0.5, 2.0, size=(45, 130)).astype(np.float32)
    m = (rng.uniform(size=(45, 1)) > 0.5)

    def build(A, B, M):
        t = (A / B).log() + (A * B).sqrt() - jt.sigmoid(A - B)
        return jt.ternary(M, t.exp(), jt.minimum(A, B) ** 2.0) * (A > B)

    fused, unfused, plans = run_both(jt, build, [a, b, m])
    assert plans == 1 and np.array_equal(fused, unfused)
    t = np.log(a / b) + np.sqrt(a * b) - 1 / (1 + np.exp(-(a - b)))
    want = np.where(m, np.exp(t), np.minimum(a, b) ** 2.0) * (a > b)
    check(fused, want.astype(np.float32), False, rtol=1e-5)


def test_unaligned_and_ragged_rows(jt):
    """Row lengths that are not whole 8-element vectors and views that start off a 32-byte boundary."""
    rng = np.random.default_rng(21)
    base = rng.normal(size=(19 * 13 + 3,)).astype(np.float32)
    t = torch.from_numpy(base).cuda()
    x = jt.array(t[3:].reshape(19, 13))
    b = jt.array(rng.normal(size=13).astype(np.float32))
    got = ((x + b) * 2.0 - 1.0).numpy()
    check(got, (base[3:].reshape(19, 13) + b.numpy()) * 2.0 - 1.0, False)
    got = ((x * x) + 1.0).sum(1).numpy()
    check(got, ((base[3:].reshape(19, 13) ** 2) + 1.0).sum(1), False)


@pytest.mark.parametrize("rows,cols", [(64, 4096), (33, 1000), (7, 10), (5, 9000), (3, 8)])
@pytest.mark.parametrize("log", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_nn_softmax_backward_kernel(jt, rows, cols, log, dtype):
    """nn.softmax / log_softmax over the last axis carry their own backward (one kernel from y and dy, as the reference's CUDA
    softmax does): against float64 formulas, and against reverse mode through the hand-written chain."""
    from jittor_b200 import nn
    rng = np.random.default_rng(rows + cols)
    x, dy = rng.normal(size=(rows, cols)).astype(np.float32), rng.normal(size=(rows, cols)).astype(np.float32)
    if dtype == "bfloat16":
        x, dy = bf16_round(x), bf16_round(dy)
        X, DY = jt.array(torch.from_numpy(x).bfloat16()), jt.array(torch.from_numpy(dy).bfloat16())
    else:
        X, DY = jt.array(x), jt.array(dy)
    y = nn.softmax(X, -1, log)
    g = jt.grad((y * DY).sum(), X)
    assert g._op.kind == "custom"
    got = g.numpy()
    xd, dd = x.astype(np.float64), dy.astype(np.float64)
    e = np.exp(xd - xd.max(-1, keepdims=True))
    sm = e / e.sum(-1, keepdims=True)
    want = dd - sm * dd.sum(-1, keepdims=True) if log else sm * (dd - (sm * dd).sum(-1, keepdims=True))
    if dtype == "bfloat16":
        check(got, bf16_round(want), False, rtol=3e-2)
    else:
        check(got, want.astype(np.float32), False, rtol=1e-5)
        if not log:
            by_hand = jt.grad((_softmax_by_hand(X) * DY).sum(), X).numpy()
            check(got, by_hand, False, rtol=1e-5)


def test_compiled_kernels_are_cached_per_program_not_per_size_or_constant(jt):
    import ctypes
    from jittor_b200 import _capi as C

    def stats():
        c, h, f = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        C.check(C.lib.b200jt_chain_jit_stats(ctypes.byref(c), ctypes.byref(h), ctypes.byref(f)), "stats")
        return c.value, h.value, f.value
    rng = np.random.default_rng(5)
    c0, h0, f0 = stats()
    for rows, k in ((64, 0.25), (128, 0.5), (256, 3.0)):
        x = rng.normal(size=(rows, 512)).astype(np.float32)
        got = ((jt.array(x) * k + 1.0).exp() * 2.0).numpy()
        check(got, np.exp(x * np.float32(k) + 1) * 2, False)
    c1, h1, f1 = stats()
    assert f1 == f0 and c1 - c0 <= 1 and h1 - h0 >= 2


@pytest.mark.parametrize("shape", [(512, 1024), (37, 771), (64, 4096)])
def test_layernorm_backward_runs_as_one_kernel(jt, shape):
    """d LayerNorm / dx built by jt.grad from the per-op rules: one plan, the same result as op by op and as torch autograd."""
    from jittor_b200 import nn
    rng = np.random.default_rng(shape[1])
    x = rng.normal(size=shape).astype(np.float32)
    dy = rng.normal(size=shape).astype(np.float32)
    g = (1 + 0.1 * rng.normal(size=shape[1])).astype(np.float32)
    b = rng.normal(size=shape[1]).astype(np.float32)

    def build(X, DY, G, B):
        return jt.grad((nn.layer_norm(X, (shape[1],), G, B) * DY).sum(), X)

    fused, unfused, plans = run_both(jt, build, [x, dy, g, b], reduces=True)
    assert plans == 1
    check(fused, unfused, False, rtol=1e-4)
    xt = torch.from_numpy(x).requires_grad_()
    torch.nn.functional.layer_norm(xt, (shape[1],), torch.from_numpy(g), torch.from_numpy(b), 1e-5).backward(torch.from_numpy(dy))
    check(fused, xt.grad.numpy(), False, rtol=1e-4)
