"""GPU parity of the callers either side of the path at sizes beyond the fixtures: slicing / scatter / gather against
the numpy oracle and against independent torch formulations, pooling forward / backward against the oracle, grouped and
transposed convolution against the oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def jt():
    import jittor_b200
    return jittor_b200


@pytest.fixture(scope="module")
def ref():
    from oracle import meta_ops_ref
    return meta_ops_ref


def test_getitem_rows_large(jt):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(1 << 16, 48, generator=g)
    idx = torch.randint(-(1 << 16), 1 << 16, (100_000,), generator=g, dtype=torch.int32)      # negatives wrap once
    got = jt.array(table)[jt.array(idx)].torch().cpu()
    assert torch.equal(got, table[idx.long()])


def test_getitem_mixed_matches_oracle(jt, ref):
    rng = np.random.default_rng(1)
    x = rng.normal(size=(37, 29, 41)).astype(np.float32)
    a = rng.integers(0, 29, size=(5, 1)).astype(np.int32)
    b = rng.integers(0, 41, size=(7,)).astype(np.int64)
    sl = (slice(30, 2, -3), a, b)
    want = ref.getitem(x, sl)
    got = jt.array(x)[slice(30, 2, -3), jt.array(a), jt.array(b)].numpy()
    assert np.array_equal(got, want)


def test_setitem_add_duplicates_int_exact(jt):
    g = torch.Generator().manual_seed(2)
    x = torch.randint(0, 10, (5000, 16), generator=g, dtype=torch.int32)
    idx = torch.randint(0, 5000, (200_000,), generator=g, dtype=torch.int32)
    v = torch.randint(0, 10, (200_000, 16), generator=g, dtype=torch.int32)
    got = jt.array(x).setitem((jt.array(idx),), jt.array(v), "add").torch().cpu()
    want = x.clone().index_add_(0, idx.long(), v)
    assert torch.equal(got, want)


def test_setitem_python_syntax_rebinds(jt):
    x = jt.array(np.zeros((4, 6), np.float32))
    x[1:3, ::2] = 5.0
    want = np.zeros((4, 6), np.float32)
    want[1:3, ::2] = 5.0
    assert np.array_equal(x.numpy(), want)
    x[jt.array(np.array([0, 3], np.int32))] = jt.array(np.arange(12, dtype=np.float32).reshape(2, 6))
    want[[0, 3]] = np.arange(12, dtype=np.float32).reshape(2, 6)
    assert np.array_equal(x.numpy(), want)


def test_scatter_gather_roundtrip(jt):
    g = torch.Generator().manual_seed(3)
    perm = torch.stack([torch.randperm(300, generator=g) for _ in range(64)]).to(torch.int32)
    src = torch.randn(64, 300, generator=g)
    out = jt.array(torch.zeros(64, 300)).scatter(1, jt.array(perm), jt.array(src))
    back = out.gather(1, jt.array(perm)).torch().cpu()
    assert torch.equal(back, src)
    assert torch.equal(out.torch().cpu(), torch.zeros(64, 300).scatter_(1, perm.long(), src))


@pytest.mark.parametrize("op,k,s,p,ceil,cip", [("maximum", 3, 2, 1, False, True), ("minimum", 2, 2, 0, False, True),
                                               ("mean", 3, 2, 1, True, False), ("mean", 3, 1, 1, False, True),
                                               ("maximum", (2, 3), (1, 2), (0, 1), True, True)])
def test_pool_matches_oracle(jt, ref, op, k, s, p, ceil, cip):
    from jittor_b200 import pool
    rng = np.random.default_rng(4)
    x = np.round(rng.normal(size=(3, 5, 33, 30)) * 2).astype(np.float32) / 2        # coarse values: ties are frequent
    layer = pool.Pool(k, s, p, ceil_mode=ceil, count_include_pad=cip, op=op)
    vx = jt.array(x)
    y = layer(vx)
    want = ref.pool2d(x, k, op, s, p, ceil, cip)
    assert np.allclose(y.numpy(), want, rtol=1e-6, atol=1e-6)
    dy = rng.normal(size=want.shape).astype(np.float32)
    dx = jt.grad((y * jt.array(dy)).sum(), vx).numpy()
    wdx = ref.pool2d_backward(x, dy, k, op, s, p, ceil, cip)
    assert np.allclose(dx, wdx, rtol=1e-5, atol=1e-5)


def test_pool_return_indices_and_bf16(jt, ref):
    from jittor_b200 import pool
    rng = np.random.default_rng(5)
    x = rng.normal(size=(2, 4, 17, 19)).astype(np.float32)
    y, idx = pool.max_pool2d(jt.array(x), 3, 2, 1, return_indices=True)
    wy, widx = ref.pool2d(x, 3, "maximum", 2, 1, return_indices=True)
    assert np.array_equal(y.numpy(), wy) and np.array_equal(idx.numpy(), widx)
    xb = torch.from_numpy(x).bfloat16()
    yb = pool.max_pool2d(jt.array(xb), 3, 2, 1).torch().float().cpu().numpy()
    assert np.array_equal(yb, ref.pool2d(xb.float().numpy(), 3, "maximum", 2, 1))


def test_grouped_and_transposed_conv_match_oracle(jt, ref):
    from jittor_b200 import nn
    rng = np.random.default_rng(6)
    x = rng.normal(size=(3, 32, 20, 23)).astype(np.float32)
    w = (rng.normal(size=(64, 4, 3, 3)) * 0.1).astype(np.float32)
    got = nn.conv2d(jt.array(x), jt.array(w), None, 2, 1, 1, groups=8).numpy()
    want = ref.conv2d_grouped(x, w, 2, 1, 1, 8)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5 * np.abs(want).max())
    wd = (rng.normal(size=(32, 1, 3, 3)) * 0.3).astype(np.float32)                    # depthwise
    got = nn.conv2d(jt.array(x), jt.array(wd), None, 1, 1, 1, groups=32).numpy()
    want = ref.conv2d_grouped(x, wd, 1, 1, 1, 32)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5 * np.abs(want).max())
    wt = (rng.normal(size=(32, 12, 4, 4)) * 0.1).astype(np.float32)
    got = nn.conv_transpose2d(jt.array(x), jt.array(wt), None, 2, 1, 1).numpy()
    want = ref.conv_transpose2d(x, wt, 2, 1, 1)
    assert got.shape == want.shape
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5 * np.abs(want).max())
    wtg = (rng.normal(size=(32, 3, 3, 3)) * 0.1).astype(np.float32)                   # 4 groups, 32 -> 12 channels
    got = nn.conv_transpose2d(jt.array(x), jt.array(wtg), None, (2, 1), (1, 0), 0, groups=4, dilation=(1, 2)).numpy()
    want = ref.conv_transpose2d(x, wtg, (2, 1), (1, 0), 0, 4, (1, 2))
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5 * np.abs(want).max())


def test_optimizer_accumulates_and_matches_torch(jt):
    from jittor_b200 import nn, optim
    g = torch.Generator().manual_seed(7)
    x, y = torch.randn(64, 10, generator=g), torch.randn(64, 3, generator=g)
    w0 = torch.randn(10, 3, generator=g)
    w = jt.array(w0.clone())
    opt = optim.SGD([w], lr=0.05, momentum=0.9, weight_decay=0.01, nesterov=True)
    tw = w0.clone().cuda().requires_grad_()
    topt = torch.optim.SGD([tw], lr=0.05, momentum=0.9, weight_decay=0.01, nesterov=True)
    for _ in range(5):
        d = nn.matmul(jt.array(x), w) - jt.array(y)
        opt.step((d * d).sum() * (1.0 / 64))
        topt.zero_grad()
        (((x.cuda() @ tw - y.cuda()) ** 2).sum() / 64).backward()
        topt.step()
    assert torch.allclose(w.torch(), tw.detach(), rtol=1e-4, atol=1e-5)
    # backward twice, then one step: the gradients add up (python/jittor/optim.py:205-219)
    w2 = jt.array(w0.clone())
    opt2 = optim.SGD([w2], lr=0.1)
    for _ in range(2):
        d = nn.matmul(jt.array(x), w2) - jt.array(y)
        opt2.backward((d * d).sum() * (1.0 / 64))
    opt2.step()
    gr = (2.0 / 64) * x.T @ (x @ w0 - y)
    assert torch.allclose(w2.torch().cpu(), w0 - 0.1 * 2 * gr, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype,stride,pad,dil", [("float32", 1, 1, 1), ("float32", 2, 1, 1), ("float32", 1, 2, 2),
                                                  ("bfloat16", 1, 1, 1)])
def test_conv_backward_matches_torch(jt, dtype, stride, pad, dil):
    """jt.grad through the reindex-lowered conv: the executor recognises the data- and weight-gradient graphs and runs
    them as transposed convolution / flipped-weight convolution and as the weight-gradient implicit GEMM."""
    from jittor_b200 import executor, nn
    g = torch.Generator().manual_seed(8)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    C = 64 if dtype == "bfloat16" else 6
    x = torch.randn(4, C, 18, 20, generator=g).to(td).cuda()
    w = (torch.randn(C, C, 3, 3, generator=g) * 0.1).to(td).cuda()
    vx, vw = jt.array(x), jt.array(w)
    y = nn.conv2d(vx, vw, None, stride, pad, dil)
    dy = torch.randn(*y.shape, generator=g).to(td).cuda()
    dx, dw = jt.grad((y * jt.array(dy)).sum(), [vx, vw])
    assert executor._match_conv_dgrad(dx) is not None
    tx, tw = x.float().requires_grad_(), w.float().requires_grad_()
    ty = torch.nn.functional.conv2d(tx, tw, None, stride, pad, dil)
    (ty * dy.float()).sum().backward()
    tol = 1e-4 if dtype == "float32" else 3e-2
    for got, want in ((dx.torch().float(), tx.grad), (dw.torch().float(), tw.grad)):
        assert got.shape == want.shape
        err = (got - want).abs().max().item()
        assert err <= tol * want.abs().max().item() + 1e-6, (err, want.abs().max().item())


def test_backward_relays_under_the_tuner_names(jt):
    """cudnn_conv_backward_x / _w are registered with the signatures ConvTuner uses (conv_tuner.cc:382-396)."""
    g = torch.Generator().manual_seed(9)
    x = torch.randn(2, 5, 9, 11, generator=g).cuda()
    w = (torch.randn(7, 5, 3, 3, generator=g) * 0.2).cuda()
    tx, tw = x.clone().requires_grad_(), w.clone().requires_grad_()
    ty = torch.nn.functional.conv2d(tx, tw, None, 2, 1, 1)
    dy = torch.randn(*ty.shape, generator=g).cuda()
    (ty * dy).sum().backward()
    make_dx = jt.get_op_info("cudnn_conv_backward_x").get_constructor()
    make_dw = jt.get_op_info("cudnn_conv_backward_w").get_constructor()
    dx = make_dx(jt.array(w), jt.array(dy), 9, 11, 2, 2, 1, 1, 1, 1)
    dw = make_dw(jt.array(x), jt.array(dy), 3, 3, 2, 2, 1, 1, 1, 1)
    assert torch.allclose(dx.torch(), tx.grad, rtol=1e-4, atol=1e-5)
    assert torch.allclose(dw.torch(), tw.grad, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16", "int32", "int64", "int16", "int8", "uint8"])
def test_getitem_setitem_every_dtype(jt, ref, dtype):
    rng = np.random.default_rng(10)
    npdt = np.float32 if dtype == "bfloat16" else np.dtype(dtype)
    x = rng.integers(0, 50, size=(40, 24)).astype(npdt)
    v = rng.integers(0, 50, size=(15, 24)).astype(npdt)
    idx = rng.permutation(40)[:15].astype(np.int32)              # unique rows: 'void' is deterministic

    def to_jt(a):
        return jt.array(torch.from_numpy(a).bfloat16()) if dtype == "bfloat16" else jt.array(a)

    def back(vr):
        return vr.torch().float().cpu().numpy() if dtype == "bfloat16" else vr.numpy()

    assert np.array_equal(back(to_jt(x)[jt.array(idx)]), ref.getitem(x, (idx,)))
    assert np.array_equal(back(to_jt(x)[3:30:4, jt.array(idx % 24)]), ref.getitem(x, (slice(3, 30, 4), idx % 24)))
    assert np.array_equal(back(to_jt(x).setitem((jt.array(idx),), to_jt(v))), ref.setitem(x, (idx,), v))
    dup = np.array([1, 1, 1, 5, 5, 0, 39, 39, 2, 2, 2, 2, 7, 8, 9], np.int32)
    got = back(to_jt(x).setitem((jt.array(dup),), to_jt(v), "add"))
    want = ref.setitem(x.astype(np.float64) if dtype in ("float16", "bfloat16") else x, (dup,), v, "add")
    if dtype in ("float16", "bfloat16"):
        assert np.allclose(got, want, rtol=2e-2, atol=1.0)      # small integers: exact up to the 16-bit rounding of sums
    else:
        assert np.array_equal(got, want.astype(npdt))
    assert np.array_equal(back(to_jt(x).setitem((jt.array(dup),), to_jt(v), "maximum")), ref.setitem(x, (dup,), v, "maximum"))


@pytest.mark.parametrize("dtype", ["float64", "float16", "bfloat16"])
@pytest.mark.parametrize("k,s,p", [(3, 2, 1), (2, 2, 0), (3, 1, 1), (4, 3, 2)])
def test_pool_other_dtypes_and_windows(jt, ref, dtype, k, s, p):
    from jittor_b200 import pool
    rng = np.random.default_rng(11)
    x = (rng.integers(-20, 20, size=(2, 3, 19, 22)) / 4).astype(np.float64)      # exactly representable in 16 bits
    td = {"float64": torch.float64, "float16": torch.float16, "bfloat16": torch.bfloat16}[dtype]
    vx = jt.array(torch.from_numpy(x).to(td))
    for op in ("maximum", "mean"):
        layer = pool.Pool(k, s, p, op=op, ceil_mode=(op == "mean"))
        y = layer(vx)
        want = ref.pool2d(x, k, op, s, p, op == "mean")
        got = y.torch().double().cpu().numpy()
        assert np.allclose(got, want, rtol=1e-2 if dtype != "float64" else 1e-12, atol=1e-2 if dtype != "float64" else 1e-12)
        dy = (rng.integers(-8, 8, size=want.shape) / 2).astype(np.float64)
        dx = jt.grad((y * jt.array(torch.from_numpy(dy).to(td))).sum(), vx).torch().double().cpu().numpy()
        wdx = ref.pool2d_backward(x, dy, k, op, s, p, op == "mean")
        assert np.allclose(dx, wdx, rtol=2e-2 if dtype != "float64" else 1e-12, atol=5e-2 if dtype != "float64" else 1e-12)


def test_average_pooling_lowering_bf16_and_adaptive(jt, ref):
    """Floor-mode avg_pool2d and the adaptive pools are the reindex + reduce lowering in the reference; the executor
    relays them to the pooling kernel. bf16: mean accumulated in float32, rounded once."""
    from jittor_b200 import pool
    rng = np.random.default_rng(12)
    x = rng.normal(size=(3, 5, 20, 26)).astype(np.float32)
    xb = torch.from_numpy(x).bfloat16()
    got = pool.avg_pool2d(jt.array(xb), 3, 2, 1).torch().float().cpu().numpy()
    want = torch.from_numpy(ref.pool2d(xb.float().numpy(), 3, "mean", 2, 1)).bfloat16().float().numpy()
    assert np.allclose(got, want, rtol=1e-2, atol=1e-2)
    got = pool.AdaptiveAvgPool2d((4, None))(jt.array(x)).numpy()
    assert np.allclose(got, ref.adaptive_pool2d(x, (4, None), "mean"), rtol=1e-5, atol=1e-6)
    got = pool.AdaptiveMaxPool2d(5)(jt.array(x)).numpy()
    assert np.array_equal(got, ref.adaptive_pool2d(x, 5, "maximum"))
    # gradient of the lowering still follows the meta-operator rules
    vx = jt.array(x)
    y = pool.avg_pool2d(vx, 2)
    dy = rng.normal(size=tuple(y.shape)).astype(np.float32)
    dx = jt.grad((y * jt.array(dy)).sum(), vx).numpy()
    assert np.allclose(dx, ref.pool2d_backward(x, dy, 2, "mean"), rtol=1e-5, atol=1e-6)
