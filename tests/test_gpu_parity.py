"""GPU parity, part 2: seeded inputs beyond the fixtures -- odd sizes, every kernel path (affine / bytecode
gather, injective / privatised / direct / generic scatter, row / column / split reductions, register-resident
and sweeping row kernels), bf16 IO -- against the oracle; and size-independent properties at the benchmark's
full sizes. Tolerances: bit-exact for gathers and integer work; fp32 |d| <= 1e-5|ref| + 1e-5 max|ref|;
bf16 results compared after rounding with rel 2e-2 (mixed the same way)."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as co
from oracle import meta_ops_ref as ref
from tests.golden_cases import check

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def jt():
    import jittor_b200
    return jittor_b200


@pytest.fixture(scope="module")
def be():
    from tests.product_backend import ProductBackend
    return ProductBackend()


def bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16().float().numpy()


def to_bf16_var(jt, a):
    return jt.array(torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16())


# ------------------------------------------------------------------------------------------------ reindex
@pytest.mark.parametrize("dtype", ["float32", "int32", "float64", "int64", "uint8", "int16", "bool"])
@pytest.mark.parametrize("shape,oshape,indexes,conds", [
    ((37, 53), (41, 59), ["i0-2", "i1-3"], []),
    ((37, 53), (53, 37), ["i1", "i0"], []),
    ((5, 6, 7), (5, 3, 7, 4), ["i0", "i1*2+i3-1", "i2"], []),
    ((16, 16), (32, 32), ["i0/2", "i1%16"], []),
    ((16, 16), (16, 16), ["i0", "i1"], ["i0 > i1", "(i0+i1)%3==0"]),
    ((9,), (1000,), ["i0%9"], []),
    ((2, 3, 8, 8), (2, 4, 3, 8, 8, 3, 3), ["i0", "i2", "i3*1-1+i5*1", "i4*1-1+i6*1"], []),
])
def test_reindex_exact(be, dtype, shape, oshape, indexes, conds):
    rng = np.random.default_rng(7)
    x = (rng.integers(0, 2, size=shape).astype(bool) if dtype == "bool"
         else rng.integers(-100, 100, size=shape).astype(dtype) if dtype != "uint8"
         else rng.integers(0, 255, size=shape).astype(dtype))
    got = be.reindex(x, list(oshape), indexes, -1 if dtype != "uint8" else 7, conds)
    want = ref.reindex(x, list(oshape), indexes, -1 if dtype != "uint8" else 7, conds)
    check(got, want, True)


def test_reindex_extras_and_large(be):
    rng = np.random.default_rng(8)
    x = rng.normal(size=(1000, 64)).astype(np.float32)
    rows = rng.integers(-5, 1005, size=(4096,)).astype(np.int32)
    check(be.reindex(x, [4096, 64], ["@e0(i0)", "i1"], 0, [], [rows]),
          ref.reindex(x, [4096, 64], ["@e0(i0)", "i1"], 0, [], [rows]), True)
    x1 = rng.normal(size=(3, 1 << 20)).astype(np.float32)
    check(be.reindex(x1, [3, (1 << 20) + 5], ["i0", "i1-2"], -5), ref.reindex(x1, [3, (1 << 20) + 5], ["i0", "i1-2"], -5), True)


# ------------------------------------------------------------------------------------------------ reindex_reduce
def zipf_indices(rng, n, bins, s=1.1):
    p = np.arange(1, bins + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(p / p.sum())
    rank = np.minimum(np.searchsorted(cdf, rng.random(n)), bins - 1)
    return rng.permutation(bins)[rank].astype(np.int32)


@pytest.mark.parametrize("bins", [7, 4096, 8192, 70001, 1 << 20])
@pytest.mark.parametrize("skew", ["uniform", "zipf"])
def test_scatter_add_int32_exact(be, bins, skew):
    rng = np.random.default_rng(bins)
    n = (1 << 20) + 13
    idx = zipf_indices(rng, n, bins) if skew == "zipf" else rng.integers(-2, bins + 2, size=n).astype(np.int32)
    val = rng.integers(0, 100, size=n).astype(np.int32)
    got = be.reindex_reduce(val, "add", [bins], ["@e0(i0)"], [], [idx])
    assert np.array_equal(got, co.scatter_add(val, idx, bins))


@pytest.mark.parametrize("bins", [64, 4096, 100000])
@pytest.mark.parametrize("skew", ["uniform", "zipf"])
def test_scatter_add_fp32(be, bins, skew):
    rng = np.random.default_rng(bins + 1)
    n = (1 << 20) + 5
    idx = zipf_indices(rng, n, bins) if skew == "zipf" else rng.integers(0, bins, size=n).astype(np.int32)
    val = rng.normal(size=n).astype(np.float32)
    got = be.reindex_reduce(val, "add", [bins], ["@e0(i0)"], [], [idx])
    want = np.zeros(bins, np.float64)
    np.add.at(want, idx, val.astype(np.float64))          # exact sum; both fp32 orders lie within tolerance of it
    check(got, want.astype(np.float32), False)
    check(co.scatter_add(val, idx, bins), want.astype(np.float32), False)


@pytest.mark.parametrize("op", ["maximum", "minimum", "multiply", "add"])
@pytest.mark.parametrize("dtype", ["float32", "int32", "float64", "int64"])
def test_scatter_ops(be, op, dtype):
    rng = np.random.default_rng(11)
    n, bins = 50000, 300
    idx = rng.integers(0, bins + 20, size=n).astype(np.int64)
    if op == "multiply":
        val = (rng.choice([1, -1, 2], size=n) if "int" in dtype else rng.uniform(0.9, 1.1, size=n)).astype(dtype)
        n = 3000
        val, idx = val[:n], idx[:n]
    else:
        val = (rng.integers(-1000, 1000, size=n) if "int" in dtype else rng.normal(size=n) * 5).astype(dtype)
    got = be.reindex_reduce(val, op, [bins + 20], ["@e0(i0)"], [], [idx])
    want = ref.reindex_reduce(val, op, [bins + 20], ["@e0(i0)"], [], [idx])
    check(got, want, "int" in dtype or op in ("maximum", "minimum"))


def test_scatter_generic_forms(be):
    rng = np.random.default_rng(12)
    y = rng.normal(size=(6, 40, 40, 3)).astype(np.float32)
    for op in ("add", "maximum", "minimum"):
        got = be.reindex_reduce(y, op, [6, 14, 14, 3], ["i0", "i1/3", "i2/3", "i3"])
        check(got, ref.reindex_reduce(y, op, [6, 14, 14, 3], ["i0", "i1/3", "i2/3", "i3"]), op != "add")
    # conv data-gradient form: overlapping windows, out-of-range taps dropped
    dy = rng.normal(size=(2, 4, 3, 8, 8, 3, 3)).astype(np.float32)
    ind = ["i0", "i2", "i3*1-1+i5*1", "i4*1-1+i6*1"]
    check(be.reindex_reduce(dy, "add", [2, 3, 8, 8], ind), ref.reindex_reduce(dy, "add", [2, 3, 8, 8], ind), False)


def test_pool_backward_permutation_exact(be):
    y = np.random.default_rng(13).normal(size=(3, 5, 28, 28, 2, 2)).astype(np.float32)
    got = be.reindex_reduce(y, "add", [3, 5, 56, 56], ["i0", "i1", "i2*2+i4", "i3*2+i5"])
    assert np.array_equal(got, co.pool2x2_bwd(y))
    # injective but with holes and out-of-range elements
    y2 = np.random.default_rng(14).normal(size=(4, 30)).astype(np.float32)
    got2 = be.reindex_reduce(y2, "add", [4, 50], ["i0", "i1*2-4"])
    assert np.array_equal(got2, ref.reindex_reduce(y2, "add", [4, 50], ["i0", "i1*2-4"]))


# ------------------------------------------------------------------------------------------------ reduce / element-wise
@pytest.mark.parametrize("shape,dims", [((1 << 22,), ()), ((3, 1 << 20), (1,)), ((1 << 20, 3), (0,)), ((64, 33, 65), (0, 2)),
                                        ((64, 33, 65), (1,)), ((7, 9, 11, 13), (1, 3)), ((300, 257), (1,)), ((5, 3), (0, 1))])
@pytest.mark.parametrize("op", ["add", "maximum", "mean", "minimum"])
def test_reduce_float(be, shape, dims, op):
    x = np.random.default_rng(21).normal(size=shape).astype(np.float32)
    got = be.reduce(x, op, dims, False)
    want = ref.reduce(x.astype(np.float64), op, dims, False).astype(np.float32)
    check(got, want, op in ("maximum", "minimum"))


@pytest.mark.parametrize("op", ["add", "multiply", "maximum", "minimum", "bitwise_xor", "bitwise_and", "bitwise_or"])
def test_reduce_int_exact(be, op):
    x = np.random.default_rng(22).integers(1, 5, size=(33, 1000, 3)).astype(np.int32)
    for dims in ((1,), (0, 2), ()):
        check(be.reduce(x, op, dims, True), ref.reduce(x, op, dims, True), True)


def test_binary_broadcast_fused(be):
    rng = np.random.default_rng(23)
    a, b = rng.normal(size=(33, 1, 65)).astype(np.float32), rng.normal(size=(1, 47, 1)).astype(np.float32)
    for op in ("add", "multiply", "subtract", "maximum", "less"):
        check(be.binary(a, b, op), ref.binary(a, b, op), True)
    x = rng.normal(size=(1 << 20,)).astype(np.float32)
    check(be.binary(x, x[::-1].copy(), "multiply"), ref.binary(x, x[::-1].copy(), "multiply"), True)


# ------------------------------------------------------------------------------------------------ fused rows
@pytest.mark.parametrize("rows,cols", [(1, 4), (33, 128), (17, 1000), (64, 1024), (5, 2048), (8, 4096), (3, 8192),
                                       (2, 8196), (3, 16384), (2, 50000), (7, 1001)])
def test_softmax_layernorm_fp32(be, rows, cols):
    rng = np.random.default_rng(rows * cols)
    x = (rng.normal(size=(rows, cols)) * 2).astype(np.float32)
    check(be.softmax(x, -1, False), co.softmax_rows(x, False), False)
    check(be.softmax(x, -1, True), co.softmax_rows(x, True), False)
    g, b = (1 + 0.02 * rng.normal(size=cols)).astype(np.float32), rng.normal(size=cols).astype(np.float32)
    check(be.layer_norm(x, (cols,), g, b), co.layernorm_rows(x, g, b), False)
    check(be.layer_norm(x, (cols,)), co.layernorm_rows(x), False)


@pytest.mark.parametrize("rows,cols", [(16, 4096), (5, 1000), (9, 264)])
def test_softmax_layernorm_bf16(jt, rows, cols):
    from jittor_b200 import nn
    rng = np.random.default_rng(5)
    xr = bf16_round(rng.normal(size=(rows, cols)))
    xv = to_bf16_var(jt, xr)
    y = nn.softmax(xv, -1)
    assert y.dtype == "bfloat16"
    check(y.numpy(), bf16_round(co.softmax_rows(xr)), False, rtol=2e-2)
    g = (1 + 0.02 * rng.normal(size=cols)).astype(np.float32)
    z = nn.layer_norm(xv, (cols,), jt.array(g), jt.array(np.zeros(cols, np.float32)))
    assert z.dtype == "bfloat16"
    check(z.numpy(), bf16_round(co.layernorm_rows(xr, g, np.zeros(cols, np.float32))), False, rtol=2e-2)


@pytest.mark.parametrize("rows,cols", [(7, 8196), (3, 16384), (5, 20000), (2, 32768), (4, 50000), (1, 65536), (300, 12000)])
def test_softmax_layernorm_rows_held_by_a_cluster(be, rows, cols):
    """Rows above 8192 float32 columns: 2 / 4 / 8 CTAs of a thread-block cluster hold a row and exchange their partial
    results through distributed shared memory (whole and ragged last vectors, more rows than resident clusters)."""
    rng = np.random.default_rng(rows + cols)
    x = (rng.normal(size=(rows, cols)) * 2).astype(np.float32)
    check(be.softmax(x, -1, False), co.softmax_rows(x, False), False)
    check(be.softmax(x, -1, True), co.softmax_rows(x, True), False)
    g, b = (1 + 0.02 * rng.normal(size=cols)).astype(np.float32), rng.normal(size=cols).astype(np.float32)
    check(be.layer_norm(x, (cols,), g, b), co.layernorm_rows(x, g, b), False)


@pytest.mark.parametrize("rows,cols", [(6, 16392), (3, 40000), (2, 131072)])
def test_softmax_layernorm_bf16_rows_held_by_a_cluster(jt, rows, cols):
    from jittor_b200 import nn
    rng = np.random.default_rng(cols)
    xr = bf16_round(rng.normal(size=(rows, cols)))
    xv = to_bf16_var(jt, xr)
    check(nn.softmax(xv, -1).numpy(), bf16_round(co.softmax_rows(xr)), False, rtol=2e-2)
    g = (1 + 0.02 * rng.normal(size=cols)).astype(np.float32)
    z = nn.layer_norm(xv, (cols,), jt.array(g), jt.array(np.zeros(cols, np.float32)))
    check(z.numpy(), bf16_round(co.layernorm_rows(xr, g, np.zeros(cols, np.float32))), False, rtol=2e-2)


# ------------------------------------------------------------------------------------------------ contractions
@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (33, 29, 47), (128, 256, 64), (300, 200, 1000), (512, 512, 512)])
def test_matmul_fp32(be, m, n, k):
    rng = np.random.default_rng(m + n + k)
    a, b = rng.normal(size=(m, k)).astype(np.float32), (rng.normal(size=(k, n)) / np.sqrt(k)).astype(np.float32)
    check(be.matmul(a, b), co.matmul(a, b), False)
    check(be.matmul_transpose(a, b.T.copy()), co.matmul(a, b), False)


@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (384, 512, 1024), (130, 70, 200)])
def test_matmul_bf16(jt, m, n, k):
    from jittor_b200 import nn
    rng = np.random.default_rng(m)
    a, b = bf16_round(rng.normal(size=(m, k)) / np.sqrt(k)), bf16_round(rng.normal(size=(k, n)))
    c = nn.matmul(to_bf16_var(jt, a), to_bf16_var(jt, b))
    assert c.dtype == "bfloat16"
    check(c.numpy(), bf16_round(co.matmul(a, b)), False, rtol=2e-2)


@pytest.mark.parametrize("shape,wshape,s,p,d", [((2, 3, 17, 13), (5, 3, 3, 3), 1, 1, 1), ((1, 16, 28, 28), (32, 16, 3, 3), 1, 1, 1),
                                                ((2, 8, 15, 15), (8, 8, 5, 5), 2, 2, 1), ((2, 4, 20, 20), (6, 4, 3, 3), 1, 2, 2),
                                                ((3, 7, 9, 9), (4, 7, 1, 1), 1, 0, 1)])
def test_conv_fp32(be, shape, wshape, s, p, d):
    rng = np.random.default_rng(sum(shape))
    x, w = rng.uniform(-1, 1, size=shape).astype(np.float32), (rng.normal(size=wshape) * 0.05).astype(np.float32)
    check(be.conv2d(x, w, s, p, d), co.conv2d(x, w, s, p, d), False)


def test_conv_bf16_bn_relu(jt):
    from jittor_b200 import nn
    rng = np.random.default_rng(3)
    x, w = bf16_round(rng.normal(size=(4, 64, 16, 16))), bf16_round(rng.normal(size=(64, 64, 3, 3)) * np.sqrt(2 / (9 * 64)))
    y = nn.conv2d(to_bf16_var(jt, x), to_bf16_var(jt, w), None, 1, 1, 1)
    assert y.dtype == "bfloat16"
    yref = co.conv2d(x, w, 1, 1, 1)
    check(y.numpy(), bf16_round(yref), False, rtol=2e-2)
    bn = nn.BatchNorm(64, is_train=True, sync=False)
    with jt.flag_scope(amp_reg=2):
        z = nn.relu(bn(y))
    assert z.dtype == "bfloat16"
    zref = co.bn_relu(bf16_round(yref), np.ones(64, np.float32), np.zeros(64, np.float32))
    check(z.numpy(), bf16_round(zref), False, rtol=2e-2)


def test_batchnorm_fp32(be):
    rng = np.random.default_rng(31)
    x = rng.normal(size=(8, 12, 14, 14)).astype(np.float32) * 2 + 0.5
    g, b = rng.uniform(0.5, 1.5, 12).astype(np.float32), rng.normal(size=12).astype(np.float32)
    check(be.batch_norm_train(x, g, b, 1e-5, True), co.bn_relu(x, g, b, 1e-5, True), False)
    check(be.batch_norm_train(x, g, b, 1e-5, False), co.bn_relu(x, g, b, 1e-5, False), False)


# ------------------------------------------------------------------------------------------------ full-size properties
def test_full_size_scatter_checksums(jt):
    """2^24 values into 2^20 bins (the benchmark's size): the sum of all bins equals the sum of all in-range
    values (exact, integers), scattering twice equals doubling (linearity), and the result equals the C oracle."""
    rng = np.random.default_rng(1)
    n, bins = 1 << 24, 1 << 20
    val = rng.integers(0, 100, size=n).astype(np.int32)
    idx = rng.integers(0, bins, size=n).astype(np.int32)
    v, e = jt.array(val), jt.array(idx)
    out = v.reindex_reduce("add", [bins], ["@e0(i0)"], extras=[e]).numpy()
    assert int(out.astype(np.int64).sum()) == int(val.astype(np.int64).sum())
    out2 = (v + v).reindex_reduce("add", [bins], ["@e0(i0)"], extras=[e]).numpy()
    assert np.array_equal(out2, out * 2)
    assert np.array_equal(out, co.scatter_add(val, idx, bins))


def test_full_size_softmax_rows_sum_to_one(jt):
    from jittor_b200 import nn
    x = torch.randn(4096, 4096, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    y = nn.softmax(jt.array(x), -1).torch()
    assert torch.allclose(y.sum(-1), torch.ones(4096, device="cuda"), atol=1e-5)
    assert (y >= 0).all()
    idem = nn.softmax(jt.array(x + 7.5), -1).torch()          # shift invariance
    assert torch.allclose(idem, y, atol=1e-6, rtol=1e-4)


def test_matmul_bf16_full_size_tensor_core(jt):
    """8192^3 (the benchmark's size) through nn.matmul -> tcgen05 kernel: 64 sampled rows against the CPU oracle
    (fp32 accumulation on bf16-rounded inputs), the whole result against a float32 torch product, and the
    kernel's bounded waits must not have expired."""
    from jittor_b200 import nn, _capi as C
    g = torch.Generator("cuda").manual_seed(4)
    n = 8192
    a = (torch.randn(n, n, device="cuda", generator=g) / n ** 0.5).bfloat16()
    b = torch.randn(n, n, device="cuda", generator=g).bfloat16()
    c = nn.matmul(jt.array(a), jt.array(b))
    assert c.dtype == "bfloat16"
    ct = c.torch()
    assert C.lib.b200jt_device_status() == 0
    rows = torch.randperm(n, generator=torch.Generator().manual_seed(1))[:64]
    want = co.matmul(a[rows.cuda()].float().cpu().numpy(), b.float().cpu().numpy())
    check(ct[rows.cuda()].float().cpu().numpy(), bf16_round(want), False, rtol=2e-2)
    ref = (a.float() @ b.float())
    assert (ct.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    # transposed forms of the tuner table reach the same kernel
    ct2 = nn.matmul_transpose(jt.array(a), jt.array(b.t().contiguous())).torch()
    assert torch.equal(ct2, ct)


# ------------------------------------------------------------------------------------------------ batched matmul (one launch)
@pytest.mark.parametrize("ashape,bshape", [((10, 3, 4), (10, 4, 5)), ((8, 1, 3, 4), (10, 4, 5)), ((2, 3, 33, 17), (2, 3, 17, 9)),
                                           ((5, 70, 40), (1, 40, 30)), ((1, 64, 64), (7, 64, 64))])
def test_batched_matmul_fp32(jt, ashape, bshape):
    from jittor_b200 import nn
    rng = np.random.default_rng(sum(ashape))
    a, b = rng.normal(size=ashape).astype(np.float32), rng.normal(size=bshape).astype(np.float32)
    got = nn.matmul(jt.array(a), jt.array(b)).numpy()
    want = ref.matmul(a, b)
    check(got, want, False)


@pytest.mark.parametrize("ashape,bshape", [((6, 256, 128), (6, 128, 256)),      # tensor-core kernel, batch in the tile index
                                           ((3, 2, 200, 72), (3, 2, 72, 136)),  # ragged tiles inside every batch slice
                                           ((4, 256, 128), (1, 128, 256)),      # shared right operand
                                           ((4, 128, 64), (4, 64, 100))])       # N % 8 != 0: CUDA-core kernel, batch in grid z
def test_batched_matmul_bf16(jt, ashape, bshape):
    from jittor_b200 import nn, _capi as C
    rng = np.random.default_rng(sum(bshape))
    a, b = bf16_round(rng.normal(size=ashape) / np.sqrt(ashape[-1])), bf16_round(rng.normal(size=bshape))
    c = nn.matmul(to_bf16_var(jt, a), to_bf16_var(jt, b))
    assert c.dtype == "bfloat16"
    want = np.matmul(a.astype(np.float64), b.astype(np.float64)).astype(np.float32)
    # per-slice oracle: fp32 accumulation on bf16-rounded inputs
    a3 = np.broadcast_to(a, want.shape[:-2] + a.shape[-2:]).reshape((-1,) + a.shape[-2:])
    b3 = np.broadcast_to(b, want.shape[:-2] + b.shape[-2:]).reshape((-1,) + b.shape[-2:])
    want = np.stack([co.matmul(x, y) for x, y in zip(a3, b3)]).reshape(want.shape)
    check(c.numpy(), bf16_round(want), False, rtol=2e-2)
    assert C.lib.b200jt_device_status() == 0


# ------------------------------------------------------------------------------------------------ BatchNorm running statistics
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batchnorm_train_then_eval(jt, dtype):
    """Three training steps move running_mean / running_var as python/jittor/nn.py:684-688 does (the fused normalise
    kernel updates them in place), and evaluation then normalises with them."""
    from jittor_b200 import nn
    rng = np.random.default_rng(17)
    Cn = 12
    bn = nn.BatchNorm(Cn, momentum=0.3, is_train=True, sync=False)
    rm, rv = np.zeros(Cn, np.float32), np.ones(Cn, np.float32)
    for step in range(3):
        x = (rng.normal(size=(6, Cn, 9, 7)) * (1 + step) + step).astype(np.float32)
        if dtype == "bfloat16":
            x = bf16_round(x)
        xv = to_bf16_var(jt, x) if dtype == "bfloat16" else jt.array(x)
        with jt.flag_scope(amp_reg=2 if dtype == "bfloat16" else 0):
            y = bn(xv)
            y.sync()
        mean = x.astype(np.float64).mean((0, 2, 3))
        var = np.maximum((x.astype(np.float64) ** 2).mean((0, 2, 3)) - mean ** 2, 0)
        rm = (rm + (mean - rm) * 0.3).astype(np.float32)
        rv = (rv + (var - rv) * 0.3).astype(np.float32)
        check(bn.running_mean.numpy(), rm, False, rtol=1e-4)
        check(bn.running_var.numpy(), rv, False, rtol=1e-4)
    assert bn.running_mean.is_stop_grad() and bn.running_var.is_stop_grad()
    bn.is_train = False
    x = rng.normal(size=(2, Cn, 5, 5)).astype(np.float32)
    got = bn(jt.array(x)).numpy()
    want = (x - rm[None, :, None, None]) / np.sqrt(rv[None, :, None, None] + 1e-5)
    check(got, want.astype(np.float32), False, rtol=1e-4)


def test_batchnorm_running_statistics_without_the_fused_plan(jt):
    """float64 inputs are normalised op by op; the running statistics still move once the output is computed."""
    from jittor_b200 import nn
    rng = np.random.default_rng(18)
    x = rng.normal(size=(4, 5, 6, 6)) + 2.0
    bn = nn.BatchNorm(5, momentum=0.1, is_train=True, sync=False)
    bn(jt.array(x)).sync()
    mean = x.mean((0, 2, 3))
    var = (x ** 2).mean((0, 2, 3)) - mean ** 2
    check(bn.running_mean.numpy(), (0.1 * mean).astype(np.float32), False, rtol=1e-5)
    check(bn.running_var.numpy(), (1 + 0.1 * (var - 1)).astype(np.float32), False, rtol=1e-5)


def test_grad_stops_at_stop_grad(jt):
    x = jt.array(np.arange(6, dtype=np.float32).reshape(2, 3))
    y = (x * 2.0).stop_grad()
    z = (y * x).sum()
    g = jt.grad(z, x).numpy()
    assert np.array_equal(g, np.arange(6, dtype=np.float32).reshape(2, 3) * 2)      # d/dx (c*x) with c = y held constant
