"""The C restatement (oracle/meta_ops.c, used for large sizes and for the timed CPU baseline) must agree with
the numpy oracle, which is pinned to the reference's outputs."""
import numpy as np

from oracle import c_oracle as co
from oracle import meta_ops_ref as ref
from tests.golden_cases import check


def test_scatter_add_exact_and_float():
    rng = np.random.default_rng(5)
    idx = rng.integers(-3, 1030, size=50000).astype(np.int32)
    vi = rng.integers(0, 100, size=50000).astype(np.int32)
    assert np.array_equal(co.scatter_add(vi, idx, 1024), ref.reindex_reduce(vi, "add", [1024], ["@e0(i0)"], (), [idx]))
    vf = rng.normal(size=50000).astype(np.float32)
    assert np.array_equal(co.scatter_add(vf, idx, 1024), ref.reindex_reduce(vf, "add", [1024], ["@e0(i0)"], (), [idx]))


def test_pool_bwd():
    y = np.random.default_rng(1).normal(size=(2, 3, 4, 5, 2, 2)).astype(np.float32)
    want = ref.reindex_reduce(y, "add", [2, 3, 8, 10], ["i0", "i1", "i2*2+i4", "i3*2+i5"])
    assert np.array_equal(co.pool2x2_bwd(y), want)


def test_rows():
    x = np.random.default_rng(2).normal(size=(9, 517)).astype(np.float32) * 3
    check(co.softmax_rows(x), ref.softmax(x, -1), False)
    check(co.softmax_rows(x, True), ref.softmax(x, -1, True), False)
    g, b = np.random.default_rng(3).normal(size=(2, 517)).astype(np.float32)
    check(co.layernorm_rows(x, g, b), ref.layer_norm(x, (517,), g, b), False)
    check(co.layernorm_rows(x), ref.layer_norm(x, (517,)), False)


def test_contractions():
    rng = np.random.default_rng(4)
    a, b = rng.normal(size=(37, 53)).astype(np.float32), rng.normal(size=(53, 29)).astype(np.float32)
    check(co.matmul(a, b), ref.matmul(a, b), False)
    x, w = rng.normal(size=(2, 5, 9, 8)).astype(np.float32), rng.normal(size=(4, 5, 3, 3)).astype(np.float32)
    for s, p, d in ((1, 1, 1), (2, 1, 1), (1, 2, 2)):
        check(co.conv2d(x, w, s, p, d), ref.conv2d(x, w, s, p, d), False)
    g, bb = rng.uniform(0.5, 1.5, 5).astype(np.float32), rng.normal(size=5).astype(np.float32)
    check(co.bn_relu(x, g, bb), ref.batch_norm_train(x, g, bb, relu=True), False)


def test_conv_weight_gradient_against_the_reference_fixtures():
    """oracle_conv2d_backward_w_f32 against the weight gradients the reference's own jt.grad produced on its CPU executor
    (tests/golden/make_golden_next.py:do_conv_grad)."""
    from tests.golden_cases import CASES, arrays
    seen = 0
    for c in CASES:
        if c["op"] != "conv_wgrad":
            continue
        A = arrays(c["file"])
        x, w, dy = (A[k] for k in c["inputs"])
        a = c["args"]
        st, pd, dl = a["stride"], a["padding"], a["dilation"]
        if any(isinstance(v, (list, tuple)) and len(set(v)) > 1 for v in (st, pd, dl)):
            continue                                        # the C restatement takes one stride / padding / dilation for both axes
        one = lambda v: int(v[0]) if isinstance(v, (list, tuple)) else int(v)
        got = co.conv2d_backward_w(x, dy, w.shape[2], w.shape[3], one(st), one(pd), one(dl))
        check(got, A[c["out"]], False)
        seen += 1
    assert seen >= 4
