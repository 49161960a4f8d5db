"""CPU tests of the host side: C-ABI surface, index-program classification, shape/dtype inference of the
Var front-end against the reference-made fixtures, and the pattern dispatcher on placeholder graphs."""
import ctypes
import os
import re

import numpy as np
import pytest

import jittor_b200 as jt
from jittor_b200 import _capi, executor, nn
from tests import golden_cases as G

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "b200jt.h")).read()
    declared = set(re.findall(r"^(?:int|size_t|const char\*)\s+(b200jt_[a-z0-9_]+)\s*\(", header, re.M))
    assert len(declared) >= 20
    bound = {name for name, _, _ in _capi.SIGNATURES}
    assert declared == bound, declared ^ bound
    for name in declared:
        assert getattr(_capi.lib, name) is not None
    assert _capi.lib.b200jt_version() >= 100


def test_no_cuda_means_loud_failure():
    import torch
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(jt.B200Error):
        jt.array([1, 2, 3])


def ph(shape, dtype="float32"):
    return jt.Var(shape, dtype)


def test_index_affine_classification():
    aff = executor.index_affine([4, 64, 32, 32, 32, 3, 3], [4, 32, 32, 32], ["i0", "i2", "i3*1-1+i5*1", "i4*2-3+i6*4"])
    coef, c0 = aff
    assert coef[2] == [0, 0, 0, 1, 0, 1, 0] and c0[2] == -1
    assert coef[3] == [0, 0, 0, 0, 2, 0, 4] and c0[3] == -3
    assert executor.index_affine([8, 8], [4, 4], ["i0/2", "i1"]) is None
    assert executor.index_affine([8, 8], [4, 4], ["i0*(4/2)", "xshape1-1-i1"]) == ([[2, 0], [0, -1]], [0, 3])
    with pytest.raises(jt.B200Error):
        executor.index_affine([8], [4], ["i0 // 2"])
    with pytest.raises(jt.B200Error):
        executor.index_affine([8], [4], ["i3"])


_PATH_CASES = [c for c in G.CASES if c["file"] == "meta_ops"]     # the callers' fixtures have their own host tests


@pytest.mark.parametrize("case", _PATH_CASES, ids=[c["name"] for c in _PATH_CASES])
def test_shape_and_dtype_inference_matches_reference(case):
    """Builds the lazy graph of every fixture on placeholder Vars: output shape and dtype must equal what
    the reference produced (nothing is computed)."""
    A = G.arrays()

    if case["args"].get("bf16_bits"):
        pytest.skip("bit-pattern case")
    ins = [ph(list(A[k].shape) or [1], str(A[k].dtype)) for k in case["inputs"]]
    ex = [ph(list(A[k].shape), str(A[k].dtype)) for k in case["extras"]]
    a, op = case["args"], case["op"]
    if op == "reindex":
        if a.get("bf16_bits"):
            pytest.skip("bit-pattern case")
        v = ins[0].reindex(a["shape"], a["indexes"], a["overflow_value"], a["overflow_conditions"], ex)
    elif op == "reindex_var":
        v = ins[0].reindex_var(ex, a["overflow_value"], a["overflow_conditions"])
    elif op == "reindex_reduce":
        v = ins[0].reindex_reduce(a["op"], a["shape"], a["indexes"], a["overflow_conditions"], ex)
    elif op == "broadcast":
        v = jt.broadcast(ins[0], a["shape"], a["dims"])
    elif op == "broadcast_var":
        v = jt.broadcast_var(ins[0], ins[1], a["dims"])
    elif op == "reduce":
        d = a["dims"]
        v = jt.reduce(ins[0], a["op"], tuple(d) if isinstance(d, list) else d, a["keepdims"])
    elif op == "binary":
        v = jt.binary(ins[0], ins[1], a["op"])
    elif op == "unary":
        v = jt.unary(ins[0], a["op"])
    elif op == "ternary":
        v = jt.ternary(*ins)
    elif op == "conv":
        v = nn.conv2d(ins[0], ins[1], ins[2] if a["bias"] else None, a["stride"], a["padding"], a["dilation"])
    elif op == "matmul":
        v = nn.matmul(ins[0], ins[1])
    elif op == "matmul_transpose":
        v = nn.matmul_transpose(ins[0], ins[1])
    elif op in ("softmax", "log_softmax"):
        v = nn.softmax(ins[0], a["dim"], op == "log_softmax")
    else:
        pytest.skip("composite case")
    assert list(v.shape) == case["out_shape"]
    assert v.dtype == case["out_dtype"]


def test_conv_pattern_is_recognised_and_solved():
    x, w = ph([4, 32, 32, 32]), ph([64, 32, 3, 3])
    y = nn.conv2d(x, w, None, 1, 1, 1)
    assert list(y.shape) == [4, 64, 32, 32]
    plan = executor._make_plan(y)
    assert plan.leaves == [x, w]                       # the 7-D intermediates are not leaves: never materialised
    m = y._op.inputs[0]
    geo = executor.conv_geometry(m._op.inputs[0], m._op.inputs[1])
    assert geo[2] == (1, 1, 1, 1, 1, 1)
    y2 = nn.conv2d(ph([2, 3, 9, 8]), ph([4, 3, 5, 3]), None, (2, 3), (1, 2), (2, 1))
    m2 = y2._op.inputs[0]
    assert executor.conv_geometry(m2._op.inputs[0], m2._op.inputs[1])[2] == (2, 3, 1, 2, 2, 1)


def test_huge_conv_never_materialises():
    x, w = ph([256, 256, 56, 56], "bfloat16"), ph([256, 256, 3, 3], "bfloat16")
    y = nn.conv2d(x, w, None, 1, 1, 1)
    assert y.dtype == "bfloat16"                       # amp_reg | 36 keeps the reduce dtype (nn.py:1008)
    assert y._op.inputs[0].numel() == 256 * 256 * 256 * 56 * 56 * 9
    assert executor._make_plan(y).leaves == [x, w]


def test_unfused_giant_intermediate_is_refused():
    x = ph([256, 256, 56, 56])
    xx = x.reindex([256, 256, 256, 56, 56, 3, 3], ["i0", "i2", "i3-1+i5", "i4-1+i6"])
    y = (xx + 1.0).sum([2, 5, 6])
    with pytest.raises(jt.B200Error):
        executor._make_plan(y)


@pytest.mark.parametrize("ashape,bshape,fn", [([8, 5], [5, 7], "matmul"), ([8, 5], [7, 5], "matmul_transpose")])
def test_matmul_pattern(ashape, bshape, fn):
    a, b = ph(ashape), ph(bshape)
    c = getattr(nn, fn)(a, b)
    plan = executor._make_plan(c)
    assert plan.leaves == [a, b]


def test_matmul_tuner_table():
    """All (reduce axis, broadcast axes) combinations map to a (trans_a, trans_b) pair or to the swapped product."""
    import itertools
    for r, da, db in itertools.permutations(range(3)):
        shape = [4, 5, 6]
        a_shape = [shape[i] for i in range(3) if i != da]
        b_shape = [shape[i] for i in range(3) if i != db]
        a, b = ph(a_shape), ph(b_shape)
        with jt.flag_scope(amp_reg=36):
            c = (a.broadcast(shape, [da]) * b.broadcast(shape, [db])).sum(r)
        assert executor._match_matmul(c) is not None, (r, da, db)


def test_softmax_layernorm_batchnorm_patterns():
    x = ph([32, 4096])
    for log in (False, True):
        assert executor._match_softmax(nn.softmax(x, -1, log)) is not None
    xb = ph([32, 4096], "bfloat16")
    yb = nn.softmax(xb, -1)
    assert yb.dtype == "bfloat16" and executor._match_softmax(yb).leaves == [xb]
    assert executor._match_softmax(nn.softmax(ph([6, 33]), 0)) is None          # not the last axis: op by op
    g, b = ph([4096]), ph([4096])
    ln = nn.layer_norm(x, (4096,), g, b)
    assert executor._match_layernorm(ln).leaves == [x, g, b]
    assert executor._match_layernorm(nn.layer_norm(x, (4096,))).leaves == [x]
    lnb = nn.layer_norm(xb, (4096,), g, b)
    assert lnb.dtype == "bfloat16" and executor._match_layernorm(lnb).leaves == [xb, g, b]
    xi = ph([6, 5, 7, 7])
    bn = nn.BatchNorm(5, is_train=True, sync=False)
    bn.weight, bn.bias = ph([5]), ph([5])
    y = bn(xi)
    assert executor._match_batchnorm(y).leaves == [xi, bn.weight, bn.bias, bn.running_mean, bn.running_var]
    assert executor._match_batchnorm(nn.relu(y)).leaves == [xi, bn.weight, bn.bias, bn.running_mean, bn.running_var]
    # conv feeding BatchNorm+ReLU: one plan from (x, w) to the activation
    xc, wc = ph([4, 8, 10, 10]), ph([16, 8, 3, 3])
    bn2 = nn.BatchNorm(16, is_train=True, sync=False)
    bn2.weight, bn2.bias = ph([16]), ph([16])
    z = nn.relu(bn2(nn.conv2d(xc, wc, None, 1, 1, 1)))
    assert executor._match_batchnorm(z).leaves == [xc, wc, bn2.weight, bn2.bias, bn2.running_mean, bn2.running_var]


def test_error_cases_of_the_reference():
    x = ph([3])
    x.reindex_reduce("add", [3], ["i0"])
    for bad in (lambda: x.reindex_reduce("add", [3], []), lambda: x.reindex_reduce("add", [3], ["i0", "i0"]),
                lambda: x.reindex_reduce("???", [3], ["i0"]), lambda: x.reindex_reduce("add", [-1], ["i0"]),
                lambda: jt.broadcast_var(ph([2]), ph([3])), lambda: jt.reduce(ph([3]), "add", 2)):
        with pytest.raises(ValueError):
            bad()
    assert list(ph([1]).broadcast([0]).shape) == [0]


def test_reindex_sources_compile_for_sm_100a():
    """The source generated for an affine reindex instance goes through NVRTC without a GPU: a conv window (ragged
    3x3 inner axes -> odometer with carries), a padded copy (vector never carries), 1- / 2- / 8-byte elements, a
    scalar-store case; a gather through an index Var is not of the compiled kind."""
    import ctypes
    from jittor_b200 import _capi as C

    def fake(i, dtype, shape):
        d = C.Tensor()
        d.ptr = 0x10000 * (i + 1)
        d.dtype = C.DTYPE_CODES[dtype]
        d.ndim = len(shape)
        for j, e in enumerate(shape):
            d.shape[j] = e
        return d

    def source(xs, ys, idx, dtype="float32", extras=()):
        x, y = fake(0, dtype, xs), fake(1, dtype, ys)
        ex = (C.Tensor * max(len(extras), 1))()
        for i, (dt_, shp) in enumerate(extras):
            ex[i] = fake(2 + i, dt_, shp)
        buf = ctypes.create_string_buffer(1 << 16)
        need, ok = ctypes.c_int64(), ctypes.c_int()
        C.check(C.lib.b200jt_reindex_source(ctypes.byref(x), ctypes.byref(y), C.strings(idx), len(idx), 0.0, C.strings([]), 0,
                                            ex, len(extras), buf, 1 << 16, ctypes.byref(need), ctypes.byref(ok)), "reindex source")
        return buf.value.decode(), need.value, bool(ok.value)

    src, need, ok = source([4, 32, 32, 32], [4, 64, 32, 32, 32, 3, 3], ["i0", "i2", "i3*1-1+i5*1", "i4*1-1+i6*1"])
    assert ok and "stage[" in src and "uint4" in src and "i1 * " not in src              # tiled form; broadcast axis: no multiply at all
    src, need, ok = source([100, 66], [100, 70], ["i0", "i1-2"])
    assert ok and "if (i1 == 70)" in src and "stage[" not in src                         # long ragged rows: odometer with a carry
    src, need, ok = source([32768, 4096], [32768, 4100], ["i0", "i1-2"])
    assert ok and "if (i1 ==" not in src and "(unsigned)a0" not in src                   # no carry, no check on the row axis
    for dtype in ("uint8", "bfloat16", "float64"):
        src, need, ok = source([64, 48], [64, 56], ["i0", "i1-4"], dtype)
        assert ok, dtype
    src, need, ok = source([5, 7], [5, 9], ["i0", "i1-1"])
    assert ok and "y[v] =" in src
    src, need, ok = source([100, 8], [10, 8], ["@e0(i0)", "i1"], extras=[("int32", [10])])
    assert need == 0 and not ok
