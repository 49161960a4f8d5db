"""Host side of getitem / setitem / scatter / gather without a GPU: the slices of every golden case are resolved by
jittor_b200.slicing on placeholder Vars, and the index expressions it hands to the kernels are evaluated by the numpy
oracle; the result must equal what the reference produced."""
import numpy as np
import pytest

import jittor_b200 as jt
from jittor_b200 import slicing
from oracle import meta_ops_ref as oracle
from tests import golden_cases as G

CASES = [c for c in G.CASES if c["op"] in ("getitem", "setitem", "scatter", "gather")]


def placeholder(a):
    return jt.Var(list(a.shape) if a.ndim else [1], str(a.dtype))


def to_vars(slices, table):
    out = []
    for s in slices:
        if isinstance(s, np.ndarray):
            v = placeholder(s)
            table[id(v)] = s
            out.append(v)
        else:
            out.append(s)
    return tuple(out)


def lowered(c):
    A = G.arrays(c["file"])
    ins = [A[k] for k in c["inputs"]]
    ex = [A[k] for k in c["extras"]]
    a, table = c["args"], {}
    x = placeholder(ins[0])
    if c["op"] == "getitem":
        y = slicing.getitem(x, to_vars(G.decode_slices(a["slices"], ex), table))
    elif c["op"] == "gather":
        iv = placeholder(ex[0]); table[id(iv)] = ex[0]
        y = slicing.gather(x, a["dim"], iv)
    elif c["op"] == "setitem":
        d = placeholder(ins[1])
        y = slicing.setitem(x, to_vars(G.decode_slices(a["slices"], ex), table), d, a["op"])
    else:
        iv = placeholder(ex[0]); table[id(iv)] = ex[0]
        d = placeholder(ins[1])
        y = slicing.scatter(x, a["dim"], iv, d, a["reduce"])
    return ins, y, table


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_lowering_reproduces_reference(case):
    ins, y, table = lowered(case)
    want = G.arrays(case["file"])[case["out"]]
    assert list(y.shape) == list(want.shape) and str(y.dtype) == str(want.dtype)
    op = y._op
    if op.kind == "reindex":
        extras = [table[id(v)] for v in op.inputs[1:]]
        got = oracle.reindex(ins[0], op.attrs["shape"], op.attrs["indexes"], 0, [], extras)
        assert np.array_equal(got, want)
        return
    assert op.kind == "custom" and op.attrs["name"] == "setitem"
    extras = [table[id(v)].reshape(list(v.shape)) for v in op.inputs[2:]]
    region = op.attrs["region"]
    flat, over = oracle._flat_index(region, ins[0].shape, op.attrs["indexes"], [], extras)
    assert not over.any()
    data = ins[1]
    if case["op"] == "scatter" and data.shape != tuple(region) and data.size != 1:
        data = data[tuple(slice(None, s) for s in region)]
    data = np.broadcast_to(data.astype(ins[0].dtype).reshape([1] * (len(region) - data.ndim) + list(data.shape)), region)
    out = ins[0].copy().reshape(-1)
    red = op.attrs["reduce"]
    if red == "void":
        out[flat.reshape(-1)] = data.reshape(-1)
    else:
        {"add": np.add, "multiply": np.multiply, "maximum": np.maximum, "minimum": np.minimum}[red].at(
            out, flat.reshape(-1), data.reshape(-1))
    G.check(out.reshape(ins[0].shape), want, want.dtype.kind in "iub")


def test_errors():
    x = jt.Var([4, 5], "float32")
    with pytest.raises(IndexError):
        slicing.resolve([4, 5], (1, 2, 3))
    with pytest.raises(IndexError):
        slicing.resolve([4, 5], (7,))
    with pytest.raises(ValueError, match="bool"):
        slicing.resolve([4, 5], (jt.Var([4], "bool"),))
    with pytest.raises(ValueError, match="Shape not match"):
        slicing.resolve([4, 5], (jt.Var([3], "int32"), jt.Var([2], "int32")))
    with pytest.raises(ValueError, match="unsupported op"):
        slicing.setitem(x, 0, 1.0, "subtract")
    with pytest.raises(ValueError, match="Data shape not match"):
        slicing.setitem(x, (slice(0, 2),), jt.Var([3, 5], "float32"))
