"""Shared driver for the golden fixtures: loads tests/golden/meta_ops.{json,npz} and runs one case
against a backend (a namespace of functions over numpy arrays with the oracle's names)."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
# meta_ops: the path itself; next_ops: its callers (slicing, scatter/gather, pooling, conv variants, optimiser step)
_FILES = ("meta_ops", "next_ops")
CASES = []
for _f in _FILES:
    for _c in json.load(open(os.path.join(HERE, "golden", _f + ".json")))["cases"]:
        _c["file"] = _f
        CASES.append(_c)
_npz = {}


def arrays(which="meta_ops"):
    if which not in _npz:
        _npz[which] = np.load(os.path.join(HERE, "golden", which + ".npz"))
    return _npz[which]


def decode_slices(enc, extras):
    """Inverse of the encoding of tests/golden/make_golden_next.py: index arrays come back as numpy arrays."""
    out = []
    for e in enc:
        if e is None:
            out.append(None)
        elif e == "...":
            out.append(Ellipsis)
        elif "i" in e:
            out.append(int(e["i"]))
        elif "s" in e:
            out.append(slice(*e["s"]))
        elif "f" in e:
            out.append(e["f"])
        else:
            out.append(extras[e["v"]])
    return tuple(out)


def case_ids():
    return [c["name"] for c in CASES]


EXACT_OPS = {"reindex", "reindex_var", "broadcast", "broadcast_var", "ternary", "getitem", "gather"}


def _kw(v):
    return tuple(v) if isinstance(v, list) else v


def run_case(c, be):
    """Returns (got, want, exact) for case `c` on backend `be`."""
    A = arrays(c.get("file", "meta_ops"))
    ins = [A[k] for k in c["inputs"]]
    ex = [A[k] for k in c["extras"]]
    want = A[c["out"]]
    a = c["args"]
    op = c["op"]
    if op == "reindex":
        if a.get("bf16_bits"):
            got = be.reindex_bf16_bits(ins[0], a["shape"], a["indexes"], a["overflow_value"])
        else:
            got = be.reindex(ins[0], a["shape"], a["indexes"], a["overflow_value"],
                             a["overflow_conditions"], ex)
    elif op == "reindex_var":
        got = be.reindex_var(ins[0], ex, a["overflow_value"], a["overflow_conditions"])
    elif op == "reindex_reduce":
        got = be.reindex_reduce(ins[0], a["op"], a["shape"], a["indexes"], a["overflow_conditions"], ex)
    elif op == "broadcast":
        got = be.broadcast(ins[0], a["shape"], a["dims"])
    elif op == "broadcast_var":
        got = be.broadcast_var(ins[0], ins[1], a["dims"])
    elif op == "reduce":
        d = a["dims"]
        got = be.reduce(ins[0], a["op"], tuple(d) if isinstance(d, list) else d, a["keepdims"])
    elif op == "binary":
        got = be.binary(ins[0], ins[1], a["op"])
    elif op == "unary":
        got = be.unary(ins[0], a["op"])
    elif op == "ternary":
        got = be.ternary(*ins)
    elif op == "conv":
        got = be.conv2d(ins[0], ins[1], a["stride"], a["padding"], a["dilation"],
                        ins[2] if a["bias"] else None)
    elif op == "matmul":
        got = be.matmul(ins[0], ins[1])
    elif op == "matmul_transpose":
        got = be.matmul_transpose(ins[0], ins[1])
    elif op in ("softmax", "log_softmax"):
        got = be.softmax(ins[0], a["dim"], op == "log_softmax")
    elif op == "layer_norm":
        got = be.layer_norm(ins[0], a["normalized_shape"], ins[1] if a["affine"] else None,
                            ins[2] if a["affine"] else None, a["eps"])
    elif op in ("batch_norm", "batch_norm_relu"):
        got = be.batch_norm_train(ins[0], ins[1], ins[2], a["eps"], op == "batch_norm_relu")
    elif op == "conv_bn_relu":
        y = be.conv2d(ins[0], ins[1], a["stride"], a["padding"], a["dilation"], None)
        got = be.batch_norm_train(y, ins[2], ins[3], a["eps"], True)
    elif op == "maxpool2x2":
        got = be.maxpool2x2(ins[0])
    elif op == "maxpool2x2_bwd":
        got = be.maxpool2x2_bwd(ins[0], ins[1])
    elif op == "grad_reindex":
        # reindex grad = reindex_reduce(add) of the upstream gradient (reindex_op.cc:76-80)
        got = be.reindex_reduce(ins[1], "add", list(ins[0].shape), a["indexes"], [], [])
    elif op == "grad_reindex_reduce_add":
        # reindex_reduce(add) grad = reindex of the upstream gradient (reindex_reduce_op.cc:48-49)
        got = be.reindex(ins[1], list(ins[0].shape), a["indexes"], 0, [], [])
    elif op == "getitem":
        got = be.getitem(ins[0], decode_slices(a["slices"], ex))
    elif op == "setitem":
        got = be.setitem(ins[0], decode_slices(a["slices"], ex), ins[1], a["op"])
    elif op == "scatter":
        got = be.scatter(ins[0], a["dim"], ex[0], ins[1], a["reduce"])
    elif op == "gather":
        got = be.gather(ins[0], a["dim"], ex[0])
    elif op == "pool2d":
        got = be.pool2d(ins[0], _kw(a["kernel_size"]), a["op"], _kw(a["stride"]), _kw(a["padding"]), a["ceil_mode"],
                        a["count_include_pad"])
    elif op == "pool2d_bwd":
        got = be.pool2d_backward(ins[0], ins[1], _kw(a["kernel_size"]), a["op"], _kw(a["stride"]), _kw(a["padding"]),
                                 a["ceil_mode"], a["count_include_pad"])
    elif op == "conv_grouped":
        got = be.conv2d_grouped(ins[0], ins[1], _kw(a["stride"]), _kw(a["padding"]), _kw(a["dilation"]), a["groups"],
                                ins[2] if a["bias"] else None)
    elif op == "conv_transpose":
        got = be.conv_transpose2d(ins[0], ins[1], _kw(a["stride"]), _kw(a["padding"]), _kw(a["output_padding"]),
                                  a["groups"], _kw(a["dilation"]), ins[2] if a["bias"] else None)
    elif op in ("conv_dgrad", "conv_wgrad"):
        got = be.conv_grad(ins[0], ins[1], ins[2], a["stride"], a["padding"], a["dilation"], op == "conv_wgrad")
    elif op == "adaptive_pool":
        got = be.adaptive_pool2d(ins[0], _kw(a["output_size"]), a["op"])
    elif op == "conv1d":
        got = be.conv1d(ins[0], ins[1], a["stride"], a["padding"], a["dilation"], a["groups"], ins[2] if a["bias"] else None)
    elif op == "optim":
        kw = {k: (tuple(v) if isinstance(v, list) else v) for k, v in a.items() if k not in ("kind", "steps")}
        got = be.optim_steps(ins[0], ins[1], ins[2], a["kind"], a["steps"], **kw)
    else:
        raise KeyError(op)
    exact = op in EXACT_OPS or (want.dtype.kind in "iub" and op != "unary")
    return np.asarray(got), want, exact


def check(got, want, exact, rtol=1e-5):
    """Bit-exact for gathers and integer work; for floating point
    |got-want| <= rtol*|want| + rtol*max|want| (the reference's own -Ofast sums are order-unstable)."""
    assert got.dtype == want.dtype, (got.dtype, want.dtype)
    assert got.shape == want.shape, (got.shape, want.shape)
    if got.size == 0:
        return
    if exact:
        assert np.array_equal(got, want, equal_nan=want.dtype.kind == "f"), \
            f"mismatch at {np.argwhere(got != want)[:5].tolist()}"
    else:
        g, w = got.astype(np.float64), want.astype(np.float64)
        fin = np.isfinite(w)
        assert np.array_equal(fin, np.isfinite(g))
        assert np.array_equal(g[~fin], w[~fin], equal_nan=True)
        scale = np.max(np.abs(w[fin])) if fin.any() else 0.0
        err = np.abs(g[fin] - w[fin])
        tol = rtol * np.abs(w[fin]) + rtol * scale
        assert (err <= tol).all(), f"max err {err.max():.3e} (scale {scale:.3e})"
