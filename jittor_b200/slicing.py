"""`Var.__getitem__` / `Var.__setitem__`, `getitem`, `setitem`, `scatter`, `gather`: the slicing surface of the reference
(python/jittor/src/ops/getitem_op.cc, setitem_op.cc; python/jittor/misc.py:1563-1645) lowered onto the meta-operators.

A tuple of slices is first resolved against the input shape exactly as GetitemOp::infer_slices does
(getitem_op.cc:66-187): every input axis ends up as one of
    loop      the axis is passed through (no slice, `:`, or covered by an ellipsis),
    slice     start + step * loop variable,
    int       a constant,
    str       a formula over the output's loop variables i0, i1, ... (what scatter/gather use for the other axes),
    var       an index Var; all index Vars broadcast against each other and their axes are placed where the FIRST index
              Var stands (this is the reference's rule; numpy moves them to the front when they are separated),
and `None` adds an output axis of size 1. getitem then is ONE reindex (gather), setitem ONE b200jt_setitem launch
(copy + scatter with the reduce op), both on the CUDA kernels of the path."""
import ctypes
import re

import numpy as np
import torch

from . import _capi as C
from . import var as V

_SETITEM_OPS = {"void", "add", "multiply", "maximum", "minimum", "bitwise_and", "bitwise_or", "bitwise_xor",
                "logical_and", "logical_or", "logical_xor"}


class _Axis:
    __slots__ = ("kind", "out", "start", "step", "value", "text", "var")

    def __init__(self, kind, out=-1, start=0, step=1, value=0, text="", var=None):
        self.kind, self.out, self.start, self.step, self.value, self.text, self.var = kind, out, start, step, value, text, var


def _as_tuple(slices):
    """A tuple of index items; lists and numpy arrays become index Vars (the reference converts them the same way)."""
    items = tuple(slices) if isinstance(slices, tuple) else (slices,)
    return tuple(V.array(s) if isinstance(s, (list, np.ndarray)) else s for s in items)


def _fill_slice(s, n):
    """Python slice semantics (Slice::fill in the reference, python/jittor/src/var_slices.h): start/stop/step resolved
    against an axis of length n; the output length follows getitem_op.cc:159-168."""
    start, stop, step = s.indices(n)
    if step > 0:
        length = max(0, (stop - start + step - 1) // step)
    else:
        length = max(0, (start - stop - step - 1) // (-step))
    return start, step, length


def resolve(in_shape, slices):
    """Returns (axes: one _Axis per input axis, out_shape, first_var_axis, var_dim)."""
    slices = list(_as_tuple(slices))
    nin = len(in_shape)
    index_vars = [s for s in slices if isinstance(s, V.Var)]
    for v in index_vars:
        if str(v.dtype) == "bool":
            raise ValueError("Please convert bool slice into jt.array")
    var_dim = max((v.ndim for v in index_vars), default=0)
    if sum(1 for s in slices if s is Ellipsis) > 1:
        raise ValueError("an index can only have a single ellipsis ('...')")
    axes, out_shape = [], []
    fov = -1
    vid, i = 0, 0
    while i < nin:
        if vid >= len(slices):
            axes.append(_Axis("loop", out=len(out_shape)))
            out_shape.append(in_shape[i])
            i += 1
            continue
        s = slices[vid]
        if isinstance(s, V.Var):
            if fov == -1:
                fov = len(out_shape)
                out_shape.extend([1] * var_dim)
            for j in range(s.ndim):
                have, want = out_shape[fov + var_dim - 1 - j], s.shape[s.ndim - 1 - j]
                if not (have == want or have == 1 or want == 1):
                    raise ValueError(f"Shape not match {have}!={want} data shape:{list(in_shape)} slice shape:{list(s.shape)}")
                if have == 1:
                    out_shape[fov + var_dim - 1 - j] = want
            axes.append(_Axis("var", var=s))
            vid += 1
            i += 1
        elif s is Ellipsis:
            remain = len(slices) - vid - 1 - sum(1 for t in slices[vid + 1:] if t is None)
            size = (nin - i) - remain
            if size < 0:
                raise ValueError("NDims not match")
            for _ in range(size):
                axes.append(_Axis("loop", out=len(out_shape)))
                out_shape.append(in_shape[i])
                i += 1
            vid += 1
        elif s is None:
            out_shape.append(1)
            vid += 1
        elif isinstance(s, str):
            axes.append(_Axis("str", text=s))
            vid += 1
            i += 1
        elif isinstance(s, slice):
            if s.start is None and s.stop is None and s.step is None:
                axes.append(_Axis("loop", out=len(out_shape)))
                out_shape.append(in_shape[i])
            else:
                start, step, length = _fill_slice(s, in_shape[i])
                axes.append(_Axis("slice", out=len(out_shape), start=start, step=step))
                out_shape.append(length)
            vid += 1
            i += 1
        else:
            try:
                v = int(s.__index__())
            except AttributeError:
                raise TypeError(f"unsupported index {s!r}") from None
            if v < 0:
                v += in_shape[i]
            if not 0 <= v < in_shape[i]:
                raise IndexError(f"slice overflow, {v} not in [0,{in_shape[i]})")
            axes.append(_Axis("int", value=v))
            vid += 1
            i += 1
    while vid < len(slices):
        s = slices[vid]
        vid += 1
        if s is None:
            out_shape.append(1)
        elif s is not Ellipsis:
            raise IndexError(f"Too many slices {slices} shape:{list(in_shape)}")
    return axes, out_shape, fov, var_dim


def _index_strings(axes, out_shape, fov, var_dim, in_shape, wrap_negative):
    """One index expression per input axis over the loop variables of `out_shape`, plus the extras list."""
    extras, exprs = [], []
    for d, ax in enumerate(axes):
        if ax.kind == "loop":
            exprs.append(f"i{ax.out}")
        elif ax.kind == "slice":
            exprs.append(f"i{ax.out}*{ax.step}+{ax.start}" if ax.step >= 0 else f"{ax.start}-i{ax.out}*{-ax.step}")
        elif ax.kind == "int":
            exprs.append(str(ax.value))
        elif ax.kind == "str":
            e = f"({ax.text})"
            plain = re.fullmatch(r"\s*i\d+\s*", ax.text) is not None       # a bare loop variable cannot be negative
            exprs.append(f"({e}<0?{e}+{in_shape[d]}:{e})" if wrap_negative and not plain else ax.text if plain else e)
        else:
            v = ax.var
            k = len(extras)
            extras.append(v)
            args = []
            for j in range(v.ndim):
                o = fov + var_dim - v.ndim + j
                args.append(f"i{o}" if v.shape[j] == out_shape[o] and v.shape[j] != 1 else "0")
            e = f"@e{k}({','.join(args)})" if args else f"@e{k}(0)"
            exprs.append(f"({e}<0?{e}+{in_shape[d]}:{e})" if wrap_negative else e)
    return exprs, extras


def getitem(x, slices):
    """x[slices] (GetitemOp, python/jittor/src/ops/getitem_op.cc:530-580): one gather. Negative values of index
    Vars and formulas wrap around once, as the reference's `if (iid<0) iid += ishape`."""
    x = V.to_var(x)
    axes, out_shape, fov, var_dim = resolve(list(x.shape), slices)
    scalar_out = not out_shape
    if scalar_out:
        out_shape = [1]
    exprs, extras = _index_strings(axes, out_shape, fov, var_dim, list(x.shape), True)
    extras = [e if e.ndim else e.reshape([1]) for e in extras]
    return V.reindex(x, out_shape, exprs, 0, [], extras)


def _setitem_run(op, xshape, yshape, eshapes):
    def run(xd, yd, *extra_data, indexes=None):
        xd, yd = xd.view(xshape), yd.view(yshape)
        extra_data = [e.view(s) for e, s in zip(extra_data, eshapes)]
        out = torch.empty_like(xd)
        ex = C.descs(list(extra_data)) if extra_data else None
        C.check(C.lib.b200jt_setitem(C.desc(xd), C.desc(yd), C.desc(out), op.encode(), C.strings(indexes), len(indexes),
                                     ex, len(extra_data), C.stream_ptr()), "setitem")
        return out
    return run


def setitem(x, slices, value, op="void"):
    """A copy of x with `x[slices] = op(x[slices], value)` applied (SetitemOp, setitem_op.cc:268-366); `value` is
    broadcast to the sliced region from the right (setitem_op.cc:72-85) and cast to x's dtype."""
    x = V.to_var(x)
    if op not in _SETITEM_OPS:
        raise ValueError(f"setitem: unsupported op {op!r}")
    axes, out_shape, fov, var_dim = resolve(list(x.shape), slices)
    if not out_shape:
        out_shape = [1]
    value = V.to_var(value)
    if value.dtype != x.dtype:
        value = value.cast(x.dtype)
    if value.ndim > len(out_shape):
        raise ValueError("Data dimension not match")
    vshape = [1] * (len(out_shape) - value.ndim) + list(value.shape)
    for a, b in zip(vshape, out_shape):
        if a != 1 and a != b:
            raise ValueError(f"Data shape not match {list(value.shape)} {out_shape}")
    if vshape != out_shape:
        value = V.broadcast(value.reshape(vshape), out_shape)
    exprs, extras = _index_strings(axes, out_shape, fov, var_dim, list(x.shape), False)
    extras = [e if e.ndim else e.reshape([1]) for e in extras]
    run = _setitem_run(op, list(x.shape), list(out_shape), [list(e.shape) for e in extras])
    node = V.Op("custom", [x, value] + extras, fn=lambda xd, yd, *ed: run(xd, yd, *ed, indexes=exprs),
                name="setitem", indexes=exprs, region=list(out_shape), reduce=op)
    return V.Var(list(x.shape), x.dtype, node)


def scatter(x, dim, index, src, reduce="void"):
    """x with src scattered along `dim` at `index` (python/jittor/misc.py:1563-1605): the other axes are the formula
    slices 'i0', 'i1', ...; src is cropped to index's shape unless it is a single element."""
    x, index, src = V.to_var(x), V.to_var(index), V.to_var(src)
    shape = list(index.shape)
    if list(src.shape) != shape and src.numel() != 1:
        src = getitem(src, tuple(slice(None, s) for s in shape))
    indexes = [f"i{i}" for i in range(len(shape))]
    indexes[dim] = index
    return setitem(x, tuple(indexes), src, reduce)


def scatter_(x, dim, index, src, reduce="void"):
    return x.assign(scatter(x, dim, index, src, reduce))


def gather(x, dim, index):
    """out[i][j][k] = x[index[i][j][k]][j][k] for dim 0, and so on (python/jittor/misc.py:1610-1645)."""
    x, index = V.to_var(x), V.to_var(index)
    indexes = [f"i{i}" for i in range(index.ndim)]
    indexes[dim] = index
    return getitem(x, tuple(indexes))


def _var_getitem(self, slices):
    return getitem(self, slices)


def _var_setitem(self, slices, value):
    """`x[slices] = value` rebinds x to the updated copy, like the reference's Var.__setitem__ (assign of setitem)."""
    self.assign(setitem(self, slices, value))


V.Var.__getitem__ = _var_getitem
V.Var.__setitem__ = _var_setitem
V.Var.getitem = getitem
V.Var.setitem = setitem
V.Var.scatter = scatter
V.Var.scatter_ = scatter_
V.Var.gather = gather
