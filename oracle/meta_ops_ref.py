"""CPU restatement (numpy) of the reference's meta-operators and of the chains its nn layer
builds from them.

TEST INFRASTRUCTURE ONLY. This module is the checker that the CUDA path is compared against; it is
imported by the tests, by the smoke check and by the CPU-baseline leg of the benchmark, never by the
shipped package. Parity pinned: every function here is checked against outputs of the reference's own
CPU executor (fixtures under tests/golden, made by tests/golden/make_golden.py).

Each function cites the reference lines (paths relative to the reference project root) it follows.
Index arithmetic uses C semantics (`/` and `%` truncate toward zero) as the reference emits the
index strings verbatim into C++ (python/jittor/src/ops/reindex_op.cc:131-137).
"""
import re

import numpy as np

# --------------------------------------------------------------------------- index expressions
_TOK = re.compile(r"\s*(?:(\d+)|(@e\d+)|([A-Za-z_]\w*)|(&&|\|\||==|!=|<=|>=|<<|>>|[-+*/%()<>!,?:&|^~]))")


def _tokenize(s):
    pos, out = 0, []
    s = s.strip()
    while pos < len(s):
        m = _TOK.match(s, pos)
        if not m:
            raise ValueError(f"bad index expression {s!r} at {pos}")
        pos = m.end()
        if m.group(1):
            out.append(("num", int(m.group(1))))
        elif m.group(2):
            out.append(("ext", int(m.group(2)[2:])))
        elif m.group(3):
            out.append(("var", m.group(3)))
        else:
            out.append(("op", m.group(4)))
    return out


_BIN_PREC = [["||"], ["&&"], ["|"], ["^"], ["&"], ["==", "!="], ["<", "<=", ">", ">="],
             ["<<", ">>"], ["+", "-"], ["*", "/", "%"]]


class _Parser:
    """Recursive-descent parser of the C integer-expression subset used in index strings."""

    def __init__(self, text):
        if "//" in text:
            raise ValueError("'//' is not an operator of the index language")
        self.t = _tokenize(text)
        self.i = 0

    def peek(self):
        return self.t[self.i] if self.i < len(self.t) else (None, None)

    def eat(self, kind=None, val=None):
        k, v = self.peek()
        if k is None or (kind and k != kind) or (val is not None and v != val):
            raise ValueError(f"unexpected token {v!r}")
        self.i += 1
        return v

    def parse(self):
        e = self.ternary()
        if self.i != len(self.t):
            raise ValueError("trailing tokens in index expression")
        return e

    def ternary(self):
        c = self.binary(0)
        if self.peek() == ("op", "?"):
            self.eat()
            a = self.ternary()
            self.eat("op", ":")
            b = self.ternary()
            return ("?", c, a, b)
        return c

    def binary(self, lvl):
        if lvl == len(_BIN_PREC):
            return self.unary()
        lhs = self.binary(lvl + 1)
        while self.peek()[0] == "op" and self.peek()[1] in _BIN_PREC[lvl]:
            op = self.eat()
            rhs = self.binary(lvl + 1)
            lhs = (op, lhs, rhs)
        return lhs

    def unary(self):
        k, v = self.peek()
        if k == "op" and v in ("-", "+", "!", "~"):
            self.eat()
            return ("u" + v, self.unary())
        return self.atom()

    def atom(self):
        k, v = self.peek()
        if k == "num":
            self.eat()
            return ("num", v)
        if k == "var":
            self.eat()
            return ("var", v)
        if k == "ext":
            self.eat()
            self.eat("op", "(")
            args = [self.ternary()]
            while self.peek() == ("op", ","):
                self.eat()
                args.append(self.ternary())
            self.eat("op", ")")
            return ("ext", v, args)
        if k == "op" and v == "(":
            self.eat()
            e = self.ternary()
            self.eat("op", ")")
            return e
        raise ValueError(f"unexpected token {v!r}")


def _cdiv(a, b):
    q = np.abs(a) // np.abs(b)
    return np.where((a < 0) != (b < 0), -q, q)


def _eval(e, env, extras):
    k = e[0]
    if k == "num":
        return np.int64(e[1])
    if k == "var":
        return env[e[1]]
    if k == "ext":
        arr = extras[e[1]]
        args = [np.asarray(_eval(a, env, extras)).astype(np.int64) for a in e[2]]
        if len(args) != arr.ndim:
            raise ValueError("@e%d: wrong number of subscripts" % e[1])
        flat = 0
        for d, a in enumerate(args):
            flat = flat * arr.shape[d] + a
        v = arr.reshape(-1)[flat]
        return np.trunc(v).astype(np.int64) if v.dtype.kind == "f" else v.astype(np.int64)
    if k == "?":
        return np.where(_eval(e[1], env, extras) != 0, _eval(e[2], env, extras), _eval(e[3], env, extras))
    if k[0] == "u" and len(e) == 2:
        a = _eval(e[1], env, extras)
        return {"u-": lambda: -a, "u+": lambda: a, "u!": lambda: (a == 0).astype(np.int64),
                "u~": lambda: ~a}[k]()
    a, b = _eval(e[1], env, extras), _eval(e[2], env, extras)
    a, b = np.asarray(a, dtype=np.int64), np.asarray(b, dtype=np.int64)
    if k == "+": return a + b
    if k == "-": return a - b
    if k == "*": return a * b
    if k == "/": return _cdiv(a, b)
    if k == "%": return a - _cdiv(a, b) * b
    if k == "<": return (a < b).astype(np.int64)
    if k == "<=": return (a <= b).astype(np.int64)
    if k == ">": return (a > b).astype(np.int64)
    if k == ">=": return (a >= b).astype(np.int64)
    if k == "==": return (a == b).astype(np.int64)
    if k == "!=": return (a != b).astype(np.int64)
    if k == "&&": return ((a != 0) & (b != 0)).astype(np.int64)
    if k == "||": return ((a != 0) | (b != 0)).astype(np.int64)
    if k == "&": return a & b
    if k == "|": return a | b
    if k == "^": return a ^ b
    if k == "<<": return a << b
    if k == ">>": return a >> b
    raise ValueError(k)


def _index_env(yshape, xshape, extras):
    """Loop variables i0..in over `yshape` plus the shape/stride symbols the generated source
    defines (reindex_op.cc:113-130)."""
    env = {}
    grids = np.indices(tuple(yshape), dtype=np.int64, sparse=True) if len(yshape) else []
    for d, g in enumerate(grids):
        env[f"i{d}"] = g
    for nm, shp in (("x", xshape), ("y", yshape)):
        st = 1
        for d in range(len(shp) - 1, -1, -1):
            env[f"{nm}shape{d}"] = np.int64(shp[d])
            env[f"{nm}stride{d}"] = np.int64(st)
            st *= shp[d]
    for k, e in enumerate(extras):
        st = 1
        for d in range(e.ndim - 1, -1, -1):
            env[f"extras{k}shape{d}"] = np.int64(e.shape[d])
            env[f"extras{k}stride{d}"] = np.int64(st)
            st *= e.shape[d]
    return env


def _flat_index(yshape, xshape, indexes, overflow_conditions, extras):
    """Returns (flat x index, overflow mask), both of shape yshape (reindex_op.cc:131-137)."""
    env = _index_env(yshape, xshape, extras)
    flat = np.zeros(tuple(yshape), dtype=np.int64)
    over = np.zeros(tuple(yshape), dtype=bool)
    for d, s in enumerate(indexes):
        xi = np.broadcast_to(_eval(_Parser(s).parse(), env, extras), tuple(yshape))
        over |= (xi < 0) | (xi >= xshape[d])
        flat = flat * xshape[d] + xi
    for s in overflow_conditions:
        over |= np.broadcast_to(_eval(_Parser(s).parse(), env, extras), tuple(yshape)) != 0
    return flat, over


# --------------------------------------------------------------------------- the four meta-ops
def reindex(x, shape, indexes, overflow_value=0, overflow_conditions=(), extras=()):
    """ReindexOp::jit_run, python/jittor/src/ops/reindex_op.cc:111-139; shape rule :82-91."""
    x = np.asarray(x)
    extras = [np.asarray(e) for e in extras]
    if len(indexes) != x.ndim:
        raise ValueError("Number of x's shape and indexes should be the same.")
    shape = list(shape) if len(shape) else list(extras[0].shape)
    if not len(shape):
        raise ValueError("Number of shape should greater than 0.")
    flat, over = _flat_index(shape, x.shape, indexes, overflow_conditions, extras)
    y = np.empty(tuple(shape), dtype=x.dtype)
    if y.size == 0:
        return y
    fill = np.array(overflow_value, dtype=np.float64).astype(x.dtype)
    y[...] = x.reshape(-1)[np.where(over, 0, flat)] if x.size else fill
    y[over] = fill
    return y


def reindex_var(x, indexes, overflow_value=0, overflow_conditions=()):
    """ReindexOp var-index constructor, reindex_op.cc:35-70: index d is `@ed(i0,..,in)`."""
    indexes = [np.asarray(i) for i in indexes]
    n = indexes[0].ndim
    args = ",".join(f"i{d}" for d in range(n))
    return reindex(x, indexes[0].shape, [f"@e{d}({args})" for d in range(len(indexes))],
                   overflow_value, overflow_conditions, indexes)


def _lowest(dt):
    dt = np.dtype(dt)
    if dt.kind == "f":
        return np.finfo(dt).min
    if dt.kind == "b":
        return False
    return np.iinfo(dt).min


def _highest(dt):
    dt = np.dtype(dt)
    if dt.kind == "f":
        return np.finfo(dt).max
    if dt.kind == "b":
        return True
    return np.iinfo(dt).max


def _init_value(op, dt):
    """init_<op> table, python/jittor/src/type/common_op_type.cc:117-118,141-151 (CPU map)."""
    if op in ("add", "mean", "void", "bitwise_or", "bitwise_xor", "logical_or", "logical_xor"):
        return np.zeros((), dt)
    if op == "multiply":
        return np.ones((), dt)
    if op == "logical_and":
        return np.ones((), dt)
    if op == "bitwise_and":
        return np.array(-1).astype(dt)
    if op == "maximum":
        return np.array(_lowest(dt), dt)
    if op == "minimum":
        return np.array(_highest(dt), dt)
    raise ValueError(f"unknown reduce op {op}")


_UFUNC_AT = {"add": np.add, "multiply": np.multiply, "maximum": np.maximum, "minimum": np.minimum,
             "bitwise_and": np.bitwise_and, "bitwise_or": np.bitwise_or, "bitwise_xor": np.bitwise_xor}


def reindex_reduce(y, op, shape, indexes, overflow_conditions=(), extras=()):
    """ReindexReduceOp::jit_run, python/jittor/src/ops/reindex_reduce_op.cc:93-131: fill x with
    init(op), then walk y in row-major order and fold each element into x[index(i)]."""
    y = np.asarray(y)
    extras = [np.asarray(e) for e in extras]
    if len(shape) != len(indexes):
        raise ValueError("Number of shape and indexes should be the same.")
    if not len(shape):
        raise ValueError("Number of shape should greater than 0.")
    if any(int(s) < 0 for s in shape):
        raise ValueError("Shape should greater than 0.")
    if op not in _UFUNC_AT and op not in ("logical_and", "logical_or", "logical_xor", "void"):
        raise ValueError(f"unknown reindex_reduce op {op!r}")
    x = np.empty(tuple(shape), dtype=y.dtype)
    x[...] = _init_value(op, y.dtype)
    if y.size == 0 or x.size == 0:
        return x
    flat, over = _flat_index(y.shape, shape, indexes, overflow_conditions, extras)
    keep = ~over.reshape(-1)
    idx = flat.reshape(-1)[keep]
    val = y.reshape(-1)[keep]
    xf = x.reshape(-1)
    if op in _UFUNC_AT:
        with np.errstate(over="ignore"):
            _UFUNC_AT[op].at(xf, idx, val)
    elif op == "void":
        xf[idx] = val
    else:
        for i, v in zip(idx, val):
            a, b = bool(xf[i]), bool(v)
            xf[i] = {"logical_and": a and b, "logical_or": a or b, "logical_xor": a != b}[op]
    return x


def _bcast_masks(xshape, yshape, dims):
    """Mask inference of BroadcastToOp: ctor python/jittor/src/ops/broadcast_to_op.cc:74-96,
    infer_shape :119-168. Returns (zshape, bcast_mask)."""
    count = len(dims)
    xdim, ydim = len(xshape), len(yshape)
    zdim = max(xdim, ydim - count) + count
    mask = 0
    for d in dims:
        if d < 0:
            d += zdim
        if not 0 <= d < zdim:
            raise ValueError(f"Wrong dims number: {dims}")
        mask |= 1 << d
    keep = 0
    z = [0] * zdim
    xi, yi = xdim - 1, ydim - 1
    for i in range(zdim - 1, -1, -1):
        bx, by = xi >= 0, yi >= 0
        xs = xshape[xi] if bx else 1
        ys = yshape[yi] if by else 1
        if mask >> i & 1:
            yi -= 1
            if keep >> i & 1:
                xi -= 1
            z[i] = ys
            continue
        m = int(xs == 1 and (ys != 1 or not bx)) << i
        mask |= m
        if bx:
            keep |= m
        if (xs == 1 or ys == 1) and xs != ys:
            z[i] = xs * ys
        else:
            if xs != ys:
                raise ValueError(f"Shape not match {list(xshape)} {list(yshape)}")
            z[i] = xs
        xi -= 1
        yi -= 1
    return z, mask, keep


def broadcast(x, shape, dims=()):
    """BroadcastToOp::jit_run, broadcast_to_op.cc:177-194: z[i] = x[i with broadcast axes zeroed]."""
    x = np.asarray(x)
    shape = list(shape)
    if not len(dims) and not _need_broadcast(x.shape, shape):
        return x.copy()
    if not len(shape):
        raise ValueError("Number of shape should greater than 0.")
    zshape, mask, keep = _bcast_masks(list(x.shape), shape, list(dims))
    # x supplies the axes that are not new: new axes are bcast bits that x does not keep
    xi = 0
    src = list(x.shape)
    kept = [i for i in range(len(zshape)) if not (mask >> i & 1) or (keep >> i & 1)]
    src = [1] * (len(kept) - len(src)) + src
    view = []
    for i in range(len(zshape)):
        if i in kept:
            view.append(src[xi])
            xi += 1
        else:
            view.append(1)
    return np.ascontiguousarray(np.broadcast_to(x.reshape(view), zshape))


def _need_broadcast(xshape, shape):
    if len(xshape) < len(shape):
        return True
    for i in range(1, len(shape) + 1):
        if xshape[-i] != shape[-i] and shape[-i] != 1:
            return True
    return False


def broadcast_var(x, y, dims=()):
    """BroadcastToOp(Var* x, Var* y, dims): same rule with y's shape (broadcast_to_op.cc:23-44)."""
    return broadcast(x, list(np.asarray(y).shape), dims)


def reduce_dtype(op, dt):
    """reduce_dtype_infer, python/jittor/src/misc/nano_string.h:268-277 (+ bool -> int32,
    reduce_op.cc:287-288)."""
    dt = np.dtype(dt)
    if dt == np.bool_:
        return np.dtype(np.int32)
    if dt.kind == "f" or op == "mean":
        return np.dtype(np.float64) if dt.itemsize == 8 else np.dtype(np.float32)
    return dt


def reduce(x, op, dims=(), keepdims=False):
    """ReduceOp::jit_run, python/jittor/src/ops/reduce_op.cc:374-399; shape rule :318-337;
    `mean` accumulates x*rcount (common_op_type.cc:141)."""
    x = np.asarray(x)
    if isinstance(dims, (int, np.integer)):
        dims = (int(dims),)
    nd = x.ndim
    axes = []
    for d in dims:
        d = d + nd if d < 0 else d
        if not 0 <= d < nd:
            raise ValueError(f"Wrong dims number: {dims}")
        axes.append(d)
    axes = tuple(sorted(set(axes))) if len(axes) else tuple(range(nd))
    ty = reduce_dtype(op, x.dtype)
    xv = x.astype(ty)
    with np.errstate(over="ignore"):
        if op == "add":
            y = np.add.reduce(xv, axis=axes, dtype=ty, keepdims=keepdims)
        elif op == "mean":
            n = 1
            for a in axes:
                n *= x.shape[a]
            rcount = np.array(1.0 / n if n else 0).astype(ty)
            y = np.add.reduce(xv * rcount, axis=axes, dtype=ty, keepdims=keepdims)
        elif op == "multiply":
            y = np.multiply.reduce(xv, axis=axes, dtype=ty, keepdims=keepdims)
        elif op in ("maximum", "minimum"):
            f = np.maximum if op == "maximum" else np.minimum
            y = f.reduce(xv, axis=axes, keepdims=keepdims, initial=_init_value(op, ty)[()])
        elif op.startswith("bitwise_"):
            y = getattr(np, op).reduce(xv, axis=axes, keepdims=keepdims)
        elif op.startswith("logical_"):
            y = getattr(np, op).reduce(xv != 0, axis=axes, keepdims=keepdims).astype(ty)
        else:
            raise ValueError(f"unknown reduce op {op}")
    y = np.asarray(y, dtype=ty)
    if y.ndim == 0:
        y = y.reshape(1)
    return y


# --------------------------------------------------------------------------- element-wise ops
_BOOL_OPS = {"less", "less_equal", "greater", "greater_equal", "equal", "not_equal",
             "logical_and", "logical_or", "logical_xor", "logical_not", "bool"}
_FLOAT_OPS = {"log", "exp", "sqrt", "mean", "divide", "sin", "asin", "sinh", "asinh", "tan", "atan",
              "tanh", "atanh", "cos", "acos", "cosh", "acosh", "sigmoid", "erf", "erfinv"}
_INT_OPS = {"round_int", "floor_int", "ceil_int", "floor_divide"}
_DTYPES = {"bool", "int8", "int16", "int32", "int64", "uint8", "uint16", "uint32", "uint64",
           "float32", "float64"}


def _dsize(dt):
    return {1: 0, 2: 1, 4: 2, 8: 3}[np.dtype(dt).itemsize]


def binary_dtype(op, a, b):
    """binary_dtype_infer, python/jittor/src/misc/nano_string.h:233-252 (amp_reg = 0)."""
    a, b = np.dtype(a), np.dtype(b)
    if op in _BOOL_OPS:
        return np.dtype(np.bool_)
    ds = max(_dsize(a), _dsize(b))
    is_float = op not in _INT_OPS and (a.kind == "f" or b.kind == "f" or op in _FLOAT_OPS)
    if is_float:
        return np.dtype(np.float64) if ds == 3 else np.dtype(np.float32)
    if a == np.bool_ and b == np.bool_:
        return np.dtype(np.bool_)
    return np.dtype({3: np.int64, 2: np.int32, 1: np.int16, 0: np.int8}[ds])


def binary(a, b, op):
    """BinaryOp, python/jittor/src/ops/binary_op.cc:421-474 (broadcast insertion) and :563-570;
    scalar semantics python/jittor/src/type/common_op_type.cc:82-152."""
    a, b = np.asarray(a), np.asarray(b)
    if a.shape != b.shape:
        a2 = broadcast_var(a, b)
        b2 = broadcast_var(b, a)
        a, b = a2, b2
    tz = binary_dtype(op, a.dtype, b.dtype)
    with np.errstate(all="ignore"):
        if op in ("add", "subtract", "multiply"):
            f = {"add": np.add, "subtract": np.subtract, "multiply": np.multiply}[op]
            z = f(a, b)
        elif op in ("divide", "floor_divide"):
            x, y = a.astype(tz), b.astype(tz)
            z = x / y if tz.kind == "f" else _cdiv(x.astype(np.int64), y.astype(np.int64))
        elif op == "mod":
            if tz.kind == "f":
                z = a - np.floor(a / b) * b
            else:
                x, y = a.astype(np.int64), b.astype(np.int64)
                z = x - _cdiv(x, y) * y
        elif op == "pow":
            z = np.power(a, b)
        elif op in ("maximum", "minimum"):
            f = np.maximum if op == "maximum" else np.minimum
            z = f(a.astype(tz), b.astype(tz))
        elif op in ("less", "less_equal", "greater", "greater_equal", "equal", "not_equal"):
            z = getattr(np, op)(a, b)
        elif op in ("logical_and", "logical_or", "logical_xor"):
            z = getattr(np, op)(a != 0, b != 0)
        elif op in ("bitwise_and", "bitwise_or", "bitwise_xor", "left_shift", "right_shift"):
            z = getattr(np, op)(a, b)
        else:
            raise ValueError(f"unknown binary op {op}")
    return np.ascontiguousarray(np.asarray(z).astype(tz))


def unary_dtype(op, a):
    """unary_dtype_infer, nano_string.h:254-266; a dtype name is a cast (unary_op.cc)."""
    a = np.dtype(a)
    if op in _DTYPES:
        return np.dtype(op)
    if op in _BOOL_OPS:
        return np.dtype(np.bool_)
    if op in _FLOAT_OPS:
        return np.dtype(np.float64) if _dsize(a) == 3 else np.dtype(np.float32)
    if op in _INT_OPS:
        return np.dtype({3: np.int64, 2: np.int32, 1: np.int16, 0: np.int8}[_dsize(a)])
    return a


def unary(a, op):
    """UnaryOp; scalar semantics common_op_type.cc:82-112 (CPU map)."""
    a = np.asarray(a)
    tz = unary_dtype(op, a.dtype)
    with np.errstate(all="ignore"):
        if op in _DTYPES:
            z = (a != 0) if op == "bool" else a
            if a.dtype.kind == "f" and tz.kind in "iu":
                z = np.trunc(a)
        elif op == "negative":
            z = -a
        elif op == "abs":
            z = np.abs(a)
        elif op == "logical_not":
            z = a == 0
        elif op == "bitwise_not":
            z = ~a
        elif op == "sigmoid":
            x = a.astype(tz)
            z = 1.0 / (1.0 + np.exp(np.minimum(-x, tz.type(30 if tz == np.float32 else 300))))
        elif op in ("round", "round_int"):
            z = np.where(a >= 0, np.floor(a + 0.5), np.ceil(a - 0.5))    # C round(): half away from 0
        elif op in ("floor", "floor_int"):
            z = np.floor(a)
        elif op in ("ceil", "ceil_int"):
            z = np.ceil(a)
        elif op == "erf":
            from math import erf
            z = np.vectorize(erf)(a.astype(np.float64))
        elif op in ("asin", "acos", "atan", "asinh", "acosh", "atanh"):
            z = getattr(np, "arc" + op[1:])(a.astype(tz))
        elif op in ("exp", "log", "sqrt", "sin", "cos", "tan", "sinh", "cosh", "tanh"):
            z = getattr(np, op)(a.astype(tz))
        else:
            raise ValueError(f"unknown unary op {op}")
    return np.ascontiguousarray(np.asarray(z).astype(tz))


def ternary(c, a, b):
    """TernaryOp, python/jittor/src/ops/ternary_op.cc: z = c ? a : b."""
    c, a, b = np.asarray(c), np.asarray(a), np.asarray(b)
    return np.where(c != 0, a, b).astype(binary_dtype("add", a.dtype, b.dtype))


# --------------------------------------------------------------------------- chains from nn.py
def conv2d(x, w, stride=1, padding=1, dilation=1, bias=None, materialize_limit=1 << 23):
    """nn.Conv.execute, groups == 1: python/jittor/nn.py:1001-1021 -- reindex to the 7-D window
    tensor, broadcast w over [0,3,4], multiply, sum over [2,5,6]. Above `materialize_limit`
    elements the same sum is formed tap by tap so the 7-D tensor is never held."""
    x, w = np.asarray(x), np.asarray(w)
    n, c, h, wd = x.shape
    co, ci, kh, kw = w.shape
    s, p, d = stride, padding, dilation
    oh = (h + p * 2 - kh * d + d - 1) // s + 1
    ow = (wd + p * 2 - kw * d + d - 1) // s + 1
    shape7 = [n, co, c, oh, ow, kh, kw]
    if int(np.prod(shape7)) <= materialize_limit:
        xx = reindex(x, shape7, ["i0", "i2", f"i3*{s}-{p}+i5*{d}", f"i4*{s}-{p}+i6*{d}"])
        ww = broadcast(w, shape7, [0, 3, 4])
        y = reduce(binary(xx, ww, "multiply"), "add", [2, 5, 6])
    else:
        y = np.zeros((n, co, oh, ow), np.float32)
        xp = np.zeros((n, c, h + 2 * p + s, wd + 2 * p + s), x.dtype)
        xp[:, :, p:p + h, p:p + wd] = x
        for a in range(kh):
            for b in range(kw):
                win = xp[:, :, a * d:a * d + oh * s:s, b * d:b * d + ow * s:s]
                y += np.einsum("nchw,oc->nohw", win, w[:, :, a, b], optimize=True).astype(np.float32)
    if bias is not None:
        y = binary(y, broadcast(np.asarray(bias), y.shape, [0, 2, 3]), "add")
    return y


def matmul(a, b):
    """nn.matmul, python/jittor/nn.py:118-159 (every branch)."""
    a, b = np.asarray(a), np.asarray(b)
    if b.ndim == 1:
        return reduce(binary(a, b, "multiply"), "add", -1)
    if a.ndim == 1:
        return reduce(binary(broadcast_var(a, b, [-1]), b, "multiply"), "add", 0)
    n, m = a.shape[-2:]
    m2, k = b.shape[-2:]
    if m != m2:
        raise ValueError(f"dimension not match, a.shape:{a.shape}, b.shape:{b.shape}")
    if b.ndim == 2 and a.ndim > 2:
        return matmul(a.reshape(-1, m), b).reshape(a.shape[:-1] + (k,))
    lc = max(a.ndim, b.ndim)
    shape = []
    for i in range(lc - 2):
        ai, bi = a.ndim - (lc - i), b.ndim - (lc - i)
        an = a.shape[ai] if ai >= 0 else 1
        bn = b.shape[bi] if bi >= 0 else 1
        shape.append(max(an, bn))
    shape += [n, m, k]
    aa = broadcast(a, shape, [-1])
    bb = broadcast(b, shape, [-3])
    return reduce(binary(aa, bb, "multiply"), "add", -2)


def matmul_transpose(a, b):
    """nn.matmul_transpose, python/jittor/nn.py:40-58: c[n,k] = sum_m a[n,m] b[k,m]."""
    a, b = np.asarray(a), np.asarray(b)
    shape = list(a.shape[:-1]) + [b.shape[0], a.shape[-1]]
    aa = broadcast(a, shape, [len(shape) - 2])
    bb = broadcast(b, shape)
    return reduce(binary(aa, bb, "multiply"), "add", len(shape) - 1)


def softmax(x, dim=None, log=False):
    """nn.softmax meta-op form, python/jittor/nn.py:527-535."""
    x = np.asarray(x)
    dt = x.dtype
    xf = x.astype(np.float32) if dt != np.float64 else x
    dims = () if dim is None else dim
    mx = reduce(xf, "maximum", dims, True)
    a = binary(xf, mx, "subtract")
    if log:
        s = reduce(unary(a, "exp"), "add", dims, True)
        ret = binary(a, unary(s, "log"), "subtract")
    else:
        e = unary(a, "exp")
        ret = binary(e, reduce(e, "add", dims, True), "divide")
    return ret.astype(dt)


def _moments_norm(x, dims, keepdims, weight, bias, eps, bdims=None):
    xmean = reduce(x, "mean", dims, keepdims)
    x2mean = reduce(binary(x, x, "multiply"), "mean", dims, keepdims)
    xvar = binary(binary(x2mean, binary(xmean, xmean, "multiply"), "subtract"),
                  np.zeros(1, np.float32), "maximum")
    w = binary(weight, unary(binary(xvar, np.full(1, eps, np.float32), "add"), "sqrt"), "divide")
    b = binary(bias, binary(xmean, w, "multiply"), "subtract")
    if bdims is not None:
        w, b = broadcast_var(w, x, bdims), broadcast_var(b, x, bdims)
    return binary(binary(x, w, "multiply"), b, "add")


def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    """nn.LayerNorm.execute, python/jittor/nn.py:778-787."""
    x = np.asarray(x, dtype=np.float32)
    dims = [-i for i in range(len(normalized_shape), 0, -1)]
    weight = np.ones(1, np.float32) if weight is None else np.asarray(weight)
    bias = np.zeros(1, np.float32) if bias is None else np.asarray(bias)
    return _moments_norm(x, dims, True, weight, bias, eps)


def batch_norm_train(x, weight, bias, eps=1e-5, relu=False):
    """nn.BatchNorm.execute, training branch without sync, python/jittor/nn.py:671-683."""
    x = np.asarray(x, dtype=np.float32)
    dims = [0] + list(range(2, x.ndim))
    y = _moments_norm(x, dims, False, np.asarray(weight), np.asarray(bias), eps, dims)
    return np.maximum(y, 0) if relu else y


def maxpool2x2(x):
    """2x2/2 max pool written as reindex + reduce(max) (the Pool reindex path, python/jittor/pool.py)."""
    n, c, h, w = x.shape
    xx = reindex(x, [n, c, h // 2, w // 2, 2, 2], ["i0", "i1", "i2*2+i4", "i3*2+i5"])
    return reduce(xx, "maximum", [4, 5])


def maxpool2x2_bwd(x, dy):
    """Gradient of maxpool2x2 by the reference's rules: reduce(max) grad = (x == bcast(out)) ? bcast(dout) : 0
    (reduce_op.cc:354-360), reindex grad = reindex_reduce(add) (reindex_op.cc:76-80)."""
    n, c, h, w = x.shape
    shape6 = [n, c, h // 2, w // 2, 2, 2]
    idx = ["i0", "i1", "i2*2+i4", "i3*2+i5"]
    xx = reindex(x, shape6, idx)
    out = reduce(xx, "maximum", [4, 5])
    cond = binary(xx, broadcast(out, shape6, [4, 5]), "equal")
    dxx = ternary(cond, broadcast(np.asarray(dy), shape6, [4, 5]), np.zeros(shape6, np.float32))
    return reindex_reduce(dxx, "add", list(x.shape), idx)


# --------------------------------------------------------------------------- getitem / setitem
def _resolve_slices(in_shape, slices):
    """GetitemOp::infer_slices, python/jittor/src/ops/getitem_op.cc:66-187. `slices`: tuple of int, slice, Ellipsis,
    None, str (formula over the output loop variables) and integer numpy arrays (index Vars).
    Returns (per input axis: ("loop", o) | ("slice", o, start, step) | ("int", v) | ("str", text) | ("var", array),
    out_shape, first output axis of the index arrays, number of axes they span)."""
    slices = list(slices) if isinstance(slices, tuple) else [slices]
    nin = len(in_shape)
    arrays = [s for s in slices if isinstance(s, np.ndarray)]
    var_dim = max((a.ndim for a in arrays), default=0)
    axes, out_shape, fov = [], [], -1
    vid = i = 0
    while i < nin:
        if vid >= len(slices):                                   # :78-85 axes past the last slice pass through
            axes.append(("loop", len(out_shape))); out_shape.append(in_shape[i]); i += 1
            continue
        s = slices[vid]
        if isinstance(s, np.ndarray):                            # :87-113 index arrays broadcast from the right
            if fov < 0:
                fov = len(out_shape)
                out_shape += [1] * var_dim
            for j in range(s.ndim):
                o = fov + var_dim - 1 - j
                n = s.shape[s.ndim - 1 - j]
                if not (out_shape[o] == n or out_shape[o] == 1 or n == 1):
                    raise ValueError("Shape not match")
                if out_shape[o] == 1:
                    out_shape[o] = n
            axes.append(("var", s)); vid += 1; i += 1
        elif s is Ellipsis:                                      # :115-130
            remain = len(slices) - vid - 1 - sum(1 for t in slices[vid + 1:] if t is None)
            for _ in range((nin - i) - remain):
                axes.append(("loop", len(out_shape))); out_shape.append(in_shape[i]); i += 1
            vid += 1
        elif s is None:                                          # :132-137
            out_shape.append(1); vid += 1
        elif isinstance(s, str):                                 # :147-150
            axes.append(("str", s)); vid += 1; i += 1
        elif isinstance(s, slice):                               # :151-176
            if s.start is None and s.stop is None and s.step is None:
                axes.append(("loop", len(out_shape))); out_shape.append(in_shape[i])
            else:
                idx = range(*s.indices(in_shape[i]))
                axes.append(("slice", len(out_shape), idx.start, idx.step)); out_shape.append(len(idx))
            vid += 1; i += 1
        else:                                                    # :139-146
            v = int(s)
            if v < 0:
                v += in_shape[i]
            if not 0 <= v < in_shape[i]:
                raise IndexError("slice overflow")
            axes.append(("int", v)); vid += 1; i += 1
    for s in slices[vid:]:                                       # :178-185
        if s is None:
            out_shape.append(1)
        elif s is not Ellipsis:
            raise IndexError("Too many slices")
    return axes, out_shape, fov, var_dim


def _slice_flat_index(in_shape, axes, out_shape, fov, var_dim, wrap):
    """Flat input offset for every point of the loop nest over out_shape (getitem_op.cc:560-577)."""
    grids = np.indices(tuple(out_shape), dtype=np.int64, sparse=True)
    env = {f"i{d}": g for d, g in enumerate(grids)}
    flat = np.zeros(tuple(out_shape), dtype=np.int64)
    for d, ax in enumerate(axes):
        kind = ax[0]
        if kind == "loop":
            iid = grids[ax[1]]
        elif kind == "slice":
            iid = grids[ax[1]] * ax[3] + ax[2]
        elif kind == "int":
            iid = np.int64(ax[1])
        elif kind == "str":
            iid = _eval(_Parser(ax[1]).parse(), env, [])
        else:
            a = ax[1]
            off = fov + var_dim - a.ndim
            sub = tuple(grids[off + j] if a.shape[j] == out_shape[off + j] else np.int64(0) for j in range(a.ndim))
            iid = a[sub].astype(np.int64) if a.ndim else a.astype(np.int64)
        iid = np.broadcast_to(iid, tuple(out_shape))
        if wrap:
            iid = np.where(iid < 0, iid + in_shape[d], iid)      # :573 `if (iid<0) iid += ishape`
        flat = flat * in_shape[d] + iid
    return flat


def getitem(x, slices):
    """GetitemOp::jit_run, python/jittor/src/ops/getitem_op.cc:512-580."""
    x = np.asarray(x)
    axes, out_shape, fov, var_dim = _resolve_slices(list(x.shape), slices)
    if not out_shape:
        out_shape = [1]
    flat = _slice_flat_index(x.shape, axes, out_shape, fov, var_dim, True)
    return x.reshape(-1)[flat]


def setitem(x, slices, data, op="void"):
    """SetitemOp::jit_run, python/jittor/src/ops/setitem_op.cc:268-366: copy, then out[iid] = op(out[iid], data[did])
    in loop order (the last duplicate wins for 'void'); data broadcasts from the right (:72-85) and is cast to x's
    dtype (`(Ti)dp[did]`)."""
    x = np.asarray(x)
    axes, out_shape, fov, var_dim = _resolve_slices(list(x.shape), slices)
    if not out_shape:
        out_shape = [1]
    flat = _slice_flat_index(x.shape, axes, out_shape, fov, var_dim, False).reshape(-1)
    data = np.broadcast_to(np.asarray(data).astype(x.dtype), tuple(out_shape)).reshape(-1)
    out = x.copy().reshape(-1)
    if op == "void":
        out[flat] = data
    else:
        uf = {"add": np.add, "multiply": np.multiply, "maximum": np.maximum, "minimum": np.minimum,
              "bitwise_and": np.bitwise_and, "bitwise_or": np.bitwise_or, "bitwise_xor": np.bitwise_xor}[op]
        uf.at(out, flat, data)
    return out.reshape(x.shape)


def scatter(x, dim, index, src, reduce="void"):
    """python/jittor/misc.py:1563-1605."""
    index, src = np.asarray(index), np.asarray(src)
    if src.shape != index.shape and src.size != 1:
        src = src[tuple(slice(None, s) for s in index.shape)]
    idx = [f"i{i}" for i in range(index.ndim)]
    idx[dim] = index
    return setitem(x, tuple(idx), src, reduce)


def gather(x, dim, index):
    """python/jittor/misc.py:1610-1645."""
    index = np.asarray(index)
    idx = [f"i{i}" for i in range(index.ndim)]
    idx[dim] = index
    return getitem(x, tuple(idx))


# --------------------------------------------------------------------------- optimiser steps
def optim_steps(x, y, w, kind, steps, lr, momentum=0, weight_decay=0, dampening=0, nesterov=False,
                eps=1e-8, betas=(0.9, 0.999), alpha=0.99):
    """`steps` updates of w on loss = sum((x @ w - y)^2) / N with the reference's SGD (python/jittor/optim.py:325-345)
    or Adam (:420-437) formulas, in float32 like the reference's graph; the gradient is 2/N * x^T (x w - y)."""
    f = np.float32
    x, y, w = x.astype(f), y.astype(f), w.astype(f).copy()
    v, m = np.zeros_like(w), np.zeros_like(w)
    for n in range(1, steps + 1):
        d = x @ w - y
        g = (x.T @ (d * f(2.0))) * f(1.0 / x.shape[0])
        if kind == "sgd":
            dp = w * f(weight_decay) + g
            v = f(momentum) * v + dp * f(1 - dampening)
            w = w - (dp + f(momentum) * v) * f(lr) if nesterov else w - v * f(lr)
        elif kind == "rmsprop":
            v = f(alpha) * v + f(1 - alpha) * g * g                                   # optim.py:384-385
            w = w - f(lr) * g / (np.sqrt(v) + f(eps))
        elif kind == "adamw":
            b0, b1 = betas                                                            # optim.py:471-491
            w = w * f(1 - lr * weight_decay)
            m = f(b0) * m + f(1 - b0) * g
            v = f(b1) * v + f(1 - b1) * g * g
            denom = np.sqrt(v) / np.sqrt(f(1 - b1 ** n)) + f(eps)
            w = w - f(lr / (1 - b0 ** n)) * m / denom
        else:
            b0, b1 = betas
            g = w * f(weight_decay) + g
            m = f(b0) * m + f(1 - b0) * g
            v = f(b1) * v + f(1 - b1) * g * g
            step = f(lr) * np.sqrt(f(1 - b1 ** n)) / f(1 - b0 ** n)
            w = w - m * step / (np.sqrt(v) + f(eps))
    return w.astype(f)


# --------------------------------------------------------------------------- pooling
def _pool_geometry(H, W, k, s, p, ceil_mode):
    """Output size rules of Pool.execute, python/jittor/pool.py:46-53."""
    if not ceil_mode:
        return (H + p[0] * 2 - k[0]) // s[0] + 1, (W + p[1] * 2 - k[1]) // s[1] + 1
    return (H + p[0] * 2 - k[0] + s[0] - 1) // s[0] + 1, (W + p[1] * 2 - k[1] + s[1] - 1) // s[1] + 1


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


def pool2d(x, kernel_size, op, stride=None, padding=0, ceil_mode=False, count_include_pad=True, return_indices=False):
    """Forward of Pool.execute (python/jittor/pool.py:42-95,187-197): the jt.code loops over the clipped window for
    maximum / minimum (always) and mean (ceil mode); mean in floor mode is reindex + reduce(mean), i.e. zero padding
    and a division by kh*kw."""
    x = np.asarray(x)
    k, s, p = _pair(kernel_size), _pair(stride if stride else kernel_size), _pair(padding)
    cip = bool(count_include_pad) and padding != 0
    N, C, H, W = x.shape
    h, w = _pool_geometry(H, W, k, s, p, ceil_mode)
    code_op = op in ("maximum", "minimum") or (op == "mean" and ceil_mode)
    y = np.empty((N, C, h, w), dtype=x.dtype)
    idx = np.full((N, C, h, w), -1, dtype=np.int32)
    acc_t = np.float64 if x.dtype == np.float64 else np.float32
    for i2 in range(h):
        for i3 in range(w):
            k2, k3 = i2 * s[0] - p[0], i3 * s[1] - p[1]
            k2_, k3_ = min(k2 + k[0], H), min(k3 + k[1], W)
            k2, k3 = max(0, k2), max(0, k3)
            win = x[:, :, k2:k2_, k3:k3_].reshape(N, C, -1)
            if op == "mean":
                count = k[0] * k[1] if (cip or not code_op) else (k2_ - k2) * (k3_ - k3)
                with np.errstate(divide="ignore", invalid="ignore"):
                    y[:, :, i2, i3] = (win.astype(acc_t).sum(-1) / acc_t(count)).astype(x.dtype)
            elif win.shape[-1] == 0:
                y[:, :, i2, i3] = _init_value(op, x.dtype)
            else:
                y[:, :, i2, i3] = win.max(-1) if op == "maximum" else win.min(-1)
                if return_indices:
                    a = win.argmax(-1)                       # first largest element (:70-79 uses a strict `<`)
                    ww = k3_ - k3
                    idx[:, :, i2, i3] = (k2 + a // ww) * W + (k3 + a % ww)
    return (y, idx) if return_indices else y


def pool2d_backward(x, dy, kernel_size, op, stride=None, padding=0, ceil_mode=False, count_include_pad=True):
    """Gradient of pool2d w.r.t. x. Code-op route (python/jittor/pool.py:96-118): per window, the first element (row
    major) equal to the pooled value receives dy (maximum / minimum), or every element receives dy/count (mean). The
    floor-mode mean is the meta-op route, whose gradient is dy/(kh*kw) on every in-range window element."""
    x, dy = np.asarray(x), np.asarray(dy)
    k, s, p = _pair(kernel_size), _pair(stride if stride else kernel_size), _pair(padding)
    cip = bool(count_include_pad) and padding != 0
    N, C, H, W = x.shape
    h, w = _pool_geometry(H, W, k, s, p, ceil_mode)
    code_op = op in ("maximum", "minimum") or (op == "mean" and ceil_mode)
    y = pool2d(x, kernel_size, op, stride, padding, ceil_mode, count_include_pad)
    dx = np.zeros(x.shape, dtype=np.float64)
    for i2 in range(h):
        for i3 in range(w):
            k2, k3 = i2 * s[0] - p[0], i3 * s[1] - p[1]
            k2_, k3_ = min(k2 + k[0], H), min(k3 + k[1], W)
            k2, k3 = max(0, k2), max(0, k3)
            if k2_ <= k2 or k3_ <= k3:
                continue
            d = dy[:, :, i2, i3].astype(np.float64)
            if op == "mean":
                count = k[0] * k[1] if (cip or not code_op) else (k2_ - k2) * (k3_ - k3)
                dx[:, :, k2:k2_, k3:k3_] += (d / count)[:, :, None, None]
            else:
                win = x[:, :, k2:k2_, k3:k3_].reshape(N, C, -1)
                hit = win == y[:, :, i2, i3][:, :, None]
                first = hit.argmax(-1)
                has = hit.any(-1)
                ww = k3_ - k3
                n_i, c_i = np.nonzero(has)
                np.add.at(dx, (n_i, c_i, k2 + first[n_i, c_i] // ww, k3 + first[n_i, c_i] % ww), d[n_i, c_i])
    return dx.astype(x.dtype)


# --------------------------------------------------------------------------- grouped / transposed convolution
def conv2d_grouped(x, w, stride=1, padding=0, dilation=1, groups=1, bias=None):
    """Conv.execute with groups > 1, python/jittor/nn.py:1022-1051, composed from this file's meta-ops exactly as
    the reference composes its own: two reindex to [N,G,oc/G,C/G,oh,ow,Kh,Kw], multiply, reindex_reduce('add')."""
    x, w = np.asarray(x), np.asarray(w)
    s, p, d = _pair(stride), _pair(padding), _pair(dilation)
    N, C, H, W = x.shape
    oc, _, Kh, Kw = w.shape
    G, CpG, ocg = groups, C // groups, oc // groups
    oh = (H + p[0] * 2 - Kh * d[0] + d[0] - 1) // s[0] + 1
    ow = (W + p[1] * 2 - Kw * d[1] + d[1] - 1) // s[1] + 1
    shape = [N, G, ocg, CpG, oh, ow, Kh, Kw]
    xx = reindex(x, shape, ["i0", f"i1*{CpG}+i3", f"i4*{s[0]}-{p[0]}+i6*{d[0]}", f"i5*{s[1]}-{p[1]}+i7*{d[1]}"])
    ww = reindex(w, shape, [f"i1*{ocg}+i2", "i3", "i6", "i7"])
    y = reindex_reduce(binary(xx, ww, "multiply"), "add", [N, oc, oh, ow], ["i0", f"i1*{ocg}+i2", "i4", "i5"])
    if bias is not None:
        y = binary(y, broadcast(np.asarray(bias), y.shape, [0, 2, 3]), "add")
    return y


def conv_transpose2d(x, w, stride=1, padding=0, output_padding=0, groups=1, dilation=1, bias=None):
    """ConvTranspose.execute, python/jittor/nn.py:1429-1491: y[n, g*oc_g+o, hi*s-p+kh*d, wi*s-p+kw*d] += x[n, g*ic_g+i,
    hi, wi] * w[g*ic_g+i, o, kh, kw]. (The reference's groups > 1 branch mixes up the per-group channel counts and is
    only meaningful for in_channels == out_channels, where it computes exactly this.)"""
    x, w = np.asarray(x), np.asarray(w)
    s, p, d, op_ = _pair(stride), _pair(padding), _pair(dilation), _pair(output_padding)
    N, C, H, W = x.shape
    _, o, Kh, Kw = w.shape
    G, icg = groups, C // groups
    h_out = (H - 1) * s[0] + op_[0] - 2 * p[0] + 1 + (Kh - 1) * d[0]
    w_out = (W - 1) * s[1] + op_[1] - 2 * p[1] + 1 + (Kw - 1) * d[1]
    y = np.zeros((N, o * G, h_out, w_out), dtype=np.float64)
    for g in range(G):
        xg = x[:, g * icg:(g + 1) * icg].astype(np.float64)
        wg = w[g * icg:(g + 1) * icg].astype(np.float64)
        for kh in range(Kh):
            for kw in range(Kw):
                contrib = np.einsum("nihw,io->nohw", xg, wg[:, :, kh, kw])
                for hi in range(H):
                    ho = hi * s[0] - p[0] + kh * d[0]
                    if not 0 <= ho < h_out:
                        continue
                    wo = np.arange(W) * s[1] - p[1] + kw * d[1]
                    ok = (wo >= 0) & (wo < w_out)
                    y[:, g * o:(g + 1) * o, ho, wo[ok]] += contrib[:, :, hi, ok]
    y = y.astype(x.dtype)
    if bias is not None:
        y = binary(y, broadcast(np.asarray(bias), y.shape, [0, 2, 3]), "add")
    return y


def conv_grad(x, w, dy, stride, padding, dilation, want_dw):
    """Gradient of sum(conv2d(x, w) * dy) w.r.t. x or w, composed from this file's meta-ops with the reference's rules:
    reduce.add <-> broadcast (python/jittor/src/ops/reduce_op.cc:339-343, broadcast_to_op.cc:112-117) and
    reindex <-> reindex_reduce.add (reindex_op.cc:76-80) applied to the lowering of python/jittor/nn.py:1009-1017."""
    x, w, dy = np.asarray(x), np.asarray(w), np.asarray(dy)
    n, c, h, wd = x.shape
    co, _, kh, kw = w.shape
    s, p, d = stride, padding, dilation
    oh, ow = dy.shape[2], dy.shape[3]
    shape7 = [n, co, c, oh, ow, kh, kw]
    idx = ["i0", "i2", f"i3*{s}-{p}+i5*{d}", f"i4*{s}-{p}+i6*{d}"]
    dm = broadcast(dy, shape7, [2, 5, 6])
    if want_dw:
        xx = reindex(x, shape7, idx)
        return reduce(binary(xx, dm, "multiply"), "add", [0, 3, 4])
    ww = broadcast(w, shape7, [0, 3, 4])
    return reindex_reduce(binary(ww, dm, "multiply"), "add", list(x.shape), idx)


def adaptive_pool2d(x, output_size, op):
    """AdaptiveAvgPool2d / AdaptiveMaxPool2d.execute, python/jittor/pool.py:405-466, from this file's reindex + reduce."""
    x = np.asarray(x)
    N, C, H, W = x.shape
    if isinstance(output_size, int):
        oh = ow = output_size
    else:
        oh = H if output_size[0] is None else output_size[0]
        ow = W if output_size[1] is None else output_size[1]
    if oh == 1 and ow == 1:
        return reduce(x, op, [2, 3], True)
    sh, sw = H // oh, W // ow
    ksh, ksw = H - (oh - 1) * sh, W - (ow - 1) * sw
    h, w = (H - ksh) // sh + 1, (W - ksw) // sw + 1
    xx = reindex(x, [N, C, h, w, ksh, ksw], ["i0", "i1", f"i2*{sh}+i4", f"i3*{sw}+i5"])
    return reduce(xx, op, [4, 5])


def conv1d(x, w, stride=1, padding=0, dilation=1, groups=1, bias=None):
    """Conv1d.execute, python/jittor/nn.py:1097-1125: a 2-D convolution with a trailing axis of extent 1."""
    x, w = np.asarray(x), np.asarray(w)
    x4, w4 = x[..., None], w[..., None]
    s, p, d = (stride, 1), (padding, 0), (dilation, 1)
    if groups == 1:
        N, C, L, _ = x4.shape
        O, _, K, _ = w4.shape
        oh = (L + p[0] * 2 - K * d[0] + d[0] - 1) // s[0] + 1
        shape7 = [N, O, C, oh, 1, K, 1]
        xx = reindex(x4, shape7, ["i0", "i2", f"i3*{s[0]}-{p[0]}+i5*{d[0]}", "i4*1-0+i6*1"])
        ww = broadcast(w4, shape7, [0, 3, 4])
        y = reduce(binary(xx, ww, "multiply"), "add", [2, 5, 6])
        if bias is not None:
            y = binary(y, broadcast(np.asarray(bias), y.shape, [0, 2, 3]), "add")
    else:
        y = conv2d_grouped(x4, w4, s, p, d, groups, bias)
    return y[..., 0]
