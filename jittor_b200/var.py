"""`Var` and the lazy op graph: the Python-facing surface of the reference's meta-operators
(`Var.reindex / reindex_var / reindex_reduce / broadcast / broadcast_var / reduce / sum / ...`,
python/jittor/src/var_holder.h:37-392 and the op headers under python/jittor/src/ops).

Every call records a node with inferred shape and dtype and computes nothing; `sync()`, `.data`,
`.numpy()` hand the graph to the executor (executor.py), which recognises the chains the reference
fuses (conv, matmul, softmax, LayerNorm, BatchNorm) and launches the CUDA kernels through the C ABI.
"""
import numbers

import numpy as np
import torch

from . import dtypes as dt
from ._capi import TORCH_DTYPES, DTYPE_NAMES, B200Error, require_cuda
from .flags import flags

MAX_DIMS = 10


class Shape(list):
    """List of ints that also equals tuples (the reference's NanoVector compares with both)."""

    def __eq__(self, other):
        return list(self) == list(other) if isinstance(other, (list, tuple)) else NotImplemented

    def __ne__(self, other):
        r = self.__eq__(other)
        return r if r is NotImplemented else not r

    __hash__ = None


class Op:
    __slots__ = ("kind", "inputs", "attrs")

    def __init__(self, kind, inputs, **attrs):
        self.kind = kind
        self.inputs = list(inputs)
        self.attrs = attrs


def _check_shape(shape):
    shape = [int(s) for s in shape]
    if len(shape) > MAX_DIMS:
        raise ValueError(f"at most {MAX_DIMS} dims are supported, got {len(shape)}")
    return shape


class Var:
    __array_priority__ = 100

    def __init__(self, shape, dtype, op=None, data=None, is_scalar=False):
        self._shape = shape if type(shape) is Shape else Shape(_check_shape(shape))
        self._dtype = dtype if type(dtype) is dt.DType else dt.canon(dtype)
        self._op = op
        self._data = data            # contiguous torch tensor on the CUDA device once computed
        self.is_scalar = is_scalar
        self._name = None
        self._const = None           # the Python number this Var was made from, if any
        self._pending = None         # handle of a collective still in flight on another stream
        self.compile_options = {}

    # ---- metadata -----------------------------------------------------------------------------
    @property
    def shape(self):
        return self._shape

    @property
    def dtype(self):
        return self._dtype

    @property
    def ndim(self):
        return len(self._shape)

    def numel(self):
        n = 1
        for s in self._shape:
            n *= s
        return n

    size = property(lambda self: self._shape)

    def name(self, n=None):
        if n is None:
            return self._name
        self._name = n
        return self

    def stop_grad(self):
        self._stop_grad = True
        return self

    def start_grad(self):
        self._stop_grad = False
        return self

    def is_stop_grad(self):
        return getattr(self, "_stop_grad", False)

    def stop_fuse(self):
        """This Var is computed on its own and stored: no fused chain reaches through it
        (python/jittor/src/var_holder.h `stop_fuse`, python/jittor/test/test_stop_fuse.py)."""
        self._stop_fuse = True
        return self

    def is_stop_fuse(self):
        return getattr(self, "_stop_fuse", False)

    def __len__(self):
        return self._shape[0]

    def __repr__(self):
        state = "" if self._data is not None else ", lazy"
        return f"jt.Var(shape={list(self._shape)}, dtype={self._dtype}{state})"

    # ---- execution ----------------------------------------------------------------------------
    def sync(self, device_sync=False, weak_sync=True):
        from . import executor
        executor.realize([self])
        if device_sync:
            torch.cuda.current_stream().synchronize()
        return self

    def wait(self):
        """Makes the current stream wait for a collective that produced this Var (no host blocking)."""
        if self._pending is not None:
            self._pending.wait()
            self._pending = None
        return self

    def torch(self):
        """The computed value as a torch CUDA tensor (no copy)."""
        self.sync()
        self.wait()
        return self._data.view(list(self._shape))

    @property
    def data(self):
        return self.numpy()

    def numpy(self):
        t = self.torch()
        if t.dtype == torch.bfloat16:
            return t.float().cpu().numpy()
        return t.cpu().numpy()

    def fetch_sync(self):
        return self.numpy()

    def fetch_into(self, host, non_blocking=True, stream=None):
        """Copies the value into a preallocated host torch tensor (pinned memory makes the copy a DMA that
        can overlap later launches). With `stream`, the copy is queued on that stream after the producing work,
        so that it overlaps the next host->device copy (PCIe is full duplex); synchronise the stream that carried
        the copy before reading `host`."""
        src = self.torch().reshape(-1)
        if stream is None:
            host.view(-1).copy_(src, non_blocking=non_blocking)
            return host
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            host.view(-1).copy_(src, non_blocking=non_blocking)
        src.record_stream(stream)
        return host

    def item(self):
        if self.numel() != 1:
            raise ValueError("item() needs a Var with exactly one element")
        return self.numpy().reshape(-1)[0].item()

    def assign(self, other):
        other = to_var(other)
        other.sync()
        self._shape, self._dtype, self._data, self._op = other._shape, other._dtype, other._data, None
        return self

    update = assign

    # ---- the four meta-operators -----------------------------------------------------------------
    def reindex(self, *args, **kw):
        return reindex(self, *args, **kw)

    def reindex_var(self, indexes, overflow_value=0, overflow_conditions=()):
        return reindex_var(self, indexes, overflow_value, overflow_conditions)

    def reindex_reduce(self, op, shape, indexes, overflow_conditions=(), extras=()):
        return reindex_reduce(self, op, shape, indexes, overflow_conditions, extras)

    def broadcast(self, shape, dims=()):
        return broadcast(self, shape, dims)

    def broadcast_var(self, y, dims=()):
        return broadcast(self, y, dims)

    def reduce(self, op, dim=(), keepdims=False, dims=None):
        return reduce(self, op, dims if dims is not None else dim, keepdims)

    def sum(self, dim=(), keepdims=False, dims=None):
        return reduce(self, "add", dims if dims is not None else dim, keepdims)

    def prod(self, dim=(), keepdims=False, dims=None):
        return reduce(self, "multiply", dims if dims is not None else dim, keepdims)

    product = prod

    def max(self, dim=(), keepdims=False, dims=None):
        return reduce(self, "maximum", dims if dims is not None else dim, keepdims)

    def min(self, dim=(), keepdims=False, dims=None):
        return reduce(self, "minimum", dims if dims is not None else dim, keepdims)

    def mean(self, dim=(), keepdims=False, dims=None):
        return reduce(self, "mean", dims if dims is not None else dim, keepdims)

    def all_(self, dim=(), keepdims=False, dims=None):
        return reduce(self, "logical_and", dims if dims is not None else dim, keepdims)

    def any_(self, dim=(), keepdims=False, dims=None):
        return reduce(self, "logical_or", dims if dims is not None else dim, keepdims)

    all = all_
    any = any_

    # ---- element-wise -------------------------------------------------------------------------
    def binary(self, other, op):
        return binary(self, other, op)

    def unary(self, op):
        return unary(self, op)

    def cast(self, dtype):
        return unary(self, dt.canon(dtype))

    astype = cast

    def float(self):
        return self.float32()

    def int(self):
        return self.int32()

    def double(self):
        return self.float64()

    def half(self):
        return self.float16()

    def _to_float(self):
        return self if self.dtype == "float64" else self.float32()

    def maximum(self, o):
        return binary(self, o, "maximum")

    def minimum(self, o):
        return binary(self, o, "minimum")

    def ternary(self, x, y):
        return ternary(self, x, y)

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (list, tuple, Shape)):
            shape = shape[0]
        return reshape(self, shape)

    view = reshape

    def transpose(self, *perm):
        if len(perm) == 1 and isinstance(perm[0], (list, tuple)):
            perm = perm[0]
        return transpose(self, perm)

    permute = transpose

    def mpi_broadcast(self, root=0):
        from . import dist
        return dist.mpi_broadcast(self, root)

    def mpi_all_reduce(self, op="add"):
        from . import dist
        return dist.mpi_all_reduce(self, op)

    def mpi_reduce(self, op="add", root=0):
        from . import dist
        return dist.mpi_reduce(self, op, root)

    def matmul(self, other):
        from . import nn
        return nn.matmul(self, other)

    __matmul__ = matmul

    def softmax(self, dim=None, log=False):
        from . import nn
        return nn.softmax(self, dim, log)

    def log_softmax(self, dim=None):
        from . import nn
        return nn.softmax(self, dim, True)

    def __bool__(self):
        return bool(self.item())


def _install_operators():
    table = {"add": "add", "sub": "subtract", "mul": "multiply", "truediv": "divide", "floordiv": "floor_divide",
             "mod": "mod", "pow": "pow", "lt": "less", "le": "less_equal", "gt": "greater", "ge": "greater_equal",
             "eq": "equal", "ne": "not_equal", "and": "bitwise_and", "or": "bitwise_or", "xor": "bitwise_xor",
             "lshift": "left_shift", "rshift": "right_shift"}
    for py, op in table.items():
        setattr(Var, f"__{py}__", (lambda op: lambda a, b: binary(a, b, op))(op))
        if py not in ("lt", "le", "gt", "ge", "eq", "ne"):
            setattr(Var, f"__r{py}__", (lambda op: lambda a, b: binary(b, a, op))(op))
    Var.__hash__ = lambda self: id(self)
    Var.__neg__ = lambda a: unary(a, "negative")
    Var.__abs__ = lambda a: unary(a, "abs")
    Var.__invert__ = lambda a: unary(a, "bitwise_not")
    for op in dt.BINARY_OPS - {"mean"}:
        if not hasattr(Var, op):
            setattr(Var, op, (lambda op: lambda a, b: binary(a, b, op))(op))
    for op in dt.UNARY_OPS - {"cast"}:
        if not hasattr(Var, op):
            setattr(Var, op, (lambda op: lambda a: unary(a, op))(op))
    for name in dt.DTYPES:
        setattr(Var, name, (lambda name: lambda a: unary(a, name))(name))
    for op in dt.REDUCE_OPS:
        setattr(Var, f"reduce_{op}", (lambda op: lambda a, dim=(), keepdims=False, dims=None:
                                      reduce(a, op, dims if dims is not None else dim, keepdims))(op))


# ------------------------------------------------------------------------------------ constructors
def array(data, dtype=None):
    """jt.array: numpy array / list / scalar / torch tensor -> Var resident on the CUDA device."""
    if isinstance(data, Var):
        return data if dtype is None or dt.canon(dtype) == data.dtype else data.cast(dtype)
    is_scalar = isinstance(data, numbers.Number)
    if is_scalar:
        # Python numbers: bool -> bool, int -> int32, float -> float32; materialised lazily
        name = dtype if dtype is not None else ("bool" if isinstance(data, bool) else
                                                "int32" if isinstance(data, numbers.Integral) else "float32")
        v = Var([1], name, Op("fill", [], value=data), is_scalar=True)
        v._const = data
        return v
    require_cuda()
    if isinstance(data, torch.Tensor):
        t = data
        if dtype is not None:
            t = t.to(TORCH_DTYPES[dt.canon(dtype)])
    else:
        a = np.asarray(data)
        if dtype is not None:
            a = a.astype(np.dtype(str(dt.canon(dtype))))
        elif a.dtype == np.float64 and not isinstance(data, np.ndarray):
            a = a.astype(np.float32)       # Python floats are float32 in the reference
        elif a.dtype == np.int64 and not isinstance(data, np.ndarray):
            a = a.astype(np.int32)
        t = torch.from_numpy(np.ascontiguousarray(a))
    if t.dtype not in DTYPE_NAMES:
        raise ValueError(f"unsupported dtype {t.dtype}")
    t = t.to("cuda", non_blocking=False).contiguous()
    shape = list(t.shape) if t.dim() else [1]
    return Var(shape, DTYPE_NAMES[t.dtype], data=t.reshape(shape))


def to_var(x):
    return x if isinstance(x, Var) else array(x)


def full(shape, value, dtype="float32"):
    """Constant-filled Var; the buffer is created when first needed."""
    return Var(_check_shape(shape), dtype, Op("fill", [], value=value))


def empty(shape, dtype="float32"):
    return full(shape, 0, dtype)


def zeros(shape, dtype="float32"):
    return full(shape, 0, dtype)


def ones(shape, dtype="float32"):
    return full(shape, 1, dtype)


# ------------------------------------------------------------------------------------ meta-operators
def _norm_list(v):
    if isinstance(v, (str, bytes)):
        raise TypeError("expected a list of strings")
    return list(v)


def reindex(x, *args, **kw):
    """x.reindex(shape, indexes, overflow_value=0, overflow_conditions=[], extras=[])  or
    x.reindex(indexes: list[Var], overflow_value=0, overflow_conditions=[])
    (python/jittor/src/ops/reindex_op.h:91,96)."""
    x = to_var(x)
    if args and len(args[0]) and isinstance(args[0][0], Var):
        return reindex_var(x, *args, **kw)
    names = ["shape", "indexes", "overflow_value", "overflow_conditions", "extras"]
    a = dict(zip(names, args))
    a.update(kw)
    shape = _check_shape(a.get("shape", []))
    indexes = _norm_list(a["indexes"])
    extras = [to_var(e) for e in a.get("extras", ())]
    if len(indexes) != x.ndim:
        raise ValueError("Number of x's shape and indexes should be the same.")
    if not shape:
        if not extras:
            raise ValueError("Number of shape should greater than 0.")
        shape = list(extras[0].shape)
    op = Op("reindex", [x] + extras, shape=shape, indexes=[str(s) for s in indexes],
            overflow_value=float(a.get("overflow_value", 0)),
            overflow_conditions=[str(s) for s in a.get("overflow_conditions", ())])
    return Var(shape, x.dtype, op)


def reindex_var(x, indexes, overflow_value=0, overflow_conditions=()):
    """Index d is the Var indexes[d] read at the output coordinate (reindex_op.cc:35-70)."""
    x = to_var(x)
    indexes = [to_var(i) for i in indexes]
    if len(indexes) != x.ndim:
        raise ValueError("Number of indexes should equal x's number of dims")
    shape = list(indexes[0].shape)
    for i in indexes:
        if list(i.shape) != shape:
            raise ValueError("all index Vars must have the same shape")
    args = ",".join(f"i{d}" for d in range(len(shape)))
    return reindex(x, shape, [f"@e{d}({args})" for d in range(len(indexes))], overflow_value,
                   overflow_conditions, indexes)


_RR_OPS = {"add", "multiply", "maximum", "minimum", "bitwise_and", "bitwise_or", "bitwise_xor",
           "logical_and", "logical_or", "logical_xor", "void"}


def reindex_reduce(y, op, shape, indexes, overflow_conditions=(), extras=()):
    """python/jittor/src/ops/reindex_reduce_op.h:86; checks of reindex_reduce_op.cc:34,65-73."""
    y = to_var(y)
    shape = [int(s) for s in shape]
    indexes = _norm_list(indexes)
    if op not in _RR_OPS:
        raise ValueError(f"reindex_reduce: unsupported op {op!r}")
    if len(shape) != len(indexes):
        raise ValueError("Number of shape and indexes should be the same.")
    if not shape:
        raise ValueError("Number of shape should greater than 0.")
    if any(s < 0 for s in shape):
        raise ValueError("Shape should greater than 0.")
    extras = [to_var(e) for e in extras]
    node = Op("reindex_reduce", [y] + extras, op=op, shape=_check_shape(shape), indexes=[str(s) for s in indexes],
              overflow_conditions=[str(s) for s in overflow_conditions])
    return Var(shape, y.dtype, node)


def bcast_masks(xshape, yshape, dims):
    """Shape / mask inference of BroadcastToOp (python/jittor/src/ops/broadcast_to_op.cc:74-96,119-168)."""
    count = len(dims)
    xdim, ydim = len(xshape), len(yshape)
    zdim = max(xdim, ydim - count) + count
    mask = 0
    for d in dims:
        d = int(d)
        if d < 0:
            d += zdim
        if not 0 <= d < zdim:
            raise ValueError(f"Wrong dims number: {list(dims)}")
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
                raise ValueError(f"Shape not match {list(xshape)} {list(yshape)} {mask}")
            z[i] = xs
        xi -= 1
        yi -= 1
    return z, mask, keep


def _need_broadcast(xshape, shape):
    if len(xshape) < len(shape):
        return True
    for i in range(1, len(shape) + 1):
        if xshape[-i] != shape[-i] and shape[-i] != 1:
            return True
    return False


def broadcast(x, shape, dims=()):
    """jt.broadcast(x, shape | y, dims=[]) (python/jittor/src/ops/broadcast_to_op.h:46,86)."""
    x = to_var(x)
    if isinstance(shape, Var):
        shape = shape.shape
    shape = [int(s) for s in shape]
    dims = [int(d) for d in dims]
    if not dims and not _need_broadcast(x.shape, shape):
        return x
    if not shape:
        raise ValueError("Number of shape should greater than 0.")
    if any(s < 0 for s in shape):
        raise ValueError("Shape should greater than 0.")
    z, mask, keep = bcast_masks(list(x.shape), shape, dims)
    return Var(z, x.dtype, Op("broadcast_to", [x], bcast_mask=mask, keepdims_mask=keep))


broadcast_var = broadcast


def reduce(x, op, dims=(), keepdims=False):
    """jt.reduce(x, op, dim | dims, keepdims) (python/jittor/src/ops/reduce_op.cc:257-337)."""
    x = to_var(x)
    if op not in dt.REDUCE_OPS:
        raise ValueError(f"unknown reduce op {op!r}")
    if isinstance(dims, numbers.Integral):
        dims = (int(dims),)
    if dims is None:
        dims = ()
    # half inputs are summed in float32 unless amp_reg bit 32 is set (reduce_op.cc:260-266)
    if not (flags.amp_reg & dt.AMP_NO_REDUCE_UPCAST) and x.dtype in ("float16", "bfloat16") and op in ("mean", "add"):
        return reduce(x.float32(), op, dims, keepdims).cast(x.dtype)
    nd = x.ndim
    if len(dims) == 0:
        mask = (1 << nd) - 1
    else:
        mask = 0
        for d in dims:
            d = int(d)
            if d < 0:
                d += nd
            if not 0 <= d < nd:
                raise ValueError(f"Wrong dims number: {list(dims)}")
            mask |= 1 << d
    keep_mask = (1 << nd) - 1 if keepdims else 0
    yshape = []
    for i in range(nd):
        if mask >> i & 1:
            if keep_mask >> i & 1:
                yshape.append(1)
        else:
            yshape.append(x.shape[i])
    if not yshape:
        yshape = [1]
    ydt = dt.reduce_dtype_infer(op, x.dtype)
    return Var(yshape, ydt, Op("reduce", [x], op=op, reduce_mask=mask, keepdims_mask=keep_mask))


class LazyVar(Var):
    """A Var whose producer graph is written down only when something reads `_op`. A caller that hands the executor a relay
    record with the result (nn.conv2d) can be planned and run without the graph; jt.grad, the fuser and the pattern
    matchers of consumers read `_op` and find the same meta-operator graph the eager construction would have made."""

    def __init__(self, shape, dtype, builder):
        Var.__init__(self, shape, dtype, None)
        del self.__dict__["_op"]
        self.__dict__["_op_builder"] = builder

    def __getattr__(self, name):               # only reached for attributes the instance does not have
        if name == "_op":
            builder = self.__dict__.pop("_op_builder", None)
            op = builder() if builder is not None else None
            self.__dict__["_op"] = op
            return op
        raise AttributeError(name)


# ------------------------------------------------------------------------------------ element-wise
def _bshape(a, b):
    """Result shape of a binary op on shapes a, b: right-aligned, size-1 axes stretch
    (python/jittor/src/ops/binary_op.cc:421-441)."""
    n = max(len(a), len(b))
    pa, pb = [1] * (n - len(a)) + list(a), [1] * (n - len(b)) + list(b)
    z = []
    for x, y in zip(pa, pb):
        if x == y or y == 1:
            z.append(x)
        elif x == 1:
            z.append(y)
        else:
            raise ValueError(f"Shape not match, x:{list(a)} y:{list(b)}")
    return z


def binary(x, y, op):
    if op not in dt.BINARY_OPS or op == "mean":
        raise ValueError(f"unknown binary op {op!r}")
    x, y = to_var(x), to_var(y)
    z = _bshape(x.shape, y.shape)
    zdt = dt.binary_dtype_infer(op, x.dtype, y.dtype, x.is_scalar, y.is_scalar)
    return Var(z, zdt, Op("binary", [x, y], op=op))


def unary(x, op):
    x = to_var(x)
    op = str(op)
    if op not in dt.UNARY_OPS and op not in dt.DTYPES:
        raise ValueError(f"unknown unary op {op!r}")
    ydt = dt.unary_dtype_infer(op, x.dtype)
    if op in dt.DTYPES and ydt == x.dtype:
        return x
    return Var(x.shape, ydt, Op("unary", [x], op=op), is_scalar=x.is_scalar)


def ternary(cond, x, y):
    cond, x, y = to_var(cond), to_var(x), to_var(y)
    z = _bshape(_bshape(cond.shape, x.shape), y.shape)
    zdt = dt.binary_dtype_infer("add", x.dtype, y.dtype, x.is_scalar, y.is_scalar)
    return Var(z, zdt, Op("ternary", [cond, x, y]))


ternary_out_hint = ternary


def reshape(x, shape):
    x = to_var(x)
    shape = [int(s) for s in shape]
    n = x.numel()
    if shape.count(-1) > 1:
        raise ValueError("only one -1 allowed in reshape")
    if -1 in shape:
        known = 1
        for s in shape:
            if s != -1:
                known *= s
        shape[shape.index(-1)] = n // known if known else 0
    m = 1
    for s in shape:
        m *= s
    if m != n:
        raise ValueError(f"cannot reshape {list(x.shape)} to {shape}")
    if not shape:
        shape = [1]
    if shape == list(x.shape):
        return x
    return Var(shape, x.dtype, Op("reshape", [x]))


def transpose(x, perm=()):
    """Axis permutation expressed as a reindex (the meta-operator form of transpose)."""
    x = to_var(x)
    perm = [int(p) % x.ndim for p in perm] if len(perm) else list(range(x.ndim))[::-1]
    inv = [0] * x.ndim
    for o, p in enumerate(perm):
        inv[p] = o
    return reindex(x, [x.shape[p] for p in perm], [f"i{inv[d]}" for d in range(x.ndim)])


def index(shape, dim, dtype="int32"):
    """jt.index(shape, dim): the coordinate along `dim` at every position (python/jittor/src/ops/index_op.h)."""
    shape = _check_shape(shape)
    one = array(np.arange(shape[dim], dtype=np.dtype(str(dt.canon(dtype)))))
    return reindex(one, shape, [f"i{dim}"])


_install_operators()
