"""General element-wise chain fusion: the part of the reference's fuser that is not a named pattern.

The reference groups any run of element-wise ops, broadcasts and reduces into one FusedOp and generates one loop nest
for it (python/jittor/src/executor.cc:276-534, python/jittor/src/fused_op.cc:41-118, python/jittor/src/op_compiler.cc:839-1045).
Here the executor asks `match(v)` for every Var no named pattern (conv, matmul, softmax, ...) claimed: starting at v it
collects the maximal region of fusable nodes, writes it as the postfix program of `b200jt_fused_chain` (statements that
reduce a row, compute per-row values, and store) and runs it as ONE launch. Nothing inside the region is materialised.

What can be fused (everything else is a leaf = an input of the chain, computed first):
  * unary / binary / ternary ops whose arithmetic the element-wise kernels do in the float32 class, with results of dtype
    float32 / bfloat16 / float16 / bool;
  * broadcast_to of a leaf (the leaf becomes a broadcast input) or of a per-row value;
  * reduce add / mean / maximum / minimum / multiply over the trailing axes of the region's full shape;
  * constants (`fill`).
"""
import ctypes
import struct

from . import _capi as C
from .var import Var

MAX_INPUTS, MAX_CODE, MAX_ROWVALS, MAX_TMP = 8, 160, 8, 6

# word = op | sub << 4 | operand kind << 10 | operand index << 13 | swap << 21 | result dtype << 24
CH_OPERAND, CH_LOAD, CH_UNARY, CH_BINARY, CH_SELECT, CH_TSTORE = 0, 1, 2, 3, 4, 5
CH_ROW_REDUCE, CH_ROW_MAP, CH_STORE, CH_STORE_ROW = 8, 9, 10, 11
K_NONE, K_INPUT, K_CONST, K_ROWVAL, K_TMP = 0, 1, 2, 3, 4

UNARY_CODES = {n: i for i, n in enumerate(
    ["cast", "negative", "abs", "logical_not", "bitwise_not", "log", "exp", "sqrt", "round", "floor", "ceil", "sin", "asin",
     "sinh", "asinh", "tan", "atan", "tanh", "atanh", "cos", "acos", "cosh", "acosh", "sigmoid", "erf", "erfinv"])}
del UNARY_CODES["bitwise_not"]                 # integer only
BINARY_CODES = {n: i for i, n in enumerate(
    ["add", "subtract", "multiply", "divide", "floor_divide", "mod", "pow", "maximum", "minimum", "less", "less_equal",
     "greater", "greater_equal", "equal", "not_equal", "logical_and", "logical_or", "logical_xor"])}
REDUCE_CODES = {"add": 0, "multiply": 2, "maximum": 7, "minimum": 8, "mean": 23}

_FLOAT = ("float32", "bfloat16", "float16")
_VALUE_DTYPES = _FLOAT + ("bool",)
_LEAF_DTYPES = _FLOAT + ("bool", "int8", "int16", "int32", "uint8")


class _Unfusable(Exception):
    pass


def _word(op, sub=0, operand=(K_NONE, 0), swap=0, dtype="float32"):
    return op | (sub << 4) | (operand[0] << 10) | (operand[1] << 13) | (swap << 21) | (C.DTYPE_CODES[str(dtype)] << 24)


def _const_word(value):
    return struct.unpack("<i", struct.pack("<f", value))[0]


def decode(words):
    """[(op, sub, kind, index, swap, dtype code, constant or None)] -- for tests and debugging."""
    out, pc = [], 0
    while pc < len(words):
        w = words[pc]
        kind = (w >> 10) & 7
        const = None
        if kind == K_CONST:
            pc += 1
            const = struct.unpack("<f", struct.pack("<i", words[pc]))[0]
        out.append((w & 15, (w >> 4) & 63, kind, (w >> 13) & 255, (w >> 21) & 1, (w >> 24) & 255, const))
        pc += 1
    return out


def _is_node(v):
    return isinstance(v, Var) and v._data is None and v._op is not None


def _const_of(v):
    """The Python number behind a constant Var (a scalar made from a number, or a `fill`), else None."""
    if not _is_node(v) or v._op.kind != "fill":
        return None
    val = v._op.attrs["value"]
    if isinstance(val, bool):
        return 1.0 if val else 0.0
    f = float(val)
    if str(v.dtype) not in _FLOAT and str(v.dtype) != "bool" and abs(f) >= 1 << 24:
        return None
    return f


def _float_class_node(v):
    """True if the element-wise kernels would compute node v in the float32 class and its result is a dtype a fused chain
    can hold."""
    if not _is_node(v) or str(v.dtype) not in _VALUE_DTYPES:
        return False
    op, ins = v._op, v._op.inputs
    for i in ins:
        if str(i.dtype) in ("float64", "int64"):
            return False
    if op.kind == "binary":
        name = op.attrs["op"]
        if name not in BINARY_CODES:
            return False
        if str(v.dtype) == "bool":               # comparisons compute in the promoted class of the operands
            return any(str(i.dtype) in _FLOAT for i in ins)
        return str(v.dtype) in _FLOAT
    if op.kind == "unary":
        name = op.attrs["op"]
        if name in C.DTYPE_CODES:                # cast: result dtype checked above; the source must fit a float32 exactly enough
            return str(ins[0].dtype) in _LEAF_DTYPES
        if name not in UNARY_CODES:
            return False
        return str(v.dtype) in _FLOAT or str(ins[0].dtype) in _FLOAT
    if op.kind == "ternary":
        return str(v.dtype) in _FLOAT
    return False


class _Builder:
    """Walks the graph under `root` and writes the program. Shapes are handled as *views*: a node's shape written with
    the rank of the region's full shape (size 1 on the axes it does not have), which is what decides whether the node is
    a full-space value, a per-row value, or something the region cannot hold (a leaf)."""

    def __init__(self, root):
        self.root = root
        self.inputs = []              # (Var, view)
        self.input_ids = {}
        self.statements = []          # finished statements (lists of words)
        self.row_slots = {}           # (id(node), axes) -> slot
        self.n_ops = 0
        if _is_node(root) and root._op.kind == "reduce":
            x = root._op.inputs[0]
            self.full = list(x.shape)
            self.k = self._trailing(root._op.attrs["reduce_mask"], x.ndim) or 0
            if not self.k:
                raise _Unfusable
        else:
            self.full = list(root.shape)
            self.k = self._find_reduce_axes(root)
        self.d = len(self.full)
        self.rows = self.cols = 1
        for i, s in enumerate(self.full):
            if i < self.d - self.k:
                self.rows *= s
            else:
                self.cols *= s

    @staticmethod
    def _trailing(mask, nd):
        k = bin(mask).count("1")
        return k if k and mask == ((1 << k) - 1) << (nd - k) else None

    def _find_reduce_axes(self, root):
        """Number of trailing axes the region's reduces fold (0 if it has none): the first reduce over the full shape
        reachable through element-wise nodes decides."""
        seen, stack = set(), [root]
        while stack and len(seen) < 256:
            v = stack.pop()
            if id(v) in seen or not _is_node(v):
                continue
            seen.add(id(v))
            op = v._op
            if op.kind == "reduce":
                x = op.inputs[0]
                if list(x.shape) == self.full and op.attrs["op"] in REDUCE_CODES:
                    k = self._trailing(op.attrs["reduce_mask"], x.ndim)
                    if k is not None:
                        return k
            elif op.kind in ("binary", "unary", "ternary", "broadcast_to"):
                stack.extend(op.inputs)
        return 0

    # ---- views -----------------------------------------------------------------------------------
    def _view(self, shape, axes):
        """Shape `shape` (rank <= len(axes), right-aligned against a node whose axes sit at `axes`) in full rank."""
        shape = list(shape)
        if len(shape) > len(axes):
            if any(s != 1 for s in shape[:len(shape) - len(axes)]):
                raise _Unfusable
            shape = shape[len(shape) - len(axes):]
        view = [1] * self.d
        for s, a in zip(shape, axes[len(axes) - len(shape):]):
            view[a] = s
        return view

    def _klass(self, view):
        if view == self.full:
            return "full"
        if self.k and all(s == 1 for s in view[self.d - self.k:]):
            return "row"
        return None

    def _input(self, v, view, ctx):
        """Registers leaf v (seen through `view`) and returns its operand."""
        if str(v.dtype) not in _LEAF_DTYPES:
            raise _Unfusable
        for s, f in zip(view, self.full):
            if s != f and s != 1:
                raise _Unfusable
        if ctx == "row" and any(s != 1 for s in view[self.d - self.k:]):
            raise _Unfusable                    # a per-row statement cannot read something that varies along the row
        key = (id(v), tuple(view))
        if key not in self.input_ids:
            if len(self.inputs) >= MAX_INPUTS:
                raise _Unfusable
            self.input_ids[key] = len(self.inputs)
            self.inputs.append((v, view))
        return (K_INPUT, self.input_ids[key])

    # ---- expressions -----------------------------------------------------------------------------
    def _fusable(self, v, view):
        if not _is_node(v) or (v.is_stop_fuse() and v is not self.root):
            return False
        op = v._op
        if op.kind in ("binary", "unary", "ternary"):
            return _float_class_node(v) and self._klass(view) is not None
        if op.kind == "reduce":
            x = op.inputs[0]
            return (self.k > 0 and list(x.shape) == self.full and op.attrs["op"] in REDUCE_CODES
                    and self._trailing(op.attrs["reduce_mask"], x.ndim) == self.k and str(v.dtype) in _FLOAT
                    and str(x.dtype) in _FLOAT)
        if op.kind == "broadcast_to":
            return self._klass(view) is not None
        return False

    def _axes_of(self, v, axes):
        if v.ndim > len(axes):                  # leading axes of extent 1 (a [1] scalar stretched over every axis) carry nothing
            if any(s != 1 for s in v.shape[:v.ndim - len(axes)]):
                raise _Unfusable
            return axes
        return axes[len(axes) - v.ndim:]

    def _through_broadcasts(self, v, axes):
        """Follows broadcast_to nodes down to what they stretch: (node, axes of that node)."""
        while True:
            if _const_of(v) is not None:
                return v, axes
            axes = self._axes_of(v, axes)
            if not (_is_node(v) and v._op.kind == "broadcast_to" and self._fusable(v, self._view(v.shape, axes))):
                return v, axes
            mask, keep = v._op.attrs["bcast_mask"], v._op.attrs["keepdims_mask"]
            axes = [axes[i] for i in range(v.ndim) if not (mask >> i & 1) or (keep >> i & 1)]
            v = v._op.inputs[0]
            self.n_ops += 1

    def _simple(self, v, axes, ctx, chain):
        """The operand that names v's value without touching the accumulator (a constant, an input, a row value, a
        temporary holding a shared sub-expression), or None if v has to be computed."""
        v, axes = self._through_broadcasts(v, axes)
        c = _const_of(v)
        if c is not None:
            return (K_CONST, 0, c)
        key = (id(v), tuple(axes))
        if key in self.row_slots:
            return (K_ROWVAL, self.row_slots[key])
        if key in chain["memo"]:
            return (K_TMP, chain["memo"][key])
        view = self._view(v.shape, axes)
        if not self._fusable(v, view):
            return self._input(v, view, ctx)
        if v._op.kind == "reduce":
            return (K_ROWVAL, self._row_reduce(v, key))
        if self._klass(view) == "row" and ctx == "full":
            return (K_ROWVAL, self._row_map(v, axes, key))
        return None

    @staticmethod
    def _put(code, op, sub=0, operand=None, swap=0, dtype="float32"):
        if op == CH_LOAD and operand[0] == K_TMP and code and code[-1] == _word(CH_TSTORE, 0, (K_TMP, operand[1])):
            return                              # the accumulator still holds what was just parked there
        code.append(_word(op, sub, operand[:2] if operand else (K_NONE, 0), swap, dtype))
        if operand is not None and operand[0] == K_CONST:
            code.append(_const_word(operand[2]))
        if len(code) > MAX_CODE:
            raise _Unfusable

    def _tmp(self, chain):
        if not chain["free"]:
            raise _Unfusable
        return chain["free"].pop()

    def _gen(self, v, axes, code, ctx, chain):
        """Appends code that leaves the value of v in the accumulator."""
        opnd = self._simple(v, axes, ctx, chain)
        if opnd is not None:
            self._put(code, CH_LOAD, operand=opnd)
            return
        v, axes = self._through_broadcasts(v, axes)
        key = (id(v), tuple(axes))
        op = v._op
        if op.kind == "unary":
            name = op.attrs["op"]
            self._gen(op.inputs[0], axes, code, ctx, chain)
            self._put(code, CH_UNARY, UNARY_CODES["cast"] if name in C.DTYPE_CODES else UNARY_CODES[name], dtype=v.dtype)
        elif op.kind == "binary":
            x, y = op.inputs
            sub = BINARY_CODES[op.attrs["op"]]
            oy = self._simple(y, axes, ctx, chain)
            if oy is not None:
                self._gen(x, axes, code, ctx, chain)
                self._put(code, CH_BINARY, sub, oy, 0, v.dtype)
            else:
                ox = self._simple(x, axes, ctx, chain)
                if ox is not None:
                    self._gen(y, axes, code, ctx, chain)
                    self._put(code, CH_BINARY, sub, ox, 1, v.dtype)
                else:
                    self._gen(y, axes, code, ctx, chain)
                    oy, t = self._simple(y, axes, ctx, chain), None
                    if oy is None:
                        t = self._tmp(chain)
                        self._put(code, CH_TSTORE, operand=(K_TMP, t))
                        oy = (K_TMP, t)
                    self._gen(x, axes, code, ctx, chain)
                    self._put(code, CH_BINARY, sub, oy, 0, v.dtype)
                    if t is not None:
                        chain["free"].append(t)
        else:                                   # ternary: cond ? x : y
            c, x, y = op.inputs
            held = []
            ops = []
            for u in (x, y):
                o = self._simple(u, axes, ctx, chain)
                if o is None:
                    self._gen(u, axes, code, ctx, chain)
                    o = self._simple(u, axes, ctx, chain)       # a shared value has parked itself in a temporary
                    if o is None:
                        t = self._tmp(chain)
                        self._put(code, CH_TSTORE, operand=(K_TMP, t))
                        held.append(t)
                        o = (K_TMP, t)
                ops.append(o)
            self._gen(c, axes, code, ctx, chain)
            self._put(code, CH_SELECT, operand=ops[0], dtype=v.dtype)
            self._put(code, CH_OPERAND, operand=ops[1])
            chain["free"] += held
        self.n_ops += 1
        # a value other nodes of this chain use again is parked in a temporary (if one is left; else it is recomputed)
        if chain["uses"].get(key, 0) > 1 and len(chain["free"]) > 1:
            t = chain["free"].pop(0)
            self._put(code, CH_TSTORE, operand=(K_TMP, t))
            chain["memo"][key] = t

    def _count_uses(self, v, axes, uses, ctx, depth=0):
        """How often each computed node is referenced inside one chain (stops at leaves, row values, constants)."""
        if depth > 64 or _const_of(v) is not None:
            return
        try:
            v, axes = self._through_broadcasts(v, axes)
        except _Unfusable:
            return
        if _const_of(v) is not None:
            return
        key = (id(v), tuple(axes))
        view = self._view(v.shape, axes)
        if key in self.row_slots or not self._fusable(v, view) or v._op.kind == "reduce":
            return
        if self._klass(view) == "row" and ctx == "full":
            return
        uses[key] = uses.get(key, 0) + 1
        if uses[key] == 1:
            for i in v._op.inputs:
                self._count_uses(i, axes, uses, ctx, depth + 1)

    def _chain(self, v, axes, ctx):
        n_ops = self.n_ops
        uses = {}
        self._count_uses(v, axes, uses, ctx)
        self.n_ops = n_ops                       # counting walks through broadcasts too; only _gen's count is kept
        chain = {"free": list(range(MAX_TMP - 1, -1, -1)), "memo": {}, "uses": uses}
        code = []
        self._gen(v, axes, code, ctx, chain)
        return code

    # ---- statements ------------------------------------------------------------------------------
    def _new_slot(self):
        if len(self.row_slots) >= MAX_ROWVALS:
            raise _Unfusable
        return len(self.row_slots)

    def _row_reduce(self, v, key):
        code = self._chain(v._op.inputs[0], list(range(self.d)), "full")
        slot = self._new_slot()
        code.append(_word(CH_ROW_REDUCE, REDUCE_CODES[v._op.attrs["op"]], (K_NONE, slot), 0, v.dtype))
        self.statements.append(code)
        self.row_slots[key] = slot
        self.n_ops += 1
        return slot

    def _row_map(self, v, axes, key):
        code = self._chain(v, axes, "row")
        slot = self._new_slot()
        code.append(_word(CH_ROW_MAP, 0, (K_NONE, slot), 0, v.dtype))
        self.statements.append(code)
        self.row_slots[key] = slot
        return slot

    def build(self):
        root = self.root
        if _is_node(root) and root._op.kind == "reduce":
            if not self._fusable(root, None):
                raise _Unfusable
            slot = self._row_reduce(root, (id(root), ()))
            self.statements.append([_word(CH_STORE_ROW, 0, (K_NONE, slot), 0, root.dtype)])
        else:
            if not self._fusable(root, list(root.shape)) or (_is_node(root) and root._op.kind == "broadcast_to"):
                raise _Unfusable
            code = self._chain(root, list(range(self.d)), "full")
            code.append(_word(CH_STORE, 0, (K_NONE, 0), 0, root.dtype))
            self.statements.append(code)
        words = [w for st in self.statements for w in st]
        if len(words) > MAX_CODE:
            raise _Unfusable
        return words


def build_program(v):
    """(words, inputs [(Var, view shape)], full shape, row axes, n fused ops) for the region rooted at v, or None."""
    from .flags import flags
    if not flags.b200_fuse_chains:
        return None
    try:
        b = _Builder(v)
        words = b.build()
    except _Unfusable:
        return None
    if b.n_ops < 2:
        return None            # a single op: the dedicated kernels do that better
    # a reduce whose rows are few and long would leave most of the GPU idle (one group of threads per row)
    if b.k and b.rows < 64 and b.cols > (1 << 14):
        return None
    return words, b.inputs, b.full, b.k, b.n_ops


def run_program(words, inputs, full, k, out):
    """Launches b200jt_fused_chain for realised inputs; `out` is the preallocated result tensor."""
    n = len(inputs)
    descs = (C.Tensor * max(n, 1))()
    for i, (var, view) in enumerate(inputs):
        descs[i] = C.desc(var._data, view)
    shp = (ctypes.c_int64 * len(full))(*full)
    code = (ctypes.c_int32 * len(words))(*words)
    C.check(C.lib.b200jt_fused_chain(descs, n, shp, len(full), k, code, len(words), C.desc(out), C.stream_ptr()),
            f"fused chain over {full} ({len(words)} words, {n} inputs)")
    return out


def program_source(words, inputs, full, k, out_shape, out_dtype="float32"):
    """The CUDA source the library generates for a program, and whether NVRTC accepts it for sm_100a: needs no GPU, nothing
    is launched. inputs: (var, view) pairs as build_program returns them (only dtype and view are used).
    Returns (source, compiled, log)."""
    n = len(inputs)
    descs = (C.Tensor * max(n, 1))()

    def fake(i, dtype, shape):
        d = C.Tensor()
        d.ptr = 0x10000 * (i + 1)                  # never dereferenced: only the alignment is looked at
        d.dtype = C.DTYPE_CODES[str(dtype)]
        d.ndim = max(len(shape), 1)
        for j, e in enumerate(list(shape) or [1]):
            d.shape[j] = int(e)
        return d
    for i, (var, view) in enumerate(inputs):
        descs[i] = fake(i, var.dtype, view)
    out = fake(n, out_dtype, out_shape)
    shp = (ctypes.c_int64 * len(full))(*full)
    code = (ctypes.c_int32 * len(words))(*words)
    cap = 1 << 18
    buf = ctypes.create_string_buffer(cap)
    needed, ok = ctypes.c_int64(0), ctypes.c_int(0)
    C.check(C.lib.b200jt_fused_chain_source(descs, n, shp, len(full), k, code, len(words), ctypes.byref(out), buf, cap,
                                            ctypes.byref(needed), ctypes.byref(ok)),
            f"fused chain source over {full}")
    log = "" if ok.value else C.lib.b200jt_last_error().decode()
    return buf.value.decode(), bool(ok.value), log
