"""Reverse-mode differentiation over the lazy graph with the reference's per-op rules:
reindex <-> reindex_reduce(add) (python/jittor/src/ops/reindex_op.cc:76-80, reindex_reduce_op.cc:45-63),
broadcast_to <-> reduce(add) (broadcast_to_op.cc:112-117, reduce_op.cc:339-362), element-wise rules
(binary_op.cc:491-550, unary_op.cc:891-966), ternary, reshape and the all-reduce (its own adjoint,
python/jittor/extern/mpi/ops/mpi_all_reduce_op.cc:67-71).

`grad(loss, targets)` builds new lazy Vars; nothing runs until they are synced, and the backward graph goes through
the same executor (so e.g. the gradient of a max-pool written with reindex + reduce(max) lands on the injective
reindex_reduce kernel)."""
from . import var as V
from . import dtypes as dt


def _bcast_like(x, ref, mask, keep):
    """broadcast_to with explicit masks (the constructor the reference's grad rules call)."""
    return V.Var(ref.shape, x.dtype, V.Op("broadcast_to", [x], bcast_mask=mask, keepdims_mask=keep))


def _reduce_masks(x, op, mask, keep):
    nd = x.ndim
    yshape = []
    for i in range(nd):
        if mask >> i & 1:
            if keep >> i & 1:
                yshape.append(1)
        else:
            yshape.append(x.shape[i])
    if not yshape:
        yshape = [1]
    return V.Var(yshape, dt.reduce_dtype_infer(op, x.dtype), V.Op("reduce", [x], op=op, reduce_mask=mask, keepdims_mask=keep))


def _unbroadcast(g, shape):
    """Sums g over the axes along which an operand of shape `shape` was stretched by a binary op."""
    gs = list(g.shape)
    if gs == list(shape):
        return g
    pad = len(gs) - len(shape)
    dims = list(range(pad)) + [pad + i for i, s in enumerate(shape) if s == 1 and gs[pad + i] != 1]
    if dims:
        g = V.reduce(g, "add", dims, True)
    return g.reshape(list(shape))


def _is_ones(v):
    """v is the constant 1 stretched to its shape (the seed of a gradient pushed through sums and casts): an unrealised chain
    of broadcast_to / float casts over fill(1)."""
    for _ in range(8):
        op = v._op
        if v._data is not None or op is None:
            return False
        if op.kind == "fill":
            return op.attrs["value"] == 1 and not isinstance(op.attrs["value"], bool)
        if op.kind == "broadcast_to" or (op.kind == "unary" and op.attrs["op"] in ("float32", "bfloat16", "float16", "float64")):
            v = op.inputs[0]
            continue
        return False
    return False


def _zeros_like(v):
    return V.full(list(v.shape), 0, v.dtype)


def _op_grad(out, dout, k):
    """Gradient w.r.t. input k of the op that produced `out` (None: no gradient flows)."""
    op = out._op
    kind, a = op.kind, op.attrs
    x = op.inputs[k]
    if kind == "reindex":
        if k != 0:
            return None
        return V.reindex_reduce(dout, "add", list(x.shape), a["indexes"], a["overflow_conditions"], op.inputs[1:])
    if kind == "reindex_reduce":
        if k != 0:
            return None
        args = (list(x.shape), a["indexes"], 0, a["overflow_conditions"], op.inputs[1:])
        if a["op"] == "add":
            return V.reindex(dout, *args)
        if a["op"] == "multiply":
            return V.reindex(dout * out, *args) / x
        if a["op"] in ("maximum", "minimum"):
            cond = V.binary(x, V.reindex(out, *args), "equal")
            return V.ternary(cond, V.reindex(dout, *args), _zeros_like(x))
        return None
    if kind == "broadcast_to":
        mask, keep = a["bcast_mask"], a["keepdims_mask"]
        if mask == 0:
            return dout
        g = _reduce_masks(dout, "add", mask, keep)
        return g.reshape(list(x.shape)) if list(g.shape) != list(x.shape) else g
    if kind == "reduce":
        mask, keep, rop = a["reduce_mask"], a["keepdims_mask"], a["op"]
        if rop == "add":
            return _bcast_like(dout, x, mask, keep)
        if rop == "mean":
            return _bcast_like(dout, x, mask, keep) * (float(out.numel()) / float(x.numel()))
        if rop == "multiply":
            return _bcast_like(dout * out, x, mask, keep) / x
        if rop in ("maximum", "minimum"):
            cond = V.binary(x, _bcast_like(out, x, mask, keep), "equal")
            return V.ternary(cond, _bcast_like(dout, x, mask, keep), _zeros_like(x))
        return None
    if kind == "binary":
        p, q = op.inputs
        bop = a["op"]
        if bop == "add":
            g = dout
        elif bop == "subtract":
            g = dout if k == 0 else -dout
        elif bop == "multiply":
            other = q if k == 0 else p
            # 1 * y is y bit for bit: the gradient of (p * q).sum() is the other factor itself, not a pass over it
            # (not when the factor is the reindex / broadcast operand of a convolution: its gradient graphs are recognised
            # with the product in place)
            same = (list(other.shape) == list(dout.shape) and str(other.dtype) == str(dout.dtype) and other.dtype.is_float()
                    and (other._op is None or other._op.kind not in ("broadcast_to", "reindex")))
            g = other if same and _is_ones(dout) else other * dout
        elif bop == "divide":
            g = dout / q if k == 0 else (-dout * p) / (q * q)
        elif bop in ("maximum", "minimum"):
            cond = V.binary(q, out, "equal")
            zeros = _zeros_like(dout)
            g = V.ternary(cond, dout, zeros) if k == 1 else V.ternary(cond, zeros, dout)
        elif bop == "pow":
            g = dout * q * V.binary(p, q - 1, "pow") if k == 0 else dout * (out * V.unary(p, "log"))
        else:
            return None
        return _unbroadcast(g, x.shape)
    if kind == "unary":
        uop = a["op"]
        if not x.dtype.is_float():
            return None
        if uop in dt.DTYPES:
            return dout.cast(x.dtype)
        if uop == "negative":
            return -dout
        if uop == "abs":
            return V.ternary(V.binary(x, 0.0, "greater_equal"), dout, -dout)
        if uop == "log":
            return dout / x
        if uop == "exp":
            return dout * out
        if uop == "sqrt":
            return dout / (out * 2.0)
        if uop == "sin":
            return dout * V.unary(x, "cos")
        if uop == "cos":
            return dout * (-V.unary(x, "sin"))
        if uop == "tanh":
            c = V.unary(x, "cosh")
            return dout / (c * c)
        if uop == "sigmoid":
            return dout * out * (1.0 - out)
        return None
    if kind == "ternary":
        if k == 0:
            return None
        cond = op.inputs[0]
        zeros = _zeros_like(dout)
        g = V.ternary(cond, dout, zeros) if k == 1 else V.ternary(cond, zeros, dout)
        return _unbroadcast(g, x.shape)
    if kind == "reshape":
        return dout.reshape(list(x.shape))
    if kind == "custom":
        rule = a.get("grad")                      # relays bring their own backward (e.g. the pooling kernels)
        return rule(out, dout, k) if rule is not None else None
    if kind == "mpi_all_reduce":
        from . import dist
        return dist.mpi_all_reduce(dout, "add")
    return None


def _grad_inputs(v):
    """The Vars a gradient flows to from v: its op's inputs, or the single input of a Var with its own backward rule."""
    vjp = getattr(v, "_vjp", None)
    return [vjp[0]] if vjp is not None else v._op.inputs


def grad(loss, targets, retain_graph=True):
    """d(sum(loss)) / d(target) for every target; a list of Vars (a single Var if `targets` is one)."""
    single = isinstance(targets, V.Var)
    tlist = [targets] if single else list(targets)
    tids = {id(t) for t in tlist}
    # nodes from which a target is reachable, in topological order
    order, needs, seen = [], {}, set()
    stack = [(loss, False)]
    while stack:
        v, done = stack.pop()
        if done:
            need = id(v) in tids
            if v._op is not None and not v.is_stop_grad():
                need = need or any(needs.get(id(i), False) for i in _grad_inputs(v))
            needs[id(v)] = need
            order.append(v)
            continue
        if id(v) in seen:
            continue
        seen.add(id(v))
        stack.append((v, True))
        if v._op is not None and id(v) not in tids and not v.is_stop_grad():     # no gradient flows through stop_grad Vars
            for i in _grad_inputs(v):
                if id(i) not in seen:
                    stack.append((i, False))
    dmap = {id(loss): V.full(list(loss.shape), 1, loss.dtype if loss.dtype.is_float() else "float32")}
    for v in reversed(order):
        if not needs.get(id(v)) or id(v) not in dmap or v._op is None or id(v) in tids:
            continue
        dout = dmap[id(v)]
        vjp = getattr(v, "_vjp", None)
        if vjp is not None:                 # a fused op that brings its own backward: one step from v to its input
            inp, rule = vjp
            if needs.get(id(inp)):
                g = rule(v, dout)
                if g.dtype != inp.dtype and inp.dtype.is_float():
                    g = g.cast(inp.dtype)
                dmap[id(inp)] = dmap[id(inp)] + g if id(inp) in dmap else g
            continue
        for k, inp in enumerate(v._op.inputs):
            if not needs.get(id(inp)):
                continue
            g = _op_grad(v, dout, k)
            if g is None:
                continue
            if g.dtype != inp.dtype and inp.dtype.is_float():
                g = g.cast(inp.dtype)
            dmap[id(inp)] = dmap[id(inp)] + g if id(inp) in dmap else g
    out = [dmap.get(id(t), None) for t in tlist]
    out = [g if g is not None else _zeros_like(t) for g, t in zip(out, tlist)]
    return out[0] if single else out
