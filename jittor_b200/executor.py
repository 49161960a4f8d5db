"""Executor: turns the lazy graph into kernel launches.

The reference's executor groups ops into FusedOps (python/jittor/src/executor.cc:276-534) and its
tuners swap recognised groups for library relays (python/jittor/src/opt/tuner/matmul_tuner.cc:21-102,
conv_tuner.cc:218-411). Here the same groups are recognised structurally on the graph and handed to
hand-written kernels:

    reduce.add(multiply(reindex(x), broadcast_to(w)))          -> conv2d
    reduce.add(multiply(broadcast_to(a), broadcast_to(b)))     -> matmul
    exp(x - max(x)) / sum(exp(x - max(x)))  (and the log form) -> fused row softmax
    x * (g / sqrt(var + eps)) + (b - mean * w)                 -> fused LayerNorm / BatchNorm (+ReLU)

Everything else runs op by op through the meta-operator kernels. Intermediates of a recognised
group are never materialised.
"""
import ctypes

import torch
import torch.distributed as tdist

from . import _capi as C
from . import dtypes as dt
from .var import Var

_MATERIALIZE_LIMIT = 1 << 33       # elements; beyond this an unfused intermediate is refused
counters = {"plans": 0}            # plans run so far: one per kernel group, the analogue of the reference's fused-op count


class Plan:
    __slots__ = ("leaves", "run")

    def __init__(self, leaves, run):
        self.leaves = leaves
        self.run = run


def realize(roots):
    for root in roots:
        stack = [root]
        plans = {}
        while stack:
            v = stack[-1]
            if v._data is not None:
                stack.pop()
                continue
            plan = plans.get(id(v))
            if plan is None:
                plan = plans[id(v)] = _make_plan(v)
            pending = [l for l in plan.leaves if l._data is None]
            if pending:
                stack.extend(pending)
                continue
            for l in plan.leaves:
                if l._pending is not None:           # produced by a collective on another stream
                    l.wait()
            out = plan.run()
            counters["plans"] += 1
            v._data = out.reshape(list(v.shape))
            plans.pop(id(v), None)
            stack.pop()
            pending_update = getattr(v, "_bn_running", None)
            if pending_update is not None:          # a BatchNorm output computed op by op: move its running statistics now
                v._bn_running = None
                module, xmean, xvar = pending_update
                module._update_running(xmean, xvar)


def _make_plan(v):
    relay = getattr(v, "_relay", None)
    if relay is not None:                       # a convolution built by nn with its relay record (its graph may not be written yet)
        kind, x, w, geo, groups = relay
        if x.dtype in ("float32", "bfloat16") and w.dtype in ("float32", "bfloat16"):
            if kind == "conv2d":
                return Plan([x, w], lambda: run_conv2d(x, w, geo, v.dtype, groups=groups))
            return Plan([x, w], lambda: run_conv2d_transpose(x, w, geo, groups, list(v.shape), v.dtype))
    if v._op is None:
        raise C.B200Error("Var has neither data nor a producer")
    for matcher in _MATCHERS:
        p = matcher(v)
        if p is not None:
            return p
    op = v._op
    for i in op.inputs:
        if i._data is None and i.numel() > _MATERIALIZE_LIMIT:
            raise C.B200Error(f"refusing to materialise an unfused intermediate of {i.numel()} elements "
                              f"(shape {list(i.shape)}); the chain around it is not one of the fused forms")
    return Plan(list(op.inputs), lambda: _RUNNERS[op.kind](v, op))


# --------------------------------------------------------------------------------- helpers
def _empty(shape, dtype):
    C.require_cuda()
    return torch.empty(list(shape), dtype=C.TORCH_DTYPES[str(dtype)], device="cuda")


def _workspace(nbytes):
    if nbytes == 0:
        return None, ctypes.c_void_p(0)
    ws = torch.empty(int(nbytes), dtype=torch.uint8, device="cuda")
    return ws, ctypes.c_void_p(ws.data_ptr())


def _cast(t, dtype):
    """Tensor converted to `dtype` by the unary cast kernel (a no-op if it already has it)."""
    if C.DTYPE_NAMES[t.dtype] == str(dtype):
        return t
    out = _empty(t.shape, dtype)
    C.check(C.lib.b200jt_unary(C.desc(t), C.desc(out), str(dtype).encode(), C.stream_ptr()), f"cast({dtype})")
    return out


def _pad_shape(shape, rank):
    return [1] * (rank - len(shape)) + list(shape)


def _node(v, kind, **attrs):
    """v is an unrealised Var produced by an op of `kind` whose attrs match."""
    if not isinstance(v, Var) or v._data is not None or v._op is None or v._op.kind != kind:
        return False
    return all(v._op.attrs.get(k) == val for k, val in attrs.items())


def _const(v):
    return getattr(v, "_const", None)


def _strip_cast(v, to):
    """If v = cast<to>(u) (unrealised), returns u."""
    if _node(v, "unary", op=to):
        return v._op.inputs[0]
    return None


# --------------------------------------------------------------------------------- single ops
def _run_reindex(v, op):
    x, extras = op.inputs[0], op.inputs[1:]
    out = _empty(v.shape, v.dtype)
    a = op.attrs
    keep = [e._data for e in extras]
    C.check(C.lib.b200jt_reindex(C.desc(x._data), C.desc(out), C.strings(a["indexes"]), len(a["indexes"]),
                                 a["overflow_value"], C.strings(a["overflow_conditions"]),
                                 len(a["overflow_conditions"]), C.descs(keep), len(keep), C.stream_ptr()),
            f"reindex {list(x.shape)}->{list(v.shape)} {a['indexes']}")
    return out


def _run_reindex_reduce(v, op):
    y, extras = op.inputs[0], op.inputs[1:]
    out = _empty(v.shape, v.dtype)
    a = op.attrs
    keep = [e._data for e in extras]
    args = (C.desc(y._data), C.desc(out), a["op"].encode(), C.strings(a["indexes"]), len(a["indexes"]),
            C.strings(a["overflow_conditions"]), len(a["overflow_conditions"]), C.descs(keep), len(keep))
    nbytes = C.lib.b200jt_reindex_reduce_workspace(*args)
    ws, wsp = _workspace(nbytes)
    C.check(C.lib.b200jt_reindex_reduce(*args, wsp, nbytes, C.stream_ptr()),
            f"reindex_reduce({a['op']}) {list(y.shape)}->{list(v.shape)} {a['indexes']}")
    return out


def _bcast_view_shape(xshape, zrank, mask, keep):
    """x's shape written with z's rank: size 1 on axes that broadcast_to creates."""
    kept = [i for i in range(zrank) if not (mask >> i & 1) or (keep >> i & 1)]
    src = _pad_shape(xshape, len(kept))
    view, k = [], 0
    for i in range(zrank):
        if i in kept:
            view.append(src[k])
            k += 1
        else:
            view.append(1)
    return view


def _run_broadcast(v, op):
    x = op.inputs[0]
    out = _empty(v.shape, v.dtype)
    mask, keep = op.attrs["bcast_mask"], op.attrs["keepdims_mask"]
    view = _bcast_view_shape(list(x.shape), v.ndim, mask, keep)
    eff = 0
    for i in range(v.ndim):
        if view[i] == 1 and v.shape[i] != 1:
            eff |= 1 << i
        elif view[i] != v.shape[i]:
            raise C.B200Error(f"broadcast: cannot stretch {list(x.shape)} to {list(v.shape)}")
    C.check(C.lib.b200jt_broadcast_to(C.desc(x._data, view), C.desc(out), eff, C.stream_ptr()), "broadcast_to")
    return out


def _run_reduce(v, op):
    x = op.inputs[0]
    mask = op.attrs["reduce_mask"]
    yfull = [1 if mask >> i & 1 else x.shape[i] for i in range(x.ndim)]
    out = _empty(v.shape, v.dtype)
    name = op.attrs["op"].encode()
    xd, yd = C.desc(x._data), C.desc(out, yfull)
    nbytes = C.lib.b200jt_reduce_workspace(xd, yd, name, mask)
    ws, wsp = _workspace(nbytes)
    C.check(C.lib.b200jt_reduce(xd, yd, name, mask, wsp, nbytes, C.stream_ptr()),
            f"reduce({op.attrs['op']}) {list(x.shape)} mask {mask:b}")
    return out


def _run_binary(v, op):
    x, y = op.inputs
    out = _empty(v.shape, v.dtype)
    r = v.ndim
    C.check(C.lib.b200jt_binary(C.desc(x._data, _pad_shape(x.shape, r)), C.desc(y._data, _pad_shape(y.shape, r)),
                                C.desc(out), op.attrs["op"].encode(), C.stream_ptr()),
            f"binary({op.attrs['op']}) {list(x.shape)} {list(y.shape)}")
    return out


def _run_unary(v, op):
    x = op.inputs[0]
    out = _empty(v.shape, v.dtype)
    C.check(C.lib.b200jt_unary(C.desc(x._data), C.desc(out), op.attrs["op"].encode(), C.stream_ptr()),
            f"unary({op.attrs['op']})")
    return out


def _run_ternary(v, op):
    c, x, y = op.inputs
    out = _empty(v.shape, v.dtype)
    r = v.ndim
    xd, yd = x._data, y._data
    C.check(C.lib.b200jt_ternary(C.desc(c._data, _pad_shape(c.shape, r)), C.desc(xd, _pad_shape(x.shape, r)),
                                 C.desc(yd, _pad_shape(y.shape, r)), C.desc(out), C.stream_ptr()), "ternary")
    return out


def _run_reshape(v, op):
    return op.inputs[0]._data.reshape(list(v.shape))


def _run_all_reduce(v, op):
    """Sum over the ranks: in stream order, or -- inside dist.overlap_collectives() -- on a side stream beside the kernels
    that follow, in which case the Var carries a handle that its first reader waits on."""
    x = op.inputs[0]._data
    if tdist.is_available() and tdist.is_initialized() and tdist.get_world_size() > 1:
        from . import dist
        out, join = dist.all_reduce_sum_overlapped(x)
        v._pending = join
        return out
    return x.clone()


def _run_fill(v, op):
    C.require_cuda()
    return torch.full(list(v.shape), op.attrs["value"], dtype=C.TORCH_DTYPES[str(v.dtype)], device="cuda")


def _run_custom(v, op):
    return op.attrs["fn"](*[i._data for i in op.inputs])


_RUNNERS = {"reindex": _run_reindex, "reindex_reduce": _run_reindex_reduce, "broadcast_to": _run_broadcast,
            "reduce": _run_reduce, "binary": _run_binary, "unary": _run_unary, "ternary": _run_ternary,
            "reshape": _run_reshape, "mpi_all_reduce": _run_all_reduce, "custom": _run_custom, "fill": _run_fill}


# --------------------------------------------------------------------------------- contraction patterns
_AFFINE_CACHE = {}


def index_affine(loop_shape, x_shape, indexes):
    """(coef[d][j], c0[d]) if all indexes are affine in the loop variables, else None (memoised)."""
    key = (tuple(loop_shape), tuple(x_shape), tuple(indexes))
    if key not in _AFFINE_CACHE:
        if len(_AFFINE_CACHE) > 4096:
            _AFFINE_CACHE.clear()
        _AFFINE_CACHE[key] = _index_affine(loop_shape, x_shape, indexes)
    return _AFFINE_CACHE[key]


def _index_affine(loop_shape, x_shape, indexes):
    n = len(indexes)
    ls = (ctypes.c_int64 * len(loop_shape))(*loop_shape)
    xs = (ctypes.c_int64 * len(x_shape))(*x_shape)
    coef = (ctypes.c_int64 * (n * C.MAX_DIMS))()
    c0 = (ctypes.c_int64 * n)()
    rc = C.lib.b200jt_index_affine(ls, len(loop_shape), xs, len(x_shape), C.strings(indexes), n, coef, c0)
    if rc < 0:
        C.check(rc, "index expression")
    if rc != 1:
        return None
    return [[coef[d * C.MAX_DIMS + j] for j in range(len(loop_shape))] for d in range(n)], list(c0)


def _mul_operands(v, rank):
    """v = reduce.add over an unrealised multiply of rank `rank`: returns (reduce op, lhs, rhs)."""
    if not _node(v, "reduce", op="add"):
        return None
    m = v._op.inputs[0]
    if not _node(m, "binary", op="multiply") or m.ndim != rank:
        return None
    a, b = m._op.inputs
    if list(a.shape) != list(m.shape) or list(b.shape) != list(m.shape):
        return None
    return v._op, a, b


def _conv_index_geometry(loop_shape, x_shape, indexes):
    """Solves (sh, sw, ph, pw, dh, dw) from the four index strings of the conv lowering over the 7-D loop nest
    [N, Co, Ci, OH, OW, KH, KW] (python/jittor/nn.py:1009-1014), as ConvTuner does with expr::match
    (python/jittor/src/opt/tuner/conv_tuner.cc:313-338). None if the strings are not that lowering."""
    N, Co, Ci, OH, OW, KH, KW = loop_shape
    aff = index_affine(list(loop_shape), list(x_shape), indexes)
    if aff is None:
        return None
    coef, c0 = aff

    def only(row, allowed):
        return all(cf == 0 or j in allowed for j, cf in enumerate(row))

    if not (coef[0] == [1, 0, 0, 0, 0, 0, 0] and c0[0] == 0 and coef[1] == [0, 0, 1, 0, 0, 0, 0] and c0[1] == 0):
        return None
    if not (only(coef[2], (3, 5)) and only(coef[3], (4, 6))):
        return None
    sh, dh, ph = coef[2][3], coef[2][5], -c0[2]
    sw, dw, pw = coef[3][4], coef[3][6], -c0[3]
    if KH == 1:
        dh = max(dh, 1)
    if KW == 1:
        dw = max(dw, 1)
    if OH == 1:
        sh = max(sh, 1)
    if OW == 1:
        sw = max(sw, 1)
    if min(sh, sw, dh, dw) < 1 or ph < 0 or pw < 0:
        return None
    H, W = x_shape[2], x_shape[3]
    if OH != (H + 2 * ph - KH * dh + dh - 1) // sh + 1 or OW != (W + 2 * pw - KW * dw + dw - 1) // sw + 1:
        return None
    return (sh, sw, ph, pw, dh, dw)


_MASK_W, _MASK_Y = 0b0011001, 0b1100100     # axes a weight / an output gradient is broadcast over in the 7-D nest


def _bcast_of(v, mask, shape4):
    """v = broadcast_to(u) over exactly the axes of `mask` with u of shape `shape4`: returns u, else None."""
    if not _node(v, "broadcast_to") or v._op.attrs["bcast_mask"] != mask or v._op.attrs["keepdims_mask"] != 0:
        return None
    u = v._op.inputs[0]
    return u if list(u.shape) == list(shape4) else None


def conv_geometry(rx, ww):
    """Checks that rx = reindex(x) and ww = broadcast_to(w) are the NCHW/OIHW conv lowering of
    python/jittor/nn.py:1009-1016. Returns (x, w, geometry) or None."""
    if not (_node(rx, "reindex") and _node(ww, "broadcast_to")):
        return None
    a = rx._op.attrs
    x = rx._op.inputs[0]
    if len(rx._op.inputs) != 1 or a["overflow_conditions"] or a["overflow_value"] != 0:
        return None
    if x.ndim != 4 or rx.ndim != 7:
        return None
    N, Co, Ci, OH, OW, KH, KW = rx.shape
    w = _bcast_of(ww, _MASK_W, [Co, Ci, KH, KW])
    if w is None or x.shape[0] != N or x.shape[1] != Ci:
        return None
    geo = _conv_index_geometry(list(rx.shape), list(x.shape), a["indexes"])
    return None if geo is None else (x, w, geo)


def _match_conv_dgrad(v):
    """dx = reindex_reduce.add(multiply(broadcast(w), broadcast(dy))) with the conv's index strings: what the reindex /
    broadcast gradient rules make of a conv, and one of the forms ConvTuner relays (conv_tuner.cc:375-397, to
    cudnn_conv_backward_x). Runs as a transposed convolution; stride-1 bf16 layers run on the tensor-core conv with
    the weights flipped and transposed (a gather by the reindex kernel)."""
    if not _node(v, "reindex_reduce", op="add") or v.ndim != 4:
        return None
    a = v._op.attrs
    m = v._op.inputs[0]
    if len(v._op.inputs) != 1 or a["overflow_conditions"] or not _node(m, "binary", op="multiply") or m.ndim != 7:
        return None
    N, Co, Ci, OH, OW, KH, KW = m.shape
    p, q = m._op.inputs
    w = _bcast_of(p, _MASK_W, [Co, Ci, KH, KW])
    dy = _bcast_of(q, _MASK_Y, [N, Co, OH, OW])
    if w is None or dy is None:
        w, dy = _bcast_of(q, _MASK_W, [Co, Ci, KH, KW]), _bcast_of(p, _MASK_Y, [N, Co, OH, OW])
    if w is None or dy is None or list(v.shape[:2]) != [N, Ci]:
        return None
    if dy.dtype not in ("float32", "bfloat16") or w.dtype not in ("float32", "bfloat16"):
        return None
    geo = _conv_index_geometry(list(m.shape), list(v.shape), a["indexes"])
    if geo is None:
        return None
    sh, sw, ph, pw, dh, dw = geo
    fp, fq = dh * (KH - 1) - ph, dw * (KW - 1) - pw
    if sh == 1 and sw == 1 and fp >= 0 and fq >= 0 and dy.dtype == "bfloat16":
        from . import var as V
        wf = V.reindex(w, [Ci, Co, KH, KW], ["i1", "i0", f"{KH - 1}-i2", f"{KW - 1}-i3"])
        return Plan([dy, wf], lambda: run_conv2d(dy, wf, (1, 1, fp, fq, dh, dw), v.dtype))
    return Plan([dy, w], lambda: run_conv2d_transpose(dy, w, geo, 1, list(v.shape), v.dtype))


def _match_conv_wgrad(v):
    """dw = reduce.add over [0,3,4] of multiply(reindex(x), broadcast(dy)) (conv_tuner.cc:375-397, relayed there to
    cudnn_conv_backward_w)."""
    got = _mul_operands(v, 7)
    if got is None:
        return None
    rop, p, q = got
    if rop.attrs["reduce_mask"] != _MASK_W or rop.attrs["keepdims_mask"] != 0:
        return None
    rx, bd = (p, q) if _node(p, "reindex") else (q, p)
    if not _node(rx, "reindex"):
        return None
    a = rx._op.attrs
    x = rx._op.inputs[0]
    if len(rx._op.inputs) != 1 or a["overflow_conditions"] or a["overflow_value"] != 0 or x.ndim != 4:
        return None
    N, Co, Ci, OH, OW, KH, KW = rx.shape
    dy = _bcast_of(bd, _MASK_Y, [N, Co, OH, OW])
    if dy is None or list(x.shape[:2]) != [N, Ci]:
        return None
    if x.dtype not in ("float32", "bfloat16") or dy.dtype not in ("float32", "bfloat16"):
        return None
    geo = _conv_index_geometry(list(rx.shape), list(x.shape), a["indexes"])
    if geo is None:
        return None

    return Plan([x, dy], lambda: run_conv2d_backward_w(x, dy, geo, [Co, Ci, KH, KW], v.dtype))


def _swap01(t):
    """[a, b, c, d] -> [b, a, c, d] by the reindex kernel (a pure permutation: tiled through shared memory)."""
    a, b, c, d = t.shape
    out = _empty([b, a, c, d], C.DTYPE_NAMES[t.dtype])
    idx = ["i1", "i0", "i2", "i3"]
    C.check(C.lib.b200jt_reindex(C.desc(t), C.desc(out), C.strings(idx), 4, 0.0, C.strings([]), 0, None, 0, C.stream_ptr()),
            "reindex (swap of the two leading axes)")
    return out


def _wgrad_as_conv(xd, dyd, geo, w_shape):
    """The weight gradient on the tensor-core convolution: dw[o,c,kh,kw] = sum over (n,oh,ow) of dy[n,o,oh,ow] *
    x[n,c,oh*s-p+kh*d, ...] IS a convolution of x with the batch and channel axes exchanged (images = in channels, channels =
    batch) by dy with its two leading axes exchanged as the filter (out channels = o, in channels = n, an OH x OW window),
    with the roles of stride and dilation exchanged; its [C, Co, KH, KW] result only needs its leading axes swapped back.
    cuDNN has a dedicated kernel for this (cudnn_conv_backward_w_op.cc:292); here the forward kernel serves, at the price of
    8x8 output patches of which KH x KW pixels are real. Returns None when the shapes miss the tensor-core path."""
    sh, sw, ph, pw, dh, dw = geo
    Co, Ci, KH, KW = w_shape
    N, _, H, W = xd.shape
    OH, OW = dyd.shape[2], dyd.shape[3]
    if xd.dtype != torch.bfloat16 or max(sh, sw, dh, dw) > 4:
        return None
    # extents of the exchanged convolution must come out as the filter's
    if (H + 2 * ph - sh * (OH - 1) - 1) // dh + 1 != KH or (W + 2 * pw - sw * (OW - 1) - 1) // dw + 1 != KW:
        return None
    if N % 8 or N < 64 or Co < 64 or Ci * KH * KW < 1024 or H < 8 or W < 8:
        return None
    xt, dyt = _swap01(xd), _swap01(dyd)                   # [C, N, H, W], [Co, N, OH, OW]
    out = _empty([Ci, Co, KH, KW], "bfloat16")
    args = (C.desc(xt), C.desc(dyt), C.desc(out), dh, dw, ph, pw, sh, sw, 1)
    nbytes = C.lib.b200jt_conv2d_workspace(*args)
    if nbytes == 0:
        return None                                       # not a tensor-core shape after all
    ws, wsp = _workspace(nbytes)
    C.check(C.lib.b200jt_conv2d(*args, ctypes.c_void_p(0), wsp, nbytes, C.stream_ptr()), "conv2d (weight gradient form)")
    return _swap01(out)


def run_conv2d_backward_w(x, dy, geo, w_shape, out_dtype):
    """Weight gradient. flags.b200_wgrad_tc: 1 (default) the tensor-core weight-gradient kernel where its shape rules hold,
    then the exchanged-axes convolution, then the CUDA-core kernel; 2 skips the dedicated kernel; 0 CUDA cores only."""
    xd = x._data.view(list(x.shape))
    dyd = _cast(dy._data.view(list(dy.shape)), x.dtype)
    from .flags import flags
    mode = int(getattr(flags, "b200_wgrad_tc", 1))
    out = _empty(w_shape, x.dtype)
    args = (C.desc(xd), C.desc(dyd), C.desc(out), *geo)
    if mode == 1:
        nbytes = C.lib.b200jt_conv2d_backward_w_workspace(*args)
        if nbytes:
            ws, wsp = _workspace(nbytes)
            C.check(C.lib.b200jt_conv2d_backward_w_tc(*args, wsp, nbytes, C.stream_ptr()),
                    f"conv2d_backward_w (tensor cores) x{list(x.shape)} dy{list(dy.shape)} geo{geo}")
            return _cast(out, out_dtype)
    if mode:
        got = _wgrad_as_conv(xd, dyd, geo, w_shape)
        if got is not None:
            return _cast(got, out_dtype)
    C.check(C.lib.b200jt_conv2d_backward_w(*args, C.stream_ptr()),
            f"conv2d_backward_w x{list(x.shape)} dy{list(dy.shape)} geo{geo}")
    return _cast(out, out_dtype)


def run_conv2d_backward_w_formats(x, dy, geo, kh, kw, xformat, wformat, yformat, out_dtype):
    """Weight gradient with the relay's layout strings (cudnn_conv_backward_w_op.h): x "abcd" / "acdb", dy (yformat) likewise,
    dw "oihw" / "ohwi". Layouts other than the defaults exist on the tensor-core kernel only."""
    Ci = x.shape[1] if xformat == "abcd" else x.shape[3]
    Co = dy.shape[1] if yformat == "abcd" else dy.shape[3]
    xd = x._data.view(list(x.shape))
    dyd = _cast(dy._data.view(list(dy.shape)), x.dtype)
    out = _empty([Co, Ci, kh, kw] if wformat == "oihw" else [Co, kh, kw, Ci], x.dtype)
    args = (C.desc(xd), C.desc(dyd), C.desc(out), *geo, xformat.encode(), wformat.encode(), yformat.encode())
    nbytes = C.lib.b200jt_conv2d_backward_w_formats_workspace(*args)
    ws, wsp = _workspace(nbytes)
    C.check(C.lib.b200jt_conv2d_backward_w_formats(*args, wsp, nbytes, C.stream_ptr()),
            f"conv2d_backward_w x{list(x.shape)} ({xformat}) dy{list(dy.shape)} ({yformat}) -> {wformat} geo{geo}")
    return _cast(out, out_dtype)


def run_conv2d_transpose(x, w, geo, groups, out_shape, out_dtype):
    sh, sw, ph, pw, dh, dw = geo
    xd = x._data
    wd = _cast(w._data, x.dtype)
    out = _empty(out_shape, x.dtype)
    C.check(C.lib.b200jt_conv2d_transpose(C.desc(xd), C.desc(wd), C.desc(out), sh, sw, ph, pw, dh, dw, groups, C.stream_ptr()),
            f"conv2d_transpose x{list(x.shape)} w{list(w.shape)} geo{geo} groups {groups}")
    return _cast(out, out_dtype)


def run_conv2d(x, w, geo, out_dtype, stats=None, groups=1):
    sh, sw, ph, pw, dh, dw = geo
    N, Ci, H, W = x.shape
    Co, _, KH, KW = w.shape
    OH = (H + 2 * ph - KH * dh + dh - 1) // sh + 1
    OW = (W + 2 * pw - KW * dw + dw - 1) // sw + 1
    xd, wd = x._data, w._data
    wd = _cast(wd, x.dtype)
    out = _empty([N, Co, OH, OW], x.dtype)
    args = (C.desc(xd), C.desc(wd), C.desc(out), sh, sw, ph, pw, dh, dw, groups)
    nbytes = C.lib.b200jt_conv2d_workspace(*args)
    ws, wsp = _workspace(nbytes)
    sp = ctypes.c_void_p(stats.data_ptr()) if stats is not None else ctypes.c_void_p(0)
    rc = C.lib.b200jt_conv2d(*args, sp, wsp, nbytes, C.stream_ptr())
    if rc:                                       # the message is only put together when there is one to show
        C.check(rc, f"conv2d x{list(x.shape)} w{list(w.shape)} geo{geo}")
    return _cast(out, out_dtype)


def run_conv2d_formats(x, w, geo, xformat, wformat, yformat, out_dtype):
    """Convolution with the relay's layout strings (cudnn_conv_op.h): x / y "abcd" or "acdb", w "oihw" or "ohwi"."""
    sh, sw, ph, pw, dh, dw = geo
    yformat = yformat or xformat
    N, Ci, H, W = x.shape if xformat == "abcd" else (x.shape[0], x.shape[3], x.shape[1], x.shape[2])
    Co, KH, KW = (w.shape[0], w.shape[2], w.shape[3]) if wformat == "oihw" else (w.shape[0], w.shape[1], w.shape[2])
    OH = (H + 2 * ph - KH * dh + dh - 1) // sh + 1
    OW = (W + 2 * pw - KW * dw + dw - 1) // sw + 1
    xd, wd = x._data, _cast(w._data, x.dtype)
    out = _empty([N, Co, OH, OW] if yformat == "abcd" else [N, OH, OW, Co], x.dtype)
    args = (C.desc(xd), C.desc(wd), C.desc(out), sh, sw, ph, pw, dh, dw, xformat.encode(), wformat.encode(), yformat.encode())
    nbytes = C.lib.b200jt_conv2d_formats_workspace(*args)
    ws, wsp = _workspace(nbytes)
    C.check(C.lib.b200jt_conv2d_formats(*args, None, wsp, nbytes, C.stream_ptr()),
            f"conv2d x{list(x.shape)} ({xformat}) w{list(w.shape)} ({wformat}) -> {yformat} geo{geo}")
    return _cast(out, out_dtype)


def _match_conv(v):
    got = _mul_operands(v, 7)
    if got is None:
        return None
    rop, a, b = got
    if rop.attrs["reduce_mask"] != 0b1100100 or rop.attrs["keepdims_mask"] != 0:
        return None
    g = conv_geometry(a, b) or conv_geometry(b, a)
    if g is None:
        return None
    x, w, geo = g
    if x.dtype not in ("float32", "bfloat16") or w.dtype not in ("float32", "bfloat16"):
        return None
    return Plan([x, w], lambda: run_conv2d(x, w, geo, v.dtype))


def run_matmul(a, b, trans_a, trans_b, out_dtype):
    ad, bd = a._data, b._data
    bd = _cast(bd, a.dtype)
    M = a.shape[1] if trans_a else a.shape[0]
    N = b.shape[0] if trans_b else b.shape[1]
    out = _empty([M, N], a.dtype)
    args = (C.desc(ad), C.desc(bd), C.desc(out), int(trans_a), int(trans_b))
    nbytes = C.lib.b200jt_matmul_workspace(*args)
    ws, wsp = _workspace(nbytes)
    C.check(C.lib.b200jt_matmul(*args, wsp, nbytes, C.stream_ptr()),
            f"matmul a{list(a.shape)} b{list(b.shape)} t{int(trans_a)}{int(trans_b)}")
    return _cast(out, out_dtype)


def _match_matmul(v):
    """reduce.add over one axis of multiply(broadcast_to(a), broadcast_to(b)), 3-D product of 2-D inputs:
    the (reduce_mask, bcast masks) -> (trans_a, trans_b) table of matmul_tuner.cc:42-82."""
    got = _mul_operands(v, 3)
    if got is None:
        return None
    rop, pa, pb = got
    if rop.attrs["keepdims_mask"] != 0 or not (_node(pa, "broadcast_to") and _node(pb, "broadcast_to")):
        return None
    rmask = rop.attrs["reduce_mask"]
    if rmask not in (1, 2, 4):
        return None
    r = rmask.bit_length() - 1
    ma, mb = pa._op.attrs["bcast_mask"], pb._op.attrs["bcast_mask"]
    if ma not in (1, 2, 4) or mb not in (1, 2, 4) or pa._op.attrs["keepdims_mask"] or pb._op.attrs["keepdims_mask"]:
        return None
    da, db = ma.bit_length() - 1, mb.bit_length() - 1       # axis each operand lacks
    if len({r, da, db}) != 3:
        return None
    a, b = pa._op.inputs[0], pb._op.inputs[0]
    if a.ndim != 2 or b.ndim != 2 or a.dtype not in ("float32", "bfloat16") or b.dtype not in ("float32", "bfloat16"):
        return None
    # a spans axes {r, db}: axis db is its "row" (M) axis; b spans {r, da}: axis da is its "column" (N) axis
    trans_a = r < db          # a stored [K, M]
    trans_b = da < r          # b stored [N, K]
    if db < da:               # output axes in order (M, N)
        return Plan([a, b], lambda: run_matmul(a, b, trans_a, trans_b, v.dtype))
    # output is [N, M] = (A.B)^T = B^T.A^T
    return Plan([a, b], lambda: run_matmul(b, a, not trans_b, not trans_a, v.dtype))


def _match_batched_matmul(v):
    """The [..., n, m, k] product of nn.matmul (python/jittor/nn.py:140-159) as one strided-batched launch."""
    if not _node(v, "reduce", op="add"):
        return None
    m = v._op.inputs[0]
    nd = m.ndim
    if nd < 4 or not _node(m, "binary", op="multiply"):
        return None
    rop = v._op
    if rop.attrs["reduce_mask"] != 1 << (nd - 2) or rop.attrs["keepdims_mask"] != 0:
        return None
    pa, pb = m._op.inputs
    if not (_node(pa, "broadcast_to") and _node(pb, "broadcast_to")):
        return None
    a, b = pa._op.inputs[0], pb._op.inputs[0]
    if not (pa._op.attrs["bcast_mask"] >> (nd - 1) & 1) or not (pb._op.attrs["bcast_mask"] >> (nd - 3) & 1):
        return None
    if list(pa.shape) != list(m.shape) or list(pb.shape) != list(m.shape):
        return None
    if a.ndim < 2 or b.ndim < 2 or a.dtype not in ("float32", "bfloat16") or b.dtype != a.dtype:
        return None
    n, k_, kk = m.shape[nd - 3], m.shape[nd - 2], m.shape[nd - 1]
    if list(a.shape[-2:]) != [n, k_] or list(b.shape[-2:]) != [k_, kk]:
        return None
    batch = list(m.shape[:nd - 3])

    def run():
        out = _empty(batch + [n, kk], a.dtype)
        ab = _pad_shape(list(a.shape[:-2]), len(batch))
        bb = _pad_shape(list(b.shape[:-2]), len(batch))
        # the longest run of trailing batch axes over which each operand is either complete or shared goes to ONE
        # launch (python/jittor/extern/cuda/cublas/ops/cublas_batched_matmul_op.cc:160 does the same for equal batch
        # shapes); leading axes with mixed stretching are walked on the host
        k0 = len(batch)
        while k0 > 0:
            ta, tb, tc = ab[k0 - 1:], bb[k0 - 1:], batch[k0 - 1:]
            if (ta == tc or all(s == 1 for s in ta)) and (tb == tc or all(s == 1 for s in tb)):
                k0 -= 1
            else:
                break
        inner = 1
        for s in batch[k0:]:
            inner *= s

        def flat(t, bshape, rows, cols):
            lead = list(bshape[:k0])
            tail = 1
            for s in bshape[k0:]:
                tail *= s
            return t.reshape(lead + [tail, rows, cols])

        a3, b3, o3 = flat(a._data, ab, n, k_), flat(b._data, bb, k_, kk), out.reshape(batch[:k0] + [inner, n, kk])
        import itertools
        for idx in itertools.product(*[range(s) for s in batch[:k0]]):
            ai = tuple(i if s != 1 else 0 for i, s in zip(idx, ab))
            bi = tuple(i if s != 1 else 0 for i, s in zip(idx, bb))
            C.check(C.lib.b200jt_batched_matmul(C.desc(a3[ai]), C.desc(b3[bi]), C.desc(o3[idx]), 0, 0, C.stream_ptr()),
                    f"batched matmul a{list(a.shape)} b{list(b.shape)}")
        return _cast(out, v.dtype)

    return Plan([a, b], run)


# --------------------------------------------------------------------------------- row softmax
def _last_axis_reduce(r, op, src=None):
    """r = reduce.<op>(u, last axis or all axes, keepdims=True); returns u."""
    if not _node(r, "reduce", op=op):
        return None
    u = r._op.inputs[0]
    nd = u.ndim
    mask = r._op.attrs["reduce_mask"]
    full = (1 << nd) - 1
    if r._op.attrs["keepdims_mask"] & mask != mask:
        return None
    if mask != 1 << (nd - 1) and mask != full:
        return None
    if src is not None and u is not src:
        return None
    return u


def _softmax_rows(u, r):
    mask = r._op.attrs["reduce_mask"]
    cols = u.shape[-1] if mask == 1 << (u.ndim - 1) else u.numel()
    return (u.numel() // cols if cols else 0), cols


def _match_pool(v):
    """y = reduce.{maximum,minimum,mean} over axes [4,5] of reindex(x, [N,C,h,w,kh,kw], [i0, i1, i2*sh-ph+i4, i3*sw-pw+i5]):
    the pooling lowering of python/jittor/pool.py:187-197 (also the adaptive pools, :419-432) as one pooling-kernel
    launch instead of a materialised window tensor. Padding reads as 0 in that lowering, which the kernel reproduces for
    mean (divide by kh*kw); maximum / minimum are only relayed when no window leaves the input."""
    if not _node(v, "reduce") or v._op.attrs["op"] not in ("maximum", "minimum", "mean"):
        return None
    if v._op.attrs["reduce_mask"] != 0b110000 or v._op.attrs["keepdims_mask"] != 0:
        return None
    rx = v._op.inputs[0]
    # 16-bit mean / add: the reduce constructor widens to float32 first (python/jittor/src/ops/reduce_op.cc:260-266) and the
    # caller narrows the result again, so rounding the kernel's float32 accumulator to 16 bits here loses nothing
    widened = _node(rx, "unary", op="float32") and str(v.dtype) == "float32"
    if widened:
        rx = rx._op.inputs[0]
    if not _node(rx, "reindex") or rx.ndim != 6 or len(rx._op.inputs) != 1:
        return None
    a = rx._op.attrs
    x = rx._op.inputs[0]
    if x.ndim != 4 or a["overflow_conditions"] or a["overflow_value"] != 0:
        return None
    if widened and str(x.dtype) not in ("float16", "bfloat16"):
        return None
    if not widened and x.dtype != v.dtype:
        return None
    if str(x.dtype) not in ("float32", "float64", "float16", "bfloat16"):
        return None
    N, Cn, h, w, kh, kw = rx.shape
    if list(x.shape[:2]) != [N, Cn] or min(h, w, kh, kw) < 1:
        return None
    aff = index_affine(list(rx.shape), list(x.shape), a["indexes"])
    if aff is None:
        return None
    coef, c0 = aff
    if coef[0] != [1, 0, 0, 0, 0, 0] or c0[0] != 0 or coef[1] != [0, 1, 0, 0, 0, 0] or c0[1] != 0:
        return None
    if coef[2][0] or coef[2][1] or coef[2][3] or coef[2][5] or coef[3][0] or coef[3][1] or coef[3][2] or coef[3][4]:
        return None
    sh, sw, ph, pw = coef[2][2], coef[3][3], -c0[2], -c0[3]
    if (kh > 1 and coef[2][4] != 1) or (kw > 1 and coef[3][5] != 1):
        return None
    sh, sw = (sh if h > 1 else max(sh, 1)), (sw if w > 1 else max(sw, 1))
    if sh < 1 or sw < 1 or ph < 0 or pw < 0:
        return None
    H, W = x.shape[2], x.shape[3]
    op = v._op.attrs["op"]
    inside = ph == 0 and pw == 0 and (h - 1) * sh + kh <= H and (w - 1) * sw + kw <= W
    if op != "mean" and not inside:
        return None

    def run():
        xd = x._data.view(list(x.shape))
        out = _empty([N, Cn, h, w], x.dtype)
        C.check(C.lib.b200jt_pool2d(C.desc(xd), C.desc(out), ctypes.c_void_p(0), op.encode(), kh, kw, sh, sw, ph, pw, 1,
                                    C.stream_ptr()), f"pool2d x{list(x.shape)} k{(kh, kw)} s{(sh, sw)} p{(ph, pw)}")
        return _cast(out, v.dtype)

    return Plan([x], run)


def _match_softmax(v):
    """softmax / log-softmax over the last axis (or over everything) written with meta-ops as in
    python/jittor/nn.py:527-535, including the float32 round trip of bfloat16 inputs."""
    root, io = v, "float32"
    if _node(v, "unary", op="bfloat16"):
        inner = v._op.inputs[0]
        if inner._data is None and inner._op is not None and inner.dtype == "float32":
            root, io = inner, "bfloat16"
    log = False
    if _node(root, "binary", op="divide"):
        e, s = root._op.inputs
        if not _node(e, "unary", op="exp") or _last_axis_reduce(s, "add", e) is None:
            return None
        a, red = e._op.inputs[0], s
    elif _node(root, "binary", op="subtract"):
        a, l = root._op.inputs
        if not _node(l, "unary", op="log"):
            return None
        s = l._op.inputs[0]
        e = _last_axis_reduce(s, "add")
        if e is None or not _node(e, "unary", op="exp") or e._op.inputs[0] is not a:
            return None
        log, red = True, s
    else:
        return None
    if not _node(a, "binary", op="subtract"):
        return None
    xf, mx = a._op.inputs
    if _last_axis_reduce(mx, "maximum", xf) is None or mx._op.attrs["reduce_mask"] != red._op.attrs["reduce_mask"]:
        return None
    if xf.dtype != "float32":
        return None
    x = xf
    if io == "bfloat16":
        x = _strip_cast(xf, "float32")
        if x is None or x.dtype != "bfloat16":
            return None          # the float32 core is matched again when `inner` itself is realised
    rows, cols = _softmax_rows(xf, red)

    def run():
        out = _empty([rows, cols], x.dtype)
        C.check(C.lib.b200jt_softmax(C.desc(x._data, [rows, cols]), C.desc(out), int(log), C.stream_ptr()), "softmax")
        return out

    return Plan([x], run)


# --------------------------------------------------------------------------------- normalisation
def _match_moments(var_node, eps_holder):
    """var_node = maximum(x2mean - xmean*xmean, 0). Returns (xmean, x2mean) nodes."""
    if not _node(var_node, "binary", op="maximum"):
        return None
    d, zero = var_node._op.inputs
    if _const(zero) != 0 or not _node(d, "binary", op="subtract"):
        return None
    x2mean, sq = d._op.inputs
    if not _node(sq, "binary", op="multiply") or sq._op.inputs[0] is not sq._op.inputs[1]:
        return None
    return sq._op.inputs[0], x2mean


def _match_scale_shift(root):
    """root = x*W + B with W = weight / sqrt(var + eps) and B = bias - xmean*W (W, B possibly wrapped in an
    explicit broadcast_to). Returns dict(x, weight, bias, eps, xmean, x2mean, wb, bb) or None."""
    if not _node(root, "binary", op="add"):
        return None
    xm, B = root._op.inputs
    if not _node(xm, "binary", op="multiply"):
        return None
    x, W = xm._op.inputs
    wb = bb = None
    if _node(W, "broadcast_to"):
        wb, W = W, W._op.inputs[0]
    if _node(B, "broadcast_to"):
        bb, B = B, B._op.inputs[0]
    if not (_node(W, "binary", op="divide") and _node(B, "binary", op="subtract")):
        return None
    weight, sd = W._op.inputs
    if not _node(sd, "unary", op="sqrt"):
        return None
    ve = sd._op.inputs[0]
    if not _node(ve, "binary", op="add"):
        return None
    var_node, eps = ve._op.inputs
    if _const(eps) is None:
        return None
    mm = _match_moments(var_node, eps)
    if mm is None:
        return None
    xmean, x2mean = mm
    bias, mw = B._op.inputs
    if not _node(mw, "binary", op="multiply") or mw._op.inputs[0] is not xmean or mw._op.inputs[1] is not W:
        return None
    return dict(x=x, weight=weight, bias=bias, eps=float(_const(eps)), xmean=xmean, x2mean=x2mean, wb=wb, bb=bb)


def _mean_of(node, src_check, unwrap=lambda n: n):
    """node = reduce.mean(u, ...) possibly followed by mpi_all_reduce(add)/world, with `unwrap` stripping a
    dtype round trip on either side of the all-reduce. Returns (reduce node, synced)."""
    synced = False
    node = unwrap(node)
    if _node(node, "binary", op="divide") and _node(node._op.inputs[0], "mpi_all_reduce"):
        node = unwrap(node._op.inputs[0]._op.inputs[0])
        synced = True
    if not _node(node, "reduce", op="mean"):
        return None
    u = node._op.inputs[0]
    if not src_check(u):
        return None
    return node, synced


def _affine_param(p, cols):
    """A LayerNorm/BatchNorm parameter: python scalar (returns its value) or float32 Var with `cols` elements."""
    c = _const(p)
    if c is not None:
        return ("const", float(c))
    if p.dtype == "float32" and p.numel() == cols:
        return ("var", p)
    return None


def _match_layernorm(v):
    root, out_cast, x_src = v, None, None
    if _node(v, "unary", op="bfloat16"):
        inner = v._op.inputs[0]
        if inner._data is None and inner._op is not None and inner.dtype == "float32":
            out_cast, root = "bfloat16", inner
    m = _match_scale_shift(root)
    if m is None or m["wb"] is not None or m["bb"] is not None:
        return None
    x = m["x"]
    if x.dtype != "float32":
        return None
    r1 = _mean_of(m["xmean"], lambda u: u is x)
    r2 = _mean_of(m["x2mean"], lambda u: _node(u, "binary", op="multiply") and u._op.inputs[0] is x and u._op.inputs[1] is x)
    if r1 is None or r2 is None or r1[1] or r2[1]:
        return None
    red = r1[0]._op
    nd = x.ndim
    mask = red.attrs["reduce_mask"]
    if r2[0]._op.attrs["reduce_mask"] != mask or red.attrs["keepdims_mask"] & mask != mask:
        return None
    k = bin(mask).count("1")
    if mask != ((1 << k) - 1) << (nd - k):          # the last k axes
        return None
    cols = 1
    for s in x.shape[nd - k:]:
        cols *= s
    rows = x.numel() // cols if cols else 0
    g, b = _affine_param(m["weight"], cols), _affine_param(m["bias"], cols)
    if g is None or b is None:
        return None
    if (g[0] == "const" and g[1] != 1.0) or (b[0] == "const" and b[1] != 0.0):
        return None
    xin = x
    if out_cast == "bfloat16":
        src = _strip_cast(x, "float32")
        if src is None or src.dtype != "bfloat16":
            return None
        xin = src
    leaves = [xin] + [p[1] for p in (g, b) if p[0] == "var"]

    def run():
        out = _empty([rows, cols], xin.dtype)
        gd = C.desc(g[1]._data, [cols]) if g[0] == "var" else None
        bd = C.desc(b[1]._data, [cols]) if b[0] == "var" else None
        C.check(C.lib.b200jt_layer_norm(C.desc(xin._data, [rows, cols]), gd, bd, C.desc(out), m["eps"],
                                        C.stream_ptr()), "layer_norm")
        return out

    return Plan(leaves, run)


def _match_batchnorm(v):
    """Training BatchNorm of python/jittor/nn.py:671-683, optionally followed by nn.relu and optionally
    fed by an unrealised conv (whose epilogue then produces the statistics)."""
    root, relu = v, False
    if _node(v, "ternary"):
        c, y, z = v._op.inputs
        if _const(z) == 0 and _node(c, "binary", op="greater") and c._op.inputs[0] is y and _const(c._op.inputs[1]) == 0:
            root, relu = y, True
        else:
            return None
    m = _match_scale_shift(root)
    if m is None or m["wb"] is None or m["bb"] is None:
        return None
    x = m["x"]
    if x.ndim < 3 or x.dtype not in ("float32", "bfloat16") or v.dtype not in ("float32", "bfloat16"):
        return None
    nd = x.ndim
    chan_mask = ((1 << nd) - 1) & ~2                      # every axis but 1
    for bnode in (m["wb"], m["bb"]):
        if bnode._op.attrs["bcast_mask"] != chan_mask or list(bnode.shape) != list(x.shape):
            return None

    def is_x(u):
        if u is x:
            return True
        return x.dtype == "bfloat16" and _strip_cast(u, "float32") is x

    def is_xx(u):
        if _node(u, "binary", op="multiply") and u._op.inputs[0] is x and u._op.inputs[1] is x:
            return True
        if x.dtype == "bfloat16":
            w = _strip_cast(u, "float32")
            return w is not None and _node(w, "binary", op="multiply") and w._op.inputs[0] is x and w._op.inputs[1] is x
        return False

    def unwrap(n):
        # bf16 means come back through cast(bf16)(mean(cast(f32)(x)))
        if x.dtype == "bfloat16" and _node(n, "unary", op="bfloat16"):
            return n._op.inputs[0]
        return n

    r1 = _mean_of(m["xmean"], is_x, unwrap)
    r2 = _mean_of(m["x2mean"], is_xx, unwrap)
    if r1 is None or r2 is None or r1[1] != r2[1]:
        return None
    for r in (r1, r2):
        if r[0]._op.attrs["reduce_mask"] != chan_mask or r[0]._op.attrs["keepdims_mask"] != 0:
            return None
    Cn = x.shape[1]
    g, b = _affine_param(m["weight"], Cn), _affine_param(m["bias"], Cn)
    if g is None or b is None:
        return None
    synced = r1[1]
    conv = None
    if x._data is None:
        cplan = _match_conv(x)
        if cplan is not None:
            got = _mul_operands(x, 7)
            geo = conv_geometry(got[1], got[2]) or conv_geometry(got[2], got[1])
            conv = geo
    leaves = ([conv[0], conv[1]] if conv else [x]) + [p[1] for p in (g, b) if p[0] == "var"]
    running = getattr(root, "_bn_running", None)
    if running is not None:
        rm, rv = running[0].running_mean, running[0].running_var
        if rm.dtype == "float32" and rv.dtype == "float32" and rm.numel() == Cn and rv.numel() == Cn:
            leaves += [rm, rv]
        else:
            running = None

    def run():
        stats = torch.empty(2 * Cn, dtype=torch.float32, device="cuda")
        if conv:
            xd = run_conv2d(conv[0], conv[1], conv[2], x.dtype, stats=stats)
            x._data = xd                       # the conv output is a by-product other consumers may want
        else:
            xd = x._data
            C.check(C.lib.b200jt_bn_stats(C.desc(xd), ctypes.c_void_p(stats.data_ptr()), C.stream_ptr()), "bn_stats")
        count = float(x.numel() // Cn)
        if synced and tdist.is_initialized() and tdist.get_world_size() > 1:
            from . import dist
            dist.all_reduce_sum(stats, out=stats)              # sum and sum of squares in ONE 2*C message
            count *= tdist.get_world_size()

        def param(p, fill):
            if p[0] == "var":
                return p[1]._data
            return torch.full((Cn,), p[1], dtype=torch.float32, device="cuda") if p[1] != fill else None

        gt, bt = param(g, 1.0), param(b, 0.0)
        out = _empty(x.shape, v.dtype)
        rmp = rvp = 0
        momentum = 0.0
        if running is not None and getattr(root, "_bn_running", None) is not None:
            root._bn_running = None                # consumed here: the kernel updates the running statistics in place
            rmp, rvp, momentum = running[0].running_mean._data.data_ptr(), running[0].running_var._data.data_ptr(), running[0].momentum
        C.check(C.lib.b200jt_bn_apply(C.desc(xd), ctypes.c_void_p(stats.data_ptr()), count,
                                      ctypes.c_void_p(gt.data_ptr() if gt is not None else 0),
                                      ctypes.c_void_p(bt.data_ptr() if bt is not None else 0),
                                      m["eps"], int(relu), C.desc(out), ctypes.c_void_p(rmp), ctypes.c_void_p(rvp),
                                      float(momentum), C.stream_ptr()), "bn_apply")
        return out

    return Plan(leaves, run)


def _match_fused_chain(v):
    """Whatever no named pattern claimed: the maximal region of element-wise ops, broadcasts and trailing-axis reduces
    under v as ONE launch of the chain interpreter (fusion.py)."""
    from . import fusion
    prog = fusion.build_program(v)
    if prog is None:
        return None
    words, inputs, full, k, _ = prog
    leaves, seen = [], set()
    for var, _view in inputs:
        if id(var) not in seen:
            seen.add(id(var))
            leaves.append(var)

    def run():
        out = _empty(v.shape, v.dtype)
        return fusion.run_program(words, inputs, full, k, out)

    return Plan(leaves, run)


_MATCHERS = [_match_conv, _match_conv_dgrad, _match_conv_wgrad, _match_pool, _match_matmul, _match_batched_matmul, _match_softmax, _match_layernorm, _match_batchnorm,
             _match_fused_chain]
