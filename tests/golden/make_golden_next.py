"""Generate `next_ops.{json,npz}`: golden fixtures for the callers either side of the meta-operator path (slicing,
scatter/gather, pooling, grouped / transposed convolution, the data-parallel optimiser step), from the reference's own
CPU implementation. Same recipe and same bridge as make_golden.py:

    HOME=/tmp/jt_home PYTHONPATH=<reference>/python nvcc_path="" use_mkl=0 use_mpi=0 \
        cache_name=oracle python tests/golden/make_golden_next.py

Slices are stored as a list of items: {"i": int} | {"s": [start, stop, step]} | "..." | null | {"f": formula} |
{"v": k} (the k-th array of the case's `extras`).
"""
import ctypes
import json
import os

import numpy as np

import jittor as jt
from jittor import nn

HERE = os.path.dirname(os.path.abspath(__file__))
jt.flags.enable_tuner = 0
rng = np.random.default_rng(20240607)
ARRAYS, CASES = {}, []


def to_jt(a):
    a = np.ascontiguousarray(a)
    v = jt.empty(list(a.shape), str(a.dtype))
    v.sync()
    if a.nbytes:
        ctypes.memmove(v.raw_ptr, a.ctypes.data, a.nbytes)
    return v


def to_np(v):
    v.sync()
    out = np.empty(tuple(v.shape), dtype=str(v.dtype))
    if out.nbytes:
        ctypes.memmove(out.ctypes.data, v.raw_ptr, out.nbytes)
    return out


def put(name, arr):
    ARRAYS[name] = np.ascontiguousarray(arr)
    return name


def case(name, op, args, inputs, out, extras=()):
    assert name not in [c["name"] for c in CASES], name
    CASES.append({"name": name, "op": op, "args": args,
                  "inputs": [put(f"{name}/in{i}", a) for i, a in enumerate(inputs)],
                  "extras": [put(f"{name}/ex{i}", a) for i, a in enumerate(extras)],
                  "out": put(f"{name}/out", out), "out_dtype": str(out.dtype), "out_shape": list(out.shape)})


def f32(*shape):
    return rng.uniform(-1, 1, size=shape).astype(np.float32)


def i32(*shape, lo=0, hi=100):
    return rng.integers(lo, hi, size=shape).astype(np.int32)


def encode(slices, extras):
    enc = []
    for s in slices if isinstance(slices, tuple) else (slices,):
        if isinstance(s, np.ndarray):
            extras.append(s)
            enc.append({"v": len(extras) - 1})
        elif isinstance(s, slice):
            enc.append({"s": [s.start, s.stop, s.step]})
        elif s is Ellipsis:
            enc.append("...")
        elif s is None:
            enc.append(None)
        elif isinstance(s, str):
            enc.append({"f": s})
        else:
            enc.append({"i": int(s)})
    return enc


def jt_slices(slices):
    return tuple(to_jt(s) if isinstance(s, np.ndarray) else s for s in (slices if isinstance(slices, tuple) else (slices,)))


def do_getitem(name, x, slices):
    extras = []
    enc = encode(slices, extras)
    y = to_jt(x).getitem(jt_slices(slices))
    case(name, "getitem", {"slices": enc}, [x], to_np(y), extras)


def do_setitem(name, x, slices, data, op="void"):
    extras = []
    enc = encode(slices, extras)
    y = to_jt(x).setitem(jt_slices(slices), to_jt(data), op)
    case(name, "setitem", {"slices": enc, "op": op}, [x, data], to_np(y), extras)


x3 = f32(4, 5, 6)
xi = i32(4, 5, 6)
do_getitem("getitem_int", x3, 1)
do_getitem("getitem_neg_int", x3, (-1, 2))
do_getitem("getitem_all_ints", x3, (1, 2, 3))
do_getitem("getitem_slice", x3, (slice(1, 3),))
do_getitem("getitem_slice_step", x3, (slice(None), slice(0, 5, 2), slice(1, None, 3)))
do_getitem("getitem_slice_neg_step", x3, (slice(None, None, -1), slice(4, 0, -2)))
do_getitem("getitem_slice_neg_bounds", x3, (slice(-3, -1), slice(None, -2)))
do_getitem("getitem_empty_slice", x3, (slice(3, 1),))
do_getitem("getitem_ellipsis", x3, (Ellipsis, 2))
do_getitem("getitem_ellipsis_mid", x3, (1, Ellipsis, slice(0, 2)))
do_getitem("getitem_none", x3, (None, slice(None), 0))
do_getitem("getitem_none_tail", x3, (slice(None), 1, None, slice(2, 4), None))
do_getitem("getitem_var_1d", x3, (np.array([3, 0, 0, 2, 1], np.int32),))
do_getitem("getitem_var_negative", x3, (np.array([-1, 0, -4], np.int32),))
do_getitem("getitem_var_int64", xi, (slice(None), np.array([4, 4, 1], np.int64)))
do_getitem("getitem_var_2d", x3, (slice(None), np.array([[0, 1, 2], [2, 3, 4]], np.int32)))
do_getitem("getitem_two_vars", x3, (np.array([[0], [3]], np.int32), np.array([1, 2, 4], np.int32)))
do_getitem("getitem_vars_broadcast", x3, (slice(None), np.array([[0, 1, 2], [2, 3, 4]], np.int32), np.array([5, 0, 1], np.int32)))
do_getitem("getitem_vars_separated", x3, (np.array([1, 2], np.int32), slice(None), np.array([0, 5], np.int32)))
do_getitem("getitem_var_slice_int", x3, (np.array([2, 2, 0], np.int32), slice(1, 4), 3))
do_getitem("getitem_formula", x3, ("i0", np.array([[0, 4], [1, 1], [2, 0], [3, 3]], np.int32), "i1"))
do_getitem("getitem_int8", rng.integers(-100, 100, size=(7, 9)).astype(np.int8), (slice(1, 6, 2), slice(None, None, -1)))
do_getitem("getitem_float64", rng.normal(size=(6, 3)), (np.array([5, 1], np.int32), 2))
do_getitem("getitem_1d_large", f32(100000), (slice(3, 99999, 7),))

do_setitem("setitem_int", x3, 1, f32(5, 6))
do_setitem("setitem_scalar", x3, (slice(1, 3), slice(None, None, 2)), np.array([7.0], np.float32))
do_setitem("setitem_slice_bcast", x3, (slice(None), slice(1, 4)), f32(6))
do_setitem("setitem_slice_bcast_mid", x3, (slice(0, 2),), f32(5, 1))
do_setitem("setitem_neg_step", xi, (slice(None, None, -1), 0), i32(4, 6))
do_setitem("setitem_ellipsis", x3, (Ellipsis, 5), f32(4, 5))
do_setitem("setitem_none", x3, (None, 2), f32(1, 5, 6))
do_setitem("setitem_var_unique", x3, (np.array([3, 0, 2], np.int32),), f32(3, 5, 6))
do_setitem("setitem_var_2axes", x3, (np.array([0, 1, 3], np.int32), np.array([4, 4, 0], np.int32)), f32(3, 6))
do_setitem("setitem_var_add_dup", x3, (np.array([1, 1, 1, 0], np.int32),), f32(4, 5, 6), "add")
do_setitem("setitem_int_add_dup", xi, (slice(None), np.array([2, 2, 4, 2], np.int32)), i32(4, 4, 6), "add")
do_setitem("setitem_var_max", x3, (np.array([1, 1, 2], np.int32),), f32(3, 5, 6), "maximum")
do_setitem("setitem_var_min", x3, (np.array([1, 1, 2], np.int32),), f32(3, 5, 6), "minimum")
do_setitem("setitem_var_mul", x3, (slice(None), np.array([0, 3], np.int32)), f32(4, 2, 6), "multiply")
do_setitem("setitem_cast_data", xi, (slice(1, 2),), f32(1, 5, 6) * 50)


def do_scatter(name, x, dim, index, src, reduce="void"):
    y = to_jt(x).scatter(dim, to_jt(index), to_jt(src), reduce)
    case(name, "scatter", {"dim": dim, "reduce": reduce}, [x, src], to_np(y), [index])


def do_gather(name, x, dim, index):
    y = to_jt(x).gather(dim, to_jt(index))
    case(name, "gather", {"dim": dim}, [x], to_np(y), [index])


srcs = np.arange(1, 11, dtype=np.int32).reshape(2, 5)
do_scatter("scatter_dim0", np.zeros((3, 5), np.int32), 0, np.array([[0, 1, 2, 0]], np.int32), srcs)
do_scatter("scatter_dim1", np.zeros((3, 5), np.int32), 1, np.array([[0, 1, 2], [0, 1, 4]], np.int32), srcs)
do_scatter("scatter_scalar_mul", np.full((2, 4), 2.0, np.float32), 1, np.array([[2], [3]], np.int32),
           np.array([1.23], np.float32), "multiply")
do_scatter("scatter_scalar_add", np.full((2, 4), 2.0, np.float32), 1, np.array([[2], [3]], np.int32),
           np.array([1.23], np.float32), "add")
perm = np.stack([rng.permutation(50) for _ in range(8)]).astype(np.int32)
do_scatter("scatter_perm_dim1", f32(8, 64), 1, perm, f32(8, 50))
do_scatter("scatter_add_dup_3d", f32(5, 6, 7), 2, i32(5, 6, 20, hi=7), f32(5, 6, 20), "add")
do_scatter("scatter_add_dup_dim0_int", i32(9, 4), 0, i32(30, 4, hi=9), i32(30, 4), "add")
do_gather("gather_dim1", np.array([[1, 2], [3, 4]], np.int32), 1, np.array([[0, 0], [1, 0]], np.int32))
do_gather("gather_dim0", np.array([[1, 2], [3, 4]], np.int32), 0, np.array([[0, 0], [1, 0]], np.int32))
do_gather("gather_3d_dim2", f32(5, 6, 7), 2, i32(5, 6, 11, hi=7))
do_gather("gather_3d_dim0_smaller", f32(5, 6, 7), 0, i32(3, 4, 7, hi=5))
do_gather("gather_int64_index", f32(10, 3), 0, rng.integers(0, 10, size=(4, 3)).astype(np.int64))



# ---- optimiser steps on a small least-squares problem: loss = sum((x @ w - y)^2) / N ------------------------------
def do_optim(name, kind, steps, **kw):
    x, y, w0 = f32(32, 6), f32(32, 3), f32(6, 3)
    w = to_jt(w0)
    vx, vy = to_jt(x), to_jt(y)
    opt = {"sgd": jt.optim.SGD, "adam": jt.optim.Adam, "adamw": jt.optim.AdamW, "rmsprop": jt.optim.RMSprop}[kind]([w], **kw)
    for _ in range(steps):
        d = jt.matmul(vx, w) - vy
        loss = (d * d).sum() * (1.0 / 32)
        opt.step(loss)
    case(name, "optim", dict(kind=kind, steps=steps, **{k: (list(v) if isinstance(v, tuple) else v) for k, v in kw.items()}),
         [x, y, w0], to_np(w))


do_optim("sgd_plain", "sgd", 3, lr=0.1)
do_optim("sgd_momentum_wd", "sgd", 4, lr=0.05, momentum=0.9, weight_decay=0.01)
do_optim("sgd_nesterov_dampening", "sgd", 4, lr=0.05, momentum=0.8, dampening=0.1, nesterov=True)
do_optim("adam_default", "adam", 4, lr=0.01)
do_optim("adam_wd_betas", "adam", 3, lr=0.02, eps=1e-6, betas=(0.8, 0.9), weight_decay=0.1)



# ---- pooling: forward, and backward through jt.grad with a random upstream gradient -------------------------------
from jittor import pool as jpool


def do_pool(name, x, kernel_size, op, stride=None, padding=0, ceil_mode=False, count_include_pad=True, backward=True):
    args = dict(kernel_size=kernel_size, op=op, stride=stride, padding=padding, ceil_mode=ceil_mode,
                count_include_pad=count_include_pad)
    vx = to_jt(x)
    layer = jpool.Pool(kernel_size, stride, padding, ceil_mode=ceil_mode, count_include_pad=count_include_pad, op=op)
    y = layer(vx)
    ynp = to_np(y)
    case(name, "pool2d", args, [x], ynp)
    if backward:
        dy = f32(*ynp.shape)
        dx = jt.grad((y * to_jt(dy)).sum(), vx)
        case(name + "_bwd", "pool2d_bwd", args, [x, dy], to_np(dx))


ties = rng.integers(0, 3, size=(2, 3, 9, 11)).astype(np.float32)        # many equal values: the first-match rule decides
do_pool("pool_max_2x2", f32(2, 3, 8, 10), 2, "maximum")
do_pool("pool_max_3x3_s2_p1", f32(2, 3, 9, 11), 3, "maximum", 2, 1)
do_pool("pool_max_ties", ties, 3, "maximum", 2, 1)
do_pool("pool_max_ties_overlap_s1", ties, 2, "maximum", 1, 0)
do_pool("pool_max_ceil", f32(1, 2, 10, 10), 3, "maximum", 2, 0, True)
do_pool("pool_max_rect", f32(2, 2, 12, 9), (3, 2), "maximum", (2, 1), (1, 0))
do_pool("pool_min_3x3_s2_p1", f32(2, 3, 9, 11), 3, "minimum", 2, 1)
do_pool("pool_min_ties", ties, 2, "minimum", 2, 0)
do_pool("pool_mean_2x2", f32(2, 3, 8, 10), 2, "mean")
do_pool("pool_mean_3x3_s2_p1", f32(2, 3, 9, 11), 3, "mean", 2, 1)
do_pool("pool_mean_p1_no_count_pad", f32(2, 3, 9, 11), 3, "mean", 2, 1, False, False)
do_pool("pool_mean_ceil", f32(1, 2, 10, 10), 3, "mean", 2, 0, True)
do_pool("pool_mean_ceil_p1_count_pad", f32(1, 2, 10, 10), 3, "mean", 2, 1, True, True)
do_pool("pool_mean_ceil_p1_no_count_pad", f32(1, 2, 10, 10), 3, "mean", 2, 1, True, False)
do_pool("pool_max_64ch", f32(2, 64, 28, 28), 3, "maximum", 2, 1)



# ---- grouped convolution and transposed convolution through the reference's nn layers ------------------------------
def do_gconv(name, x, w, stride, padding, dilation, groups, bias=None):
    m = nn.Conv(x.shape[1], w.shape[0], (w.shape[2], w.shape[3]), stride, padding, dilation, groups, bias is not None)
    m.weight = to_jt(w)
    if bias is not None:
        m.bias = to_jt(bias)
    y = m(to_jt(x))
    case(name, "conv_grouped", dict(stride=stride, padding=padding, dilation=dilation, groups=groups, bias=bias is not None),
         [x, w] + ([bias] if bias is not None else []), to_np(y))


def do_tconv(name, x, w, stride, padding, output_padding, groups, dilation, bias=None):
    m = nn.ConvTranspose(x.shape[1], w.shape[1] * groups, (w.shape[2], w.shape[3]), stride, padding, output_padding,
                         groups, bias is not None, dilation)
    m.weight = to_jt(w)
    if bias is not None:
        m.bias = to_jt(bias)
    y = m(to_jt(x))
    case(name, "conv_transpose", dict(stride=stride, padding=padding, output_padding=output_padding, groups=groups,
                                      dilation=dilation, bias=bias is not None),
         [x, w] + ([bias] if bias is not None else []), to_np(y))


def wgt(*shape):
    return (rng.normal(size=shape) * 0.2).astype(np.float32)


do_gconv("gconv_g2", f32(2, 8, 9, 9), wgt(12, 4, 3, 3), 1, 1, 1, 2)
do_gconv("gconv_g4_s2_bias", f32(2, 8, 10, 11), wgt(8, 2, 3, 3), 2, 1, 1, 4, f32(8))
do_gconv("gconv_g2_dilated", f32(1, 6, 12, 12), wgt(4, 3, 3, 3), 1, 2, 2, 2)
do_gconv("gconv_depthwise", f32(2, 16, 10, 10), wgt(16, 1, 3, 3), 1, 1, 1, 16)
do_gconv("gconv_depthwise_mult2_s2", f32(2, 6, 11, 9), wgt(12, 1, 3, 3), 2, 1, 1, 6)
do_gconv("gconv_g8_1x1", f32(2, 64, 7, 7), wgt(64, 8, 1, 1), 1, 0, 1, 8)
do_tconv("tconv_basic", f32(2, 4, 5, 6), wgt(4, 3, 3, 3), 1, 0, 0, 1, 1)
do_tconv("tconv_s2_p1_op1_bias", f32(2, 4, 5, 6), wgt(4, 6, 3, 3), 2, 1, 1, 1, 1, f32(6))
do_tconv("tconv_s3_k2", f32(1, 3, 4, 4), wgt(3, 5, 2, 2), 3, 0, 2, 1, 1)
do_tconv("tconv_dilated", f32(1, 3, 6, 6), wgt(3, 2, 3, 3), 1, 1, 0, 1, 2)
do_tconv("tconv_rect_kernel", f32(2, 3, 5, 7), wgt(3, 4, 2, 4), (2, 1), (0, 1), 0, 1, 1)
do_tconv("tconv_g2_in_eq_out", f32(2, 6, 5, 5), wgt(6, 3, 3, 3), 2, 1, 1, 2, 1)
do_tconv("tconv_g4_in_eq_out", f32(1, 8, 4, 6), wgt(8, 2, 4, 4), 2, 1, 0, 4, 1, f32(8))



# ---- gradients of the reindex-lowered conv (data and weight) through jt.grad --------------------------------------
def do_conv_grad(name, x, w, stride, padding, dilation):
    m = nn.Conv(x.shape[1], w.shape[0], (w.shape[2], w.shape[3]), stride, padding, dilation, 1, False)
    vx, vw = to_jt(x), to_jt(w)
    m.weight = vw
    y = m(vx)
    dy = f32(*y.shape)
    dx, dw = jt.grad((y * to_jt(dy)).sum(), [vx, vw])
    args = dict(stride=stride, padding=padding, dilation=dilation)
    case(name + "_dx", "conv_dgrad", args, [x, w, dy], to_np(dx))
    case(name + "_dw", "conv_wgrad", args, [x, w, dy], to_np(dw))


do_conv_grad("conv_grad_s1_p1", f32(2, 5, 9, 10), wgt(7, 5, 3, 3), 1, 1, 1)
do_conv_grad("conv_grad_s2_p1", f32(2, 4, 11, 9), wgt(6, 4, 3, 3), 2, 1, 1)
do_conv_grad("conv_grad_dilated", f32(1, 3, 12, 12), wgt(4, 3, 3, 3), 1, 2, 2)
do_conv_grad("conv_grad_1x1_s2", f32(2, 8, 8, 8), wgt(5, 8, 1, 1), 2, 0, 1)



# ---- adaptive pooling (meta-operator lowering in the reference) ----------------------------------------------------
def do_adaptive(name, x, output_size, op):
    layer = (jpool.AdaptiveAvgPool2d if op == "mean" else jpool.AdaptiveMaxPool2d)(output_size)
    case(name, "adaptive_pool", {"output_size": list(output_size) if isinstance(output_size, tuple) else output_size, "op": op},
         [x], to_np(layer(to_jt(x))))


do_adaptive("adaptive_avg_7", f32(2, 3, 21, 30), 7, "mean")
do_adaptive("adaptive_avg_1", f32(2, 3, 9, 11), 1, "mean")
do_adaptive("adaptive_avg_rect_none", f32(1, 4, 10, 13), (None, 4), "mean")
do_adaptive("adaptive_max_5x3", f32(2, 3, 17, 10), (5, 3), "maximum")



# ---- Conv1d through the reference's layer ---------------------------------------------------------------------------
def do_conv1d(name, x, w, stride, padding, dilation, groups, bias=None):
    m = nn.Conv1d(x.shape[1], w.shape[0], w.shape[2], stride, padding, dilation, groups, bias is not None)
    m.weight = to_jt(w)
    if bias is not None:
        m.bias = to_jt(bias)
        m._conv[0].bias = m.bias
    y = m(to_jt(x))
    case(name, "conv1d", dict(stride=stride, padding=padding, dilation=dilation, groups=groups, bias=bias is not None),
         [x, w] + ([bias] if bias is not None else []), to_np(y))


do_conv1d("conv1d_basic", f32(2, 6, 40), wgt(8, 6, 3), 1, 0, 1, 1)
do_conv1d("conv1d_s2_p1_bias", f32(3, 4, 33), wgt(5, 4, 5), 2, 1, 1, 1, f32(5))
do_conv1d("conv1d_dilated_grouped", f32(2, 8, 50), wgt(12, 2, 3), 1, 2, 2, 4)


do_optim("adamw_wd", "adamw", 4, lr=0.02, weight_decay=0.1)
do_optim("rmsprop_default", "rmsprop", 4, lr=0.01)
do_optim("rmsprop_alpha", "rmsprop", 3, lr=0.02, eps=1e-6, alpha=0.9)

np.savez_compressed(os.path.join(HERE, "next_ops.npz"), **ARRAYS)
with open(os.path.join(HERE, "next_ops.json"), "w") as f:
    json.dump({"generator": "tests/golden/make_golden_next.py", "reference_version": jt.__version__, "cases": CASES},
              f, indent=1)
print("cases:", len(CASES), "arrays:", len(ARRAYS), "npz bytes:", os.path.getsize(os.path.join(HERE, "next_ops.npz")))
