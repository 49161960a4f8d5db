"""Generate the golden fixtures in this folder from the reference's own CPU implementation.

Run once, in a container that has the reference checkout (it is never needed at test time):

    HOME=/tmp/jt_home PYTHONPATH=<reference>/python nvcc_path="" use_mkl=0 use_mpi=0 \
        cache_name=oracle python tests/golden/make_golden.py

The reference is imported as `jittor`; every case below is executed by its CPU executor
(g++-compiled JIT kernels, tuners disabled: no vendor library is involved) and the inputs,
arguments and outputs are written to `meta_ops.npz` + `meta_ops.json`.

The reference's numpy bridge assumes the numpy-1 struct layout, so arrays are moved through
`Var.raw_ptr` with `ctypes.memmove` instead of `jt.array()` / `Var.numpy()`.

A case is a dict {name, op, args, inputs:[npz keys], extras:[npz keys], out: npz key}. The same
manifest drives the CPU tests of the oracle and the GPU parity tests of the CUDA path.
"""
import ctypes
import json
import os
import re
import sys

import numpy as np

import jittor as jt
from jittor import nn

HERE = os.path.dirname(os.path.abspath(__file__))
jt.flags.enable_tuner = 0

ARRAYS = {}
CASES = []


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


def guarded(fn):
    """The reference rejects some inputs at JIT-compile time; such a case is reported and skipped."""
    def wrapper(name, *a, **k):
        try:
            fn(name, *a, **k)
        except Exception as e:  # noqa: BLE001
            msg = str(e)
            m = re.search(r"error: [^\n]*", msg)
            print("SKIPPED (reference failed):", name, "--", m.group(0) if m else msg[-200:])
    return wrapper


def case(name, op, args, inputs, out, extras=()):
    """inputs/extras: numpy arrays; out: numpy array produced by the reference."""
    assert name not in [c["name"] for c in CASES], name
    rec = {"name": name, "op": op, "args": args,
           "inputs": [put(f"{name}/in{i}", a) for i, a in enumerate(inputs)],
           "extras": [put(f"{name}/ex{i}", a) for i, a in enumerate(extras)],
           "out": put(f"{name}/out", out),
           "out_dtype": str(out.dtype), "out_shape": list(out.shape)}
    CASES.append(rec)


rng = np.random.default_rng(20240)


def f32(*shape, lo=-1.0, hi=1.0):
    return rng.uniform(lo, hi, size=shape).astype(np.float32)


def i32(*shape, lo=0, hi=100):
    return rng.integers(lo, hi, size=shape).astype(np.int32)


# ---------------------------------------------------------------- reindex
@guarded
def do_reindex(name, x, shape, indexes, overflow_value=0, overflow_conditions=(), extras=()):
    v = to_jt(x)
    ex = [to_jt(e) for e in extras]
    y = v.reindex(shape, list(indexes), overflow_value, list(overflow_conditions), ex)
    case(name, "reindex", {"shape": list(shape), "indexes": list(indexes),
                           "overflow_value": overflow_value,
                           "overflow_conditions": list(overflow_conditions)},
         [x], to_np(y), extras)


do_reindex("reindex_pad", f32(10), [17], ["i0-3"], -1)
do_reindex("reindex_pad_i32", i32(10), [17], ["i0-3"], -7)
do_reindex("reindex_pad_f64", rng.normal(size=10), [17], ["i0-3"], 5)
do_reindex("reindex_pad_i64", rng.integers(-2**40, 2**40, size=10), [17], ["i0-3"], -1)
do_reindex("reindex_pad_u8", rng.integers(0, 255, size=33).astype(np.uint8), [40], ["i0-3"], 9)
do_reindex("reindex_pad_i8", rng.integers(-128, 127, size=33).astype(np.int8), [40], ["i0-3"], -9)
do_reindex("reindex_pad_i16", rng.integers(-3000, 3000, size=33).astype(np.int16), [40], ["i0-4"], -9)
do_reindex("reindex_matmul_a", f32(10, 10), [10, 10, 10], ["i0", "i1"])
do_reindex("reindex_matmul_b", f32(10, 10), [10, 10, 10], ["i1", "i2"])
do_reindex("reindex_transpose", f32(7, 5), [5, 7], ["i1", "i0"])
do_reindex("reindex_flip", f32(4, 9), [4, 9], ["i0", "8-i1"])
do_reindex("reindex_conv_nhwc", f32(2, 5, 5, 2), [2, 7, 7, 3, 3, 2, 2],
           ["i0", "i1-i3", "i2-i4", "i5"])
do_reindex("reindex_convT_nhwc", f32(2, 4, 4, 2), [2, 10, 10, 3, 3, 2, 2],
           ["i0", "(i1-i3)/2", "(i2-i4)/2", "i5"], 0, ["(i1-i3)%2", "(i2-i4)%2"])
do_reindex("reindex_conv_nchw_s2p1d2", f32(2, 3, 9, 8), [2, 4, 3, 4, 4, 3, 3],
           ["i0", "i2", "i3*2-1+i5*2", "i4*2-1+i6*2"])
do_reindex("reindex_conv_nchw_s1p1", f32(2, 3, 6, 6), [2, 4, 3, 6, 6, 3, 3],
           ["i0", "i2", "i3*1-1+i5*1", "i4*1-1+i6*1"])
do_reindex("reindex_divmod_neg", f32(6, 6), [9, 9], ["(i0-4)/2+2", "(i1-4)%3+2"])
do_reindex("reindex_cond_cmp", f32(6, 6), [6, 6], ["i0", "i1"], 3, ["i0 > i1", "i0+i1==4"])
do_reindex("reindex_cond_logic", f32(6, 6), [6, 6], ["i1", "i0"], -2, ["i0<2 && i1>=3 || i0==5"])
do_reindex("reindex_shape_syms", f32(5, 6), [5, 6], ["xshape0-1-i0", "yshape1-1-i1"], 0)
do_reindex("reindex_extras_1d", f32(10, 10), [8, 8], ["@e0(i0)", "@e1(i1)"],
           0, (), [i32(8, lo=-2, hi=12), i32(8, lo=-2, hi=12)])
do_reindex("reindex_extras_2d", f32(10, 10), [8, 8], ["@e0(i0,i1)", "@e1(i1,i0)+1"],
           -1, (), [i32(8, 8, lo=-2, hi=12), i32(8, 8, lo=0, hi=9)])
do_reindex("reindex_extras_nested", f32(10, 10), [8, 8], ["@e0(0)", "@e1(0,i0/@e0(0))"],
           0, (), [np.array([1], dtype=np.int32), i32(10, 10, lo=0, hi=10)])
do_reindex("reindex_extras_i64", f32(50), [20], ["@e0(i0)"], 0, (),
           [rng.integers(-5, 55, size=20)])
do_reindex("reindex_gather_rows", f32(16, 33), [9, 33], ["@e0(i0)", "i1"], 0, (),
           [i32(9, lo=0, hi=16)])
do_reindex("reindex_bool", rng.integers(0, 2, size=(5, 5)).astype(bool), [7, 7], ["i0-1", "i1-1"], 1)
do_reindex("reindex_zero_size", f32(4, 4), [0, 4], ["i0", "i1"])
do_reindex("reindex_big_rows", f32(3, 1000), [3, 1003], ["i0", "i1-2"], -5)


@guarded
def do_reindex_var(name, x, idx):
    v = to_jt(x)
    y = v.reindex_var([to_jt(i) for i in idx], 0, [])
    case(name, "reindex_var", {"overflow_value": 0, "overflow_conditions": []}, [x], to_np(y), idx)


do_reindex_var("reindex_var_2d", f32(5, 5), [i32(4, 5, 5, lo=-1, hi=6), i32(4, 5, 5, lo=-1, hi=6)])

# bf16 is a pure bit copy for a gather; stored as uint16 bit patterns
xb = (f32(12, 12).view(np.uint32) >> 16).astype(np.uint16)
xv = to_jt((xb.astype(np.uint32) << 16).view(np.float32)).bfloat16()
yv = xv.reindex([14, 14], ["i0-1", "i1-1"], -1.0).float32()
case("reindex_bf16_bits", "reindex",
     {"shape": [14, 14], "indexes": ["i0-1", "i1-1"], "overflow_value": -1.0,
      "overflow_conditions": [], "bf16_bits": True},
     [xb], (to_np(yv).view(np.uint32) >> 16).astype(np.uint16))


# ---------------------------------------------------------------- reindex_reduce
@guarded
def do_rr(name, y, op, shape, indexes, overflow_conditions=(), extras=()):
    v = to_jt(y)
    ex = [to_jt(e) for e in extras]
    x = v.reindex_reduce(op, list(shape), list(indexes), list(overflow_conditions), ex)
    case(name, "reindex_reduce", {"op": op, "shape": list(shape), "indexes": list(indexes),
                                  "overflow_conditions": list(overflow_conditions)},
         [y], to_np(x), extras)


for op in ["add", "maximum", "minimum", "multiply"]:
    do_rr(f"rr_pool_{op}", f32(3, 10, 10, 4, lo=0.0, hi=1.0), op, [3, 4, 4, 4],
          ["i0", "i1/3", "i2/3", "i3"])
    do_rr(f"rr_pool_{op}_i32", i32(2, 7, 7, 3, lo=-9, hi=10), op, [2, 3, 3, 3],
          ["i0", "i1/3", "i2/3", "i3"])
for op in ["maximum", "minimum"]:
    do_rr(f"rr_{op}_neg_f32", f32(4, 9, lo=-5.0, hi=-1.0), op, [4, 5], ["i0", "i1/2"])
    do_rr(f"rr_{op}_hole_f32", f32(4, 9, lo=-5.0, hi=5.0), op, [4, 12], ["i0", "i1*2"])
    do_rr(f"rr_{op}_f64", rng.normal(size=(4, 9)), op, [4, 5], ["i0", "i1/2"])
    do_rr(f"rr_{op}_i64", rng.integers(-2**40, 2**40, size=(4, 9)), op, [4, 12], ["i0", "i1/2"])
for op in ["bitwise_and", "bitwise_or", "bitwise_xor"]:
    do_rr(f"rr_{op}_i32", i32(64, lo=0, hi=2**20), op, [8], ["i0%8"])
do_rr("rr_scatter_add_i32", i32(4096, lo=0, hi=100), "add", [257], ["@e0(i0)"], (),
      [i32(4096, lo=-3, hi=260)])
do_rr("rr_scatter_add_f32", f32(4096), "add", [64], ["@e0(i0)"], (), [i32(4096, lo=0, hi=64)])
do_rr("rr_scatter_add_f64", rng.normal(size=4096), "add", [64], ["@e0(i0)"], (),
      [i32(4096, lo=0, hi=64)])
do_rr("rr_scatter_add_i64", rng.integers(-2**40, 2**40, size=4096), "add", [64], ["@e0(i0)"], (),
      [i32(4096, lo=0, hi=64)])
do_rr("rr_scatter_max_f32", f32(4096, lo=-3, hi=3), "maximum", [100], ["@e0(i0)"], (),
      [i32(4096, lo=0, hi=90)])
do_rr("rr_scatter_min_i32", i32(4096, lo=-50, hi=50), "minimum", [100], ["@e0(i0)"], (),
      [i32(4096, lo=0, hi=90)])
do_rr("rr_scatter_2d", f32(3, 3), "add", [4, 4], ["@e0(i0,i1)", "@e0(i1,i0)"], (),
      [i32(3, 3, lo=-1, hi=5)])
do_rr("rr_scatter_e0_rows", i32(3, 3), "add", [4, 4], ["@e0(i0)", "@e0(i1)"], (),
      [np.array([-1, -2, -3, -4], dtype=np.int32)])
do_rr("rr_pool_bwd_perm", f32(2, 3, 4, 5, 2, 2), "add", [2, 3, 8, 10],
      ["i0", "i1", "i2*2+i4", "i3*2+i5"])
do_rr("rr_cond", f32(6, 6), "add", [6], ["i0"], ["i1 > i0"])
do_rr("rr_identity", f32(3), "add", [3], ["i0"])
do_rr("rr_conv_dgrad_form", f32(2, 4, 3, 4, 4, 3, 3), "add", [2, 3, 6, 6],
      ["i0", "i2", "i3*1-1+i5*1", "i4*1-1+i6*1"])


# ---------------------------------------------------------------- broadcast
@guarded
def do_bcast(name, x, shape, dims=()):
    z = jt.broadcast(to_jt(x), list(shape), list(dims))
    case(name, "broadcast", {"shape": list(shape), "dims": list(dims)}, [x], to_np(z))


@guarded
def do_bcast_var(name, x, y, dims=()):
    z = jt.broadcast_var(to_jt(x), to_jt(y), list(dims))
    case(name, "broadcast_var", {"dims": list(dims)}, [x, y], to_np(z))


def gen(shape, dt=np.int32):
    return np.arange(int(np.prod(shape))).reshape(shape).astype(dt)


for k, (s1, s2) in enumerate([([1], [3]), ([3, 1], [3]), ([3, 1, 3], [1, 3, 1]),
                              ([2, 3, 4], [2, 3, 4, 1, 1, 1]), ([2, 3], [2, 3, 1, 1]),
                              ([2, 1, 3, 1, 4], [1, 3, 4])]):
    do_bcast(f"bcast_shape_{k}", gen(s1), s2)
    do_bcast_var(f"bcast_var_{k}", gen(s1), gen(s2))
do_bcast("bcast_dims_m1", np.array([1, 2], dtype=np.int32), [2, 2], [-1])
do_bcast("bcast_dims_m2", np.array([1, 2], dtype=np.int32), [2, 2], [-2])
do_bcast("bcast_conv_w", f32(4, 3, 3, 3), [2, 4, 3, 5, 5, 3, 3], [0, 3, 4])
do_bcast("bcast_mm_a", f32(5, 7), [5, 7, 6], [-1])
do_bcast("bcast_mm_b", f32(7, 6), [5, 7, 6], [-3])
do_bcast("bcast_f64", rng.normal(size=(3, 1)), [3, 4])
do_bcast("bcast_u8", rng.integers(0, 255, size=(1, 5)).astype(np.uint8), [4, 5])
do_bcast("bcast_bn_w", f32(5), [2, 5, 3, 3], [0, 2, 3])


# ---------------------------------------------------------------- reduce
@guarded
def do_reduce(name, x, op, dims, keepdims=False):
    v = to_jt(x)
    y = jt.reduce(v, op, dims, keepdims) if dims != () else jt.reduce(v, op, keepdims=keepdims)
    case(name, "reduce", {"op": op, "dims": list(dims) if isinstance(dims, (tuple, list)) else dims,
                          "keepdims": keepdims}, [x], to_np(y))


ia = (gen([2, 3, 4, 5]) % 7 + 1).astype(np.int32)
idims = [(), (0,), (1,), (2,), (3,), (0, 2), (1, 3), (1, 2, 3), 2, 3, -1, (-1, -3)]
for k, d in enumerate(idims):
    do_reduce(f"reduce_add_i32_d{k}", ia, "add", d)
    do_reduce(f"reduce_add_i32_keep_d{k}", ia, "add", d, True)
for op in ["add", "multiply", "maximum", "minimum", "bitwise_and", "bitwise_or", "bitwise_xor",
           "logical_and", "logical_or", "logical_xor", "mean"]:
    do_reduce(f"reduce_{op}_i32_all", ia, op, ())
    do_reduce(f"reduce_{op}_i32_13", ia, op, (1, 3))
fa = f32(4, 6, 5, 7)
for op in ["add", "multiply", "maximum", "minimum", "mean"]:
    for k, d in enumerate([(), (3,), (0,), (1, 2), (0, 2, 3), (1, 3)]):
        do_reduce(f"reduce_{op}_f32_d{k}", fa, op, d)
do_reduce("reduce_add_f32_rows", f32(33, 1000), "add", (1,))
do_reduce("reduce_max_f32_rows_keep", f32(33, 1000), "maximum", (1,), True)
do_reduce("reduce_add_f32_cols", f32(1000, 33), "add", (0,))
do_reduce("reduce_mean_f32_bn", f32(6, 5, 7, 7), "mean", (0, 2, 3))
do_reduce("reduce_add_f64", rng.normal(size=(9, 11)), "add", (1,))
do_reduce("reduce_add_i64", rng.integers(-2**40, 2**40, size=(9, 11)), "add", (0,))
do_reduce("reduce_add_bool", rng.integers(0, 2, size=(9, 11)).astype(bool), "add", (0,))
do_reduce("reduce_max_neg_f32", f32(5, 9, lo=-9, hi=-1), "maximum", (1,))


# ---------------------------------------------------------------- element-wise
@guarded
def do_binary(name, a, b, op):
    z = jt.binary(to_jt(a), to_jt(b), op)
    case(name, "binary", {"op": op}, [a, b], to_np(z))


@guarded
def do_unary(name, a, op):
    z = jt.unary(to_jt(a), op)
    case(name, "unary", {"op": op}, [a], to_np(z))


for op in ["add", "subtract", "multiply", "divide", "maximum", "minimum", "equal", "less",
           "greater", "not_equal", "less_equal", "greater_equal", "pow"]:
    do_binary(f"binary_{op}_f32", f32(5, 7, lo=0.1, hi=2.0), f32(5, 7, lo=0.1, hi=2.0), op)
    do_binary(f"binary_{op}_f32_bcast", f32(5, 7, lo=0.1, hi=2.0), f32(5, 1, lo=0.1, hi=2.0), op)
for op in ["add", "subtract", "multiply", "divide", "maximum", "minimum", "equal", "mod",
           "floor_divide", "bitwise_and", "bitwise_or", "bitwise_xor", "left_shift", "right_shift"]:
    do_binary(f"binary_{op}_i32", i32(5, 7, lo=-20, hi=20), i32(5, 7, lo=1, hi=5), op)
do_binary("binary_add_i32_f32", i32(5, 7), f32(5, 7), "add")
do_binary("binary_mul_bcast_both", f32(3, 1, 5), f32(1, 4, 1), "multiply")
for op in ["exp", "sqrt", "log", "abs", "negative", "float32", "int32", "float64", "tanh", "sigmoid",
           "floor", "ceil", "round", "logical_not", "bool", "int8", "uint8", "int64", "erf", "sin", "cos"]:
    do_unary(f"unary_{op}_f32", f32(5, 7, lo=0.1, hi=3.0), op)
do_unary("unary_float32_i32", i32(5, 7, lo=-20, hi=20), "float32")
do_unary("unary_negative_i32", i32(5, 7, lo=-20, hi=20), "negative")
do_unary("unary_abs_i32", i32(5, 7, lo=-20, hi=20), "abs")

c3, a3, b3 = rng.integers(0, 2, size=(5, 7)).astype(bool), f32(5, 7), f32(5, 7)
case("ternary_f32", "ternary", {}, [c3, a3, b3], to_np(jt.ternary(to_jt(c3), to_jt(a3), to_jt(b3))))


# ---------------------------------------------------------------- fused chains (nn callers)
@guarded
def do_conv(name, x, w, stride, padding, dilation, bias=None):
    co, ci, kh, kw = w.shape
    m = nn.Conv(ci, co, (kh, kw), stride, padding, dilation, bias=bias is not None)
    m.weight = to_jt(w)
    ins = [x, w]
    if bias is not None:
        m.bias = to_jt(bias)
        ins.append(bias)
    y = m(to_jt(x))
    case(name, "conv", {"stride": stride, "padding": padding, "dilation": dilation,
                        "bias": bias is not None}, ins, to_np(y))


r1 = np.random.default_rng(0)   # config-0 of the benchmark list: seed = config index
x1 = r1.uniform(-1, 1, size=(4, 32, 32, 32)).astype(np.float32)
w1 = (r1.normal(size=(64, 32, 3, 3)) * 0.05).astype(np.float32)
do_conv("conv_c1_full", x1, w1, 1, 1, 1)
do_conv("conv_small_s1p1", f32(2, 3, 6, 6), f32(4, 3, 3, 3), 1, 1, 1)
do_conv("conv_small_s2p1", f32(2, 3, 9, 8), f32(4, 3, 3, 3), 2, 1, 1)
do_conv("conv_small_s1p2d2", f32(2, 3, 9, 8), f32(4, 3, 3, 3), 1, 2, 2)
do_conv("conv_small_s3p0", f32(1, 2, 11, 10), f32(5, 2, 3, 3), 3, 0, 1)
do_conv("conv_small_1x1", f32(2, 6, 5, 5), f32(7, 6, 1, 1), 1, 0, 1)
do_conv("conv_small_5x3_bias", f32(2, 3, 9, 8), f32(4, 3, 5, 3), 1, 1, 1, f32(4))
do_conv("conv_mid_16c", f32(2, 16, 14, 14), f32(32, 16, 3, 3) * 0.2, 1, 1, 1)


@guarded
def do_matmul(name, a, b):
    c = nn.matmul(to_jt(a), to_jt(b))
    case(name, "matmul", {}, [a, b], to_np(c))


do_matmul("matmul_2d", f32(33, 47), f32(47, 29))
do_matmul("matmul_2d_128", f32(128, 256) * 0.1, f32(256, 192) * 0.1)
do_matmul("matmul_vec_b", f32(9, 7), f32(7))
do_matmul("matmul_vec_a", f32(9), f32(9, 7))
do_matmul("matmul_3d_2d", f32(3, 5, 7), f32(7, 4))
do_matmul("matmul_bcast", f32(4, 1, 3, 6), f32(5, 6, 2))
for ta in (0, 1):
    for tb in (0, 1):
        a = f32(*( (31, 17) if not ta else (17, 31)))
        b = f32(*( (17, 23) if not tb else (23, 17)))
        c = nn.matmul_transpose(to_jt(a), to_jt(b)) if (ta, tb) == (0, 1) else None
        if c is not None:
            case("matmul_transpose_b", "matmul_transpose", {}, [a, b], to_np(c))


@guarded
def do_softmax(name, x, dim, log=False):
    y = nn.softmax(to_jt(x), dim, log)
    case(name, "log_softmax" if log else "softmax", {"dim": dim}, [x], to_np(y))


xs = (rng.normal(size=(8, 4096))).astype(np.float32)
do_softmax("softmax_rows_4096", xs, -1)
do_softmax("log_softmax_rows_4096", xs, -1, True)
do_softmax("softmax_rows_odd", (rng.normal(size=(7, 1001)) * 3).astype(np.float32), -1)
do_softmax("softmax_rows_tiny", f32(5, 3), 1)
do_softmax("softmax_dim0", f32(6, 33), 0)
do_softmax("softmax_mid", f32(3, 8, 5), 1)
do_softmax("softmax_all", f32(6, 33), None)
do_softmax("log_softmax_large_mag", (np.array([[-1e5, 0.0, 1e5, 3.0]] * 3)).astype(np.float32), -1, True)
do_softmax("softmax_rows_20000", (rng.normal(size=(3, 20000))).astype(np.float32), -1)


@guarded
def do_layernorm(name, x, nshape, gamma=None, beta=None, eps=1e-5):
    m = nn.LayerNorm(nshape, eps, gamma is not None)
    ins = [x]
    if gamma is not None:
        m.weight, m.bias = to_jt(gamma), to_jt(beta)
        ins += [gamma, beta]
    y = m(to_jt(x))
    case(name, "layer_norm", {"normalized_shape": list(nshape), "eps": eps,
                              "affine": gamma is not None}, ins, to_np(y))


g4096 = (1 + 0.02 * rng.normal(size=4096)).astype(np.float32)
do_layernorm("layernorm_rows_4096", xs, (4096,), g4096, np.zeros(4096, np.float32))
do_layernorm("layernorm_rows_odd", f32(7, 1001), (1001,), f32(1001), f32(1001))
do_layernorm("layernorm_noaffine", f32(9, 257), (257,))
do_layernorm("layernorm_2d_shape", f32(4, 6, 10), (6, 10), f32(6, 10), f32(6, 10))


@guarded
def do_batchnorm(name, x, gamma, beta, eps=1e-5, relu=False):
    m = nn.BatchNorm(x.shape[1], eps, is_train=True, sync=False)
    m.weight, m.bias = to_jt(gamma), to_jt(beta)
    y = m(to_jt(x))
    if relu:
        y = nn.relu(y)
    case(name, "batch_norm_relu" if relu else "batch_norm", {"eps": eps}, [x, gamma, beta], to_np(y))


do_batchnorm("batchnorm_train", f32(6, 5, 7, 7), f32(5, lo=0.5, hi=1.5), f32(5))
do_batchnorm("batchnorm_train_relu", f32(6, 5, 7, 7), f32(5, lo=0.5, hi=1.5), f32(5), relu=True)

# conv -> global-batch BatchNorm(train) -> relu: the single-process oracle of the sharded run
xc, wc = f32(4, 8, 10, 10), (rng.normal(size=(16, 8, 3, 3)) * 0.1).astype(np.float32)
mc = nn.Conv(8, 16, 3, 1, 1, bias=False); mc.weight = to_jt(wc)
mb = nn.BatchNorm(16, is_train=True, sync=False)
yc = nn.relu(mb(mc(to_jt(xc))))
case("conv_bn_relu", "conv_bn_relu", {"stride": 1, "padding": 1, "dilation": 1, "eps": 1e-5},
     [xc, wc, np.ones(16, np.float32), np.zeros(16, np.float32)], to_np(yc))

# max-pool 2x2 forward as reindex + reduce(max), and its backward as reindex_reduce(add)
xp = f32(2, 3, 8, 10)
vp = to_jt(xp)
xxp = vp.reindex([2, 3, 4, 5, 2, 2], ["i0", "i1", "i2*2+i4", "i3*2+i5"])
yp = xxp.reduce("maximum", [4, 5])
case("maxpool2x2_fwd", "maxpool2x2", {}, [xp], to_np(yp))
dyp = f32(2, 3, 4, 5)
dxp = jt.grad((yp * to_jt(dyp)).sum(), vp)
case("maxpool2x2_bwd", "maxpool2x2_bwd", {}, [xp, dyp], to_np(dxp))

# gradients of the meta-ops themselves (duality rules)
xg = f32(3, 10)
vg = to_jt(xg)
mg = f32(3, 14)
dg = jt.grad((vg.reindex([3, 14], ["i0", "i1-2"]) * to_jt(mg)).sum(), vg)
case("grad_reindex", "grad_reindex", {"shape": [3, 14], "indexes": ["i0", "i1-2"]}, [xg, mg], to_np(dg))
mg2 = f32(3, 4)
dg2 = jt.grad((vg.reindex_reduce("add", [3, 4], ["i0", "i1/3"]) * to_jt(mg2)).sum(), vg)
case("grad_reindex_reduce_add", "grad_reindex_reduce_add", {"shape": [3, 4], "indexes": ["i0", "i1/3"]},
     [xg, mg2], to_np(dg2))

np.savez_compressed(os.path.join(HERE, "meta_ops.npz"), **ARRAYS)
with open(os.path.join(HERE, "meta_ops.json"), "w") as f:
    json.dump({"generator": "tests/golden/make_golden.py", "reference_version": jt.__version__,
               "cases": CASES}, f, indent=1)
print("cases:", len(CASES), "arrays:", len(ARRAYS),
      "npz bytes:", os.path.getsize(os.path.join(HERE, "meta_ops.npz")))
