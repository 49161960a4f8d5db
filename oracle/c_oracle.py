"""ctypes access to oracle/_build/liboracle.so (the C restatement in meta_ops.c). Test infrastructure only."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "liboracle.so")


def build():
    subprocess.check_call(["make", "-C", _HERE, "--no-print-directory"], stdout=subprocess.DEVNULL)


def load():
    src = os.path.join(_HERE, "meta_ops.c")
    if not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        build()
    return ctypes.CDLL(_LIB)


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = load()
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


_i64 = ctypes.c_int64


def scatter_add(y, e0, bins):
    y, e0 = np.ascontiguousarray(y), np.ascontiguousarray(e0, dtype=np.int32)
    x = np.empty(bins, dtype=y.dtype)
    fn = lib().oracle_scatter_add_i32 if y.dtype == np.int32 else lib().oracle_scatter_add_f32
    fn(_p(y), _p(e0), _i64(y.size), _p(x), _i64(bins))
    return x


def pool2x2_bwd(y):
    y = np.ascontiguousarray(y, dtype=np.float32)
    N, C, H, W = y.shape[:4]
    x = np.empty((N, C, 2 * H, 2 * W), np.float32)
    lib().oracle_pool2x2_bwd_f32(_p(y), _p(x), _i64(N), _i64(C), _i64(H), _i64(W))
    return x


def softmax_rows(x, log=False):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    lib().oracle_softmax_rows_f32(_p(x), _p(y), _i64(x.shape[0]), _i64(x.shape[1]), ctypes.c_int(int(log)))
    return y


def layernorm_rows(x, gamma=None, beta=None, eps=1e-5):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    g = None if gamma is None else np.ascontiguousarray(gamma, dtype=np.float32)
    b = None if beta is None else np.ascontiguousarray(beta, dtype=np.float32)
    lib().oracle_layernorm_rows_f32(_p(x), _p(g), _p(b), _p(y), _i64(x.shape[0]), _i64(x.shape[1]), ctypes.c_float(eps))
    return y


def matmul(a, b):
    a, b = np.ascontiguousarray(a, dtype=np.float32), np.ascontiguousarray(b, dtype=np.float32)
    c = np.empty((a.shape[0], b.shape[1]), np.float32)
    lib().oracle_matmul_f32(_p(a), _p(b), _p(c), _i64(a.shape[0]), _i64(a.shape[1]), _i64(b.shape[1]))
    return c


def conv2d(x, w, stride=1, padding=1, dilation=1):
    x, w = np.ascontiguousarray(x, dtype=np.float32), np.ascontiguousarray(w, dtype=np.float32)
    N, C, H, W = x.shape
    Co, _, KH, KW = w.shape
    OH = (H + padding * 2 - KH * dilation + dilation - 1) // stride + 1
    OW = (W + padding * 2 - KW * dilation + dilation - 1) // stride + 1
    y = np.empty((N, Co, OH, OW), np.float32)
    lib().oracle_conv2d_f32(_p(x), _p(w), _p(y), _i64(N), _i64(C), _i64(H), _i64(W), _i64(Co), _i64(KH), _i64(KW),
                            _i64(stride), _i64(padding), _i64(dilation))
    return y


def conv2d_backward_w(x, dy, kh, kw, stride=1, padding=1, dilation=1):
    x, dy = np.ascontiguousarray(x, dtype=np.float32), np.ascontiguousarray(dy, dtype=np.float32)
    N, C, H, W = x.shape
    Co = dy.shape[1]
    dw = np.empty((Co, C, kh, kw), np.float32)
    lib().oracle_conv2d_backward_w_f32(_p(x), _p(dy), _p(dw), _i64(N), _i64(C), _i64(H), _i64(W), _i64(Co), _i64(kh), _i64(kw),
                                       _i64(stride), _i64(padding), _i64(dilation))
    return dw


def bn_relu(x, gamma, beta, eps=1e-5, relu=True):
    x = np.ascontiguousarray(x, dtype=np.float32)
    N, C = x.shape[:2]
    HW = int(np.prod(x.shape[2:]))
    y = np.empty_like(x)
    g, b = np.ascontiguousarray(gamma, dtype=np.float32), np.ascontiguousarray(beta, dtype=np.float32)
    lib().oracle_bn_relu_f32(_p(x), _p(g), _p(b), _p(y), _i64(N), _i64(C), _i64(HW), ctypes.c_float(eps), ctypes.c_int(int(relu)))
    return y
