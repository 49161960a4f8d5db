"""Pooling with the reference's interface and rules (python/jittor/pool.py:20-197, 530-573): `Pool`, `pool`,
`MaxPool2d`, `AvgPool2d`, `max_pool2d`, `avg_pool2d`. The reference runs hand-written jt.code loops for maximum /
minimum (and for mean in ceil mode) and falls back to reindex + reduce otherwise; here the same two routes exist:

  * `pool_use_code_op` (default True): the fixed CUDA kernels of csrc/pool.cu (b200jt_pool2d / _backward), which follow
    the jt.code bodies: clipped windows, first-match gradient for maximum / minimum;
  * otherwise, and for mean in floor mode exactly as in the reference (pool.py:46-50,187-197): the meta-operator lowering
    x.reindex([N,C,h,w,kh,kw], ...).reduce(op, [4,5]), whose overflow value 0 stands for the padding."""
import ctypes

import torch

from . import _capi as C
from . import var as V
from .nn import Module

pool_use_code_op = True


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


def _run_pool(op, k, s, p, cip, oshape, want_indices, keep=None):
    """Forward relay. For maximum / minimum the index map is always written (one extra int32 per output); `keep`, a dict
    shared with the backward relay, holds on to it so that the backward needs neither x nor a scan."""
    with_idx = op != "mean"

    def run(xd):
        xd = xd.contiguous()
        y = torch.empty(oshape, dtype=xd.dtype, device=xd.device)
        idx = torch.empty(oshape, dtype=torch.int32, device=xd.device) if with_idx else None
        C.check(C.lib.b200jt_pool2d(C.desc(xd), C.desc(y), ctypes.c_void_p(idx.data_ptr() if with_idx else 0),
                                    op.encode(), k[0], k[1], s[0], s[1], p[0], p[1], int(cip), C.stream_ptr()), "pool2d")
        if keep is not None and with_idx:
            keep["idx"] = idx
        return idx if want_indices else y
    return run


def _run_pool_bwd(op, k, s, p, cip, xshape, oshape, keep):
    def run(xd, yd, dyd):
        xd, yd, dyd = xd.view(xshape).contiguous(), yd.view(oshape).contiguous(), dyd.view(oshape).contiguous()
        dx = torch.empty_like(xd)
        idx = keep.get("idx")
        if idx is not None:
            C.check(C.lib.b200jt_pool2d_backward_indices(C.desc(xd), C.desc(yd), ctypes.c_void_p(idx.data_ptr()), C.desc(dyd),
                                                         C.desc(dx), k[0], k[1], s[0], s[1], p[0], p[1], C.stream_ptr()),
                    "pool2d_backward_indices")
            return dx
        C.check(C.lib.b200jt_pool2d_backward(C.desc(xd), C.desc(yd), C.desc(dyd), C.desc(dx), op.encode(),
                                             k[0], k[1], s[0], s[1], p[0], p[1], int(cip), C.stream_ptr()), "pool2d_backward")
        return dx
    return run


class Pool(Module):
    def __init__(self, kernel_size, stride=None, padding=0, dilation=None, return_indices=None, ceil_mode=False,
                 count_include_pad=True, op="maximum"):
        assert dilation is None
        assert return_indices is None or op == "maximum"
        self.return_indices = return_indices
        self.kernel_size = _pair(kernel_size)
        self.op = op
        self.stride = _pair(stride if stride else kernel_size)
        self.padding = _pair(padding)
        self.ceil_mode = ceil_mode
        self.count_include_pad = count_include_pad and padding != 0
        for item in self.kernel_size:
            if item <= 0:
                raise RuntimeError(f"kernel_size must be greater than zero, but got {item}")
        for item in self.stride:
            if item <= 0:
                raise RuntimeError(f"stride must be greater than zero, but got {item}")
        for item in self.padding:
            if item < 0:
                raise RuntimeError(f"padding must be non-negative, but got {item}")

    def execute(self, x):
        x = V.to_var(x)
        N, Cn, H, W = x.shape
        k, s, p = self.kernel_size, self.stride, self.padding
        if H <= k[0] or W <= k[1]:
            raise RuntimeError("size of var should be larger than kernel_size")
        if not self.ceil_mode:
            h = (H + p[0] * 2 - k[0]) // s[0] + 1
            w = (W + p[1] * 2 - k[1]) // s[1] + 1
            use_code_op = self.op in ("maximum", "minimum")
        else:
            h = (H + p[0] * 2 - k[0] + s[0] - 1) // s[0] + 1
            w = (W + p[1] * 2 - k[1] + s[1] - 1) // s[1] + 1
            use_code_op = self.op in ("maximum", "minimum", "mean")
        if not (use_code_op and pool_use_code_op):
            xx = x.reindex([N, Cn, h, w, k[0], k[1]],
                           ["i0", "i1", f"i2*{s[0]}-{p[0]}+i4", f"i3*{s[1]}-{p[1]}+i5"])
            return xx.reduce(self.op, [4, 5])
        oshape, xshape, op, cip = [N, Cn, h, w], list(x.shape), self.op, self.count_include_pad
        keep = {}

        def grad_rule(out, dout, which):
            node = V.Op("custom", [x, out, dout], fn=_run_pool_bwd(op, k, s, p, cip, xshape, oshape, keep), name="pool2d_backward")
            return V.Var(xshape, x.dtype, node)

        y = V.Var(oshape, x.dtype, V.Op("custom", [x], fn=_run_pool(op, k, s, p, cip, oshape, False, keep), name="pool2d",
                                         grad=grad_rule))
        if not self.return_indices:
            return y
        idx = V.Var(oshape, "int32", V.Op("custom", [x], fn=_run_pool(op, k, s, p, cip, oshape, True), name="pool2d_indices"))
        return y, idx


def pool(x, kernel_size, op, padding=0, stride=None):
    return Pool(kernel_size, stride, padding, op=op)(x)


pool2d = pool


class AvgPool2d(Module):
    def __init__(self, kernel_size, stride=None, padding=0, ceil_mode=False, count_include_pad=True):
        self.layer = Pool(kernel_size=kernel_size, stride=stride, padding=padding, ceil_mode=ceil_mode,
                          count_include_pad=count_include_pad, op="mean")

    def execute(self, x):
        return self.layer(x)


class MaxPool2d(Module):
    def __init__(self, kernel_size, stride=None, padding=0, dilation=None, return_indices=None, ceil_mode=False):
        self._layer = Pool(kernel_size=kernel_size, stride=stride, padding=padding, dilation=dilation,
                           return_indices=return_indices, ceil_mode=ceil_mode, op="maximum")

    def execute(self, x):
        return self._layer(x)


def avg_pool2d(x, kernel_size, stride=None, padding=0, ceil_mode=False, count_include_pad=True):
    return AvgPool2d(kernel_size, stride, padding, ceil_mode, count_include_pad)(x)


def max_pool2d(x, kernel_size, stride=None, padding=0, dilation=None, return_indices=None, ceil_mode=False):
    return MaxPool2d(kernel_size, stride, padding, dilation, return_indices, ceil_mode)(x)


def _adaptive_geometry(x, output_size, who):
    if isinstance(output_size, int):
        oh = ow = output_size
    elif isinstance(output_size, (tuple, list)):
        oh = x.shape[2] if output_size[0] is None else output_size[0]
        ow = x.shape[3] if output_size[1] is None else output_size[1]
    else:
        raise TypeError(f"{who} only support int, tuple or list input. Not support {type(output_size)} yet.")
    return oh, ow


def _adaptive(x, output_size, op, who):
    """AdaptiveAvgPool2d / AdaptiveMaxPool2d.execute (python/jittor/pool.py:405-466): stride floor(H/oh), window
    H - (oh-1)*stride, written with the meta-operators exactly as the reference does (so the gradient is theirs too)."""
    x = V.to_var(x)
    oh, ow = _adaptive_geometry(x, output_size, who)
    if oh == 1 and ow == 1:
        return x.reduce(op, [2, 3], keepdims=True)
    N, Cn, H, W = x.shape
    sh, sw = H // oh, W // ow
    ksh, ksw = H - (oh - 1) * sh, W - (ow - 1) * sw
    h, w = (H - ksh) // sh + 1, (W - ksw) // sw + 1
    xx = x.reindex([N, Cn, h, w, ksh, ksw], ["i0", "i1", f"i2*{sh}+i4", f"i3*{sw}+i5"])
    return xx.reduce(op, [4, 5])


class AdaptiveAvgPool2d(Module):
    def __init__(self, output_size):
        self.output_size = output_size

    def execute(self, x):
        return _adaptive(x, self.output_size, "mean", "AdaptiveAvgPool2d")


class AdaptiveMaxPool2d(Module):
    def __init__(self, output_size, return_indices=False):
        self.output_size, self.return_indices = output_size, return_indices

    def execute(self, x):
        if self.return_indices:
            x = V.to_var(x)
            oh, ow = _adaptive_geometry(x, self.output_size, "AdaptiveMaxPool2d")
            if not (oh == 1 and ow == 1):
                sh, sw = x.shape[2] // oh, x.shape[3] // ow
                k = (x.shape[2] - (oh - 1) * sh, x.shape[3] - (ow - 1) * sw)
                return MaxPool2d(kernel_size=k, stride=(sh, sw), return_indices=True)(x)
        return _adaptive(x, self.output_size, "maximum", "AdaptiveMaxPool2d")
