"""Adapter that runs a golden / parity case through the public jittor_b200 API (numpy in, numpy out)."""
import numpy as np
import torch

import jittor_b200 as jt
from jittor_b200 import nn


def _np(v):
    return v.numpy()


def _jt_slices(slices):
    return tuple(jt.array(s) if isinstance(s, np.ndarray) else s for s in slices)


class ProductBackend:
    @staticmethod
    def conv1d(x, w, stride, padding, dilation, groups, bias=None):
        return _np(nn.conv1d(jt.array(x), jt.array(w), None if bias is None else jt.array(bias), stride, padding, dilation,
                             groups))

    @staticmethod
    def adaptive_pool2d(x, output_size, op):
        from jittor_b200 import pool
        layer = (pool.AdaptiveAvgPool2d if op == "mean" else pool.AdaptiveMaxPool2d)(output_size)
        return _np(layer(jt.array(x)))

    @staticmethod
    def conv_grad(x, w, dy, stride, padding, dilation, want_dw):
        vx, vw = jt.array(x), jt.array(w)
        y = nn.conv2d(vx, vw, None, stride, padding, dilation)
        return _np(jt.grad((y * jt.array(dy)).sum(), vw if want_dw else vx))

    @staticmethod
    def conv2d_grouped(x, w, stride, padding, dilation, groups, bias=None):
        return _np(nn.conv2d(jt.array(x), jt.array(w), None if bias is None else jt.array(bias), stride, padding,
                             dilation, groups))

    @staticmethod
    def conv_transpose2d(x, w, stride, padding, output_padding, groups, dilation, bias=None):
        return _np(nn.conv_transpose2d(jt.array(x), jt.array(w), None if bias is None else jt.array(bias), stride,
                                       padding, output_padding, groups, dilation))

    @staticmethod
    def pool2d(x, kernel_size, op, stride=None, padding=0, ceil_mode=False, count_include_pad=True):
        from jittor_b200 import pool
        layer = pool.Pool(kernel_size, stride, padding, ceil_mode=ceil_mode, count_include_pad=count_include_pad, op=op)
        return _np(layer(jt.array(x)))

    @staticmethod
    def pool2d_backward(x, dy, kernel_size, op, stride=None, padding=0, ceil_mode=False, count_include_pad=True):
        from jittor_b200 import pool
        layer = pool.Pool(kernel_size, stride, padding, ceil_mode=ceil_mode, count_include_pad=count_include_pad, op=op)
        vx = jt.array(x)
        return _np(jt.grad((layer(vx) * jt.array(dy)).sum(), vx))

    @staticmethod
    def optim_steps(x, y, w, kind, steps, **kw):
        from jittor_b200 import optim
        w = jt.array(w)
        vx, vy = jt.array(x), jt.array(y)
        opt = {"sgd": optim.SGD, "adam": optim.Adam, "adamw": optim.AdamW, "rmsprop": optim.RMSprop}[kind]([w], **kw)
        for _ in range(steps):
            d = nn.matmul(vx, w) - vy
            loss = (d * d).sum() * (1.0 / x.shape[0])
            opt.step(loss)
        return _np(w)

    @staticmethod
    def getitem(x, slices):
        return _np(jt.array(x)[_jt_slices(slices)])

    @staticmethod
    def setitem(x, slices, data, op="void"):
        return _np(jt.array(x).setitem(_jt_slices(slices), jt.array(data), op))

    @staticmethod
    def scatter(x, dim, index, src, reduce="void"):
        return _np(jt.array(x).scatter(dim, jt.array(index), jt.array(src), reduce))

    @staticmethod
    def gather(x, dim, index):
        return _np(jt.array(x).gather(dim, jt.array(index)))

    @staticmethod
    def reindex(x, shape, indexes, overflow_value=0, overflow_conditions=(), extras=()):
        return _np(jt.array(x).reindex(shape, indexes, overflow_value, list(overflow_conditions),
                                        [jt.array(e) for e in extras]))

    @staticmethod
    def reindex_bf16_bits(bits, shape, indexes, fill):
        t = torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)
        y = jt.array(t).reindex(shape, indexes, fill)
        return y.torch().view(torch.int16).cpu().numpy().astype(np.uint16)

    @staticmethod
    def reindex_var(x, indexes, overflow_value=0, overflow_conditions=()):
        return _np(jt.array(x).reindex_var([jt.array(i) for i in indexes], overflow_value, list(overflow_conditions)))

    @staticmethod
    def reindex_reduce(y, op, shape, indexes, overflow_conditions=(), extras=()):
        return _np(jt.array(y).reindex_reduce(op, shape, indexes, list(overflow_conditions),
                                               [jt.array(e) for e in extras]))

    @staticmethod
    def broadcast(x, shape, dims=()):
        return _np(jt.broadcast(jt.array(x), shape, dims))

    @staticmethod
    def broadcast_var(x, y, dims=()):
        return _np(jt.broadcast_var(jt.array(x), jt.array(y), dims))

    @staticmethod
    def reduce(x, op, dims=(), keepdims=False):
        return _np(jt.reduce(jt.array(x), op, dims, keepdims))

    @staticmethod
    def binary(a, b, op):
        return _np(jt.binary(jt.array(a), jt.array(b), op))

    @staticmethod
    def unary(a, op):
        return _np(jt.unary(jt.array(a), op))

    @staticmethod
    def ternary(c, a, b):
        return _np(jt.ternary(jt.array(c), jt.array(a), jt.array(b)))

    @staticmethod
    def conv2d(x, w, stride=1, padding=1, dilation=1, bias=None):
        return _np(nn.conv2d(jt.array(x), jt.array(w), None if bias is None else jt.array(bias),
                             stride, padding, dilation))

    @staticmethod
    def matmul(a, b):
        return _np(nn.matmul(jt.array(a), jt.array(b)))

    @staticmethod
    def matmul_transpose(a, b):
        return _np(nn.matmul_transpose(jt.array(a), jt.array(b)))

    @staticmethod
    def softmax(x, dim=None, log=False):
        return _np(nn.softmax(jt.array(x), dim, log))

    @staticmethod
    def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5):
        return _np(nn.layer_norm(jt.array(x), tuple(normalized_shape),
                                 None if weight is None else jt.array(weight),
                                 None if bias is None else jt.array(bias), eps))

    @staticmethod
    def batch_norm_train(x, weight, bias, eps=1e-5, relu=False):
        m = nn.BatchNorm(x.shape[1], eps, is_train=True, sync=False)
        m.weight, m.bias = jt.array(weight), jt.array(bias)
        y = m(jt.array(x))
        return _np(nn.relu(y) if relu else y)

    @staticmethod
    def maxpool2x2(x):
        return _np(nn.max_pool2x2(jt.array(x)))

    @staticmethod
    def maxpool2x2_bwd(x, dy):
        # the reference's gradient rules written out: reduce(max) grad then reindex grad
        v = jt.array(x)
        n, c, h, w = x.shape
        shape6 = [n, c, h // 2, w // 2, 2, 2]
        idx = ["i0", "i1", "i2*2+i4", "i3*2+i5"]
        xx = v.reindex(shape6, idx)
        out = xx.reduce("maximum", [4, 5])
        cond = xx == out.broadcast(shape6, [4, 5])
        dxx = jt.ternary(cond, jt.array(dy).broadcast(shape6, [4, 5]), jt.zeros(shape6))
        return _np(dxx.reindex_reduce("add", list(x.shape), idx))
