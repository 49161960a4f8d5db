"""The nn callers of the meta-operator path, written with the same meta-op expressions as the reference
so that the executor sees the same graphs: matmul (python/jittor/nn.py:118-159), Conv (:1001-1021),
softmax (:523-535), LayerNorm (:766-787), BatchNorm (:651-689), relu (:166-183), Pool via reindex."""
import numpy as np

from . import var as V
from . import dtypes
from .flags import flags, flag_scope
from .var import Var, to_var


class Module:
    def __call__(self, *a, **k):
        return self.execute(*a, **k)

    def execute(self, *a, **k):
        raise NotImplementedError

    def parameters(self):
        """Vars held by this module and its sub-modules (also inside lists / tuples / dicts), in attribute order."""
        out, seen = [], set()

        def visit(obj):
            if isinstance(obj, Var):
                if id(obj) not in seen:
                    seen.add(id(obj))
                    out.append(obj)
            elif isinstance(obj, Module):
                for v in obj.__dict__.values():
                    visit(v)
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    visit(v)
            elif isinstance(obj, dict):
                for v in obj.values():
                    visit(v)

        visit(self)
        return out

    def mpi_param_broadcast(self, root=0):
        """python/jittor/__init__.py:1761-1764."""
        from . import dist
        if not dist.in_mpi():
            return
        for p in self.parameters():
            p.update(p.mpi_broadcast(root))


class Function(Module):
    """An op with a hand-written backward (python/jittor/__init__.py:1865-2004): `execute(*args)` computes the outputs,
    `grad(*output_gradients)` returns one gradient per input (None where there is none). Gradients that did not reach
    an output arrive as None. Each output is re-issued as a pass-through node that carries the backward rule, so
    `jt.grad` never differentiates through the body of `execute`."""

    def __call__(self, *args):
        outs = self.execute(*args)
        single = isinstance(outs, Var)
        outs = [outs] if single else list(outs)
        var_pos = [i for i, a in enumerate(args) if isinstance(a, Var)]
        var_args = [args[i] for i in var_pos]

        def rule_for(k_out):
            def rule(out, dout, k):
                if k == 0:
                    return None                      # input 0 is the value computed by execute
                douts = [None] * len(outs)
                douts[k_out] = dout
                grads = self.grad(*douts)
                grads = [grads] if isinstance(grads, Var) or grads is None else list(grads)
                pos = var_pos[k - 1]
                return grads[pos] if pos < len(grads) else None
            return rule

        wrapped = []
        for k_out, o in enumerate(outs):
            if not isinstance(o, Var):
                wrapped.append(o)
                continue
            node = V.Op("custom", [o] + var_args, fn=lambda first, *rest: first, grad=rule_for(k_out), name="function")
            wrapped.append(Var(o.shape, o.dtype, node))
        return wrapped[0] if single else tuple(wrapped)

    def grad(self, *douts):
        raise NotImplementedError

    @classmethod
    def apply(cls, *args, **kw):
        return cls()(*args, **kw)


def matmul_transpose(a, b):
    """c[..., n, k] = sum_m a[..., n, m] * b[k, m]  (python/jittor/nn.py:40-58)."""
    a, b = to_var(a), to_var(b)
    assert a.shape[-1] == b.shape[-1], (a.shape, b.shape)
    if a.ndim != 2:
        aa = a.reshape((-1, a.shape[-1]))
        cc = matmul_transpose(aa, b)
        return cc.reshape(list(a.shape[:-1]) + [-1])
    assert a.ndim == 2 and b.ndim == 2
    shape = list(a.shape)[:-1] + list(b.shape)
    with flag_scope(amp_reg=flags.amp_reg | 36):
        a = a.broadcast(shape, [len(shape) - 2])
        b = b.broadcast(shape)
        return (a * b).sum(len(shape) - 1)


def matmul(a, b):
    """Broadcast-multiply-sum matrix product, every branch of python/jittor/nn.py:118-159."""
    a, b = to_var(a), to_var(b)
    with flag_scope(amp_reg=flags.amp_reg | 36):
        len_a, len_b = a.ndim, b.ndim
        if len_b == 1:
            return (a * b).sum(-1)
        if len_a == 1:
            return (a.broadcast(b, [-1]) * b).sum(0)
        shape = []
        len_c = max(len_a, len_b)
        (n, m), (m_, k) = a.shape[-2:], b.shape[-2:]
        assert m == m_, f"dimension not match, a.shape:{a.shape}, b.shape:{b.shape}"
        if len_b == 2 and len_a > 2:
            aa = a.reshape((-1, m))
            cc = matmul(aa, b)
            return cc.reshape(list(a.shape[:-1]) + [k])
        for i in range(len_c - 2):
            ai = len_a - (len_c - i)
            bi = len_b - (len_c - i)
            an = a.shape[ai] if ai >= 0 else 1
            bn = b.shape[bi] if bi >= 0 else 1
            if an != 1 and bn != 1:
                assert an == bn, f"dimension not match, a.shape:{a.shape}, b.shape:{b.shape}"
            shape.append(max(an, bn))
        shape.extend([n, m, k])
        a = a.broadcast(shape, [-1])
        b = b.broadcast(shape, [-3])
        return (a * b).sum(-2)


bmm = matmul


def relu(x):
    x = to_var(x)
    return V.ternary(x > 0.0, x, 0.0)


def _softmax_backward(y, dout, log, cols):
    """dx from the forward output and the output gradient in one launch (b200jt_softmax_backward): what the reference's
    CUDA softmax brings as its own backward kernel (python/jittor/other/code_softmax.py:109-147)."""
    from . import _capi as C
    dout = to_var(dout)
    if dout.dtype != y.dtype:
        dout = dout.cast(y.dtype)
    if list(dout.shape) != list(y.shape):
        dout = dout.broadcast(y.shape)
    rows = y.numel() // cols if cols else 0

    def run(yt, dyt):
        import torch
        dx = torch.empty_like(yt)
        C.check(C.lib.b200jt_softmax_backward(C.desc(yt, [rows, cols]), C.desc(dyt.contiguous(), [rows, cols]), C.desc(dx, [rows, cols]),
                                              int(log), C.stream_ptr()), "softmax_backward")
        return dx

    return Var(y.shape, y.dtype, V.Op("custom", [y, dout], fn=run, name="softmax_backward"))


def softmax(x, dim=None, log=False):
    x0 = x = to_var(x)
    if dim is None:
        dim = ()
    dtype, x = x.dtype, x._to_float()
    if log:
        a = x - x.max(dim, keepdims=True)
        ret = a - a.exp().sum(dim, keepdims=True).log()
    else:
        e = (x - x.max(dim, keepdims=True)).exp()
        ret = e / e.sum(dim, keepdims=True)
    ret = ret.cast(dtype)
    # over the last axis (or over everything) the backward is one fused kernel, as the forward is
    whole = dim == () or dim == []
    last = isinstance(dim, int) and dim % max(x0.ndim, 1) == x0.ndim - 1
    if (whole or last) and str(dtype) in ("float32", "bfloat16") and x0.numel() > 0 and ret is not x0:
        cols = x0.numel() if whole else x0.shape[-1]
        ret._vjp = (x0, lambda y, dout: _softmax_backward(y, dout, log, cols))
    return ret


def log_softmax(x, dim=None):
    return softmax(x, dim, True)


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


def conv2d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    """Conv.execute (python/jittor/nn.py:1001-1056). groups == 1: reindex x to the 7-D window tensor, broadcast w over
    [0,3,4], multiply, sum over [2,5,6]. groups > 1: x and w are both re-indexed to [N,G,oc/G,C/G,oh,ow,Kh,Kw], multiplied
    and folded by reindex_reduce('add') (nn.py:1022-1051). The executor recognises the first form by its index
    expressions; the second carries a relay record (the role of the reference's compile_options {"G","C"} hint) so that
    it runs as one grouped implicit-GEMM launch instead of materialising the 8-D product."""
    x, weight = to_var(x), to_var(weight)
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    N, C, H, W = x.shape
    out_channels, Cw, Kh, Kw = weight.shape
    oh = (H + padding[0] * 2 - Kh * dilation[0] + dilation[0] - 1) // stride[0] + 1
    ow = (W + padding[1] * 2 - Kw * dilation[1] + dilation[1] - 1) // stride[1] + 1
    assert oh > 0 and ow > 0
    if groups != 1:
        G, CpG, ocg = groups, C // groups, out_channels // groups
        assert C % G == 0 and out_channels % G == 0 and Cw == CpG
        shape = [N, G, ocg, CpG, oh, ow, Kh, Kw]
        xx = x.reindex(shape, ["i0", f"i1*{CpG}+i3",
                               f"i4*{stride[0]}-{padding[0]}+i6*{dilation[0]}",
                               f"i5*{stride[1]}-{padding[1]}+i7*{dilation[1]}"])
        ww = weight.reindex(shape, [f"i1*{ocg}+i2", "i3", "i6", "i7"])
        y = (xx * ww).reindex_reduce("add", [N, out_channels, oh, ow], ["i0", f"i1*{ocg}+i2", "i4", "i5"])
        y._relay = ("conv2d", x, weight, stride + padding + dilation, G)
        if bias is not None:
            y = y + to_var(bias).broadcast(y.shape, [0, 2, 3])
        return y
    assert C == Cw
    amp = flags.amp_reg | 36

    def graph():
        with flag_scope(amp_reg=amp):
            xx = x.reindex([N, out_channels, C, oh, ow, Kh, Kw], [
                "i0",
                "i2",
                f"i3*{stride[0]}-{padding[0]}+i5*{dilation[0]}",
                f"i4*{stride[1]}-{padding[1]}+i6*{dilation[1]}",
            ])
            ww = weight.broadcast(xx.shape, [0, 3, 4])
            yy = xx * ww
            return yy.sum([2, 5, 6])

    # The four-op graph is written down when something reads it (jt.grad, a consumer's pattern match, the fuser); a plain
    # forward call runs from the relay record alone: the executor would only find the same operands and geometry in the
    # index strings. Shape and dtype are what the graph's own inference gives.
    with flag_scope(amp_reg=amp):
        ydt = dtypes.reduce_dtype_infer("add", dtypes.binary_dtype_infer("multiply", x.dtype, weight.dtype, x.is_scalar, weight.is_scalar))
    y = V.LazyVar([N, out_channels, oh, ow], ydt, lambda: graph()._op)
    y._relay = ("conv2d", x, weight, stride + padding + dilation, 1)
    if bias is not None:
        y = y + to_var(bias).broadcast(y.shape, [0, 2, 3])
    return y


def conv1d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    """Conv1d.execute (python/jittor/nn.py:1097-1125): the signal gets a trailing axis of extent 1, the weight
    [O, C/groups, K] likewise, and the 2-D convolution runs with kernel (K, 1), stride (s, 1), padding (p, 0)."""
    x, weight = to_var(x), to_var(weight)
    if x.ndim != 3:
        raise ValueError("Input shape must be `(N, C, L)`!")
    N, C, L = x.shape
    O, Cg, K = weight.shape
    y = conv2d(x.reshape([N, C, L, 1]), weight.reshape([O, Cg, K, 1]), bias, (stride, 1), (padding, 0), (dilation, 1), groups)
    return y.reshape([N, O, y.shape[2]])


class Conv1d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True):
        assert in_channels > 0, "in_channels must be positive"
        assert out_channels > 0, "out_channels must be positive"
        if groups <= 0:
            raise ValueError("groups must be a positive integer")
        assert in_channels % groups == 0, "in_channels must be divisible by groups"
        assert out_channels % groups == 0, "out_channels must be divisible by groups"
        self.in_channels, self.out_channels, self.groups = in_channels, out_channels, groups
        self.kernel_size, self.stride, self.padding, self.dilation = kernel_size, stride, padding, dilation
        rng = np.random.default_rng(0)
        bound = 1.0 / np.sqrt(in_channels * kernel_size)
        self.weight = V.array(rng.uniform(-bound, bound, (out_channels, in_channels // groups, kernel_size)).astype(np.float32))
        self.bias = V.array(rng.uniform(-bound, bound, (out_channels,)).astype(np.float32)) if bias else None

    def execute(self, x):
        assert x.shape[1] == self.in_channels
        return conv1d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


def conv_transpose2d(x, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1):
    """ConvTranspose.execute (python/jittor/nn.py:1429-1491): weight is [Cin, Cout/groups, Kh, Kw]; x and w are broadcast
    (groups == 1) or re-indexed (groups > 1) to the full loop nest, multiplied, and scattered into the output with
    reindex_reduce('add'). The result Var carries a relay record so that the nest runs as one implicit-GEMM launch
    (gather form) instead of being materialised."""
    x, weight = to_var(x), to_var(weight)
    stride, padding, dilation, output_padding = _pair(stride), _pair(padding), _pair(dilation), _pair(output_padding)
    if x.ndim != 4:
        raise RuntimeError(f"Expected 4D (batched) input to conv_transpose2d, but got input of size: {list(x.shape)}")
    assert output_padding[0] < max(stride[0], dilation[0]) and output_padding[1] < max(stride[1], dilation[1]), \
        "output padding must be smaller than max(stride, dilation)"
    N, C, H, W = x.shape
    i, o, h, w = weight.shape
    assert C == i
    h_out = (H - 1) * stride[0] + output_padding[0] - 2 * padding[0] + 1 + (h - 1) * dilation[0]
    w_out = (W - 1) * stride[1] + output_padding[1] - 2 * padding[1] + 1 + (w - 1) * dilation[1]
    hid = f"*{stride[0]}-{padding[0]}+"
    wid = f"*{stride[1]}-{padding[1]}+"
    if groups == 1:
        shape = [N, i, o, H, W, h, w]
        xx = x.broadcast(shape, (2, 5, 6))
        ww = weight.broadcast(shape, (0, 3, 4))
        y = (ww * xx).reindex_reduce("add", [N, o, h_out, w_out],
                                     ["i0", "i2", f"i3{hid}i5*{dilation[0]}", f"i4{wid}i6*{dilation[1]}"])
    else:
        G, CpG, oc = groups, C // groups, o * groups
        shape = [N, G, o, CpG, H, W, h, w]
        xx = x.reindex(shape, ["i0", f"i1*{CpG}+i3", "i4", "i5"])
        ww = weight.reindex(shape, [f"i1*{CpG}+i3", "i2", "i6", "i7"])
        y = (ww * xx).reindex_reduce("add", [N, oc, h_out, w_out],
                                     ["i0", f"i1*{o}+i2", f"i4{hid}i6*{dilation[0]}", f"i5{wid}i7*{dilation[1]}"])
    y._relay = ("conv2d_transpose", x, weight, stride + padding + dilation, groups)
    if bias is not None:
        y = y + to_var(bias).broadcast(y.shape, [0, 2, 3])
    return y


class ConvTranspose(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, groups=1, bias=True,
                 dilation=1):
        assert in_channels % groups == 0, "in_channels must be divisible by groups"
        assert out_channels % groups == 0, "out_channels must be divisible by groups"
        self.in_channels, self.out_channels, self.groups = in_channels, out_channels, groups
        self.kernel_size = _pair(kernel_size)
        self.stride, self.padding, self.dilation = _pair(stride), _pair(padding), _pair(dilation)
        self.output_padding = _pair(output_padding)
        Kh, Kw = self.kernel_size
        rng = np.random.default_rng(0)
        bound = 1.0 / np.sqrt(out_channels // groups * Kh * Kw)
        self.weight = V.array(rng.uniform(-bound, bound, (in_channels, out_channels // groups, Kh, Kw)).astype(np.float32))
        self.bias = V.array(rng.uniform(-bound, bound, (out_channels,)).astype(np.float32)) if bias else None

    def execute(self, x):
        return conv_transpose2d(x, self.weight, self.bias, self.stride, self.padding, self.output_padding, self.groups,
                                self.dilation)


ConvTranspose2d = ConvTranspose


class Conv(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True):
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size = _pair(kernel_size)
        self.stride, self.padding, self.dilation, self.groups = _pair(stride), _pair(padding), _pair(dilation), groups
        Kh, Kw = self.kernel_size
        fan = in_channels * Kh * Kw
        bound = 1.0 / np.sqrt(fan)
        rng = np.random.default_rng(0)
        self.weight = V.array(rng.uniform(-bound, bound, (out_channels, in_channels // groups, Kh, Kw)).astype(np.float32))
        self.bias = V.array(rng.uniform(-bound, bound, (out_channels,)).astype(np.float32)) if bias else None

    def execute(self, x):
        return conv2d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


Conv2d = Conv


class LayerNorm(Module):
    def __init__(self, normalized_shape, eps=1e-5, elementwise_affine=True):
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        self.weight = V.ones(self.normalized_shape) if elementwise_affine else 1.0
        self.bias = V.zeros(self.normalized_shape) if elementwise_affine else 0.0

    def execute(self, x):
        x = to_var(x)
        dtype = x.dtype
        # fp32_guard (python/jittor/nn.py:731-750): half inputs are normalised in float32
        guard = dtype in ("float16", "bfloat16")
        if guard:
            x = x.float32()
        dims = [-i for i in range(len(self.normalized_shape), 0, -1)]
        xmean = x.mean(dims=dims, keepdims=True)
        x2mean = (x * x).mean(dims=dims, keepdims=True)
        xvar = (x2mean - xmean * xmean).maximum(0.0)
        w = self.weight / (xvar + self.eps).sqrt()
        b = self.bias - xmean * w
        y = x * w + b
        return y.cast(dtype) if guard else y


def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    m = LayerNorm(normalized_shape, eps, weight is not None)
    if weight is not None:
        m.weight, m.bias = to_var(weight), to_var(bias)
    return m(x)


class BatchNorm(Module):
    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, is_train=True, sync=True):
        self.sync, self.num_features, self.is_train = sync, num_features, is_train
        self.eps, self.momentum, self.affine = eps, momentum, affine
        self.weight = V.ones((num_features,)) if affine else 1.0
        self.bias = V.zeros((num_features,)) if affine else 0.0
        self.running_mean = V.zeros((num_features,)).stop_grad()
        self.running_var = V.ones((num_features,)).stop_grad()

    def _update_running(self, xmean, xvar):
        """running += (batch - running) * momentum (python/jittor/nn.py:684-688), for results the fused kernels did not
        produce; the fused BatchNorm plan does the same inside its normalise kernel."""
        for name, batch in (("running_mean", xmean), ("running_var", xvar)):
            run = getattr(self, name)
            new = (run + (batch.reshape((-1,)).float32() - run) * self.momentum).float32()
            run.assign(new).stop_grad()

    def execute(self, x):
        from . import dist
        x = to_var(x)
        dims = [0] + list(range(2, x.ndim))
        if self.is_train:
            xmean = x.mean(dims=dims)
            x2mean = (x * x).mean(dims=dims)
            if self.sync and dist.in_mpi():
                xmean = xmean.mpi_all_reduce("mean")
                x2mean = x2mean.mpi_all_reduce("mean")
            xvar = (x2mean - xmean * xmean).maximum(0.0)
            w = self.weight / (xvar + self.eps).sqrt()
            b = self.bias - xmean * w
            norm_x = x * w.broadcast(x, dims) + b.broadcast(x, dims)
            # the running statistics move when norm_x is computed: the executor either folds the update into the fused
            # normalise kernel or calls _update_running once the batch statistics exist
            norm_x._bn_running = (self, xmean, xvar)
            return norm_x
        w = self.weight / (self.running_var + self.eps).sqrt()
        b = self.bias - self.running_mean * w
        return x * w.broadcast(x, dims) + b.broadcast(x, dims)


BatchNorm2d = BatchNorm


class ReLU(Module):
    def execute(self, x):
        return relu(x)


def max_pool2x2(x):
    """2x2 stride-2 max pooling through reindex + reduce(max) (the reindex path of python/jittor/pool.py)."""
    x = to_var(x)
    N, C, H, W = x.shape
    xx = x.reindex([N, C, H // 2, W // 2, 2, 2], ["i0", "i1", "i2*2+i4", "i3*2+i5"])
    return xx.reduce("maximum", [4, 5])
