"""jittor_b200: the meta-operator hot path of Jittor (reindex, reindex_reduce, broadcast, reduce and the
element-wise chains fused around them) on hand-written sm_100a CUDA kernels, behind the reference's
Python surface. Compute goes through csrc/libb200jt.so only; there is no CPU fallback."""
from . import _capi
from ._capi import B200Error
from .flags import flags, flag_scope
from .var import (Var, array, to_var, empty, zeros, ones, reindex, reindex_var, reindex_reduce, broadcast,
                  broadcast_var, reduce, binary, unary, ternary, ternary_out_hint, reshape, transpose, index)
from . import dtypes, executor, nn, dist, op_register
from .op_register import code, has_op, get_op_info, register_op, compile_custom_op, compile_custom_ops
from .dtypes import binary_dtype_infer
from .grad import grad
from .nn import Function, Module
from . import slicing, optim, pool
from .slicing import getitem, setitem, scatter, scatter_, gather

__version__ = "0.1.0"


def _reduce_alias(op):
    def f(x, dim=(), keepdims=False, dims=None):
        return reduce(x, op, dims if dims is not None else dim, keepdims)
    f.__name__ = op
    return f


sum = _reduce_alias("add")
prod = product = _reduce_alias("multiply")
max = _reduce_alias("maximum")
min = _reduce_alias("minimum")
mean = _reduce_alias("mean")
all_ = _reduce_alias("logical_and")
any_ = _reduce_alias("logical_or")
for _op in dtypes.REDUCE_OPS:
    globals()[f"reduce_{_op}"] = _reduce_alias(_op)
for _op in dtypes.BINARY_OPS - {"mean"}:
    globals().setdefault(_op, (lambda _op: lambda a, b: binary(a, b, _op))(_op))
for _op in dtypes.UNARY_OPS - {"cast"}:
    globals().setdefault(_op, (lambda _op: lambda a: unary(a, _op))(_op))
for _op in dtypes.DTYPES:
    globals()[_op] = (lambda _op: lambda a: unary(to_var(a), _op))(_op)
float = float32   # noqa: F821
int = int32       # noqa: F821
matmul = nn.matmul


# the reference re-exports the pooling layers and optimisers from jittor.nn (python/jittor/nn.py:21-22)
for _name in ("Pool", "MaxPool2d", "AvgPool2d", "AdaptiveAvgPool2d", "AdaptiveMaxPool2d", "pool", "avg_pool2d", "max_pool2d"):
    setattr(nn, _name, getattr(pool, _name))
for _name in ("Optimizer", "SGD", "Adam", "AdamW", "RMSprop"):
    setattr(nn, _name, getattr(optim, _name))
op_register._register_builtins()


def cast(x, dtype):
    return to_var(x).cast(dtype)


def sync(vars, device_sync=False):
    executor.realize(list(vars))
    if device_sync:
        import torch
        torch.cuda.current_stream().synchronize()


def sync_all(device_sync=False):
    if device_sync:
        import torch
        torch.cuda.synchronize()


def fetch_sync(vars):
    return [v.numpy() for v in vars]
