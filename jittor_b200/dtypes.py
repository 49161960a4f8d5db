"""dtype names and the reference's dtype-inference rules
(python/jittor/src/misc/nano_string.h:199-277, op classes python/jittor/src/misc/nano_string.cc:46-146)."""
import numpy as np

from .flags import flags as _FLAGS

DTYPES = ("bool", "int8", "int16", "int32", "int64", "uint8", "float16", "bfloat16", "float32", "float64")
_DSIZE = {"bool": 0, "int8": 0, "uint8": 0, "int16": 1, "float16": 1, "bfloat16": 1,
          "int32": 2, "float32": 2, "int64": 3, "float64": 3}
_FLOATS = {"float16", "bfloat16", "float32", "float64"}

BOOL_OPS = {"bool", "logical_not", "less", "less_equal", "greater", "greater_equal", "equal", "not_equal",
            "logical_and", "logical_or", "logical_xor"}
FLOAT_OPS = {"log", "exp", "sqrt", "mean", "divide", "sin", "asin", "sinh", "asinh", "tan", "atan", "tanh",
             "atanh", "cos", "acos", "cosh", "acosh", "sigmoid", "erf", "erfinv"}
INT_OPS = {"round_int", "floor_int", "ceil_int", "floor_divide"}
WHITE_OPS = {"exp", "pow"}
UNARY_OPS = {"abs", "negative", "logical_not", "bitwise_not", "log", "exp", "sqrt", "round", "floor", "ceil",
             "round_int", "floor_int", "ceil_int", "cast", "sin", "asin", "sinh", "asinh", "tan", "atan", "tanh",
             "atanh", "cos", "acos", "cosh", "acosh", "sigmoid", "erf", "erfinv"}
BINARY_OPS = {"pow", "maximum", "minimum", "add", "subtract", "multiply", "divide", "floor_divide", "mod", "less",
              "less_equal", "greater", "greater_equal", "equal", "not_equal", "left_shift", "right_shift",
              "logical_and", "logical_or", "logical_xor", "bitwise_and", "bitwise_or", "bitwise_xor", "mean"}
REDUCE_OPS = ("maximum", "minimum", "add", "multiply", "logical_and", "logical_or", "logical_xor",
              "bitwise_and", "bitwise_or", "bitwise_xor", "mean")

AMP_PREFER32, AMP_PREFER16, AMP_KEEP_REDUCE, AMP_KEEP_WHITE, AMP_ARRAY_PREFER, AMP_NO_REDUCE_UPCAST = 1, 2, 4, 8, 16, 32


_ALIASES = {"float": "float32", "int": "int32", "double": "float64", "half": "float16"}


class DType(str):
    """A dtype name that also compares equal to the numpy dtype of the same name and to the reference's short names
    ("float", "int", "double", "half": python/jittor/src/misc/nano_string.cc aliases)."""

    def __eq__(self, other):
        if isinstance(other, str):
            return str.__eq__(self, _ALIASES.get(other, other))
        try:
            return str.__eq__(self, np.dtype(other).name)
        except TypeError:
            return False

    def __ne__(self, other):
        return not self.__eq__(other)

    __hash__ = str.__hash__

    def is_float(self):
        return str(self) in _FLOATS

    def is_int(self):
        return str(self) not in _FLOATS


def canon(dt):
    """Accepts a name, a numpy dtype / type, a torch dtype or a Python type; returns the name."""
    if type(dt) is DType:
        return dt
    if isinstance(dt, str):
        name = _ALIASES.get(dt, dt)
    elif dt is float:
        name = "float32"
    elif dt is int:
        name = "int32"
    elif dt is bool:
        name = "bool"
    else:
        import torch
        if isinstance(dt, torch.dtype):
            from ._capi import DTYPE_NAMES
            name = DTYPE_NAMES[dt]
        else:
            name = np.dtype(dt).name
    if name not in DTYPES:
        raise ValueError(f"unsupported dtype {dt!r}")
    return DType(name)


def is_float(dt):
    return dt in _FLOATS


def dsize(dt):
    return _DSIZE[str(dt)]


def _float_dtype(ds, has_scalar=False, has_bf16=False):
    amp = _FLAGS.amp_reg
    if not has_scalar:
        if amp & AMP_PREFER32:
            return "float32"
        if amp & AMP_PREFER16:
            return "bfloat16" if has_bf16 else "float16"
    return "float64" if ds == 3 else "float32" if ds == 2 else ("bfloat16" if has_bf16 else "float16")


def _int_dtype(ds):
    return {3: "int64", 2: "int32", 1: "int16", 0: "int8"}[ds]


_BIN_CACHE = {}


def binary_dtype_infer(op, x, y, xscalar=False, yscalar=False):
    key = (op, str(x), str(y), xscalar, yscalar, _FLAGS.amp_reg)
    r = _BIN_CACHE.get(key)
    if r is None:
        r = _BIN_CACHE[key] = _binary_dtype_infer(op, x, y, xscalar, yscalar)
    return r


def _binary_dtype_infer(op, x, y, xscalar=False, yscalar=False):
    if op in BOOL_OPS:
        return DType("bool")
    ds = max(dsize(x), dsize(y))
    if xscalar:
        ds = dsize(y)
    if yscalar:
        ds = dsize(x)
    isf = op not in INT_OPS and (is_float(x) or is_float(y) or op in FLOAT_OPS)
    has_bf16 = x == "bfloat16" or y == "bfloat16"
    if isf:
        if op in WHITE_OPS and not (_FLAGS.amp_reg & AMP_KEEP_WHITE):
            return DType("float64" if ds == 3 else "float32")
        return DType(_float_dtype(ds, xscalar or yscalar, has_bf16))
    if x == "bool" and y == "bool":
        return DType("bool")
    return DType(_int_dtype(ds))


def unary_dtype_infer(op, x):
    if op in DTYPES:
        return DType(op)
    if op in BOOL_OPS:
        return DType("bool")
    ds = dsize(x)
    if op in FLOAT_OPS:
        if op in WHITE_OPS and not (_FLAGS.amp_reg & AMP_KEEP_WHITE):
            return DType("float64" if ds == 3 else "float32")
        return DType(_float_dtype(ds, False, x == "bfloat16"))
    if op in INT_OPS:
        return DType(_int_dtype(ds))
    return DType(x)


def reduce_dtype_infer(op, x):
    if x == "bool":
        return DType("int32")
    isf = is_float(x) or op in FLOAT_OPS
    ds = dsize(x)
    if isf:
        if _FLAGS.amp_reg & AMP_KEEP_REDUCE:
            return DType(_float_dtype(ds, False, x == "bfloat16"))
        return DType("float64" if ds == 3 else "float32")
    return DType(x)
