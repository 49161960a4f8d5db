"""ctypes binding of libb200jt.so (declared in include/b200jt.h).

The library is the only compute path of this package: if it is missing the import fails with
instructions to build it, and a call without a CUDA device raises -- there is no CPU fallback.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libb200jt.so")

MAX_DIMS = 10

DTYPE_CODES = {"bool": 0, "int8": 1, "int16": 2, "int32": 3, "int64": 4, "uint8": 5,
               "float16": 6, "bfloat16": 7, "float32": 8, "float64": 9}
TORCH_DTYPES = {"bool": torch.bool, "int8": torch.int8, "int16": torch.int16, "int32": torch.int32,
                "int64": torch.int64, "uint8": torch.uint8, "float16": torch.float16,
                "bfloat16": torch.bfloat16, "float32": torch.float32, "float64": torch.float64}
DTYPE_NAMES = {v: k for k, v in TORCH_DTYPES.items()}


class Tensor(ctypes.Structure):
    """struct b200jt_tensor"""
    _fields_ = [("ptr", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32),
                ("shape", ctypes.c_int64 * MAX_DIMS)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build the CUDA library first "
            f"(`make -C {os.path.join(_HERE, 'csrc')}` or `python -c 'import __graft_entry__ as g; g.build()'`). "
            "jittor_b200 has no CPU fallback.")
    return ctypes.CDLL(LIB_PATH)


lib = _load()

_TP = ctypes.POINTER(Tensor)
_SP = ctypes.POINTER(ctypes.c_char_p)
_vp, _i, _d, _u32, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_double, ctypes.c_uint32, ctypes.c_size_t
_FP = ctypes.c_void_p   # float* device pointers are passed as raw addresses

# every symbol of include/b200jt.h: (name, restype, argtypes)
SIGNATURES = [
    ("b200jt_last_error", ctypes.c_char_p, []),
    ("b200jt_version", _i, []),
    ("b200jt_index_affine", _i, [ctypes.POINTER(ctypes.c_int64), _i, ctypes.POINTER(ctypes.c_int64), _i, _SP, _i,
                                 ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]),
    ("b200jt_reindex", _i, [_TP, _TP, _SP, _i, _d, _SP, _i, _TP, _i, _vp]),
    ("b200jt_reindex_source", _i, [_TP, _TP, _SP, _i, _d, _SP, _i, _TP, _i, ctypes.c_char_p, ctypes.c_int64,
                                   ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(_i)]),
    ("b200jt_reindex_reduce_workspace", _sz, [_TP, _TP, ctypes.c_char_p, _SP, _i, _SP, _i, _TP, _i]),
    ("b200jt_reindex_reduce", _i, [_TP, _TP, ctypes.c_char_p, _SP, _i, _SP, _i, _TP, _i, _vp, _sz, _vp]),
    ("b200jt_reindex_reduce_noalloc_max_scratch", _sz, []),
    ("b200jt_reindex_reduce_noalloc", _i, [_TP, _TP, ctypes.c_char_p, _SP, _i, _SP, _i, _TP, _i, _vp]),
    ("b200jt_setitem", _i, [_TP, _TP, _TP, ctypes.c_char_p, _SP, _i, _TP, _i, _vp]),
    ("b200jt_broadcast_to", _i, [_TP, _TP, _u32, _vp]),
    ("b200jt_reduce_workspace", _sz, [_TP, _TP, ctypes.c_char_p, _u32]),
    ("b200jt_reduce", _i, [_TP, _TP, ctypes.c_char_p, _u32, _vp, _sz, _vp]),
    ("b200jt_binary", _i, [_TP, _TP, _TP, ctypes.c_char_p, _vp]),
    ("b200jt_unary", _i, [_TP, _TP, ctypes.c_char_p, _vp]),
    ("b200jt_ternary", _i, [_TP, _TP, _TP, _TP, _vp]),
    ("b200jt_fused_chain", _i, [_TP, _i, ctypes.POINTER(ctypes.c_int64), _i, _i, ctypes.POINTER(ctypes.c_int32), _i, _TP, _vp]),
    ("b200jt_fused_chain_source", _i, [_TP, _i, ctypes.POINTER(ctypes.c_int64), _i, _i, ctypes.POINTER(ctypes.c_int32), _i, _TP,
                                       ctypes.c_char_p, ctypes.c_int64, ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(_i)]),
    ("b200jt_chain_jit_stats", _i, [ctypes.POINTER(_i), ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    ("b200jt_softmax", _i, [_TP, _TP, _i, _vp]),
    ("b200jt_softmax_backward", _i, [_TP, _TP, _TP, _i, _vp]),
    ("b200jt_layer_norm", _i, [_TP, _TP, _TP, _TP, _d, _vp]),
    ("b200jt_matmul_workspace", _sz, [_TP, _TP, _TP, _i, _i]),
    ("b200jt_matmul", _i, [_TP, _TP, _TP, _i, _i, _vp, _sz, _vp]),
    ("b200jt_batched_matmul", _i, [_TP, _TP, _TP, _i, _i, _vp]),
    ("b200jt_device_status", _i, []),
    ("b200jt_conv2d_workspace", _sz, [_TP, _TP, _TP, _i, _i, _i, _i, _i, _i, _i]),
    ("b200jt_conv2d", _i, [_TP, _TP, _TP, _i, _i, _i, _i, _i, _i, _i, _FP, _vp, _sz, _vp]),
    ("b200jt_conv2d_formats_workspace", _sz, [_TP, _TP, _TP, _i, _i, _i, _i, _i, _i, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p]),
    ("b200jt_conv2d_formats", _i, [_TP, _TP, _TP, _i, _i, _i, _i, _i, _i, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p,
                                   _FP, _vp, _sz, _vp]),
    ("b200jt_conv2d_transpose", _i, [_TP, _TP, _TP, _i, _i, _i, _i, _i, _i, _i, _vp]),
    ("b200jt_conv2d_backward_w", _i, [_TP, _TP, _TP, _i, _i, _i, _i, _i, _i, _vp]),
    ("b200jt_conv2d_backward_w_workspace", _sz, [_TP, _TP, _TP, _i, _i, _i, _i, _i, _i]),
    ("b200jt_conv2d_backward_w_tc", _i, [_TP, _TP, _TP, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    ("b200jt_conv2d_backward_w_formats_workspace", _sz, [_TP, _TP, _TP, _i, _i, _i, _i, _i, _i, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p]),
    ("b200jt_conv2d_backward_w_formats", _i, [_TP, _TP, _TP, _i, _i, _i, _i, _i, _i, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p,
                                              _vp, _sz, _vp]),
    ("b200jt_bn_stats", _i, [_TP, _FP, _vp]),
    ("b200jt_bn_apply", _i, [_TP, _FP, _d, _FP, _FP, _d, _i, _TP, _FP, _FP, _d, _vp]),
    ("b200jt_pool2d", _i, [_TP, _TP, _vp, ctypes.c_char_p, _i, _i, _i, _i, _i, _i, _i, _vp]),
    ("b200jt_pool2d_backward", _i, [_TP, _TP, _TP, _TP, ctypes.c_char_p, _i, _i, _i, _i, _i, _i, _i, _vp]),
    ("b200jt_pool2d_backward_indices", _i, [_TP, _TP, _vp, _TP, _TP, _i, _i, _i, _i, _i, _i, _vp]),
    ("b200jt_peer_segment_bytes", _sz, [_sz]),
    ("b200jt_peer_segment_create", _i, [_sz, ctypes.POINTER(_vp), ctypes.c_char_p]),
    ("b200jt_peer_segment_destroy", _i, [_vp]),
    ("b200jt_peer_comm_create", _i, [_i, _i, _vp, ctypes.c_char_p, _sz, _d, ctypes.POINTER(_vp)]),
    ("b200jt_peer_comm_destroy", _i, [_vp]),
    ("b200jt_peer_max_bytes", _sz, [_vp]),
    ("b200jt_peer_comm_set_max_blocks", _i, [_vp, _i]),
    ("b200jt_set_sm_reserve", _i, [_i]),
    ("b200jt_probe_rate", _i, [ctypes.c_char_p, _i, _vp, ctypes.c_int64, ctypes.POINTER(ctypes.c_double)]),
    ("b200jt_peer_all_reduce", _i, [_vp, _vp, _vp, ctypes.c_int64, _i, ctypes.c_char_p, _vp]),
    ("b200jt_peer_comm_create_local", _i, [_i, _sz, _d, ctypes.POINTER(_vp)]),
    ("b200jt_peer_all_reduce_local", _i, [ctypes.POINTER(_vp), _i, ctypes.POINTER(_vp), ctypes.POINTER(_vp),
                                          ctypes.c_int64, _i, ctypes.c_char_p, _vp]),
]
for _name, _res, _args in SIGNATURES:
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


class B200Error(RuntimeError):
    pass


def check(rc, what=""):
    if rc != 0:
        msg = lib.b200jt_last_error().decode(errors="replace")
        raise B200Error(f"{what}: {msg} (status {rc})" if what else f"{msg} (status {rc})")


def require_cuda():
    if not torch.cuda.is_available():
        raise B200Error("jittor_b200 needs a CUDA device (sm_100a); there is no CPU fallback")


def desc(t, shape=None):
    """b200jt_tensor for a contiguous torch tensor, optionally viewed with another shape of equal size."""
    if not t.is_contiguous():
        raise B200Error("internal: non-contiguous tensor passed to the C ABI")
    shp = list(t.shape) if shape is None else list(shape)
    if len(shp) == 0:
        shp = [1]
    if len(shp) > MAX_DIMS:
        raise B200Error(f"tensors have at most {MAX_DIMS} dims, got {len(shp)}")
    d = Tensor()
    d.ptr = t.data_ptr() if t.numel() else None
    d.dtype = DTYPE_CODES[DTYPE_NAMES[t.dtype]]
    d.ndim = len(shp)
    for i, s in enumerate(shp):
        d.shape[i] = int(s)
    return d


def strings(items):
    arr = (ctypes.c_char_p * max(len(items), 1))()
    for i, s in enumerate(items):
        arr[i] = s.encode()
    return arr


def descs(tensors):
    arr = (Tensor * max(len(tensors), 1))()
    for i, t in enumerate(tensors):
        arr[i] = desc(t)
    return arr


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
