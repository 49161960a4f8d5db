"""Op registry and the inline-CUDA op `jt.code`.

The reference keeps a name -> constructor registry (python/jittor/src/ops/op_register.h:14-33; `has_op`,
`get_op_info(name).get_constructor`) that its tuners use to find relay ops and that `compile_custom_ops` fills with
user ops. Here the registry maps the same names to Python callables over Vars: the built-in meta-operators, the relay
names the tuners look up (`cublas_matmul`, `cudnn_conv`, `nccl_all_reduce`), and anything registered with
`register_op`.

`code(shape, dtype, inputs, cuda_src=..., cuda_header=...)` is the inline op of python/jittor/src/ops/code_op.h:24-46
with the macro set of python/jittor/src/ops/code_op.cc:186-231: `@ARGS_DEF`, `@ARGS`, `@PRECALC`, `@inK(i,j,..)`,
`@out(i,..)` / `@outK(..)`, `inK_shapeJ`, `inK_strideJ`, `inK_type`, leading `__global__` / `__device__` functions
hoisted out of the body. The source is compiled with nvcc for sm_100a into a cache directory, loaded with ctypes and
launched on the current stream. C++ op classes in the reference's custom-op form are built by custom_op.py against a
stand-in for the core headers.
"""
import ctypes
import hashlib
import os
import re
import subprocess
import tempfile

from . import var as V
from ._capi import B200Error, TORCH_DTYPES, require_cuda

_REGISTRY = {}


class OpInfo:
    def __init__(self, name, fn, doc=""):
        self.name, self.fn, self.doc = name, fn, doc

    def get_constructor(self, *signature):
        return self.fn

    def __call__(self, *a, **k):
        return self.fn(*a, **k)


def register_op(name, fn, doc=""):
    """Registers `fn(*vars, **attrs) -> Var` under `name` (the role of op_registe)."""
    _REGISTRY[name] = OpInfo(name, fn, doc)
    return fn


def has_op(name):
    return name in _REGISTRY


def get_op_info(name):
    if name not in _REGISTRY:
        raise KeyError(f"Op {name} not registered")
    return _REGISTRY[name]


def compile_custom_op(header, source, op_name=None, warp=True):
    """C++ op classes in the reference's custom-op form: see custom_op.py."""
    from . import custom_op
    return custom_op.compile_custom_op(header, source, op_name, warp)


def compile_custom_ops(filenames, extra_flags="", return_module=False, **kw):
    from . import custom_op
    return custom_op.compile_custom_ops(filenames, extra_flags, return_module, **kw)


def _register_builtins():
    from . import nn, dist
    register_op("reindex", V.reindex)
    register_op("reindex_reduce", V.reindex_reduce)
    register_op("broadcast_to", V.broadcast)
    register_op("reduce", V.reduce)
    register_op("binary", V.binary)
    register_op("unary", V.unary)
    register_op("ternary", V.ternary)
    register_op("code", code)

    def cublas_matmul(a, b, trans_a, trans_b):
        """Relay signature of matmul_tuner.cc:93-95."""
        a, b = V.to_var(a), V.to_var(b)
        if trans_a:
            a = a.transpose(1, 0)
        return nn.matmul_transpose(a, b) if trans_b else nn.matmul(a, b)

    def cudnn_conv(x, w, strideh, stridew, paddingh, paddingw, dilationh=1, dilationw=1, groups=1,
                   xformat="abcd", wformat="oihw", yformat=""):
        """Relay signature of conv_tuner.cc:370-373. Layouts as ConvTuner derives them (conv_tuner.cc:292-341): x / y "abcd"
        (NCHW) or "acdb" (NHWC, the tensor-core kernel's own operand layout: no layout pass on that side), w "oihw" or
        "ohwi"; an empty yformat follows xformat."""
        if xformat == "abcd" and wformat == "oihw" and yformat in ("", "abcd"):
            return nn.conv2d(x, w, None, (strideh, stridew), (paddingh, paddingw), (dilationh, dilationw), groups)
        if xformat not in ("abcd", "acdb") or wformat not in ("oihw", "ohwi") or yformat not in ("", "abcd", "acdb"):
            raise ValueError(f"unknown conv layouts x {xformat!r} w {wformat!r} y {yformat!r}")
        if groups != 1:
            raise NotImplementedError("acdb / ohwi layouts with groups > 1")
        from . import executor
        x, w = V.to_var(x), V.to_var(w)
        yf = yformat or xformat
        n, h, wd_ = (x.shape[0], x.shape[2], x.shape[3]) if xformat == "abcd" else (x.shape[0], x.shape[1], x.shape[2])
        co, kh, kw = (w.shape[0], w.shape[2], w.shape[3]) if wformat == "oihw" else (w.shape[0], w.shape[1], w.shape[2])
        oh = (h + 2 * paddingh - kh * dilationh + dilationh - 1) // strideh + 1
        ow = (wd_ + 2 * paddingw - kw * dilationw + dilationw - 1) // stridew + 1
        shape = [n, co, oh, ow] if yf == "abcd" else [n, oh, ow, co]
        geo = (strideh, stridew, paddingh, paddingw, dilationh, dilationw)
        return _relayed(x, w, shape, lambda xd, wd: executor.run_conv2d_formats(x, w, geo, xformat, wformat, yf, x.dtype))

    def _relayed(x, w_or_dy, shape, run):
        """A Var produced by one relay launch (inputs synced by the executor first)."""
        node = V.Op("custom", [V.to_var(x), V.to_var(w_or_dy)], fn=run, name="relay")
        return V.Var(shape, V.to_var(x).dtype, node)

    def cudnn_conv_backward_x(w, dy, height, width, strideh, stridew, paddingh, paddingw, dilationh=1, dilationw=1, groups=1,
                              xformat="abcd", wformat="oihw", yformat="abcd"):
        """Relay signature of conv_tuner.cc:382-389: dx[N, Cin, height, width] from w (OIHW) and dy."""
        if xformat != "abcd" or wformat != "oihw" or yformat != "abcd" or groups != 1:
            raise NotImplementedError("only abcd / oihw layouts, groups == 1")
        from . import executor
        w, dy = V.to_var(w), V.to_var(dy)
        shape = [dy.shape[0], w.shape[1], height, width]
        geo = (strideh, stridew, paddingh, paddingw, dilationh, dilationw)
        return _relayed(dy, w, shape, lambda dyd, wd: executor.run_conv2d_transpose(dy, w, geo, 1, shape, dy.dtype))

    def cudnn_conv_backward_w(x, dy, kh, kw, strideh, stridew, paddingh, paddingw, dilationh=1, dilationw=1, groups=1,
                              xformat="abcd", wformat="oihw", yformat="abcd"):
        """Relay signature of conv_tuner.cc:390-396: dw[Cout, Cin, kh, kw] from x and dy. xformat / yformat "acdb": x / dy are
        channels-last (read by the tensor-core kernel as they are); wformat "ohwi": dw comes out [Cout, kh, kw, Cin]."""
        if xformat not in ("abcd", "acdb") or wformat not in ("oihw", "ohwi") or yformat not in ("abcd", "acdb"):
            raise ValueError(f"unknown conv layouts x {xformat!r} w {wformat!r} y {yformat!r}")
        if groups != 1:
            raise NotImplementedError("weight gradient relay with groups > 1")
        from . import executor
        x, dy = V.to_var(x), V.to_var(dy)
        geo = (strideh, stridew, paddingh, paddingw, dilationh, dilationw)
        if xformat == "abcd" and wformat == "oihw" and yformat == "abcd":
            shape = [dy.shape[1], x.shape[1], kh, kw]
            return _relayed(x, dy, shape, lambda xd, dyd: executor.run_conv2d_backward_w(x, dy, geo, shape, x.dtype))
        ci = x.shape[1] if xformat == "abcd" else x.shape[3]
        co = dy.shape[1] if yformat == "abcd" else dy.shape[3]
        shape = [co, ci, kh, kw] if wformat == "oihw" else [co, kh, kw, ci]
        return _relayed(x, dy, shape, lambda xd, dyd: executor.run_conv2d_backward_w_formats(
            x, dy, geo, kh, kw, xformat, wformat, yformat, x.dtype))

    register_op("cublas_matmul", cublas_matmul)
    register_op("cudnn_conv", cudnn_conv)
    register_op("cudnn_conv_backward_x", cudnn_conv_backward_x)
    register_op("cudnn_conv_backward_w", cudnn_conv_backward_w)
    register_op("nccl_all_reduce", lambda x: dist.mpi_all_reduce(x, "add"))
    register_op("mpi_all_reduce", dist.mpi_all_reduce)
    register_op("mpi_reduce", dist.mpi_reduce)
    register_op("mpi_broadcast", dist.mpi_broadcast)
    register_op("nccl_reduce", lambda x, root=0: dist.mpi_reduce(x, "add", root))
    register_op("nccl_broadcast", lambda x, root=0: dist.mpi_broadcast(x, root))


# ----------------------------------------------------------------------------------------------- jt.code
_CTYPES = {"bool": "bool", "int8": "int8_t", "int16": "int16_t", "int32": "int32_t", "int64": "int64_t", "uint8": "uint8_t",
           "float16": "__half", "bfloat16": "__nv_bfloat16", "float32": "float", "float64": "double"}
_CACHE_DIR = os.environ.get("JITTOR_B200_CACHE", os.path.join(os.path.expanduser("~"), ".cache", "jittor_b200"))
_LOADED = {}


def _split_leading_functions(src):
    """Leading functions (text starting with '_', i.e. __global__/__device__, up to the matching brace) are hoisted
    in front of the entry function; the rest is its body (code_op.cc:155-178)."""
    i, n, head = 0, len(src), []
    while i < n:
        if src[i] in " \t\n":
            head.append(src[i])
            i += 1
        elif src[i] == "_":
            depth = 0
            while i < n:
                head.append(src[i])
                if src[i] == "{":
                    depth += 1
                elif src[i] == "}":
                    depth -= 1
                    if depth == 0:
                        i += 1
                        break
                i += 1
        else:
            break
    return "".join(head), src[i:]


def expand_code_source(cuda_src, cuda_header, in_meta, out_meta):
    """Returns the full .cu text. in_meta / out_meta: lists of (dtype name, ndim)."""
    names = [f"in{i}" for i in range(len(in_meta))] + [f"out{i}" for i in range(len(out_meta))]
    metas = list(in_meta) + list(out_meta)
    args_def, args, precalc, defines = [], [], [], []
    for nm, (dt, nd) in zip(names, metas):
        defines.append(f"typedef {_CTYPES[dt]} {nm}_type;")
        defines.append(f"#define {nm}_stride{nd - 1} 1")
        args_def.append(f"{nm}_type* __restrict__ {nm}_p")
        args.append(f"{nm}_p")
        for j in range(nd):
            args_def.append(f"index_t {nm}_shape{j}")
            args.append(f"{nm}_shape{j}")
        for j in range(nd - 2, -1, -1):
            precalc.append(f"auto {nm}_stride{j} = {nm}_stride{j + 1} * {nm}_shape{j + 1};")
    args_def.append("int __tmp")
    args.append("0")

    def access(m):
        nm = m.group(1)
        if nm == "out":
            nm = "out0"
        idx = [s.strip() for s in _split_args(m.group(2))]
        return f"{nm}_p[" + "+".join(f"({e})*{nm}_stride{j}" for j, e in enumerate(idx)) + "]"

    def expand(text):
        text = text.replace("@ARGS_DEF", ", ".join(args_def)).replace("@ARGS", ", ".join(args))
        text = text.replace("@PRECALC", "\n".join(precalc))
        prev = None
        while prev != text:          # nested accesses resolve inside-out
            prev = text
            text = re.sub(r"@(in\d+|out\d*)\(([^()@]*(?:\([^()@]*\)[^()@]*)*)\)", access, text)
        if "@" in text:
            bad = re.search(r"@\w+", text)
            raise B200Error(f"jt.code: unsupported macro {bad.group(0) if bad else '@'}")
        # launches without an explicit stream go to the stream the executor passes in
        return re.sub(r"<<<\s*([^,<>]+?)\s*,\s*([^,<>]+?)\s*>>>", r"<<<\1, \2, 0, __stream>>>", text)

    head, body = _split_leading_functions(cuda_src)
    unpack = []
    k = 0
    for nm, (dt, nd) in zip(names, metas):
        unpack.append(f"    {nm}_type* __restrict__ {nm}_p = ({nm}_type*)__ptrs[{names.index(nm)}];")
        for j in range(nd):
            unpack.append(f"    index_t {nm}_shape{j} = (index_t)__shapes[{k}];")
            k += 1
    return "\n".join([
        "#include <cuda_runtime.h>", "#include <cuda_bf16.h>", "#include <cuda_fp16.h>", "#include <stdint.h>",
        "typedef int64_t int64; typedef int32_t int32; typedef float float32; typedef double float64;",
        "typedef int index_t;", *defines, "static cudaStream_t __stream = 0;", expand(cuda_header or ""), expand(head),
        'extern "C" int b200jt_code_entry(void** __ptrs, const int64_t* __shapes, void* __s) {',
        "    __stream = (cudaStream_t)__s;", *unpack, expand(body),
        "    return (int)cudaGetLastError();", "}", ""])


def _split_args(s):
    out, depth, cur = [], 0, []
    for ch in s:
        if ch == "," and depth == 0:
            out.append("".join(cur))
            cur = []
        else:
            depth += ch == "("
            depth -= ch == ")"
            cur.append(ch)
    out.append("".join(cur))
    return out


def compile_code_source(text):
    """nvcc -> shared object in the cache directory (keyed by the source hash); returns its path."""
    key = hashlib.sha1(text.encode()).hexdigest()[:20]
    so = os.path.join(_CACHE_DIR, f"code_{key}.so")
    if not os.path.exists(so):
        os.makedirs(_CACHE_DIR, exist_ok=True)
        with tempfile.TemporaryDirectory() as tmp:
            cu = os.path.join(tmp, f"code_{key}.cu")
            with open(cu, "w") as f:
                f.write(text)
            cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-shared",
                   "-Xcompiler", "-fPIC", "-o", so + ".tmp", cu]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise B200Error("jt.code: nvcc failed\n" + res.stderr[-4000:] + "\n--- source ---\n" + text)
            os.replace(so + ".tmp", so)
    return so


def _alias(text, name, target):
    """@alias(name, target) of python/jittor/src/ops/code_op.cc:108-117: `@name(..)`, `name_shapeK`, `name_strideK`,
    `name_type`, `name_p` mean the same as for `target`."""
    text = re.sub(rf"@{name}\(", f"@{target}(", text)
    return re.sub(rf"\b{name}_(shape\d+|stride\d+|type|p)\b", rf"{target}_\1", text)


def code(shape, dtype, inputs=(), cpu_src="", cpu_grad_src=(), cpu_header="", cuda_src="", cuda_grad_src=(), cuda_header="",
         data=None):
    """Inline CUDA op, python/jittor/src/ops/code_op.h:24-46,265-271. `shape` / `dtype` may be lists for several outputs
    (then a list of Vars is returned). `cuda_grad_src[k]` is the source of the gradient with respect to input k: it is run
    as another inline op with the shape and dtype of that input, whose inputs are the forward inputs followed by the output
    gradient (`@dout(..)`) and the forward outputs (`@pout(..)`, `@poutK(..)`), python/jittor/src/ops/code_op.cc:100-127."""
    if not cuda_src:
        raise B200Error("jt.code: only cuda_src is supported (there is no CPU path)")
    if data:
        raise B200Error("jt.code: the `data` dictionary is not supported; pass scalars as one-element inputs")
    multi = len(shape) > 0 and isinstance(shape[0], (list, tuple, V.Shape))
    shapes = [list(s) for s in shape] if multi else [list(shape)]
    dtypes = list(dtype) if multi else [dtype]
    inputs = [V.to_var(i) for i in inputs]
    in_meta = [(str(v.dtype), v.ndim) for v in inputs]
    out_meta = [(str(V.dt.canon(d)), len(s)) for d, s in zip(dtypes, shapes)]
    text = expand_code_source(cuda_src, cuda_header, in_meta, out_meta)
    cuda_grad_src = list(cuda_grad_src or ())

    def grad_rule(out, dout, k):
        if k >= len(cuda_grad_src) or not cuda_grad_src[k] or multi:
            return None
        n = len(inputs)
        src, header = cuda_grad_src[k], cuda_header
        for name, target in (("dout", f"in{n}"), ("pout0", f"in{n + 1}"), ("pout", f"in{n + 1}")):
            src, header = _alias(src, name, target), _alias(header, name, target)
        return code(list(inputs[k].shape), inputs[k].dtype, inputs + [dout, out], cuda_src=src, cuda_header=header)

    def run(*tensors):
        import torch
        require_cuda()
        so = compile_code_source(text)
        lib = _LOADED.get(so)
        if lib is None:
            lib = _LOADED[so] = ctypes.CDLL(so)
            lib.b200jt_code_entry.restype = ctypes.c_int
            lib.b200jt_code_entry.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p]
        outs = [torch.empty(s, dtype=TORCH_DTYPES[m[0]], device="cuda") for s, m in zip(shapes, out_meta)]
        allt = list(tensors) + outs
        ptrs = (ctypes.c_void_p * len(allt))(*[t.data_ptr() for t in allt])
        dims = [d for t, (_, nd) in zip(allt, in_meta + out_meta) for d in (list(t.shape) + [1] * nd)[:nd]]
        shp = (ctypes.c_int64 * max(len(dims), 1))(*dims)
        rc = lib.b200jt_code_entry(ptrs, shp, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise B200Error(f"jt.code: CUDA error {rc} after launch")
        return outs

    if not multi:
        return V.Var(shapes[0], out_meta[0][0], V.Op("custom", inputs, fn=lambda *t: run(*t)[0], grad=grad_rule))
    # several outputs: one node computes all of them, the others pick their tensor from it
    box = {}

    def run_all(*t):
        box["outs"] = run(*t)
        return box["outs"][0]

    first = V.Var(shapes[0], out_meta[0][0], V.Op("custom", inputs, fn=run_all))
    rest = [V.Var(s, m[0], V.Op("custom", [first], fn=(lambda k: lambda _f: box["outs"][k])(k)))
            for k, (s, m) in enumerate(zip(shapes[1:], out_meta[1:]), start=1)]
    return [first] + rest
