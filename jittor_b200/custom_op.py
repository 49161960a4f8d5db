"""`compile_custom_ops` / `compile_custom_op`: user ops written as C++ classes in the reference's documented form
(python/jittor/compiler.py:624-771, python/jittor/test/test_custom_op.py:12-107).

An op is a header declaring `struct XxxOp : Op` (Var* members, a constructor, `name()`, `DECLARE_jit_run`) and a source
with two halves: outside `JIT` the constructor (which calls `create_output`) and `jit_prepare` (which adds the defines of
the JIT key); inside `JIT` the `jit_run` body, compiled once per key with those defines. The reference parses the header
with regular expressions, generates `make_<name>` bindings and registers the op by name; this module does the same against
a small stand-in for the core headers (shim/jittor_shim.h):

  stage 1  g++: shim + header + non-JIT half -> a library that constructs the op (so output shapes and dtypes are known
           when the lazy Var is made) and reports the jit defines;
  stage 2  per key: shim + header + JIT half with `-DJIT -DJIT_cuda` (nvcc, sm_100a) when the source has a CUDA branch,
           else `-DJIT_cpu` (g++): `jit_run` is called on the SAME op object the first library built.

A CUDA op launches on the default stream with device pointers; a host-only op (like the reference's own test ops) runs
on host copies of its inputs and its outputs are uploaded -- that is the user's code, not a compute path of this package.
Ops that need more of the core than the shim offers fail to compile, and the compiler's message is passed on.
"""
import ctypes
import hashlib
import os
import re
import subprocess
import tempfile
import types
import weakref

from . import var as V
from ._capi import B200Error, TORCH_DTYPES, require_cuda
from .op_register import _CACHE_DIR, register_op

_SHIM_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "shim")
_LIBS = {}


class _OpDecl:
    """What the reference's header scan extracts (python/jittor/compiler.py:421-454)."""

    def __init__(self, header):
        m = re.search(r"struct\s+(\w+)Op\s*:\s*Op\s*\{(.*?)\n\s*\}\s*;", header, re.S)
        if not m:
            raise B200Error("compile_custom_op: no `struct XxxOp : Op { ... };` found in the header")
        self.cls = m.group(1) + "Op"
        body = m.group(2)
        nm = re.search(r'name\s*\(\s*\)\s*const\s*(?:override)?\s*\{\s*return\s*"(\w+)"', body)
        self.name = nm.group(1) if nm else re.sub(r"(?<!^)(?=[A-Z])", "_", m.group(1)).lower()
        ctor = re.search(rf"\b{self.cls}\s*\(([^)]*)\)\s*;", body)
        if not ctor:
            raise B200Error(f"compile_custom_op: {self.cls} declares no constructor")
        self.params = []
        for raw in [p.strip() for p in ctor.group(1).split(",") if p.strip()]:
            default = None
            if "=" in raw:
                raw, default = [s.strip() for s in raw.split("=", 1)]
            pm = re.match(r"(.*?)(\w+)$", raw)
            ctype = re.sub(r"\s+", "", pm.group(1))
            self.params.append((self._kind(ctype, raw), pm.group(2), default))

    @staticmethod
    def _kind(ctype, raw):
        t = ctype.replace("const", "").replace("&", "").replace("std::", "")
        table = {"Var*": "var", "vector<Var*>": "vars", "NanoVector": "shape", "NanoString": "nstr", "string": "str",
                 "bool": "bool", "int": "int", "int32": "int", "int64": "int", "uint": "int", "uint32": "int", "uint64": "int",
                 "float": "float", "float32": "float", "float64": "float", "double": "float"}
        if t not in table:
            raise B200Error(f"compile_custom_op: constructor parameter `{raw}` has a type the binding generator does not know")
        return table[t]


_CONVERT = {
    "var": "(Var*)a[{i}]",
    "vars": "[&]{{ void** p = (void**)a[{i}]; std::vector<Var*> v; for (long k = 0; k < (long)(intptr_t)p[0]; k++) v.push_back((Var*)p[k + 1]); return v; }}()",
    "shape": "[&]{{ const int64_t* p = (const int64_t*)a[{i}]; NanoVector v; for (int64_t k = 0; k < p[0]; k++) v.push_back(p[k + 1]); return v; }}()",
    "nstr": "NanoString((const char*)a[{i}])",
    "str": "std::string((const char*)a[{i}])",
    "bool": "(*(const double*)a[{i}] != 0)",
    "int": "(long long)(*(const double*)a[{i}])",
    "float": "(*(const double*)a[{i}])",
}


def _stage1_source(decl, header, source):
    args = ", ".join(_CONVERT[k].format(i=i) for i, (k, _, _) in enumerate(decl.params))
    return f'''#include "jittor_shim.h"
{_strip_includes(header)}
{_strip_includes(source)}
namespace jittor {{ void {decl.cls}::jit_run() {{}} }}
using namespace jittor;
static thread_local std::string g_err;
static thread_local std::string g_defines;
extern "C" {{
void* b200jt_var_new(int ndim, const int64_t* shape, const char* dtype) {{
    Var* v = new Var(); v->dtype_ = NanoString(dtype);
    NanoVector s; for (int i = 0; i < ndim; i++) s.push_back(shape[i]);
    v->set_shape(s); return v;
}}
void b200jt_var_set_ptr(void* v, void* p) {{ ((Var*)v)->mem_ptr = p; }}
void b200jt_var_free(void* v) {{ delete (Var*)v; }}
const char* b200jt_op_error() {{ return g_err.c_str(); }}
void* b200jt_op_new(void** a) {{
    try {{ return new {decl.cls}({args}); }}
    catch (const std::exception& e) {{ g_err = e.what(); return nullptr; }}
}}
int b200jt_op_n_outputs(void* op) {{ return (int)((Op*)op)->outputs_.size(); }}
int b200jt_op_output(void* op, int i, int64_t* shape, char* dtype) {{
    Var* v = ((Op*)op)->outputs_[i];
    for (int k = 0; k < v->shape.size(); k++) shape[k] = v->shape[k];
    strcpy(dtype, v->dtype_.to_cstring());
    return v->shape.size();
}}
void b200jt_op_output_set_ptr(void* op, int i, void* p) {{ ((Op*)op)->outputs_[i]->mem_ptr = p; }}
const char* b200jt_op_defines(void* op) {{
    JK jk; ((Op*)op)->jit_prepare(jk); g_defines = jk.defines; return g_defines.c_str();
}}
void b200jt_op_free(void* op) {{ delete (Op*)op; }}
}}
'''


def _stage2_source(decl, header, source, defines, cuda):
    defs = "\n".join(f"#define {k} {v}" for k, v in defines)
    return f'''#define JIT 1
#define {"JIT_cuda" if cuda else "JIT_cpu"} 1
{defs}
#include "jittor_shim.h"
{_strip_includes(header)}
{_strip_includes(source)}
extern "C" int b200jt_op_run(void* op) {{
    try {{ ((jittor::{decl.cls}*)op)->jittor::{decl.cls}::jit_run(); }} catch (const std::exception&) {{ return -1; }}
    return {"(int)cudaGetLastError()" if cuda else "0"};
}}
'''


def _strip_includes(text):
    """The user's sources include the reference's core headers and their own header by name; both are already in the
    translation unit, so quoted includes are dropped (system includes stay)."""
    text = re.sub(r'^\s*#\s*include\s+"[^"]+"\s*$', "", text, flags=re.M)
    return re.sub(r"^\s*#\s*pragma\s+once\s*$", "", text, flags=re.M)


def _build(text, cuda, tag):
    key = hashlib.sha1((text + ("cuda" if cuda else "cpu")).encode()).hexdigest()[:20]
    so = os.path.join(_CACHE_DIR, f"{tag}_{key}.so")
    if not os.path.exists(so):
        os.makedirs(_CACHE_DIR, exist_ok=True)
        with tempfile.TemporaryDirectory() as tmp:
            src = os.path.join(tmp, f"{tag}_{key}." + ("cu" if cuda else "cc"))
            with open(src, "w") as f:
                f.write(text)
            if cuda:
                cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-shared",
                       "-Xcompiler", "-fPIC", "-I", _SHIM_DIR, "-o", so + ".tmp", src]
            else:
                cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I", _SHIM_DIR, "-o", so + ".tmp", src]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise B200Error(f"compile_custom_op: {cmd[0]} failed (the op may need parts of the reference's core that the "
                                "shim header does not provide)\n" + res.stderr[-4000:])
            os.replace(so + ".tmp", so)
    if so not in _LIBS:
        _LIBS[so] = ctypes.CDLL(so)
    return _LIBS[so]


class _OpState:
    """Keeps one constructed op object (and the stand-in Vars of its inputs) alive as long as its output Var."""

    def __init__(self, op, keep):
        self.op, self.keep = op, keep


class CustomOp:
    """One compiled op: calling it builds the lazy Var(s), like the generated `make_<name>` of the reference."""

    def __init__(self, header, source):
        self.decl = _OpDecl(header)
        self.header, self.source = header, source
        # the reference compiles for CUDA when the source has a CUDA branch; otherwise jit_run is host code
        self.cuda = "JIT_cuda" in source or "<<<" in source
        lib = self.lib = _build(_stage1_source(self.decl, header, source), False, f"op_{self.decl.name}")
        lib.b200jt_var_new.restype = ctypes.c_void_p
        lib.b200jt_var_new.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int64), ctypes.c_char_p]
        lib.b200jt_var_set_ptr.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.b200jt_var_free.argtypes = [ctypes.c_void_p]
        lib.b200jt_op_error.restype = ctypes.c_char_p
        lib.b200jt_op_new.restype = ctypes.c_void_p
        lib.b200jt_op_new.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
        lib.b200jt_op_n_outputs.argtypes = [ctypes.c_void_p]
        lib.b200jt_op_output.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int64), ctypes.c_char_p]
        lib.b200jt_op_output_set_ptr.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        lib.b200jt_op_defines.restype = ctypes.c_char_p
        lib.b200jt_op_defines.argtypes = [ctypes.c_void_p]
        lib.b200jt_op_free.argtypes = [ctypes.c_void_p]
        self.__name__ = self.decl.name

    # ---- argument marshalling ---------------------------------------------------------------------
    def _shim_var(self, v, keep):
        shp = (ctypes.c_int64 * max(v.ndim, 1))(*v.shape)
        h = self.lib.b200jt_var_new(v.ndim, shp, str(v.dtype).encode())
        keep.append(("var", h))
        return h

    def _marshal(self, args, kwargs):
        params = self.decl.params
        if len(args) > len(params):
            raise TypeError(f"{self.decl.name}() takes at most {len(params)} arguments")
        values, keep, var_inputs, shim_inputs = [], [], [], []
        for i, (kind, name, default) in enumerate(params):
            if i < len(args):
                val = args[i]
            elif name in kwargs:
                val = kwargs[name]
            elif default is not None:
                val = self._default(kind, default)
            else:
                raise TypeError(f"{self.decl.name}() missing argument {name!r}")
            if kind == "var":
                v = V.to_var(val)
                h = self._shim_var(v, keep)
                var_inputs.append(v)
                shim_inputs.append(h)
                values.append(ctypes.c_void_p(h))
            elif kind == "vars":
                vs = [V.to_var(x) for x in val]
                hs = [self._shim_var(v, keep) for v in vs]
                var_inputs += vs
                shim_inputs += hs
                arr = (ctypes.c_void_p * (len(hs) + 1))(len(hs), *hs)
                keep.append(("buf", arr))
                values.append(ctypes.cast(arr, ctypes.c_void_p))
            elif kind == "shape":
                dims = [int(s) for s in val]
                arr = (ctypes.c_int64 * (len(dims) + 1))(len(dims), *dims)
                keep.append(("buf", arr))
                values.append(ctypes.cast(arr, ctypes.c_void_p))
            elif kind in ("nstr", "str"):
                s = str(V.dt.canon(val)) if kind == "nstr" and str(val) in ("float", "int", "double", "half") else str(val)
                buf = ctypes.create_string_buffer(s.encode())
                keep.append(("buf", buf))
                values.append(ctypes.cast(buf, ctypes.c_void_p))
            else:
                d = ctypes.c_double(float(val))
                keep.append(("buf", d))
                values.append(ctypes.cast(ctypes.pointer(d), ctypes.c_void_p))
        return values, keep, var_inputs, shim_inputs

    @staticmethod
    def _default(kind, text):
        text = text.strip()
        if kind == "nstr":
            return text[3:] if text.startswith("ns_") else text.strip('"')
        if kind == "str":
            return text.strip('"')
        if kind == "bool":
            return text in ("true", "1")
        if kind == "shape":
            return [int(s) for s in re.findall(r"-?\d+", text)]
        if kind in ("int", "float"):
            return float(text.rstrip("fFlL"))
        raise B200Error(f"no default conversion for {text!r}")

    # ---- graph construction ------------------------------------------------------------------------
    def __call__(self, *args, **kwargs):
        lib = self.lib
        values, keep, var_inputs, shim_inputs = self._marshal(args, kwargs)
        argv = (ctypes.c_void_p * max(len(values), 1))(*[v.value if isinstance(v, ctypes.c_void_p) else v for v in values])
        op = lib.b200jt_op_new(argv)
        if not op:
            for kind, h in keep:
                if kind == "var":
                    lib.b200jt_var_free(h)
            raise B200Error(f"{self.decl.cls}: " + lib.b200jt_op_error().decode(errors="replace"))
        outs = []
        for i in range(lib.b200jt_op_n_outputs(op)):
            shp, dt = (ctypes.c_int64 * 10)(), ctypes.create_string_buffer(16)
            nd = lib.b200jt_op_output(op, i, shp, dt)
            outs.append(([int(shp[k]) for k in range(nd)], dt.value.decode()))
        defines = [tuple(d.split("=", 1)) for d in lib.b200jt_op_defines(op).decode().split(";") if d]
        state = _OpState(op, keep)
        weakref.finalize(state, _release, lib, op, [h for kind, h in keep if kind == "var"])
        box = {}

        def run(*tensors):
            import torch
            require_cuda()
            jit = _build(_stage2_source(self.decl, self.header, self.source, defines, self.cuda), self.cuda,
                         f"jit_{self.decl.name}")
            jit.b200jt_op_run.argtypes = [ctypes.c_void_p]
            dev = "cuda" if self.cuda else "cpu"
            ins = [t if self.cuda else t.cpu() for t in tensors]
            res = [torch.empty(s, dtype=TORCH_DTYPES[d], device=dev) for s, d in outs]
            for h, t in zip(shim_inputs, ins):
                lib.b200jt_var_set_ptr(h, ctypes.c_void_p(t.data_ptr()))
            for i, t in enumerate(res):
                lib.b200jt_op_output_set_ptr(state.op, i, ctypes.c_void_p(t.data_ptr()))
            cur = torch.cuda.current_stream()
            if self.cuda and cur != torch.cuda.default_stream():       # the op launches on the default stream
                torch.cuda.default_stream().wait_stream(cur)
            rc = jit.b200jt_op_run(state.op)
            if rc != 0:
                raise B200Error(f"{self.decl.cls}::jit_run failed (status {rc})")
            if self.cuda and cur != torch.cuda.default_stream():
                cur.wait_stream(torch.cuda.default_stream())
            box["outs"] = [t if self.cuda else t.cuda() for t in res]
            return box["outs"][0]

        first = V.Var(outs[0][0], outs[0][1], V.Op("custom", var_inputs, fn=run, name=self.decl.name))
        first._custom_state = state
        if len(outs) == 1:
            return first
        rest = [V.Var(s, d, V.Op("custom", [first], fn=(lambda k: lambda _f: box["outs"][k])(k)))
                for k, (s, d) in enumerate(outs[1:], start=1)]
        return [first] + rest


def _release(lib, op, shim_vars):
    lib.b200jt_op_free(op)
    for h in shim_vars:
        lib.b200jt_var_free(h)


def compile_custom_op(header, source, op_name=None, warp=True):
    """python/jittor/compiler.py:624-660: header and source given as strings (without the namespace / include
    boilerplate when `warp`); returns the op's constructor function and registers it under its name."""
    if warp:
        header = "namespace jittor {\n" + header + "\n}\n"
        source = "namespace jittor {\n" + source + "\n}\n"
    op = CustomOp(header, source)
    if op_name is not None and op_name != op.decl.name:
        raise B200Error(f"compile_custom_op: the header's name() says {op.decl.name!r}, not {op_name!r}")
    register_op(op.decl.name, op)
    return op


def compile_custom_ops(filenames, extra_flags="", return_module=False, **_kw):
    """python/jittor/compiler.py:661-771: pairs `<name>_op.h` / `<name>_op.cc` from a list of files; returns a module
    whose attributes are the ops' constructor functions."""
    heads, srcs = {}, {}
    for fn in filenames:
        base = os.path.basename(fn)
        stem, ext = os.path.splitext(base)
        if not stem.endswith("_op"):
            raise B200Error(f"compile_custom_ops: {base} is not named <name>_op.h / <name>_op.cc")
        (heads if ext in (".h", ".hpp") else srcs)[stem] = fn
    mod = types.ModuleType("custom_ops")
    for stem, h in heads.items():
        if stem not in srcs:
            raise B200Error(f"compile_custom_ops: {stem}.h has no {stem}.cc")
        op = CustomOp(open(h).read(), open(srcs[stem]).read())
        register_op(op.decl.name, op)
        setattr(mod, op.decl.name, op)
    return mod
