"""The inline-CUDA op and the op registry (the plugin boundary). Mirrors the reference's
python/jittor/test/test_code_op.py:259-334 (forward parts) and test_custom_op.py's registration checks."""
import numpy as np
import pytest

import jittor_b200 as jt
from jittor_b200 import op_register

SRC_1D = '''
    __global__ static void kernel1(@ARGS_DEF) {
        @PRECALC
        int i = threadIdx.x + blockIdx.x * blockDim.x;
        int stride = blockDim.x * gridDim.x;
        for (; i<in0_shape0; i+=stride)
            @out(i) = @in0(i)*@in1(i);
    }
        kernel1<<<(in0_shape0-1)/1024+1, 1024>>>(@ARGS);
'''
SRC_2D = '''
    __global__ static void kernel1(@ARGS_DEF) {
        @PRECALC
        for (int i=blockIdx.x; i<in0_shape0; i+=gridDim.x)
        for (int j=threadIdx.x; j<in0_shape1; j+=blockDim.x)
            @out(i,j) = @in0(i,j)*@in1(i,j);
    }
    kernel1<<<32, 32>>>(@ARGS);
'''
SRC_2OUT = '''
    __global__ static void kernel2(@ARGS_DEF) {
        @PRECALC
        for (int i=blockIdx.x; i<in0_shape0; i+=gridDim.x)
        for (int j=threadIdx.x; j<in0_shape1; j+=blockDim.x) {
            @out0(i,j) = @in2(i,j)*@in1(i,j);
            @out1(i,j) = @in2(i,j)*@in0(i,j);
        }
    }
    kernel2<<<32, 32>>>(@ARGS);
'''


def test_registry_names():
    for name in ("reindex", "reindex_reduce", "broadcast_to", "reduce", "binary", "cublas_matmul", "cudnn_conv",
                 "nccl_all_reduce", "code"):
        assert jt.has_op(name)
    assert not jt.has_op("no_such_op")
    with pytest.raises(KeyError):
        jt.get_op_info("no_such_op")
    jt.register_op("my_double", lambda x: x + x)
    y = jt.get_op_info("my_double").get_constructor()(jt.Var([3], "float32"))
    assert list(y.shape) == [3] and y._op.kind == "binary"
    a, b = jt.Var([8, 5], "float32"), jt.Var([7, 5], "float32")
    c = jt.get_op_info("cublas_matmul")(a, b, False, True)
    assert list(c.shape) == [8, 7]
    with pytest.raises(jt.B200Error):
        jt.compile_custom_op("", "", "x")
    with pytest.raises(TypeError):
        jt.code([3], "float32", [], cuda_src="x", cuda_grad=["y"])          # unknown keyword arguments are an error


def test_macro_expansion_and_compile():
    text = op_register.expand_code_source(SRC_2D, "", [("float32", 2), ("float32", 2)], [("float32", 2)])
    assert "@" not in text and "<<<32, 32, 0, __stream>>>" in text
    assert "out0_p[(i)*out0_stride0+(j)*out0_stride1]" in text
    so = op_register.compile_code_source(text)       # nvcc cross-compiles for sm_100a without a GPU
    assert so.endswith(".so")
    with pytest.raises(jt.B200Error):
        op_register.expand_code_source("@nonsense(1);", "", [("float32", 1)], [("float32", 1)])


@pytest.mark.gpu
def test_code_cuda_forward():
    rng = np.random.default_rng(0)
    a, b = rng.random(100000, dtype=np.float32), rng.random(100000, dtype=np.float32)
    va, vb = jt.array(a), jt.array(b)
    c = jt.code(va.shape, va.dtype, [va, vb], cuda_src=SRC_1D)
    assert np.array_equal(c.numpy(), a * b)
    a2, b2 = rng.random((100, 100), dtype=np.float32), rng.random((100, 100), dtype=np.float32)
    v2, w2 = jt.array(a2), jt.array(b2)
    c2 = jt.code(v2.shape, v2.dtype, [v2, w2], cuda_src=SRC_2D)
    assert np.array_equal(c2.numpy(), a2 * b2)
    g = rng.random((100, 100), dtype=np.float32)
    da, db = jt.code([v2.shape, w2.shape], [v2.dtype, w2.dtype], [v2, w2, jt.array(g)], cuda_src=SRC_2OUT)
    assert np.array_equal(da.numpy(), g * b2) and np.array_equal(db.numpy(), g * a2)
    # a code op composes with the meta-operators
    assert np.allclose((c2 + 1.0).sum(1).numpy(), (a2 * b2 + 1).sum(1), rtol=1e-5)


GRAD_A_1D = '''
    __global__ static void kernel2(@ARGS_DEF) {
        @PRECALC
        int i = threadIdx.x + blockIdx.x * blockDim.x;
        int stride = blockDim.x * gridDim.x;
        for (; i<in0_shape0; i+=stride)
            @out(i) = @dout(i)*@in1(i);
    }
        kernel2<<<(in0_shape0-1)/1024+1, 1024>>>(@ARGS);
'''
GRAD_B_1D = GRAD_A_1D.replace("kernel2", "kernel3").replace("@in1(i)", "@in0(i)")
GRAD_A_2D = '''
    __global__ static void kernel(@ARGS_DEF) {
        @PRECALC
        for (int i=blockIdx.x; i<in0_shape0; i+=gridDim.x)
        for (int j=threadIdx.x; j<in0_shape1; j+=blockDim.x)
            @out(i,j) = @dout(i,j)*@in1(i,j);
    }
    kernel<<<32, 32>>>(@ARGS);
'''
GRAD_B_2D = '''
    __global__ static void kernel(@ARGS_DEF) {
        @PRECALC
        @pout(0,0);
        for (int i=blockIdx.x; i<in0_shape0; i+=gridDim.x)
        for (int j=threadIdx.x; j<in0_shape1; j+=blockDim.x)
            @out(i,j) = @dout(i,j)*@in0(i,j) + 0*pout_shape1;
    }
    kernel<<<32, 32>>>(@ARGS);
'''


def test_grad_sources_become_code_ops_with_aliases():
    a, b = jt.Var([100], "float32"), jt.Var([100], "float32")
    c = jt.code(a.shape, a.dtype, [a, b], cuda_src=SRC_1D, cuda_grad_src=[GRAD_A_1D, GRAD_B_1D])
    da, db = jt.grad(c, [a, b])
    assert da.shape == [100] and da._op.kind == "custom" and len(da._op.inputs) == 4      # a, b, dout, c
    assert da._op.inputs[:2] == [a, b] and da._op.inputs[3] is c
    assert db._op.kind == "custom"
    only_a = jt.code(a.shape, a.dtype, [a, b], cuda_src=SRC_1D, cuda_grad_src=[GRAD_A_1D])
    _, gb = jt.grad(only_a, [a, b])
    assert gb._op.kind == "fill"                                                           # no source: zero gradient


@pytest.mark.gpu
def test_code_cuda_gradients():
    """python/jittor/test/test_code_op.py:259-334: forward and both gradient sources, 1-D and 2-D, with @dout / @pout."""
    rng = np.random.default_rng(1)
    a, b = rng.random(100000, dtype=np.float32), rng.random(100000, dtype=np.float32)
    va, vb = jt.array(a), jt.array(b)
    c = jt.code(va.shape, va.dtype, [va, vb], cuda_src=SRC_1D, cuda_grad_src=[GRAD_A_1D, GRAD_B_1D])
    da, db = jt.grad(c, [va, vb])
    assert np.allclose(c.data, a * b) and np.allclose(da.data, b) and np.allclose(db.data, a)
    a2, b2 = rng.random((100, 100), dtype=np.float32), rng.random((100, 100), dtype=np.float32)
    v2, w2 = jt.array(a2), jt.array(b2)
    c2 = jt.code(v2.shape, v2.dtype, [v2, w2], cuda_src=SRC_2D, cuda_grad_src=[GRAD_A_2D, GRAD_B_2D])
    da2, db2 = jt.grad((c2 * 3.0).sum(), [v2, w2])
    assert np.allclose(da2.data, 3 * b2) and np.allclose(db2.data, 3 * a2)


@pytest.mark.gpu
def test_function_with_code_backward():
    """python/jittor/test/test_code_op.py:336-376 (a Function whose backward is a two-output code op) and the doc example of
    python/jittor/__init__.py:1874-1888."""
    class Func(jt.Function):
        def execute(self, a, b):
            self.save_vars = a, b
            return jt.code(a.shape, a.dtype, [a, b], cuda_src=SRC_2D)

        def grad(self, grad):
            a, b = self.save_vars
            return jt.code([a.shape, b.shape], [a.dtype, b.dtype], [a, b, grad], cuda_src=SRC_2OUT)

    rng = np.random.default_rng(2)
    a, b = rng.random((100, 100), dtype=np.float32), rng.random((100, 100), dtype=np.float32)
    va, vb = jt.array(a), jt.array(b)
    c = Func()(va, vb)
    da, db = jt.grad(c, [va, vb])
    assert np.allclose(c.data, a * b) and np.allclose(da.data, b) and np.allclose(db.data, a)

    class MyFunc(jt.Function):
        def execute(self, x, y):
            self.x, self.y = x, y
            return x * y, x / y

        def grad(self, grad0, grad1):
            return (None if grad0 is None else grad0 * self.y), (None if grad1 is None else grad1 * self.x)

    x, y = jt.array(np.float32([3.0])), jt.array(np.float32([4.0]))
    p, q = MyFunc.apply(x, y)
    dx, dy = jt.grad(p + q * 3.0, [x, y])
    assert dx.item() == 4 and dy.item() == 9
