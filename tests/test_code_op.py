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
    with pytest.raises(NotImplementedError):
        jt.compile_custom_op("", "", "x")


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
