"""compile_custom_ops / compile_custom_op with the op sources of the reference's own test
(python/jittor/test/test_custom_op.py:12-107 -- the header / source pair written to files, and the pair passed as strings)
plus an op with inputs, attributes and a CUDA branch. Parsing, the constructor library, output shape inference and the
jit defines are checked without a GPU; running the ops is a GPU test."""
import os

import numpy as np
import pytest

import jittor_b200 as jt

HEADER = """
#pragma once
#include "op.h"

namespace jittor {

struct CustomOp : Op {
    Var* output;
    CustomOp(NanoVector shape, NanoString dtype=ns_float32);

    const char* name() const override { return "custom"; }
    DECLARE_jit_run;
};

} // jittor
"""

SRC = """
#include "var.h"
#include "custom_op.h"

namespace jittor {
#ifndef JIT
CustomOp::CustomOp(NanoVector shape, NanoString dtype) {
    output = create_output(shape, dtype);
}

void CustomOp::jit_prepare(JK& jk) {
    add_jit_define(jk, "T", output->dtype());
}

#else // JIT
#ifdef JIT_cpu
void CustomOp::jit_run() {
    index_t num = output->num;
    auto* __restrict__ x = output->ptr<T>();
    for (index_t i=0; i<num; i++)
        x[i] = (T)i;
}
#else
void CustomOp::jit_run() {
}
#endif // JIT_cpu
#endif // JIT

} // jittor
"""

MY_HEADER = """
struct MyOp : Op {
    Var* output;
    MyOp(NanoVector shape, NanoString dtype=ns_float32);

    const char* name() const override { return "my"; }
    DECLARE_jit_run;
};
"""

MY_SRC = """
#ifndef JIT
MyOp::MyOp(NanoVector shape, NanoString dtype) {
    output = create_output(shape, dtype);
}

void MyOp::jit_prepare(JK& jk) {
    add_jit_define(jk, "T", output->dtype());
}

#else // JIT
void MyOp::jit_run() {
    index_t num = output->num;
    auto* __restrict__ x = output->ptr<T>();
    for (index_t i=0; i<num; i++)
        x[i] = (T)-i;
}
#endif // JIT
"""

# an op with two inputs, a scalar attribute and a CUDA kernel: z = alpha * x + y, and a second output with the row sums of x
AXPY_HEADER = """
struct AxpyRowsOp : Op {
    Var* x, * y, * z, * rows;
    float alpha;
    AxpyRowsOp(Var* x, Var* y, float alpha=1.0);

    const char* name() const override { return "axpy_rows"; }
    DECLARE_jit_run;
};
"""

AXPY_SRC = """
#ifndef JIT
AxpyRowsOp::AxpyRowsOp(Var* x, Var* y, float alpha) : x(x), y(y), alpha(alpha) {
    CHECK(x->shape == y->shape);
    z = create_output(x->shape, x->dtype());
    rows = create_output({x->shape[0]}, x->dtype());
}
void AxpyRowsOp::jit_prepare(JK& jk) {
    add_jit_define(jk, "T", x->dtype());
    add_jit_define(jk, "COLS", x->shape[1]);
}
#else // JIT
#ifdef JIT_cuda
static __global__ void axpy_kernel(const T* x, const T* y, T* z, T* rows, float alpha, int n_rows) {
    for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
        T acc = 0;
        for (int c = threadIdx.x; c < COLS; c += blockDim.x) {
            z[r * COLS + c] = alpha * x[r * COLS + c] + y[r * COLS + c];
            acc += x[r * COLS + c];
        }
        for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
        if (threadIdx.x == 0) rows[r] = acc;
    }
}
void AxpyRowsOp::jit_run() {
    axpy_kernel<<<64, 32>>>(x->ptr<T>(), y->ptr<T>(), z->ptr<T>(), rows->ptr<T>(), alpha, (int)x->shape[0]);
}
#endif
#endif // JIT
"""


def test_header_scan_and_output_inference(tmp_path):
    hname, ccname = str(tmp_path / "custom_op.h"), str(tmp_path / "custom_op.cc")
    open(hname, "w").write(HEADER)
    open(ccname, "w").write(SRC)
    cops = jt.compile_custom_ops([hname, ccname])
    a = cops.custom([3, 4, 5], "float")
    assert a.shape == [3, 4, 5] and a.dtype == "float32"
    assert jt.has_op("custom") and jt.get_op_info("custom").get_constructor() is cops.custom
    b = cops.custom([7], "int32")
    assert b.shape == [7] and b.dtype == "int32"
    assert cops.custom([2, 2]).dtype == "float32"                     # the header's default argument


def test_op_with_inputs_attributes_and_two_outputs():
    op = jt.compile_custom_op(AXPY_HEADER, AXPY_SRC, "axpy_rows")
    x, y = jt.Var([6, 40], "float32"), jt.Var([6, 40], "float32")
    z, rows = op(x, y, 2.5)
    assert z.shape == [6, 40] and rows.shape == [6] and z.dtype == "float32"
    assert z._op.inputs == [x, y]
    with pytest.raises(jt.B200Error, match="Check failed"):
        op(x, jt.Var([6, 41], "float32"))                             # the constructor's own CHECK reaches the caller
    with pytest.raises(TypeError):
        op(x)


def test_unknown_parameter_types_and_missing_core_are_reported():
    with pytest.raises(jt.B200Error, match="type the binding generator does not know"):
        jt.compile_custom_op("""struct BadOp : Op {
            Var* y;
            BadOp(std::map<int,int> m);
            const char* name() const override { return "bad"; }
            DECLARE_jit_run;
        };""", "", "bad")
    with pytest.raises(jt.B200Error, match="failed"):
        jt.compile_custom_op(MY_HEADER.replace("MyOp", "NeedOp").replace('"my"', '"need"'),
                             "#ifndef JIT\nNeedOp::NeedOp(NanoVector s, NanoString d) { output = create_output(s, d); exe.run_sync({}, true); }\nvoid NeedOp::jit_prepare(JK& jk) {}\n#endif\n", "need")


@pytest.mark.gpu
def test_reference_custom_ops_run(tmp_path):
    hname, ccname = str(tmp_path / "custom_op.h"), str(tmp_path / "custom_op.cc")
    open(hname, "w").write(HEADER)
    open(ccname, "w").write(SRC)
    cops = jt.compile_custom_ops([hname, ccname])
    a = cops.custom([3, 4, 5], "float")
    na = a.data
    assert a.shape == [3, 4, 5] and a.dtype == "float"
    assert (na.flatten() == range(3 * 4 * 5)).all(), na
    my_op = jt.compile_custom_op(MY_HEADER, MY_SRC, "my")
    a = my_op([3, 4, 5], "float")
    na = a.data
    assert a.shape == [3, 4, 5] and a.dtype == "float"
    assert (-na.flatten() == range(3 * 4 * 5)).all(), na
    # the result is an ordinary Var: it feeds the built-in kernels
    assert float((a * 2.0).sum().item()) == -2.0 * sum(range(60))


@pytest.mark.gpu
def test_custom_cuda_op_runs_on_device_pointers():
    op = jt.compile_custom_op(AXPY_HEADER, AXPY_SRC, "axpy_rows")
    rng = np.random.default_rng(0)
    x, y = rng.normal(size=(70, 33)).astype(np.float32), rng.normal(size=(70, 33)).astype(np.float32)
    z, rows = op(jt.array(x), jt.array(y), 0.5)
    assert np.allclose(z.numpy(), 0.5 * x + y, atol=1e-6)
    assert np.allclose(rows.numpy(), x.sum(1), atol=1e-4)
    z2, _ = jt.get_op_info("axpy_rows")(jt.array(x) + 1.0, jt.array(y))            # lazy input, default alpha
    assert np.allclose(z2.numpy(), x + 1.0 + y, atol=1e-6)
