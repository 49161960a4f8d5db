"""Host logic of the general chain fusion (no GPU): which regions become one program, how their statements are ordered,
and what stays a leaf. Mirrors the grouping cases of python/jittor/test/test_fused_op.py:144-176 (reduce + broadcast in
one fused op) and python/jittor/test/test_stop_fuse.py."""
import jittor_b200 as jt
from jittor_b200 import fusion, nn, executor
from jittor_b200 import var as var_mod

OPS = {0: "OPND", 1: "LOAD", 2: "UN", 3: "BIN", 4: "SEL", 5: "TST", 8: "RRED", 9: "RMAP", 10: "STORE", 11: "STROW"}


def ph(shape, dtype="float32"):
    return jt.Var(shape, dtype)


def ops(words):
    return [OPS[d[0]] for d in fusion.decode(words)]


def test_scale_shift_is_one_map():
    x, w, b = ph([64, 4096]), ph([4096]), ph([4096])
    words, inputs, full, k, n = fusion.build_program(x * w + b)
    assert ops(words) == ["LOAD", "BIN", "BIN", "STORE"] and k == 0 and full == [64, 4096]
    assert sorted(view for _, view in inputs) == [[1, 4096], [1, 4096], [64, 4096]]
    assert {id(v) for v in executor._match_fused_chain(x * w + b).leaves} == {id(x), id(w), id(b)}


def test_shared_subexpression_uses_a_temporary():
    x, b = ph([64, 4096]), ph([4096])
    words, inputs, _, _, _ = fusion.build_program(nn.relu(x + b))
    assert ops(words) == ["LOAD", "BIN", "TST", "BIN", "SEL", "OPND", "STORE"]        # x + b is computed once and parked
    assert len(inputs) == 2


def test_multiply_then_row_sum_is_one_reduce_statement():
    a, b = ph([32, 100]), ph([32, 100])
    words, inputs, full, k, _ = fusion.build_program((a * b).sum(1))
    assert ops(words) == ["LOAD", "BIN", "RRED", "STROW"] and k == 1 and full == [32, 100]
    words, _, _, k, _ = fusion.build_program((a * b).sum(1, keepdims=True))
    assert ops(words)[-1] == "STROW" and k == 1


def test_reduce_then_broadcast_back_orders_the_statements():
    x = ph([32, 100])
    y = (x - x.mean(1, keepdims=True)) / ((x * x).mean(1, keepdims=True) + 1e-5).sqrt()
    words, inputs, _, k, _ = fusion.build_program(y)
    o = ops(words)
    assert k == 1 and len(inputs) == 1
    assert o.count("RRED") == 2 and o.count("RMAP") == 1 and o[-1] == "STORE"
    assert o.index("RMAP") > max(i for i, s in enumerate(o) if s == "RRED") - 100      # the per-row map follows its reduce
    # explicit broadcast_to of a per-row value without keepdims
    m = x.max(1)
    z = x - m.broadcast(x, [1])
    words, inputs, _, k, _ = fusion.build_program(z)
    assert ops(words) == ["LOAD", "RRED", "LOAD", "BIN", "STORE"] and len(inputs) == 1


def _softmax_by_hand(x):
    """The meta-op softmax without nn.softmax's own backward rule, so that jt.grad differentiates the chain itself."""
    e = (x - x.max(-1, keepdims=True)).exp()
    return e / e.sum(-1, keepdims=True)


def test_nn_softmax_brings_its_own_backward():
    x, dy = ph([128, 1000]), ph([128, 1000])
    y = nn.softmax(x, -1)
    g = jt.grad((y * dy).sum(), x)
    assert g._op.kind == "custom" and g._op.attrs["name"] == "softmax_backward" and g._op.inputs[0] is y
    g0 = jt.grad((nn.softmax(x, 0) * dy).sum(), x)                      # not the last axis: plain reverse mode
    assert g0._op.kind != "custom"


def test_softmax_backward_is_one_program():
    x, dy = ph([128, 1000]), ph([128, 1000])
    g = jt.grad((_softmax_by_hand(x) * dy).sum(), x)
    prog = fusion.build_program(g)
    assert prog is not None
    words, inputs, full, k, _ = prog
    assert k == 1 and full == [128, 1000] and {id(v) for v, _ in inputs} == {id(x), id(dy)}
    assert ops(words)[-1] == "STORE"


def test_what_is_not_fused():
    x = ph([32, 100])
    assert fusion.build_program(x + 1.0) is None                         # a single op keeps its dedicated kernel
    xi = ph([32, 100], "int32")
    assert fusion.build_program(xi * 2 + 1) is None                      # integer arithmetic is not the float32 class
    xd = ph([32, 100], "float64")
    assert fusion.build_program(xd * 2.0 + 1.0) is None
    col = (x * 2.0).sum(0)                                               # a reduce over leading axes is not a row reduce
    assert fusion.build_program(col) is None
    y = (x * 2.0).stop_fuse()                                            # stop_fuse makes a leaf
    words, inputs, _, _, _ = fusion.build_program((y + 1.0) * 3.0)
    assert [id(v) for v, _ in inputs] == [id(y)]
    with jt.flag_scope(b200_fuse_chains=0):
        assert fusion.build_program(x * 2.0 + 1.0) is None


def test_named_patterns_keep_their_kernels():
    x = ph([32, 4096])
    v = nn.softmax(x, -1)
    first = next(m for m in executor._MATCHERS if m(v) is not None)
    assert first is executor._match_softmax
    a, b = ph([64, 32]), ph([32, 48])
    v = nn.matmul(a, b)
    assert next(m for m in executor._MATCHERS if m(v) is not None) is executor._match_matmul


def test_bf16_chain_keeps_node_dtypes():
    xb, w = ph([8, 16, 6, 6], "bfloat16"), ph([16])
    with jt.flag_scope(amp_reg=2):
        v = nn.relu(xb * w.broadcast(xb, [0, 2, 3]))
    words, inputs, full, k, _ = fusion.build_program(v)
    assert v.dtype == "bfloat16" and fusion.decode(words)[-1][5] == 7             # STORE carries the bfloat16 code
    assert sorted(view for _, view in inputs) == [[1, 16, 1, 1], [8, 16, 6, 6]]


# ---- a reference interpreter of the program, in numpy: checks what the builder emits without a GPU -------------------
import numpy as np

from oracle import meta_ops_ref as ref

_UN = {v: k for k, v in fusion.UNARY_CODES.items()}
_BIN = {v: k for k, v in fusion.BINARY_CODES.items()}
_RED = {v: k for k, v in fusion.REDUCE_CODES.items()}
_DT = ["bool", "int8", "int16", "int32", "int64", "uint8", "float16", "bfloat16", "float32", "float64"]


def interpret(words, inputs, full, k, arrays):
    """Evaluates a program on numpy arrays (arrays[i] is the value of inputs[i][0]); float32 arithmetic, results of
    float32 / bool nodes only (enough for the host tests)."""
    d = len(full)
    rows_shape = full[:d - k]
    vals = [np.asarray(arrays[id(v)], dtype=np.float32).reshape(view) for v, view in inputs]
    rowval, tmp, acc, out = {}, {}, None, None
    dec = fusion.decode(words)
    i = 0

    def operand(e):
        _, _, kind, idx, _, _, const = e
        return {1: lambda: vals[idx], 2: lambda: np.float32(const), 3: lambda: rowval[idx], 4: lambda: tmp[idx]}[kind]()

    while i < len(dec):
        op, sub, kind, idx, swap, dt, const = dec[i]
        if op == 1:
            acc = operand(dec[i])
        elif op == 2:
            acc = acc if _UN[sub] == "cast" else ref.unary(np.asarray(acc, np.float32), _UN[sub])
        elif op == 3:
            o = operand(dec[i])
            a, b = (o, acc) if swap else (acc, o)
            acc = ref.binary(np.asarray(a, np.float32), np.asarray(b, np.float32), _BIN[sub])
        elif op == 4:
            o1 = operand(dec[i])
            i += 1
            o2 = operand(dec[i])
            acc = np.where(np.asarray(acc) != 0, o1, o2)
        elif op == 5:
            tmp[idx] = acc
        elif op == 8:
            full_acc = np.broadcast_to(np.asarray(acc, np.float32), full)
            axes = tuple(range(d - k, d))
            f = {"add": np.sum, "mean": np.mean, "maximum": np.max, "minimum": np.min, "multiply": np.prod}[_RED[sub]]
            rowval[idx] = f(full_acc.astype(np.float64), axis=axes, keepdims=True).astype(np.float32)
        elif op == 9:
            rowval[idx] = np.broadcast_to(np.asarray(acc, np.float32), rows_shape + [1] * k)
        elif op == 10:
            out = np.broadcast_to(acc, full)
        elif op == 11:
            out = np.broadcast_to(rowval[idx], rows_shape + [1] * k).reshape(rows_shape or [1])
        if op not in (5, 8, 9) and dt == 0 and op in (2, 3, 4):
            acc = np.asarray(acc) != 0
        i += 1
    return np.asarray(out)


def _check_program(build, shapes, seed=0):
    rng = np.random.default_rng(seed)
    vars_ = [ph(s) for s in shapes]
    arrays = {id(v): rng.uniform(0.5, 1.5, size=s).astype(np.float32) for v, s in zip(vars_, shapes)}
    v = build(*vars_)
    prog = fusion.build_program(v)
    assert prog is not None
    words, inputs, full, k, _ = prog
    got = interpret(words, inputs, full, k, arrays)
    return got.reshape(list(v.shape)), [arrays[id(x)] for x in vars_]


def test_programs_compute_the_right_thing():
    got, (x, w, b) = _check_program(lambda X, W, B: X * W + B, [(6, 16), (16,), (16,)])
    assert np.allclose(got, x * w + b)
    got, (x, w) = _check_program(lambda X, W: 2.0 - X / W, [(6, 16), (16,)])
    assert np.allclose(got, 2.0 - x / w)
    got, (x, w, b) = _check_program(lambda X, W, B: (X + W) * (X - B) / (X * B + W), [(6, 16), (16,), (16,)])
    assert np.allclose(got, (x + w) * (x - b) / (x * b + w), rtol=1e-5)
    got, (x, b) = _check_program(lambda X, B: nn.relu(X - B), [(6, 16), (16,)])
    assert np.allclose(got, np.maximum(x - b, 0))
    got, (x,) = _check_program(lambda X: (X - X.mean(1, keepdims=True)) / ((X * X).mean(1, keepdims=True) + 1e-5).sqrt(), [(5, 24)])
    assert np.allclose(got, (x - x.mean(1, keepdims=True)) / np.sqrt((x * x).mean(1, keepdims=True) + 1e-5), rtol=1e-4, atol=1e-6)
    got, (x, y) = _check_program(lambda X, Y: (X * Y).sum(1), [(5, 24), (5, 24)])
    assert np.allclose(got, (x * y).sum(1), rtol=1e-5)


def test_softmax_backward_program_matches_the_formula():
    got, (x, dy) = _check_program(lambda X, DY: jt.grad((_softmax_by_hand(X) * DY).sum(), X), [(7, 33), (7, 33)], seed=3)
    e = np.exp(x - x.max(1, keepdims=True))
    y = e / e.sum(1, keepdims=True)
    want = y * (dy - (y * dy).sum(1, keepdims=True))
    assert np.allclose(got, want, rtol=1e-4, atol=1e-6)


def test_generated_sources_compile_for_sm_100a():
    """Every kind of program goes through the generator and NVRTC (no GPU involved): map with column / row / general
    broadcasts, flat maps with a ragged tail, rows kernels of both group widths, bf16 and fp16 nodes, select."""
    cases = [
        lambda: ph([64, 4096]) * ph([4096]) + ph([4096]),
        lambda: nn.relu(ph([64, 4096]) + ph([4096])),
        lambda: (ph([7, 33]) * 2.0 + 1.0).exp(),
        lambda: ph([4, 1, 8]) * ph([1, 5, 8]) + ph([4, 5, 1]),
        lambda: ph([6, 16]) * ph([6, 1]) - ph([1]),
        lambda: (ph([64, 4096]) * ph([64, 4096])).sum(1),
        lambda: (ph([64, 100]) * ph([64, 100])).reduce("maximum", 1),
        lambda: (lambda X: (X - X.mean(1, keepdims=True)) / ((X * X).mean(1, keepdims=True) + 1e-5).sqrt())(ph([5, 24])),
        lambda: (lambda X: (X - X.mean(1, keepdims=True)) / ((X * X).mean(1, keepdims=True) + 1e-5).sqrt())(ph([5, 2400])),
        lambda: nn.relu(ph([64, 4096], "bfloat16") * ph([4096], "bfloat16")),
        lambda: (ph([64, 40], "float16") + ph([40], "float16")).sigmoid(),
        lambda: (ph([7, 33]).tanh() % 0.7) ** 2.0,
    ]
    for i, f in enumerate(cases):
        v = f()
        prog = fusion.build_program(v)
        assert prog is not None, i
        words, inputs, full, k, _ = prog
        src, ok, log = fusion.program_source(words, inputs, full, k, list(v.shape), v.dtype)
        assert ok, (i, log)
        assert ("chain_jit_map_kernel" in src) != ("chain_jit_rows_kernel" in src)


def test_layernorm_backward_is_one_program():
    """The gradient of LayerNorm with respect to its input, as jt.grad builds it from the per-op rules: four row reduces and
    a store sweep over x, dy and gamma in ONE program (five temporaries), checked with the numpy interpreter against the
    closed form."""
    rng = np.random.default_rng(11)
    X, DY, G, B = ph([6, 40]), ph([6, 40]), ph([40]), ph([40])
    arrays = {id(X): rng.normal(size=(6, 40)).astype(np.float32), id(DY): rng.normal(size=(6, 40)).astype(np.float32),
              id(G): (1 + 0.1 * rng.normal(size=40)).astype(np.float32), id(B): rng.normal(size=40).astype(np.float32)}
    dx = jt.grad((nn.layer_norm(X, (40,), G, B) * DY).sum(), X)
    prog = fusion.build_program(dx)
    assert prog is not None
    words, inputs, full, k, _ = prog
    assert ops(words).count("RRED") == 4 and ops(words)[-1] == "STORE" and len(inputs) == 3
    got = interpret(words, inputs, full, k, arrays).reshape(6, 40)
    x, dy, g = (arrays[id(v)].astype(np.float64) for v in (X, DY, G))
    mean, var = x.mean(1, keepdims=True), x.var(1, keepdims=True)
    xh, rstd = (x - mean) / np.sqrt(var + 1e-5), 1 / np.sqrt(var + 1e-5)
    dyg = dy * g
    want = rstd * (dyg - dyg.mean(1, keepdims=True) - xh * (dyg * xh).mean(1, keepdims=True))
    assert np.allclose(got, want, rtol=1e-3, atol=1e-4)
    src, ok, log = fusion.program_source(words, inputs, full, k, [6, 40], "float32")
    assert ok, log


def test_scalar_stretched_over_every_axis_is_a_broadcast_input():
    """The gradient of `.sum()` is a [1] value broadcast over all axes of its operand; multiplied by another tensor it must
    be one map kernel (the scalar as a broadcast input), not a materialised tensor of ones."""
    x, dy = ph([8, 16, 12, 12], "bfloat16"), ph([8, 16, 12, 12], "bfloat16")
    seed = ph([1], "float32")
    full = jt.Var([8, 16, 12, 12], "float32", var_mod.Op("broadcast_to", [seed], bcast_mask=15, keepdims_mask=0))   # the reduce rule's form
    z = full.bfloat16() * dy
    words, inputs, shape, k, n = fusion.build_program(z)
    assert ops(words) == ["LOAD", "UN", "BIN", "STORE"] and k == 0 and shape == [8, 16, 12, 12]
    assert sorted(view for _, view in inputs) == [[1, 1, 1, 1], [8, 16, 12, 12]]
    src, ok, log = fusion.program_source(words, inputs, shape, k, shape, "bfloat16")
    assert ok, log
    # as jt.grad builds it: a scaled sum leaves broadcast(scale) * dy, one map kernel; a plain sum leaves dy itself
    g = jt.grad((x * dy).sum() * 3.0, x)
    assert fusion.build_program(g) is not None
    assert jt.grad((x * dy).sum(), x) is dy
